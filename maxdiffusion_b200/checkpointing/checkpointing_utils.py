"""Checkpoint manager with the Orbax directory layout: `<dir>/<step>/<item_name>/...`.

Item names per checkpoint type are the reference's (src/maxdiffusion/checkpointing/checkpointing_utils.py:42-116):
Wan `{wan_config, wan_state | low_noise_transformer_state + high_noise_transformer_state}`, Flux `{flux_state,
flux_config, vae_state, vae_config, scheduler, scheduler_config, text_encoder_2_state, text_encoder_2_config}`,
SD/SDXL `{unet_config, vae_config, text_encoder_config, scheduler_config, unet_state, vae_state,
text_encoder_state, tokenizer_config}` (+ `text_encoder_2_*`), Z-Image `{transformer_state, vae_state,
text_encoder_state, z_image_config}`, `iter` for the data iterator.

The layout (directory names, item names, tree paths, array orientation) is the reference's; the bytes are NOT
Orbax / tensorstore: an Orbax reader cannot open these checkpoints and this manager cannot open Orbax ones. A state
item is a directory with `state.safetensors` (keys = '/'-joined tree paths, arrays in the reference's flax
orientation), `_METADATA` (tree paths, shapes, dtypes) and, for sharded optimizer state, one
`process_<rank>.safetensors` per rank of the shard group plus `_sharding` (group size); JSON items are a single
`metadata` file; each step directory carries `_CHECKPOINT_METADATA`. Saves go to a temporary directory that rank 0
creates (the other ranks wait for it through the rendezvous store, or by polling when there is none) and renames
once every rank's shard file is there; a rank that does not show up within `timeout_s` makes the save raise instead
of committing a checkpoint with missing files. Optionally the write runs on a background thread
(`enable_async_checkpointing`).
"""
from __future__ import annotations

import json
import os
import re
import shutil
import threading
import time
from typing import Dict, Optional, Sequence

import numpy as np
import torch

WAN_CHECKPOINT = "WAN_CHECKPOINT"
FLUX_CHECKPOINT = "FLUX_CHECKPOINT"
STABLE_DIFFUSION_CHECKPOINT = "STABLE_DIFUSSION_CHECKPOINT"
STABLE_DIFFUSION_XL_CHECKPOINT = "STABLE_DIFFUSION_XL_CHECKPOINT"
LTX2_CHECKPOINT = "LTX2_CHECKPOINT"
Z_IMAGE_CHECKPOINT = "Z_IMAGE_CHECKPOINT"

ITEM_NAMES = {
    WAN_CHECKPOINT: ("low_noise_transformer_state", "high_noise_transformer_state", "wan_state", "wan_config"),
    FLUX_CHECKPOINT: ("flux_state", "flux_config", "vae_state", "vae_config", "scheduler", "scheduler_config",
                      "text_encoder_2_state", "text_encoder_2_config"),
    STABLE_DIFFUSION_CHECKPOINT: ("unet_config", "vae_config", "text_encoder_config", "scheduler_config", "unet_state",
                                  "vae_state", "text_encoder_state", "tokenizer_config"),
    STABLE_DIFFUSION_XL_CHECKPOINT: ("unet_config", "vae_config", "text_encoder_config", "scheduler_config",
                                     "unet_state", "vae_state", "text_encoder_state", "tokenizer_config",
                                     "text_encoder_2_state", "text_encoder_2_config"),
    LTX2_CHECKPOINT: ("ltx2_state", "ltx2_config"),
    Z_IMAGE_CHECKPOINT: ("transformer_state", "vae_state", "text_encoder_state", "z_image_config"),
}


def item_names_for(checkpoint_type: str, dataset_type: str = "") -> tuple:
  names = ITEM_NAMES[checkpoint_type]
  return names + ("iter",) if dataset_type == "grain" else names


def _to_torch(a):
  if isinstance(a, torch.Tensor):
    return a.detach().cpu().contiguous()
  return torch.from_numpy(np.ascontiguousarray(a))


class CheckpointManager:

  def __init__(self, directory: str, item_names: Sequence[str], enable_async: bool = True, rank: int = 0,
               save_interval_steps: int = 1, max_to_keep: Optional[int] = None, store=None, timeout_s: float = 600.0):
    self.directory = directory
    self.store = store          # key-value store shared by the ranks (torch.distributed store), or None
    self.timeout_s = timeout_s
    self._saves = 0
    self.item_names = tuple(item_names)
    self.enable_async = enable_async
    self.rank = rank
    self.max_to_keep = max_to_keep
    self._thread: Optional[threading.Thread] = None
    self._error: Optional[BaseException] = None
    if directory and rank == 0:
      os.makedirs(directory, exist_ok=True)

  # ---- steps -------------------------------------------------------------------------------
  def all_steps(self) -> list[int]:
    if not self.directory or not os.path.isdir(self.directory):
      return []
    steps = []
    for name in os.listdir(self.directory):
      if re.fullmatch(r"\d+", name) and os.path.exists(os.path.join(self.directory, name, "_CHECKPOINT_METADATA")):
        steps.append(int(name))
    return sorted(steps)

  def latest_step(self) -> Optional[int]:
    steps = self.all_steps()
    return steps[-1] if steps else None

  # ---- save --------------------------------------------------------------------------------
  def save(self, step: int, items: Dict[str, object], sharded: Optional[Dict[str, Dict[str, torch.Tensor]]] = None,
           world_size: int = 1, shard_rank: Optional[int] = None) -> None:
    """`items`: name -> dict (JSON item) or flat {path: array} (state item), written by rank 0.
    `sharded`: name -> {key: tensor}, written as `process_<shard_rank>.safetensors` inside the item by every rank that
    passes one (`world_size` files are expected in all; `shard_rank` defaults to the manager's rank)."""
    for name in list(items) + list(sharded or {}):
      if name not in self.item_names:
        raise ValueError(f"item '{name}' is not one of {self.item_names}")
    self.wait_until_finished()
    host_items = {}
    for name, payload in (items.items() if self.rank == 0 else ()):  # only rank 0 writes the replicated items
      if self._is_json(payload):
        host_items[name] = ("json", payload)
      else:
        host_items[name] = ("state", {k: _to_torch(v) for k, v in payload.items()})
    host_sharded = {n: {k: _to_torch(v) for k, v in d.items()} for n, d in (sharded or {}).items()}

    def work():
      try:
        self._write(step, host_items, host_sharded, world_size, self.rank if shard_rank is None else shard_rank)
      except BaseException as e:  # surfaced by wait_until_finished
        self._error = e

    if self.enable_async:
      self._thread = threading.Thread(target=work, daemon=True)
      self._thread.start()
    else:
      work()
      self.wait_until_finished()

  @staticmethod
  def _is_json(payload) -> bool:
    return isinstance(payload, dict) and not any(isinstance(v, (torch.Tensor, np.ndarray)) for v in payload.values())

  def _announce(self, key: str) -> None:
    if self.store is not None:
      self.store.set(key, "1")

  def _await(self, key: str, path: str, what: str) -> None:
    """Waits until `key` is in the store (or, without a store, until `path` exists); raises after `timeout_s`."""
    deadline = time.time() + self.timeout_s
    while True:
      if self.store is not None:
        try:
          if self.store.check([key]):
            return
        except Exception:
          pass
      elif os.path.exists(path):
        return
      if time.time() > deadline:
        raise TimeoutError(f"checkpoint step {what}: not seen within {self.timeout_s:.0f} s")
      time.sleep(0.05)

  def _write(self, step, host_items, host_sharded, world_size, shard_rank):
    from safetensors.torch import save_file

    final = os.path.join(self.directory, str(step))
    tmp = final + ".orbax-checkpoint-tmp"
    self._saves += 1
    tag = f"mdb_ckpt/{os.path.abspath(self.directory)}/{step}/{self._saves}"
    if self.rank == 0:
      if os.path.isdir(tmp):
        shutil.rmtree(tmp)  # left over from a run that died while saving; nobody writes into it yet
      os.makedirs(tmp, exist_ok=True)
      for name, (kind, payload) in host_items.items():
        d = os.path.join(tmp, name)
        os.makedirs(d, exist_ok=True)
        if kind == "json":
          with open(os.path.join(d, "metadata"), "w") as f:
            json.dump(payload, f, indent=1, default=str)
        else:
          save_file(payload, os.path.join(d, "state.safetensors"))
          meta = {k: {"shape": list(v.shape), "dtype": str(v.dtype).replace("torch.", "")} for k, v in payload.items()}
          with open(os.path.join(d, "_METADATA"), "w") as f:
            json.dump({"tree_metadata": meta, "format": "safetensors-per-item"}, f)
      for name in host_sharded:
        os.makedirs(os.path.join(tmp, name), exist_ok=True)
      with open(os.path.join(tmp, "_tmp_ready"), "w") as f:
        f.write(tag)
      self._announce(tag + "/tmp")
    elif host_sharded:
      self._await(tag + "/tmp", os.path.join(tmp, "_tmp_ready"), f"{step}: temporary directory of rank 0")
    for name, tensors in host_sharded.items():
      d = os.path.join(tmp, name)
      save_file(tensors, os.path.join(d, f"process_{shard_rank}.safetensors"))
      with open(os.path.join(d, f"process_{shard_rank}.done"), "w") as f:
        f.write("ok")
      self._announce(f"{tag}/{name}/{shard_rank}")
    if self.rank == 0:
      for name in host_sharded:
        for r in range(world_size):
          self._await(f"{tag}/{name}/{r}", os.path.join(tmp, name, f"process_{r}.done"), f"{step}: shard file of rank {r}")
        with open(os.path.join(tmp, name, "_sharding"), "w") as f:
          json.dump({"world_size": world_size}, f)
      os.remove(os.path.join(tmp, "_tmp_ready"))
      with open(os.path.join(tmp, "_CHECKPOINT_METADATA"), "w") as f:
        json.dump({"step": step, "item_names": list(host_items) + list(host_sharded), "commit_timestamp": time.time()}, f)
      if os.path.isdir(final):
        shutil.rmtree(final)
      os.replace(tmp, final)
      if self.max_to_keep:
        for old in self.all_steps()[:-self.max_to_keep]:
          shutil.rmtree(os.path.join(self.directory, str(old)), ignore_errors=True)

  def wait_until_finished(self) -> None:
    if self._thread is not None:
      self._thread.join()
      self._thread = None
    if self._error is not None:
      err, self._error = self._error, None
      raise err

  # ---- restore -----------------------------------------------------------------------------
  def restore_json(self, step: int, name: str) -> dict:
    with open(os.path.join(self.directory, str(step), name, "metadata")) as f:
      return json.load(f)

  single_replica = False   # `enable_single_replica_ckpt_restoring`: one rank reads, the others receive

  def restore_state(self, step: int, name: str) -> Dict[str, torch.Tensor]:
    """The tensors of a state item. With `single_replica` and several ranks, rank 0 alone reads the file and
    broadcasts names, shapes and contents; the other ranks never touch the disk (what the reference's
    `enable_single_replica_ckpt_restoring` does for replicas on a shared file system,
    src/maxdiffusion/checkpointing/checkpointing_utils.py:246-267). Every rank has to make the call."""
    from safetensors.torch import load_file

    path = os.path.join(self.directory, str(step), name, "state.safetensors")
    import torch.distributed as dist

    if not (self.single_replica and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
      return load_file(path)
    src = 0
    state = load_file(path) if dist.get_rank() == src else None
    meta = [[(k, tuple(v.shape), v.dtype) for k, v in state.items()] if state is not None else None]
    dist.broadcast_object_list(meta, src=src)
    # collectives of the default group run on its own device type
    device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    out = {}
    for key, shape, dtype in meta[0]:
      t = state[key].to(device) if state is not None else torch.empty(shape, dtype=dtype, device=device)
      dist.broadcast(t, src=src)
      out[key] = t.cpu()
    return out

  def restore_sharded(self, step: int, name: str) -> list[Dict[str, torch.Tensor]]:
    """Every rank's shard file, in rank order (the caller re-shards for the current topology)."""
    from safetensors.torch import load_file

    d = os.path.join(self.directory, str(step), name)
    with open(os.path.join(d, "_sharding")) as f:
      world = json.load(f)["world_size"]
    return [load_file(os.path.join(d, f"process_{r}.safetensors")) for r in range(world)]

  def has_item(self, step: int, name: str) -> bool:
    return os.path.isdir(os.path.join(self.directory, str(step), name))


def create_checkpoint_manager(checkpoint_dir: str, checkpoint_type: str, enable_async: bool = True,
                              dataset_type: str = "", rank: int = 0, store=None, single_replica: bool = False) -> CheckpointManager:
  mgr = CheckpointManager(checkpoint_dir, item_names_for(checkpoint_type, dataset_type), enable_async, rank, store=store)
  mgr.single_replica = bool(single_replica)
  return mgr
