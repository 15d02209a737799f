"""Wan checkpointing: periodic / final saves of the transformer (+ optimizer) and resume, and the
pretrained-weights cache in checkpoint layout.

Reference: `WanCheckpointer` and its 2.1 / 2.2 / I2V / VACE subclasses
(src/maxdiffusion/checkpointing/wan_checkpointer.py:54-231, wan_checkpointer_2_1.py:26-82,
wan_checkpointer_2_2.py:26-106). Items: `wan_config` (JSON of the transformer config) and `wan_state` (2.2:
`high_noise_transformer_state`, `low_noise_transformer_state`) holding the parameters under the reference's flax
tree paths; with `save_optimizer` the AdamW moments of every rank are stored next to them and re-sharded on restore,
so a run can resume on a different number of GPUs. Unlike the reference, whose restored optimizer state is dropped
(src/maxdiffusion/trainers/base_wan_trainer.py:267 discards the result of `state.replace`), the moments and the
step counter are installed.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import max_logging
from ..loaders.wan_loader import diffusers_to_flax_tree, diffusers_to_ours, flax_tree_to_diffusers, ours_to_diffusers
from ..parallel.tensor import full_from_shards, gather_full, shard_of_full, tensor_parallel_specs
from .checkpointing_utils import WAN_CHECKPOINT, create_checkpoint_manager


def _param_names(trainer):
  names = [[n for n, _ in b.named_parameters()] for b in trainer.model.blocks]
  block_ids = {id(p) for b in trainer.model.blocks for p in b.parameters()}
  root = [n for n, p in trainer.model.named_parameters() if id(p) not in block_ids]
  return names, root


def _tensor_axis(trainer):
  """(size, this rank's index, group, per-block {parameter name: slice spec}) of the trainer's tensor axis."""
  T = trainer.mesh.size("tensor")
  if T == 1:
    return 1, 0, None, [{} for _ in trainer.model.blocks]
  return (T, trainer.mesh.index_in("tensor"), trainer.mesh.group("tensor"),
          [tensor_parallel_specs(b) for b in trainer.model.blocks])


def _specs_by_name(trainer, i, blk_names):
  """Slice specs of block i's parameters for a run that is NOT tensor parallel itself (it restores the moments of one
  that was): which parameters a tensor-parallel run splits follows from the block's structure alone."""
  out = []
  for n in blk_names:
    leaf = n.rsplit(".", 1)[-1]
    if n.endswith(("to_qkv.weight", "to_qkv.bias")):
      out.append(("col", 3))
    elif n.endswith(("to_kv.weight", "to_kv.bias", "add_kv_proj.weight", "add_kv_proj.bias")):
      out.append(("col", 2))
    elif n.endswith(("to_q.weight", "to_q.bias", "ffn_in.weight", "ffn_in.bias")) or leaf in ("norm_q", "norm_k", "norm_added_k"):
      out.append(("col", 1))
    elif n.endswith(("to_out.weight", "ffn_out.weight")):
      out.append(("row", 1))
    else:
      out.append(None)
  return out


def _reshard_flat_over_tensor_axis(flats, full_shapes, specs, group, T: int, t_rank: int) -> torch.Tensor:
  """Flat per-block moments written by `len(flats)` tensor ranks -> the flat buffer of tensor rank `t_rank` of `T`.

  Every saved buffer is cut into its per-parameter views (the slice shapes follow from the full shapes and the specs,
  the offsets from the flat layout's alignment rule), the slices are joined into full tensors and cut again for the
  restoring run; `group` is the restoring run's flat layout of the block."""
  from ..parallel.fsdp import _ALIGN

  saved_t = len(flats)
  fulls = []
  offs = [0] * saved_t
  for shape, spec in zip(full_shapes, specs):
    parts = []
    for t in range(saved_t):
      local = shard_of_full(torch.empty(shape, device="meta"), spec, saved_t, t).shape
      numel = 1
      for d in local:
        numel *= d
      parts.append(flats[t][offs[t]:offs[t] + numel].view(local))
      offs[t] += (numel + _ALIGN - 1) // _ALIGN * _ALIGN
    fulls.append(full_from_shards(parts, spec) if spec is not None else parts[0])
  out = flats[0].new_zeros(group.numel)
  for full, spec, off in zip(fulls, specs, group.offsets):
    piece = shard_of_full(full, spec, T, t_rank).reshape(-1)
    out[off:off + piece.numel()].copy_(piece)
  return out


class WanCheckpointer:

  def __init__(self, config, checkpoint_type: str = WAN_CHECKPOINT):
    self.config = config
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    self.rank = rank
    self.world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    store = None
    if self.world > 1:
      try:
        store = dist.distributed_c10d._get_default_store()
      except Exception:
        store = None
    self.manager = create_checkpoint_manager(config.get("checkpoint_dir", ""), checkpoint_type,
                                             enable_async=bool(config.get("enable_async_checkpointing", True)),
                                             dataset_type=str(config.get("dataset_type", "")), rank=rank, store=store,
                                             single_replica=bool(config.get("enable_single_replica_ckpt_restoring", False)))

  # ---- training state ----------------------------------------------------------------------
  def save(self, step: int, trainer) -> None:
    names, root = _param_names(trainer)
    eng = trainer.engine
    T, t_rank, t_group, specs = _tensor_axis(trainer)
    full = {}
    for i, (g, blk_names) in enumerate(zip(eng.groups, names)):
      flat = eng.full_block_flat(i)  # collective when sharded: every rank takes part, only rank 0 keeps the result
      for n, v in zip(blk_names, g.views(flat)):
        if T > 1 and specs[i].get(n) is not None:
          # a tensor-parallel rank holds its heads / FFN units only: the full parameter is assembled over the tensor axis
          v = gather_full(v, specs[i][n], t_group)
        if self.rank == 0:
          full[f"blocks.{i}.{n}"] = v.to("cpu")
      del flat
    cfg = trainer.wan_cfg
    items = {}
    if self.rank == 0:
      for n, v in zip(root, eng.root.views(eng.root_flat)):
        full[n] = v.to("cpu")
      tree = diffusers_to_flax_tree(ours_to_diffusers(full, cfg.in_channels, tuple(cfg.patch_size)),
                                    scan_layers=bool(self.config.get("scan_layers", True)))
      items = {"wan_config": cfg.to_dict(), "wan_state": tree}
    sharded = None
    writers = 1
    if self.config.get("save_optimizer", False):
      # The moments are sharded over the engine's shard group only; replicas (the `data` axis, and `tensor`) hold
      # identical copies, so exactly one replica writes: the ranks whose shard group contains global rank 0. Files are
      # numbered by the rank INSIDE the shard group, which is what `maybe_restore` re-shards by.
      # The ranks of the tensor axis hold the moments of different slices, so every one of them writes too: file
      # t * (ranks of a shard group) + (rank inside the shard group) for tensor rank t.
      shard_ranks = trainer.mesh.ranks("shard") if eng.world > 1 else [self.rank]
      writers = eng.world * T
      first_replica = trainer.mesh.coords.get("data", 0) == 0 if T > 1 else (0 in shard_ranks or self.world == 1)
      if first_replica:
        st = eng.optimizer_state()
        shard = {"step": torch.tensor([st["step"]]), "root_m": st["root_m"], "root_v": st["root_v"]}
        for i, (m, v) in enumerate(zip(st["m"], st["v"])):
          shard[f"m.{i}"], shard[f"v.{i}"] = m, v
        sharded = {"wan_state": shard}
      if self.rank == 0:
        items["wan_config"]["_train_step"] = int(step)
        items["wan_config"]["_tensor_parallel"] = int(T)
    self.manager.save(step, items, sharded=sharded, world_size=writers, shard_rank=t_rank * eng.world + eng.rank)
    max_logging.log(f"saved checkpoint for step {step} to {self.manager.directory}")

  def maybe_restore(self, trainer) -> Optional[int]:
    """Restores the latest step into the trainer (weights, and moments when present). Returns the step or None."""
    self.manager.wait_until_finished()
    step = self.manager.latest_step()
    if step is None:
      return None
    tree = {k: v.numpy() if v.dtype != torch.bfloat16 else v.float().numpy() for k, v in self.manager.restore_state(step, "wan_state").items()}
    ours = diffusers_to_ours(flax_tree_to_diffusers(tree))
    names, root = _param_names(trainer)
    eng = trainer.engine
    T, t_rank, _t_group, specs = _tensor_axis(trainer)
    for i, blk_names in enumerate(names):
      eng.load_full_block(i, [shard_of_full(ours[f"blocks.{i}.{n}"], specs[i].get(n), T, t_rank).to(eng.device, eng.param_dtype)
                              for n in blk_names])
    for n, view in zip(root, eng.root.views(eng.root_flat)):
      view.copy_(ours[n].to(eng.device, eng.param_dtype).reshape(view.shape))
    if os.path.exists(os.path.join(self.manager.directory, str(step), "wan_state", "_sharding")):
      shards = self.manager.restore_sharded(step, "wan_state")
      saved_t = int(self.manager.restore_json(step, "wan_config").get("_tensor_parallel", 1))
      per_t = len(shards) // saved_t  # files of one tensor rank of the saving run: the ranks of its shard group
      state = {"step": int(shards[0]["step"][0]), "root_m": shards[0]["root_m"], "root_v": shards[0]["root_v"], "m": [], "v": []}
      for i, (g, blk_names) in enumerate(zip(eng.groups, names)):
        for key in ("m", "v"):
          # flat moments of the whole block as every tensor rank of the saving run held them
          flats = [torch.cat([s[f"{key}.{i}"] for s in shards[t * per_t:(t + 1) * per_t]]) for t in range(saved_t)]
          if saved_t == T:
            full = flats[t_rank]
          else:
            full = _reshard_flat_over_tensor_axis(flats, [ours[f"blocks.{i}.{n}"].shape for n in blk_names],
                                                  [specs[i].get(n) for n in blk_names] if T > 1 else
                                                  _specs_by_name(trainer, i, blk_names), g, T, t_rank)
          if full.numel() < g.numel:
            full = torch.cat([full, full.new_zeros(g.numel - full.numel())])
          state[key].append(full[eng.rank * g.shard_numel:(eng.rank + 1) * g.shard_numel] if eng.world > 1 else full[:g.numel])
      eng.load_optimizer_state(state)
    max_logging.log(f"restored checkpoint of step {step} from {self.manager.directory}")
    return int(step)

  # ---- inference ---------------------------------------------------------------------------
  def restore_into_pipeline(self, pipe, step: Optional[int] = None) -> None:
    step = step if step is not None else self.manager.latest_step()
    if step is None:
      raise FileNotFoundError(f"no checkpoint under {self.manager.directory}")
    pairs = [("wan_state", pipe.transformer)]
    if pipe.transformer_2 is not None:
      pairs = [("high_noise_transformer_state", pipe.transformer), ("low_noise_transformer_state", pipe.transformer_2)]
    missing = [item for item, _ in pairs if not self.manager.has_item(step, item)]
    if missing:
      # a one-expert checkpoint cannot fill a two-expert pipeline and the other way round: say which item is absent
      present = [n for n in ("wan_state", "high_noise_transformer_state", "low_noise_transformer_state") if self.manager.has_item(step, n)]
      raise ValueError(f"checkpoint step {step} under {self.manager.directory} has no {missing} (it holds {present}): the "
                       "pipeline variant and the checkpoint do not match")
    for item, model in pairs:
      tree = {k: (v.float().numpy() if v.dtype == torch.bfloat16 else v.numpy()) for k, v in self.manager.restore_state(step, item).items()}
      ours = diffusers_to_ours(flax_tree_to_diffusers(tree))
      dtype = next(model.parameters()).dtype
      model.load_state_dict({k: v.to(dtype) for k, v in ours.items()})

  def save_pipeline(self, step: int, pipe) -> None:
    cfg = pipe.transformer.cfg
    def tree(m):
      return diffusers_to_flax_tree(ours_to_diffusers(m.state_dict(), cfg.in_channels, tuple(cfg.patch_size)))
    items = {"wan_config": cfg.to_dict()}
    if pipe.transformer_2 is not None:
      items["high_noise_transformer_state"], items["low_noise_transformer_state"] = tree(pipe.transformer), tree(pipe.transformer_2)
    else:
      items["wan_state"] = tree(pipe.transformer)
    self.manager.save(step, items)
    self.manager.wait_until_finished()

  def load_pretrained_pipeline_or_diffusers(self, pipeline_cls, device=None):
    """`pretrained_orbax_dir` cache: restore from it when it holds a checkpoint, else load the diffusers weights and
    write the cache for the next start (reference: wan_checkpointer.py:61-174)."""
    cache_dir = self.config.get("pretrained_orbax_dir", "")
    if cache_dir:
      cache = WanCheckpointer(self.config.replace(checkpoint_dir=cache_dir))
      if cache.manager.latest_step() is not None:
        pipe = pipeline_cls.from_config(self.config, device=device)
        cache.restore_into_pipeline(pipe)
        return pipe
    pipe = pipeline_cls.from_pretrained(self.config, device=device)
    if cache_dir and self.rank == 0:
      WanCheckpointer(self.config.replace(checkpoint_dir=cache_dir)).save_pipeline(0, pipe)
    return pipe

  # ---- one call for the generate / train entry points -------------------------------------------
  pipeline_module, pipeline_name = "maxdiffusion_b200.pipelines.wan.wan_pipeline", "WanPipeline2_1"

  @classmethod
  def pipeline_cls(cls):
    import importlib

    return getattr(importlib.import_module(cls.pipeline_module), cls.pipeline_name)

  def load_checkpoint(self, step: Optional[int] = None, device=None):
    """(pipeline, step): the pipeline of this checkpointer's model variant restored from `checkpoint_dir` at `step`
    (latest when None) if a checkpoint exists there, else built from the pretrained / cached weights with step None
    (reference: `WanCheckpointer2_1.load_checkpoint`, src/maxdiffusion/checkpointing/wan_checkpointer_2_1.py)."""
    pcls = self.pipeline_cls()
    have = self.manager.latest_step() if self.manager is not None else None
    if have is not None:
      pipe = pcls.from_config(self.config, device=device)
      self.restore_into_pipeline(pipe, step)
      return pipe, step if step is not None else have
    if self.config.get("random_init", False):
      return pcls.from_config(self.config, device=device), None
    return self.load_pretrained_pipeline_or_diffusers(pcls, device=device), None


class WanCheckpointer2_1(WanCheckpointer):
  pipeline_name = "WanPipeline2_1"


class WanCheckpointer2_2(WanCheckpointer):
  """Two experts: items `high_noise_transformer_state` / `low_noise_transformer_state`."""
  pipeline_name = "WanPipeline2_2"


class WanCheckpointerI2V_2_1(WanCheckpointer):
  pipeline_name = "WanPipelineI2V_2_1"


class WanCheckpointerI2V_2_2(WanCheckpointer):
  pipeline_name = "WanPipelineI2V_2_2"
