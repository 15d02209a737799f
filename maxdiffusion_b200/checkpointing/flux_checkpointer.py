"""Flux checkpointing: training state of the transformer (+ optimizer shards), pipeline construction from a checkpoint
or from pretrained weights.

Reference: src/maxdiffusion/checkpointing/flux_checkpointer.py (items `flux_state`, `flux_config`, `vae_state`,
`vae_config`, `scheduler`, `scheduler_config`, `text_encoder_2_*`, :147-161; `load_checkpoint` / `load_diffusers_checkpoint`
:163-311). The transformer state is stored under its parameter names; the optimizer moments of every rank go next to
it as `process_<rank>.safetensors` and are only restored on the same topology.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import max_logging
from .checkpointing_utils import FLUX_CHECKPOINT, create_checkpoint_manager


def _names(model, blocks):
  names = [[n for n, _ in b.named_parameters()] for b in blocks]
  ids = {id(p) for b in blocks for p in b.parameters()}
  root = [n for n, p in model.named_parameters() if id(p) not in ids]
  return names, root


def _block_prefixes(model):
  out = []
  for i in range(len(model.transformer_blocks)):
    out.append(f"transformer_blocks.{i}.")
  for i in range(len(model.single_transformer_blocks)):
    out.append(f"single_transformer_blocks.{i}.")
  return out


class FluxCheckpointer:

  def __init__(self, config, checkpoint_type: str = FLUX_CHECKPOINT):
    self.config = config
    init = dist.is_available() and dist.is_initialized()
    self.rank = dist.get_rank() if init else 0
    self.world = dist.get_world_size() if init else 1
    self.manager = create_checkpoint_manager(config.get("checkpoint_dir", ""), checkpoint_type,
                                             enable_async=bool(config.get("enable_async_checkpointing", True)),
                                             dataset_type=str(config.get("dataset_type", "")), rank=self.rank,
                                             single_replica=bool(config.get("enable_single_replica_ckpt_restoring", False)))

  # ---- training state ------------------------------------------------------------------------
  def save(self, step: int, trainer) -> None:
    model, eng = trainer.model, trainer.engine
    names, root = _names(model, model.blocks)
    prefixes = _block_prefixes(model)
    full = eng.gather_state_dict([[prefixes[i] + n for n in blk] for i, blk in enumerate(names)], root)
    items = {"flux_state": full, "flux_config": model.cfg.to_dict()}
    sharded = None
    if self.config.get("save_optimizer", False):
      st = eng.optimizer_state()
      opt = {f"m.{i}": t for i, t in enumerate(st["m"])} | {f"v.{i}": t for i, t in enumerate(st["v"])}
      opt.update(root_m=st["root_m"], root_v=st["root_v"], step=torch.tensor([st["step"]]))
      # optimizer shards ride in the scheduler item's directory of the reference layout
      sharded = {"scheduler": opt}
    self.manager.save(step, items, sharded=sharded, world_size=self.world)

  def maybe_restore(self, trainer) -> Optional[int]:
    step = self.manager.latest_step() if self.manager is not None else None
    if step is None:
      return None
    self.manager.wait_until_finished()
    state = self.manager.restore_state(step, "flux_state")
    model, eng = trainer.model, trainer.engine
    names, root = _names(model, model.blocks)
    prefixes = _block_prefixes(model)
    for i, blk in enumerate(names):
      eng.load_full_block(i, [state[prefixes[i] + n].to(eng.device, eng.param_dtype) for n in blk])
    for n, v in zip(root, eng.root.views(eng.root_flat)):
      v.copy_(state[n].to(v))
    if self.manager.has_item(step, "scheduler"):
      shards = self.manager.restore_sharded(step, "scheduler")
      if len(shards) == self.world:
        mine = shards[self.rank]
        eng.load_optimizer_state({"step": int(mine["step"][0]), "m": [mine[f"m.{i}"] for i in range(len(eng.m))],
                                  "v": [mine[f"v.{i}"] for i in range(len(eng.v))], "root_m": mine["root_m"], "root_v": mine["root_v"]})
      else:
        max_logging.log(f"optimizer state was saved on {len(shards)} ranks, now {self.world}: moments start from zero")
    max_logging.log(f"restored Flux training state from step {step}")
    return step

  # ---- pipelines -----------------------------------------------------------------------------
  def load_pipeline(self, device=None):
    """`FluxPipeline` with the transformer of the latest checkpoint step if there is one, else pretrained / random."""
    from ..pipelines.flux.flux_pipeline import FluxPipeline

    step = self.manager.latest_step() if self.manager is not None else None
    if self.config.get("random_init", False) or step is not None:
      pipe = FluxPipeline.from_config(self.config, device=device)
    else:
      from ..loaders.flux_loader import load_flux_pipeline

      pipe = load_flux_pipeline(self.config, device=device)
    if step is not None:
      state = self.manager.restore_state(step, "flux_state")
      dtype = next(pipe.transformer.parameters()).dtype
      pipe.transformer.load_state_dict({k: v.to(dtype) for k, v in state.items()})
      max_logging.log(f"restored the Flux transformer from step {step}")
    return pipe
