"""Stable Diffusion / SDXL checkpointing (reference: src/maxdiffusion/checkpointing/base_stable_diffusion_checkpointer.py,
items :235-258: `unet_config`, `unet_state`, `vae_*`, `text_encoder_*`, `text_encoder_2_*` for SDXL, `scheduler_config`,
`tokenizer_config`, `iter` for grain datasets :162-176).

`save` writes the UNet (the trained component) with its config and the scheduler config; VAE and text encoders are
frozen during training and are re-read from the pretrained folder, unless `train_text_encoder` is set, in which case
the text-encoder state is stored too. The flat ZeRO-2 optimizer state is stored per rank.
"""
from __future__ import annotations

from dataclasses import asdict
from typing import Optional

import torch
import torch.distributed as dist

from .. import max_logging
from .checkpointing_utils import STABLE_DIFFUSION_CHECKPOINT, STABLE_DIFFUSION_XL_CHECKPOINT, create_checkpoint_manager


class BaseStableDiffusionCheckpointer:

  def __init__(self, config, checkpoint_type: Optional[str] = None):
    self.config = config
    if checkpoint_type is None:
      xl = "xl" in str(config.get("model_name", "")).lower() or "xl" in str(config.get("pretrained_model_name_or_path", "")).lower()
      checkpoint_type = STABLE_DIFFUSION_XL_CHECKPOINT if xl else STABLE_DIFFUSION_CHECKPOINT
    self.checkpoint_type = checkpoint_type
    init = dist.is_available() and dist.is_initialized()
    self.rank = dist.get_rank() if init else 0
    self.world = dist.get_world_size() if init else 1
    self.manager = create_checkpoint_manager(config.get("checkpoint_dir", ""), checkpoint_type,
                                             enable_async=bool(config.get("enable_async_checkpointing", True)),
                                             dataset_type=str(config.get("dataset_type", "")), rank=self.rank,
                                             single_replica=bool(config.get("enable_single_replica_ckpt_restoring", False)))

  def save(self, step: int, trainer, data_iterator=None) -> None:
    unet = trainer.unet
    cfg = {k: (list(v) if isinstance(v, tuple) else v) for k, v in asdict(unet.cfg).items()}
    items = {"unet_config": cfg, "unet_state": {k: v.detach() for k, v in unet.state_dict().items()},
             "scheduler_config": trainer.scheduler.config.to_dict()}
    if self.config.get("train_text_encoder", False) and trainer.text_encoders:
      items["text_encoder_state"] = {k: v.detach() for k, v in trainer.text_encoders[0].state_dict().items()}
    if data_iterator is not None and hasattr(data_iterator, "get_state") and "iter" in self.manager.item_names:
      items["iter"] = data_iterator.get_state()
    sharded = None
    if self.config.get("save_optimizer", False):
      o = trainer.optimizer
      sharded = {"tokenizer_config": {"m": o.m, "v": o.v, "step": torch.tensor([o.step_count])}}
    self.manager.save(step, items, sharded=sharded, world_size=self.world)

  def maybe_restore(self, trainer, data_iterator=None) -> Optional[int]:
    step = self.manager.latest_step() if self.manager is not None else None
    if step is None:
      return None
    self.manager.wait_until_finished()
    state = self.manager.restore_state(step, "unet_state")
    dtype = next(trainer.unet.parameters()).dtype
    trainer.unet.load_state_dict({k: v.to(dtype) for k, v in state.items()})
    trainer.optimizer.flat.copy_(trainer.optimizer.flat_group.pack_from_params())
    trainer.optimizer.flat_group.point_params_to(trainer.optimizer.flat)
    if self.manager.has_item(step, "text_encoder_state") and trainer.text_encoders:
      trainer.text_encoders[0].load_state_dict(self.manager.restore_state(step, "text_encoder_state"))
    if self.manager.has_item(step, "tokenizer_config"):
      shards = self.manager.restore_sharded(step, "tokenizer_config")
      if len(shards) == self.world and "m" in shards[self.rank]:
        mine = shards[self.rank]
        trainer.optimizer.m.copy_(mine["m"])
        trainer.optimizer.v.copy_(mine["v"])
        trainer.optimizer.step_count = int(mine["step"][0])
    if data_iterator is not None and hasattr(data_iterator, "set_state") and self.manager.has_item(step, "iter"):
      data_iterator.set_state(self.manager.restore_json(step, "iter"))
    max_logging.log(f"restored Stable Diffusion training state from step {step}")
    return step

  def restore_iterator(self, data_iterator) -> bool:
    """Puts a data source that can save its position (`get_state` / `set_state`: grain) back where the latest
    checkpoint left it (item `iter`)."""
    step = self.manager.latest_step() if self.manager is not None else None
    if step is None or not hasattr(data_iterator, "set_state") or not self.manager.has_item(step, "iter"):
      return False
    data_iterator.set_state(self.manager.restore_json(step, "iter"))
    return True

  def load_pipeline(self, pipeline_cls, device=None):
    step = self.manager.latest_step() if self.manager is not None else None
    if self.config.get("random_init", False):
      pipe = pipeline_cls.from_config(self.config, device=device)
    else:
      from ..loaders.sd_loader import load_sd_pipeline

      pipe = load_sd_pipeline(self.config, pipeline_cls)
    if step is not None:
      dtype = next(pipe.unet.parameters()).dtype
      pipe.unet.load_state_dict({k: v.to(dtype) for k, v in self.manager.restore_state(step, "unet_state").items()})
      max_logging.log(f"restored the UNet from step {step}")
    return pipe
