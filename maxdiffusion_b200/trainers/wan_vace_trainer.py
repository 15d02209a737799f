"""Wan VACE training: the flow-matching step of `WanTrainer` with `conditioning_latents` fed to the control branch.

reference: src/maxdiffusion/trainers/wan_vace_trainer.py:140-197 (`conditioning_latents` -> `control_hidden_states`).
"""
from __future__ import annotations

import torch

from ..models.wan.transformer_wan_vace import WAN_VACE_PRESETS, WanVACEConfig, WanVACEModel
from .wan_trainer import WanTrainer


def resolve_wan_vace_config(config) -> WanVACEConfig:
  preset = str(config.get("wan_preset", "") or "")
  if preset not in WAN_VACE_PRESETS:
    name = str(config.get("pretrained_model_name_or_path", "")).lower()
    preset = "wan2.1-vace-1.3b" if "1.3b" in name else "wan2.1-vace-14b"
  cfg = dict(WAN_VACE_PRESETS[preset])
  cfg.update(config.get("wan_config_overrides", None) or {})
  return WanVACEConfig(**cfg)


class WanVACETrainer(WanTrainer):
  model_cls = WanVACEModel
  resolve_config = staticmethod(resolve_wan_vace_config)

  def model_kwargs(self, batch: dict) -> dict:
    cond = batch.get("conditioning_latents")
    if cond is None:
      # synthetic data: zero control video, all-ones mask channels
      lat = batch["latents"]
      cond = torch.zeros((lat.shape[0], self.wan_cfg.vace_in_channels, *lat.shape[2:]), device=self.device, dtype=self.dtype)
      cond[:, 2 * lat.shape[1]:] = 1.0
    return {"control_hidden_states": cond.to(self.device, self.dtype)}
