"""Parameter counts per top-level sub-module of any model family, built on the meta device (no memory is used).

  python -m maxdiffusion_b200.pedagogical_examples.parameter_count wan2.1-t2v-14b
  python -m maxdiffusion_b200.pedagogical_examples.parameter_count flux-dev | sdxl | sd15
"""
from __future__ import annotations

import sys
from collections import OrderedDict

import torch


def build(name: str) -> torch.nn.Module:
  from ..models.flux.transformer_flux import FLUX_PRESETS, FluxConfig, FluxTransformer2DModel
  from ..models.unet_2d_condition import UNET_PRESETS, UNet2DConditionModel, UNetConfig
  from ..models.wan.transformer_wan import WAN_PRESETS, WanConfig, WanModel

  with torch.device("meta"):
    if name in WAN_PRESETS:
      return WanModel(WanConfig(**WAN_PRESETS[name]))
    if name in FLUX_PRESETS:
      return FluxTransformer2DModel(FluxConfig(**FLUX_PRESETS[name]))
    if name in UNET_PRESETS:
      return UNet2DConditionModel(UNetConfig(**UNET_PRESETS[name]))
  raise KeyError(f"unknown preset {name}; Wan: {sorted(WAN_PRESETS)}, Flux: {sorted(FLUX_PRESETS)}, UNet: {sorted(UNET_PRESETS)}")


def count(model: torch.nn.Module) -> "OrderedDict[str, int]":
  out: "OrderedDict[str, int]" = OrderedDict()
  for n, p in model.named_parameters():
    top = n.split(".")[0]
    out[top] = out.get(top, 0) + p.numel()
  out["total"] = sum(p.numel() for p in model.parameters())
  return out


def run(name: str) -> "OrderedDict[str, int]":
  c = count(build(name))
  for k, v in c.items():
    print(f"{k:>28}: {v / 1e6:12.2f} M")
  return c


if __name__ == "__main__":
  run(sys.argv[1] if len(sys.argv) > 1 else "wan2.1-t2v-14b")
