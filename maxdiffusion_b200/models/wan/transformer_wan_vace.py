"""Wan VACE: video-conditioned editing through a control branch whose hints are added to the main stream.

Reference: src/maxdiffusion/models/wan/transformers/transformer_wan_vace.py (`WanVACETransformerBlock` :37-290,
`WanVACEModel` :294-640). The control video latents (with mask channels, `vace_in_channels`) are patch-embedded
by their own projection; `len(vace_layers)` control blocks (a Wan block; the first adds `proj_in(control) + x`)
run once on the control stream, each emitting `proj_out(control)`; the hint of control block j is added, times
`control_hidden_states_scale[j]`, after main block `vace_layers[j]`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn

from ..layers import Linear
from .transformer_wan import WAN_PRESETS, WanBlock, WanConfig, WanModel


@dataclass
class WanVACEConfig(WanConfig):
  vace_layers: Sequence[int] = (0, 5, 10, 15, 20, 25, 30, 35)
  vace_in_channels: int = 96


WAN_VACE_PRESETS = {
    "wan2.1-vace-14b": dict(WAN_PRESETS["wan2.1-t2v-14b"], vace_layers=(0, 5, 10, 15, 20, 25, 30, 35), vace_in_channels=96),
    "wan2.1-vace-1.3b": dict(WAN_PRESETS["wan2.1-t2v-1.3b"], vace_layers=tuple(range(0, 30, 2)), vace_in_channels=96),
    "tiny": dict(WAN_PRESETS["tiny"], vace_layers=(0, 1), vace_in_channels=20),
}


class WanVACEBlock(WanBlock):

  def __init__(self, cfg: WanConfig, apply_input_projection: bool, apply_output_projection: bool = True):
    super().__init__(cfg)
    self.proj_in = Linear(cfg.dim, cfg.dim) if apply_input_projection else None
    self.proj_out = Linear(cfg.dim, cfg.dim) if apply_output_projection else None

  def forward(self, x, control, context, temb6, rope, pctx=None, cached_kv=None):
    """Returns (hint, control): the projected conditioning and the updated control stream."""
    if self.proj_in is not None:
      control = self.proj_in(control) + x
    control = super().forward(control, context, temb6, rope, pctx, None, cached_kv)
    hint = self.proj_out(control) if self.proj_out is not None else None
    return hint, control


class WanVACEModel(WanModel):

  def __init__(self, cfg: WanVACEConfig, remat_policy: str = "NONE"):
    super().__init__(cfg, remat_policy)
    pt, ph, pw = cfg.patch_size
    self.vace_patch_embedding = Linear(cfg.vace_in_channels * pt * ph * pw, cfg.dim)
    self.vace_blocks = nn.ModuleList([WanVACEBlock(cfg, apply_input_projection=(i == 0)) for i in range(len(cfg.vace_layers))])

  def compute_kv_cache(self, encoder_hidden_states, encoder_hidden_states_image=None):
    """(control-branch K/V, main K/V) per layer (reference :449-497)."""
    main = super().compute_kv_cache(encoder_hidden_states, encoder_hidden_states_image)
    dtype = self.patch_embedding.weight.dtype
    context = self.condition_embedder.text(encoder_hidden_states.to(dtype))
    return [blk.attn2.compute_kv(context, None) for blk in self.vace_blocks], main

  def forward(self, hidden_states, timestep, encoder_hidden_states, control_hidden_states,
              control_hidden_states_scale: Optional[Sequence[float]] = None, pctx=None, kv_cache=None, rope=None,
              return_tokens: bool = False, encoder_hidden_states_image=None, **kw):
    if encoder_hidden_states_image is not None:
      raise NotImplementedError("image conditioning is not part of the VACE model")
    cfg = self.cfg
    n = len(cfg.vace_layers)
    scales = [1.0] * n if control_hidden_states_scale is None else [float(s) for s in control_hidden_states_scale]
    if len(scales) != n:
      raise ValueError(f"Length of `control_hidden_states_scale` {len(scales)} should be equal to {n}.")
    dtype = self.patch_embedding.weight.dtype
    ctl_tokens, _ = self.patchify(control_hidden_states.to(dtype))
    vace_kv, main_kv = kv_cache if kv_cache is not None else (None, None)

    def control_branch(x, context, temb6, rope_, pctx_):
      tok = pctx_.shard_sequence(ctl_tokens) if pctx_ is not None else ctl_tokens
      control = self.vace_patch_embedding(tok)
      hints = {}
      for j, blk in enumerate(self.vace_blocks):
        hint, control = blk(x, control, context, temb6, rope_, pctx_, vace_kv[j] if vace_kv is not None else None)
        hints[int(cfg.vace_layers[j])] = hint * scales[j]
      return hints

    return super().forward(hidden_states, timestep, encoder_hidden_states, None, pctx=pctx, kv_cache=main_kv, rope=rope,
                           return_tokens=return_tokens, hints=control_branch, **kw)
