"""LTX-Video (0.9.x, 2B / 13B) transformer: PixArt-style blocks with fractional 3-D RoPE and skip-layer guidance.

Reference: src/maxdiffusion/models/ltx_video/transformers/transformer3d.py (`Transformer3DModel` :25-244,
`FreqsCisPrecomputer` :258-325), `attention.py` (`BasicTransformerBlock` :64-312, `Attention` :315-912),
`adaln.py` (`AdaLayerNormSingle`), `caption_projection.py`, `symmetric_patchifier.py`,
`utils/skip_layer_strategy.py`.
  * tokens = latents patchified with patch size 1; RoPE from fractional coordinates `indices_grid / max_pos`
    (seconds, pixels) with `theta ** linspace(0, 1, dim // 6) * pi / 2`, interleaved, left-padded with cos = 1;
  * block: RMSNorm (no affine) -> AdaLN-single (6-row scale_shift_table + timestep embedding) -> self-attention with
    q/k RMSNorm over the full inner dimension and RoPE -> gate; cross-attention to the projected captions (no
    modulation); FFN (GELU-tanh) with scale/shift/gate;
  * skip-layer (spatio-temporal) guidance: `skip_layer_mask[block, batch]` = 0 makes the self-attention of that
    sample return its values (`AttentionValues`), skip the attention (`AttentionSkip`), or keep the residual only;
  * output: LayerNorm (no affine) * (1 + scale) + shift with the 2-row table, linear projection.
Parameter names follow the LTX-Video checkpoint.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..embeddings import PixArtAlphaTextProjection
from ..layers import Linear, RMSNorm
from ..ltx2.attention_ltx2 import LTX2Attention
from ..ltx2.transformer_ltx2 import FeedForward, LTX2AdaLayerNormSingle, _ada, _gated_add, _mod


class SkipLayerStrategy(enum.Enum):
  AttentionSkip = enum.auto()
  AttentionValues = enum.auto()
  Residual = enum.auto()
  TransformerBlock = enum.auto()


@dataclass
class LTXVideoConfig:
  in_channels: int = 128
  out_channels: int = 128
  num_attention_heads: int = 32
  attention_head_dim: int = 128
  num_layers: int = 48
  cross_attention_dim: int = 4096
  caption_channels: int = 4096
  activation_fn: str = "gelu-approximate"
  attention_bias: bool = True
  norm_eps: float = 1e-6
  qk_norm: str = "rms_norm"
  positional_embedding_theta: float = 10000.0
  positional_embedding_max_pos: Sequence[int] = (20, 2048, 2048)
  timestep_scale_multiplier: float = 1000.0
  adaptive_norm: str = "single_scale_shift"

  @property
  def inner_dim(self):
    return self.num_attention_heads * self.attention_head_dim

  @classmethod
  def from_dict(cls, d):
    return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})


LTXV_PRESETS = {
    "ltxv-13b": dict(num_attention_heads=32, num_layers=48),
    "ltxv-2b": dict(num_attention_heads=16, num_layers=28, cross_attention_dim=2048),
    "tiny": dict(in_channels=8, out_channels=8, num_attention_heads=2, attention_head_dim=24, num_layers=3,
                 cross_attention_dim=48, caption_channels=16),
}


def fractional_rope(indices_grid: torch.Tensor, max_pos: Sequence[int], theta: float, dim: int):
  """indices_grid [B, 3, N] (frame time in seconds, y, x in pixels) -> (cos, sin) [B, N, dim]."""
  frac = torch.stack([indices_grid[:, i].double() / max_pos[i] for i in range(3)], dim=-1)       # [B, N, 3]
  idx = torch.pow(torch.tensor(theta, dtype=torch.float64), torch.linspace(0.0, 1.0, dim // 6, dtype=torch.float64)).to(frac.device) * math.pi / 2
  freqs = (idx * (frac.unsqueeze(-1) * 2 - 1)).transpose(-1, -2).reshape(frac.shape[0], frac.shape[1], -1)
  cos, sin = freqs.cos().float().repeat_interleave(2, dim=-1), freqs.sin().float().repeat_interleave(2, dim=-1)
  pad = dim % 6
  if pad:
    cos = torch.cat([torch.ones_like(cos[..., :pad]), cos], dim=-1)
    sin = torch.cat([torch.zeros_like(sin[..., :pad]), sin], dim=-1)
  return cos, sin


class BasicTransformerBlock(nn.Module):

  def __init__(self, c: LTXVideoConfig):
    super().__init__()
    d = c.inner_dim
    self.norm1, self.norm2 = RMSNorm(d, c.norm_eps, elementwise_affine=False), RMSNorm(d, c.norm_eps, elementwise_affine=False)
    self.attn1 = LTX2Attention(d, c.num_attention_heads, c.attention_head_dim, bias=c.attention_bias, eps=c.norm_eps)
    self.attn2 = LTX2Attention(d, c.num_attention_heads, c.attention_head_dim, context_dim=c.cross_attention_dim,
                               bias=c.attention_bias, eps=c.norm_eps)
    self.ff = FeedForward(d, c.activation_fn)
    self.n_ada = 4 if c.adaptive_norm == "single_scale" else 6
    self.scale_shift_table = nn.Parameter(torch.randn(self.n_ada, d) / d ** 0.5)

  def forward(self, x, rope, text, text_mask, temb, skip_mask=None, strategy: Optional[SkipLayerStrategy] = None):
    """skip_mask: [B, 1, 1] with 0 for the samples whose self-attention is perturbed in this block."""
    ada = _ada(self.scale_shift_table, temb, self.n_ada)
    if self.n_ada == 6:
      shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = ada
    else:
      scale_msa, gate_msa, scale_mlp, gate_mlp = ada
      shift_msa = shift_mlp = torch.zeros_like(scale_msa)
    h = _mod(self.norm1(x), scale_msa, shift_msa)
    if skip_mask is not None and strategy == SkipLayerStrategy.TransformerBlock:
      keep = skip_mask.to(x.dtype)
    else:
      keep = None
    values_mask = skip_mask if (skip_mask is not None and strategy in (None, SkipLayerStrategy.AttentionValues)) else None
    a = self.attn1(h, rotary_emb=rope, perturbation_mask=values_mask)
    if skip_mask is not None and strategy in (SkipLayerStrategy.AttentionSkip, SkipLayerStrategy.Residual):
      a = a * skip_mask.to(a.dtype)  # the perturbed samples keep the residual stream only
    y = _gated_add(x, a, gate_msa)
    y = y + self.attn2(y, encoder_hidden_states=text, attention_mask=text_mask)
    y = _gated_add(y, self.ff(_mod(self.norm2(y), scale_mlp, shift_mlp)), gate_mlp)
    return y if keep is None else (keep * y + (1 - keep) * x)


class Transformer3DModel(nn.Module):

  def __init__(self, cfg: LTXVideoConfig):
    super().__init__()
    self.cfg = cfg
    d = cfg.inner_dim
    self.patchify_proj = Linear(cfg.in_channels, d)
    self.adaln_single = LTX2AdaLayerNormSingle(d, 4 if cfg.adaptive_norm == "single_scale" else 6)
    self.caption_projection = PixArtAlphaTextProjection(cfg.caption_channels, d) if cfg.caption_channels else None
    self.transformer_blocks = nn.ModuleList([BasicTransformerBlock(cfg) for _ in range(cfg.num_layers)])
    self.scale_shift_table = nn.Parameter(torch.randn(2, d) / d ** 0.5)
    self.proj_out = Linear(d, cfg.out_channels)

  def create_skip_layer_mask(self, batch_size: int, num_conds: int, ptb_index: int, skip_block_list=None):
    """[num_layers, batch_size * num_conds] with 0 at the perturbed condition of the listed blocks (reference :148-161)."""
    if not skip_block_list:
      return None
    mask = torch.ones((self.cfg.num_layers, batch_size * num_conds))
    for b in skip_block_list:
      mask[b, ptb_index::num_conds] = 0
    return mask

  def forward(self, hidden_states, indices_grid, encoder_hidden_states, timestep, encoder_attention_mask=None,
              skip_layer_mask=None, skip_layer_strategy: Optional[SkipLayerStrategy] = None):
    """hidden_states [B,N,C]; indices_grid [B,3,N]; timestep [B] or [B,N] in [0,1]; skip_layer_mask [L,B]."""
    cfg = self.cfg
    dtype = self.patchify_proj.weight.dtype
    B = hidden_states.shape[0]
    x = self.patchify_proj(hidden_states.to(dtype))
    rope = fractional_rope(indices_grid, cfg.positional_embedding_max_pos, cfg.positional_embedding_theta, cfg.inner_dim)
    t = timestep.float() * cfg.timestep_scale_multiplier
    temb, emb = self.adaln_single(t.flatten(), dtype)
    temb, emb = temb.reshape(B, -1, temb.shape[-1]), emb.reshape(B, -1, emb.shape[-1])
    text = encoder_hidden_states.to(dtype)
    if self.caption_projection is not None:
      text = self.caption_projection(text)
    mask = None
    if encoder_attention_mask is not None and not bool(encoder_attention_mask.bool().all()):
      mask = encoder_attention_mask.bool()
    for i, blk in enumerate(self.transformer_blocks):
      sm = None
      if skip_layer_mask is not None and not bool(skip_layer_mask[i].bool().all()):
        sm = skip_layer_mask[i].to(x.device).view(B, 1, 1)
      x = blk(x, rope, text, mask, temb, sm, skip_layer_strategy)
    shift = self.scale_shift_table.float()[None, None, 0] + emb.float()
    scale = self.scale_shift_table.float()[None, None, 1] + emb.float()
    x = _mod(F.layer_norm(x.float(), (x.shape[-1],), eps=1e-6).to(x.dtype), scale, shift)
    return self.proj_out(x)
