"""Flux.2-Klein transformer (4B / 9B): double-stream and single-stream blocks with ONE set of modulation vectors
shared by all blocks of a kind, SwiGLU MLPs, bias-free projections, 4-axis RoPE (theta 2000).

Reference: `NNXFlux2KleinTransformer2DModel` and its blocks
(src/maxdiffusion/models/flux/transformers/transformer_flux_flax.py:1279-2025):
  * `double_stream_modulation_img/txt` (dim -> 6 dim) and `single_stream_modulation` (dim -> 3 dim) are applied once
    to silu(temb) at the top of the model (:1964-1969); every block splits them the same way;
  * double block (:1544-1686): LN(no affine) * (1 + scale) + shift on both streams, fused qkv per stream, per-head
    RMSNorm on q and k, joint attention over [txt ; img] with RoPE, per-stream output projection, gated residual,
    then a SwiGLU feed-forward (`linear_in` dim -> 2 * 3 dim, silu(x1) * x2, `linear_out`) with gated residual;
  * single block (:1688-1808): `linear1` dim -> 3 dim + 2 * 3 dim in one GEMM, attention on the qkv part, SwiGLU on
    the rest, `linear2` on concat[attn, mlp], gate, residual;
  * output: AdaLayerNormContinuous + bias-free projection to `in_channels` (:1936-1946).
Parameter names follow the diffusers `Flux2Transformer2DModel` checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as OF
from ..layers import Linear, RMSNorm, sinusoidal_embedding
from .transformer_flux import _MLPEmbedder, flux_rope_tables


@dataclass
class Flux2KleinConfig:
  patch_size: int = 1
  in_channels: int = 128
  num_layers: int = 5
  num_single_layers: int = 20
  attention_head_dim: int = 128
  num_attention_heads: int = 24
  joint_attention_dim: int = 7680
  pooled_projection_dim: int = 0      # Klein has no pooled text vector; > 0 adds the CLIP-style projection
  guidance_embeds: bool = False
  axes_dims_rope: Sequence[int] = (32, 32, 32, 32)
  theta: float = 2000.0
  mlp_ratio: float = 3.0
  scale_shift_order: str = "scale_shift"

  @property
  def dim(self) -> int:
    return self.num_attention_heads * self.attention_head_dim

  @classmethod
  def from_dict(cls, d):
    d = dict(d)
    if "axes_dim" in d and "axes_dims_rope" not in d:
      d["axes_dims_rope"] = d.pop("axes_dim")
    if "rope_theta" in d and "theta" not in d:
      d["theta"] = d.pop("rope_theta")
    return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

  def to_dict(self):
    return {k: (list(v) if isinstance(v, tuple) else v) for k, v in self.__dict__.items()}


FLUX2_KLEIN_PRESETS = {
    "flux2-klein-4b": dict(num_layers=5, num_single_layers=20, num_attention_heads=24, joint_attention_dim=7680),
    "flux2-klein-9b": dict(num_layers=8, num_single_layers=24, num_attention_heads=32, joint_attention_dim=12288),
    "tiny": dict(in_channels=128, num_layers=1, num_single_layers=2, num_attention_heads=2, attention_head_dim=32,
                 joint_attention_dim=48, axes_dims_rope=(8, 8, 8, 8)),
}


def _rope_qk(x, norm: RMSNorm, rope, heads: int):
  """Per-head RMSNorm then RoPE on interleaved pairs; fused kernel when the head width is 128."""
  return OF.rms_norm_rope(x, norm.weight, rope[0], rope[1], heads=heads, per_head=True, eps=norm.eps)


class SwiGLUFeedForward(nn.Module):

  def __init__(self, dim: int, mult: float):
    super().__init__()
    inner = int(dim * mult)
    self.linear_in, self.linear_out = Linear(dim, 2 * inner, bias=False), Linear(inner, dim, bias=False)

  def forward(self, x):
    a, b = self.linear_in(x).chunk(2, dim=-1)
    return self.linear_out(F.silu(a) * b)


class Flux2DoubleBlock(nn.Module):

  def __init__(self, cfg: Flux2KleinConfig):
    super().__init__()
    dim, d = cfg.dim, cfg.attention_head_dim
    self.heads = cfg.num_attention_heads
    self.to_qkv, self.add_qkv_proj = Linear(dim, 3 * dim, bias=False), Linear(dim, 3 * dim, bias=False)
    self.to_out, self.to_add_out = Linear(dim, dim, bias=False), Linear(dim, dim, bias=False)
    self.norm_q, self.norm_k = RMSNorm(d, 1e-6), RMSNorm(d, 1e-6)
    self.norm_added_q, self.norm_added_k = RMSNorm(d, 1e-6), RMSNorm(d, 1e-6)
    self.ff, self.ff_context = SwiGLUFeedForward(dim, cfg.mlp_ratio), SwiGLUFeedForward(dim, cfg.mlp_ratio)

  def forward(self, img, txt, mod_img, mod_txt, rope_img, rope_txt):
    B, Si, C = img.shape
    St, H = txt.shape[1], self.heads
    sh_i, sc_i, g_i, sh2_i, sc2_i, g2_i = mod_img
    sh_t, sc_t, g_t, sh2_t, sc2_t, g2_t = mod_txt
    qi, ki, vi = self.to_qkv(OF.layer_norm_mod(img, scale=sc_i, shift=sh_i)).chunk(3, dim=-1)
    qt, kt, vt = self.add_qkv_proj(OF.layer_norm_mod(txt, scale=sc_t, shift=sh_t)).chunk(3, dim=-1)
    q = torch.cat([_rope_qk(qt, self.norm_added_q, rope_txt, H), _rope_qk(qi, self.norm_q, rope_img, H)], dim=1)
    k = torch.cat([_rope_qk(kt, self.norm_added_k, rope_txt, H), _rope_qk(ki, self.norm_k, rope_img, H)], dim=1)
    v = torch.cat([vt.unflatten(-1, (H, C // H)), vi.unflatten(-1, (H, C // H))], dim=1)
    o = OF.attention(q, k, v).reshape(B, St + Si, C)
    img = OF.linear_gated_residual(o[:, St:], self.to_out.weight, None, img, g_i)
    txt = OF.linear_gated_residual(o[:, :St], self.to_add_out.weight, None, txt, g_t)
    img = OF.gated_residual(img, self.ff(OF.layer_norm_mod(img, scale=sc2_i, shift=sh2_i)), g2_i)
    txt = OF.gated_residual(txt, self.ff_context(OF.layer_norm_mod(txt, scale=sc2_t, shift=sh2_t)), g2_t)
    return img, txt


class Flux2SingleBlock(nn.Module):

  def __init__(self, cfg: Flux2KleinConfig):
    super().__init__()
    dim, d = cfg.dim, cfg.attention_head_dim
    self.heads, self.hidden = cfg.num_attention_heads, int(cfg.dim * cfg.mlp_ratio)
    self.to_qkv_mlp_proj = Linear(dim, 3 * dim + 2 * self.hidden, bias=False)
    self.to_out = Linear(dim + self.hidden, dim, bias=False)
    self.norm_q, self.norm_k = RMSNorm(d, 1e-6), RMSNorm(d, 1e-6)

  def forward(self, x, mod, rope):
    B, S, C = x.shape
    H = self.heads
    shift, scale, gate = mod
    f = self.to_qkv_mlp_proj(OF.layer_norm_mod(x, scale=scale, shift=shift))
    q, k, v, mlp = f[..., :C], f[..., C:2 * C], f[..., 2 * C:3 * C], f[..., 3 * C:]
    o = OF.attention(_rope_qk(q, self.norm_q, rope, H), _rope_qk(k, self.norm_k, rope, H),
                     v.unflatten(-1, (H, C // H))).reshape(B, S, C)
    a, b = mlp.chunk(2, dim=-1)
    return OF.linear_gated_residual(torch.cat([o, F.silu(a) * b], dim=-1), self.to_out.weight, None, x, gate)


class Flux2KleinTransformer2DModel(nn.Module):
  """`forward(hidden_states [B,S,in], encoder_hidden_states [B,T,joint], timestep [B], img_ids, txt_ids, guidance)`."""

  def __init__(self, cfg: Flux2KleinConfig):
    super().__init__()
    self.cfg = cfg
    dim = cfg.dim
    self.x_embedder = Linear(cfg.in_channels, dim, bias=False)
    self.context_embedder = Linear(cfg.joint_attention_dim, dim, bias=False)
    self.time_embedder = _MLPEmbedder(256, dim)
    self.guidance_embedder = _MLPEmbedder(256, dim) if cfg.guidance_embeds else None
    self.text_embedder = _MLPEmbedder(cfg.pooled_projection_dim, dim) if cfg.pooled_projection_dim else None
    self.double_stream_modulation_img = Linear(dim, 6 * dim, bias=False)
    self.double_stream_modulation_txt = Linear(dim, 6 * dim, bias=False)
    self.single_stream_modulation = Linear(dim, 3 * dim, bias=False)
    self.transformer_blocks = nn.ModuleList([Flux2DoubleBlock(cfg) for _ in range(cfg.num_layers)])
    self.single_transformer_blocks = nn.ModuleList([Flux2SingleBlock(cfg) for _ in range(cfg.num_single_layers)])
    self.norm_out = Linear(dim, 2 * dim, bias=False)
    self.proj_out = Linear(dim, cfg.in_channels, bias=False)

  def forward(self, hidden_states, encoder_hidden_states, timestep, img_ids, txt_ids, guidance=None,
              pooled_projections=None):
    cfg = self.cfg
    dtype = self.x_embedder.weight.dtype
    img = self.x_embedder(hidden_states.to(dtype))
    txt = self.context_embedder(encoder_hidden_states.to(dtype))
    temb = self.time_embedder(sinusoidal_embedding(timestep * 1000.0, 256).to(dtype))
    if self.guidance_embedder is not None:
      g = guidance if guidance is not None else torch.ones_like(timestep)
      temb = temb + self.guidance_embedder(sinusoidal_embedding(g * 1000.0, 256).to(dtype))
    if self.text_embedder is not None and pooled_projections is not None:
      temb = temb + self.text_embedder(pooled_projections.to(dtype))
    ts = F.silu(temb).float()
    mod_img = F.linear(ts, self.double_stream_modulation_img.weight.float()).chunk(6, dim=-1)
    mod_txt = F.linear(ts, self.double_stream_modulation_txt.weight.float()).chunk(6, dim=-1)
    mod_single = F.linear(ts, self.single_stream_modulation.weight.float()).chunk(3, dim=-1)
    img_ids = img_ids[0] if img_ids.dim() == 3 else img_ids
    txt_ids = txt_ids[0] if txt_ids.dim() == 3 else txt_ids
    rope_img = flux_rope_tables(img_ids, cfg.axes_dims_rope, cfg.theta)
    rope_txt = flux_rope_tables(txt_ids, cfg.axes_dims_rope, cfg.theta)
    rope_all = (torch.cat([rope_txt[0], rope_img[0]]), torch.cat([rope_txt[1], rope_img[1]]))
    for blk in self.transformer_blocks:
      img, txt = blk(img, txt, mod_img, mod_txt, rope_img, rope_txt)
    x = torch.cat([txt, img], dim=1)
    for blk in self.single_transformer_blocks:
      x = blk(x, mod_single, rope_all)
    img = x[:, txt.shape[1]:].contiguous()
    a, b = F.linear(ts, self.norm_out.weight.float()).chunk(2, dim=-1)
    scale, shift = (a, b) if cfg.scale_shift_order == "scale_shift" else (b, a)
    return self.proj_out(OF.layer_norm_mod(img, scale=scale, shift=shift))
