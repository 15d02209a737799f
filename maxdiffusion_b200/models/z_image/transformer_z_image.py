"""Z-Image / Z-Image-Turbo single-stream DiT over one joint [image | caption] sequence.

Behaviour follows the reference (src/maxdiffusion/models/z_image/transformer_z_image.py):
  * 2x2x1 patchify of [C, F, H, W] latents, captions and image tokens each padded to a multiple of 32 with a
    learned pad token (`_pad`, :755-779); 3-axis RoPE ids: captions at (1 + i, 0, 0), image patches at
    (caption_len + 1 + f, h, w) (:856-870);
  * timestep embedder (256 sinusoidal features -> 1024 -> 256), caption RMSNorm + Linear;
  * 2 noise-refiner blocks (image tokens, modulated), 2 context-refiner blocks (captions, not modulated),
    then `n_layers` modulated blocks over the concatenation (:873-950);
  * block = sandwich RMSNorms, scale-only AdaLN with tanh gates, per-head q/k RMSNorm, real RoPE on interleaved
    pairs, bias-free SwiGLU with hidden 8/3 dim (:356-462, :125-172, :175-350);
  * final layer: LayerNorm (no affine) * (1 + Linear(silu(adaln))) -> Linear to the patch dimension.

Parameter names follow the released checkpoint (`layers.N.attention.to_q.weight`, `noise_refiner.N...`,
`all_x_embedder.2-1`, `all_final_layer.2-1`, `cap_embedder.0/1`, `t_embedder.mlp.0/2`, `x_pad_token`,
`cap_pad_token`) so the safetensors shards load without renaming.

head_dim is 128 (3840 / 30), so attention runs on the tcgen05 flash kernel; q/k RMSNorm + RoPE is the fused
`rms_norm_rope` kernel; the gated residual adds are the fused `gated_residual` kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as OF
from ..layers import Linear, RMSNorm

ADALN_EMBED_DIM = 256
SEQ_MULTI_OF = 32


@dataclass
class ZImageConfig:
  in_channels: int = 16
  dim: int = 3840
  n_layers: int = 30
  n_refiner_layers: int = 2
  n_heads: int = 30
  norm_eps: float = 1e-5
  qk_norm: bool = True
  cap_feat_dim: int = 2560
  rope_theta: float = 256.0
  t_scale: float = 1000.0
  axes_dims: Sequence[int] = (32, 48, 48)
  axes_lens: Sequence[int] = (1536, 512, 512)


ZIMAGE_PRESETS = {
    "z-image": ZImageConfig(),
    "z-image-turbo": ZImageConfig(),
    "tiny": ZImageConfig(in_channels=4, dim=64, n_layers=2, n_refiner_layers=1, n_heads=4, cap_feat_dim=32,
                         axes_dims=(4, 6, 6), axes_lens=(128, 32, 32)),
}


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> torch.Tensor:
  half = dim // 2
  freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
  args = t.float()[:, None] * freqs[None]
  return torch.cat([args.cos(), args.sin()], dim=-1)


class ZImageRope:
  """Per-axis cos/sin tables; `__call__(ids [.., 3])` -> (cos, sin) [.., head_dim/2] (reference :520-556)."""

  def __init__(self, theta: float, axes_dims: Sequence[int], axes_lens: Sequence[int]):
    self.axes_dims, self.axes_lens = tuple(axes_dims), tuple(axes_lens)
    self.cos, self.sin = [], []
    for dim, length in zip(self.axes_dims, self.axes_lens):
      ang = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
      phase = torch.arange(length, dtype=torch.float32)[:, None] * ang[None]
      self.cos.append(phase.cos())
      self.sin.append(phase.sin())

  def __call__(self, ids: torch.Tensor):
    cos = torch.cat([c.to(ids.device)[ids[..., a]] for a, c in enumerate(self.cos)], dim=-1)
    sin = torch.cat([s.to(ids.device)[ids[..., a]] for a, s in enumerate(self.sin)], dim=-1)
    return cos, sin


def _rope_interleaved(x, cos, sin):
  """x: [B,S,H,D]; cos/sin: [B,S,D/2]."""
  xf = x.float().reshape(*x.shape[:-1], -1, 2)
  re, im = xf[..., 0], xf[..., 1]
  c, s = cos[:, :, None, :], sin[:, :, None, :]
  return torch.stack([re * c - im * s, re * s + im * c], dim=-1).reshape(x.shape).to(x.dtype)


class ZImageAttention(nn.Module):

  def __init__(self, dim: int, heads: int, qk_norm: bool, eps: float):
    super().__init__()
    self.heads, self.dim_head = heads, dim // heads
    self.to_q, self.to_k, self.to_v = (Linear(dim, dim, bias=False) for _ in range(3))
    self.to_out = nn.ModuleList([Linear(dim, dim, bias=False)])
    self.norm_q = RMSNorm(self.dim_head, eps) if qk_norm else None
    self.norm_k = RMSNorm(self.dim_head, eps) if qk_norm else None
    self.eps = eps

  def forward(self, x, freqs, mask=None, shared_positions: bool = True):
    B, S, _ = x.shape
    cos, sin = freqs
    q, k = self.to_q(x), self.to_k(x)
    v = self.to_v(x).view(B, S, self.heads, self.dim_head)
    if shared_positions and self.norm_q is not None and self.dim_head == 128:
      # fused per-head RMSNorm + RoPE (all batch rows share the position ids)
      q = OF.rms_norm_rope(q, self.norm_q.weight, cos[0], sin[0], heads=self.heads, per_head=True, eps=self.eps)
      k = OF.rms_norm_rope(k, self.norm_k.weight, cos[0], sin[0], heads=self.heads, per_head=True, eps=self.eps)
    else:
      q, k = q.view(B, S, self.heads, self.dim_head), k.view(B, S, self.heads, self.dim_head)
      if self.norm_q is not None:
        q, k = self.norm_q(q), self.norm_k(k)
      q, k = _rope_interleaved(q, cos, sin), _rope_interleaved(k, cos, sin)
    if mask is None:
      o = OF.attention(q, k, v)
    elif mask.dtype == torch.bool and mask.dim() == 2:
      o = OF.attention(q, k, v, keep_mask=mask)  # kept keys are compacted for the flash kernel
    else:
      o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                         attn_mask=mask[:, None, None, :]).transpose(1, 2)
    return self.to_out[0](o.reshape(B, S, -1))


class ZImageFeedForward(nn.Module):
  """w2(silu(w1 x) * w3 x), bias-free."""

  def __init__(self, dim: int, hidden: int):
    super().__init__()
    self.w1, self.w2, self.w3 = Linear(dim, hidden, bias=False), Linear(hidden, dim, bias=False), Linear(dim, hidden, bias=False)

  def forward(self, x):
    gate = self.w1(x, activation=None if torch.is_grad_enabled() else "silu")
    if torch.is_grad_enabled():
      gate = F.silu(gate)
    return self.w2(gate * self.w3(x))


def _select(noisy, clean, noise_mask):
  return torch.where(noise_mask[..., None] == 1, noisy[:, None, :], clean[:, None, :])


class ZImageTransformerBlock(nn.Module):

  def __init__(self, dim: int, heads: int, eps: float, qk_norm: bool, modulation: bool = True):
    super().__init__()
    self.modulation = modulation
    self.attention = ZImageAttention(dim, heads, qk_norm, 1e-5)
    self.feed_forward = ZImageFeedForward(dim, int(dim / 3 * 8))
    self.attention_norm1, self.ffn_norm1 = RMSNorm(dim, eps), RMSNorm(dim, eps)
    self.attention_norm2, self.ffn_norm2 = RMSNorm(dim, eps), RMSNorm(dim, eps)
    if modulation:
      self.adaLN_modulation = nn.ModuleList([Linear(min(dim, ADALN_EMBED_DIM), 4 * dim)])

  def forward(self, x, freqs, mask=None, adaln=None, noise_mask=None, adaln_noisy=None, adaln_clean=None,
              shared_positions=True):
    if not self.modulation:
      x = x + self.attention_norm2(self.attention(self.attention_norm1(x), freqs, mask, shared_positions))
      return x + self.ffn_norm2(self.feed_forward(self.ffn_norm1(x)))
    if noise_mask is None:
      mod = self.adaLN_modulation[0](adaln).float()
      scale_msa, gate_msa, scale_mlp, gate_mlp = mod.chunk(4, dim=-1)  # [B, dim] each
      h = (self.attention_norm1(x).float() * (1.0 + scale_msa[:, None])).to(x.dtype)
      a = self.attention_norm2(self.attention(h, freqs, mask, shared_positions))
      x = OF.gated_residual(x, a, torch.tanh(gate_msa))
      h = (self.ffn_norm1(x).float() * (1.0 + scale_mlp[:, None])).to(x.dtype)
      return OF.gated_residual(x, self.ffn_norm2(self.feed_forward(h)), torch.tanh(gate_mlp))
    # per-token choice between the modulation of noisy and of clean tokens (reference :451-459)
    n = self.adaLN_modulation[0](adaln_noisy).float().chunk(4, dim=-1)
    c = self.adaLN_modulation[0](adaln_clean).float().chunk(4, dim=-1)
    scale_msa = 1.0 + _select(n[0], c[0], noise_mask)
    gate_msa = _select(torch.tanh(n[1]), torch.tanh(c[1]), noise_mask)
    scale_mlp = 1.0 + _select(n[2], c[2], noise_mask)
    gate_mlp = _select(torch.tanh(n[3]), torch.tanh(c[3]), noise_mask)
    h = (self.attention_norm1(x).float() * scale_msa).to(x.dtype)
    x = (x.float() + gate_msa * self.attention_norm2(self.attention(h, freqs, mask, shared_positions)).float()).to(x.dtype)
    h = (self.ffn_norm1(x).float() * scale_mlp).to(x.dtype)
    return (x.float() + gate_mlp * self.ffn_norm2(self.feed_forward(h)).float()).to(x.dtype)


class ZImageFinalLayer(nn.Module):

  def __init__(self, dim: int, out_dim: int):
    super().__init__()
    self.linear = Linear(dim, out_dim)
    self.adaLN_modulation = nn.ModuleList([nn.SiLU(), Linear(min(dim, ADALN_EMBED_DIM), dim)])

  def forward(self, x, c):
    scale = self.adaLN_modulation[1](F.silu(c)).float()
    # LayerNorm without affine, times (1 + scale): the AdaLN kernel with shift = 0
    h = OF.layer_norm_mod(x, scale=scale, shift=torch.zeros_like(scale), eps=1e-6)
    return self.linear(h)


class _TimestepEmbedder(nn.Module):

  def __init__(self, out_size: int, mid_size: int, freq: int = 256):
    super().__init__()
    self.freq = freq
    self.mlp = nn.ModuleList([Linear(freq, mid_size), nn.SiLU(), Linear(mid_size, out_size)])

  def forward(self, t, dtype):
    x = timestep_embedding(t, self.freq).to(dtype)
    return self.mlp[2](F.silu(self.mlp[0](x)))


class ZImageTransformer2DModel(nn.Module):
  """`forward(x, t, cap_feats)`: x is a list of [C, F, H, W] latents (or one [B, C, F, H, W] tensor), cap_feats a
  list of [L_i, cap_feat_dim] caption features; returns a list of [C, F, H, W] predictions."""

  def __init__(self, cfg: ZImageConfig):
    super().__init__()
    self.cfg = cfg
    if cfg.dim // cfg.n_heads != sum(cfg.axes_dims):
      raise ValueError("Z-Image head_dim must equal sum(axes_dims)")
    patch_dim = 2 * 2 * 1 * cfg.in_channels
    self.all_x_embedder = nn.ModuleDict({"2-1": Linear(patch_dim, cfg.dim)})
    self.all_final_layer = nn.ModuleDict({"2-1": ZImageFinalLayer(cfg.dim, patch_dim)})
    self.t_embedder = _TimestepEmbedder(min(cfg.dim, ADALN_EMBED_DIM), 1024)
    self.cap_embedder = nn.ModuleList([RMSNorm(cfg.cap_feat_dim, cfg.norm_eps), Linear(cfg.cap_feat_dim, cfg.dim)])
    self.x_pad_token = nn.Parameter(torch.zeros(1, cfg.dim))
    self.cap_pad_token = nn.Parameter(torch.zeros(1, cfg.dim))
    mk = lambda mod: ZImageTransformerBlock(cfg.dim, cfg.n_heads, cfg.norm_eps, cfg.qk_norm, mod)
    self.noise_refiner = nn.ModuleList([mk(True) for _ in range(cfg.n_refiner_layers)])
    self.context_refiner = nn.ModuleList([mk(False) for _ in range(cfg.n_refiner_layers)])
    self.layers = nn.ModuleList([mk(True) for _ in range(cfg.n_layers)])
    self.rope = ZImageRope(cfg.rope_theta, cfg.axes_dims, cfg.axes_lens)

  # ---- token layout --------------------------------------------------------------------------
  @staticmethod
  def patchify(image: torch.Tensor):
    C, Fr, H, W = image.shape
    if H % 2 or W % 2:
      raise ValueError("Z-Image latents must be divisible by the 1x2x2 patch size")
    ht, wt = H // 2, W // 2
    p = image.reshape(C, Fr, 1, ht, 2, wt, 2).permute(1, 3, 5, 2, 4, 6, 0)
    return p.reshape(Fr * ht * wt, -1), (Fr, H, W), (Fr, ht, wt)

  def unpatchify(self, tokens: torch.Tensor, size):
    Fr, H, W = size
    C = self.cfg.in_channels
    n = Fr * (H // 2) * (W // 2)
    p = tokens[:n].reshape(Fr, H // 2, W // 2, 1, 2, 2, C)
    return p.permute(6, 0, 3, 1, 4, 2, 5).reshape(C, Fr, H, W)

  def _pad(self, feature, grid, start):
    for axis, (s, n, mx) in enumerate(zip(start, grid, self.rope.axes_lens)):
      if s + n > mx:
        raise ValueError(f"position ids along axis {axis} (start {s}, size {n}) exceed axes_lens[{axis}] = {mx}")
    original = feature.shape[0]
    pad = (-original) % SEQ_MULTI_OF
    total = original + pad
    axes = [torch.arange(s, s + n, device=feature.device) for s, n in zip(start, grid)]
    pos = torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=-1).reshape(-1, 3)
    if pos.shape[0] < total:  # pad tokens take position (0, 0, 0)
      pos = torch.cat([pos, pos.new_zeros((total - pos.shape[0], 3))])
    if pad:
      feature = torch.cat([feature, feature[-1:].expand(pad, -1)])
    mask = torch.arange(total, device=feature.device) >= original
    return feature, pos[:total], mask

  @staticmethod
  def _stack(feats, poss, masks):
    mx = max(f.shape[0] for f in feats)
    out_f, out_p, out_m = [], [], []
    for f, p, m in zip(feats, poss, masks):
      miss = mx - f.shape[0]
      if miss:
        f = F.pad(f, (0, 0, 0, miss))
        p = F.pad(p, (0, 0, 0, miss))
        m = F.pad(m, (0, miss), value=True)
      out_f.append(f), out_p.append(p), out_m.append(m)
    lengths = [f.shape[0] for f in feats]
    real = None
    if any(l != mx for l in lengths):
      real = torch.stack([torch.arange(mx, device=feats[0].device) < l for l in lengths])
    return torch.stack(out_f), torch.stack(out_p), torch.stack(out_m), real

  # ---- forward -------------------------------------------------------------------------------
  def forward(self, x, t: torch.Tensor, cap_feats):
    cfg = self.cfg
    if torch.is_tensor(x):
      x = list(x)
    if torch.is_tensor(cap_feats):
      cap_feats = list(cap_feats)
    if len(x) != len(cap_feats):
      raise ValueError("x and cap_feats must have one item per batch element")
    dtype = x[0].dtype
    adaln = self.t_embedder(t * cfg.t_scale, dtype)
    cf, cp, cm, xf, xp, xm, sizes = [], [], [], [], [], [], []
    for image, caption in zip(x, cap_feats):
      cap_len = caption.shape[0] + (-caption.shape[0]) % SEQ_MULTI_OF
      c, pos, m = self._pad(caption, (cap_len, 1, 1), (1, 0, 0))
      patches, size, tokens = self.patchify(image)
      p, ipos, im = self._pad(patches, tokens, (cap_len + 1, 0, 0))
      cf.append(c), cp.append(pos), cm.append(m)
      xf.append(p), xp.append(ipos), xm.append(im), sizes.append(size)
    caps, cap_pos, cap_pad, cap_real = self._stack(cf, cp, cm)
    imgs, img_pos, img_pad, img_real = self._stack(xf, xp, xm)
    shared = all(torch.equal(img_pos[0], p) for p in img_pos[1:]) and all(torch.equal(cap_pos[0], p) for p in cap_pos[1:])

    img = self.all_x_embedder["2-1"](imgs)
    img = torch.where(img_pad[..., None], self.x_pad_token.to(img.dtype), img)
    cap = self.cap_embedder[1](self.cap_embedder[0](caps))
    cap = torch.where(cap_pad[..., None], self.cap_pad_token.to(cap.dtype), cap)
    img_freqs, cap_freqs = self.rope(img_pos), self.rope(cap_pos)

    for blk in self.noise_refiner:
      img = blk(img, img_freqs, img_real, adaln, shared_positions=shared)
    for blk in self.context_refiner:
      cap = blk(cap, cap_freqs, cap_real, shared_positions=shared)

    joint = torch.cat([img, cap], dim=1)
    freqs = (torch.cat([img_freqs[0], cap_freqs[0]], dim=1), torch.cat([img_freqs[1], cap_freqs[1]], dim=1))
    mask = None
    if img_real is not None or cap_real is not None:
      B = joint.shape[0]
      ones = lambda n: torch.ones((B, n), dtype=torch.bool, device=joint.device)
      mask = torch.cat([img_real if img_real is not None else ones(img.shape[1]),
                        cap_real if cap_real is not None else ones(cap.shape[1])], dim=1)
    for blk in self.layers:
      joint = blk(joint, freqs, mask, adaln, shared_positions=shared)
    out = self.all_final_layer["2-1"](joint, adaln)
    return [self.unpatchify(out[i], size) for i, size in enumerate(sizes)]
