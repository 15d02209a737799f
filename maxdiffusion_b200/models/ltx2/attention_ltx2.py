"""LTX-2 attention and rotary position embeddings.

Reference: src/maxdiffusion/models/ltx2/attention_ltx2.py
  * `LTX2RotaryPosEmbed` (:105-326): fractional coordinates — video (frame / fps with the causal offset, h, w in
    pixels), audio (seconds) — are taken at patch mid-points, divided by the base extents, mapped to [-1, 1] and
    multiplied by `theta ** linspace(0, 1, dim // (2 n_axes)) * pi / 2`; `interleaved` layout repeats every
    frequency twice (left-padded with cos = 1, sin = 0 up to `dim`), `split` layout keeps `dim / 2` frequencies
    reshaped per head;
  * `LTX2Attention` (:329-611): q / k / v projections with bias, RMSNorm over the FULL inner dimension on q and k,
    RoPE on q (and on k with its own table for audio<->video attention), optional STG perturbation
    `v + mask * (attn - v)` (:592-595), optional per-head gate `2 * sigmoid(Linear(x))` (:597-603), output projection.
Video heads are 128 wide and run on the tcgen05 flash kernel; audio heads are 64 wide.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as OF
from ..layers import Linear, RMSNorm


def apply_rotary_emb(x, freqs):
  """Interleaved pairs: out = x * cos + [-x_odd, x_even] * sin; x [B,S,D], cos/sin broadcastable to it."""
  cos, sin = freqs
  xr = x.float().reshape(*x.shape[:-1], -1, 2)
  rot = torch.stack([-xr[..., 1], xr[..., 0]], dim=-1).reshape(x.shape)
  return (x.float() * cos + rot * sin).to(x.dtype)


def apply_split_rotary_emb(x, freqs):
  """Split halves per head: x [B,S,H*D]; cos/sin [B,H,S,D/2]."""
  cos, sin = freqs
  B, H, S, r = cos.shape
  xh = x.float().reshape(B, S, H, 2, r).permute(0, 2, 1, 3, 4)
  a, b = xh[..., 0, :], xh[..., 1, :]
  out = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-2)
  return out.permute(0, 2, 1, 3, 4).reshape(x.shape).to(x.dtype)


class LTX2RotaryPosEmbed(nn.Module):

  def __init__(self, dim: int, patch_size: int = 1, patch_size_t: int = 1, base_num_frames: int = 20,
               base_height: int = 2048, base_width: int = 2048, sampling_rate: int = 16000, hop_length: int = 160,
               scale_factors: Sequence[int] = (8, 32, 32), theta: float = 10000.0, causal_offset: int = 1,
               modality: str = "video", rope_type: str = "interleaved", num_attention_heads: int = 32):
    super().__init__()
    if rope_type not in ("interleaved", "split"):
      raise ValueError(f"rope_type={rope_type} not supported. Choose between 'interleaved' and 'split'.")
    if modality not in ("video", "audio"):
      raise ValueError(f"Modality {modality} is not supported. Supported modalities are `video` and `audio`.")
    self.dim, self.patch_size, self.patch_size_t = dim, patch_size, patch_size_t
    self.base = (base_num_frames, base_height, base_width)
    self.sampling_rate, self.hop_length, self.scale_factors = sampling_rate, hop_length, tuple(scale_factors)
    self.theta, self.causal_offset, self.modality, self.rope_type, self.heads = theta, causal_offset, modality, rope_type, num_attention_heads

  def prepare_video_coords(self, batch: int, num_frames: int, height: int, width: int, fps: float = 24.0, device=None):
    """[B, 3, n_patches, 2]: (start, end) of every latent patch in seconds / pixels."""
    gf = torch.arange(0, num_frames, self.patch_size_t, dtype=torch.float32, device=device)
    gh = torch.arange(0, height, self.patch_size, dtype=torch.float32, device=device)
    gw = torch.arange(0, width, self.patch_size, dtype=torch.float32, device=device)
    grid = torch.stack(torch.meshgrid(gf, gh, gw, indexing="ij"), dim=0)
    delta = torch.tensor([self.patch_size_t, self.patch_size, self.patch_size], dtype=torch.float32, device=device).view(3, 1, 1, 1)
    coords = torch.stack([grid, grid + delta], dim=-1).reshape(3, -1, 2)[None].repeat(batch, 1, 1, 1)
    coords = coords * torch.tensor(self.scale_factors, dtype=torch.float32, device=device).view(1, 3, 1, 1)
    coords[:, 0] = (coords[:, 0] + self.causal_offset - self.scale_factors[0]).clamp(min=0) / fps
    return coords

  def prepare_audio_coords(self, batch: int, num_frames: int, shift: int = 0, device=None):
    """[B, 1, n_patches, 2] in seconds."""
    gf = torch.arange(shift, num_frames + shift, self.patch_size_t, dtype=torch.float32, device=device)
    s = self.scale_factors[0]
    to_s = lambda g: (g * s + self.causal_offset - s).clamp(min=0) * self.hop_length / self.sampling_rate
    coords = torch.stack([to_s(gf), to_s(gf + self.patch_size_t)], dim=-1)
    return coords[None, None].repeat(batch, 1, 1, 1)

  def prepare_coords(self, *a, **k):
    return self.prepare_video_coords(*a, **k) if self.modality == "video" else self.prepare_audio_coords(*a, **k)

  def forward(self, coords: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    if coords.dim() == 4:
      n = coords.shape[1]
      grid = ((coords[..., 0] + coords[..., 1]) / 2.0).transpose(1, 2)  # [B, patches, n]
    elif coords.dim() == 3:
      n, grid = coords.shape[-1], coords
    else:
      raise ValueError(f"coords must be 3D or 4D, got {coords.dim()}D")
    maxpos = torch.tensor(self.base[:n] if self.modality == "video" else self.base[:1], dtype=torch.float64, device=coords.device)
    grid = grid.double() / maxpos.view(1, 1, -1)
    steps = self.dim // (2 * n)
    base = torch.pow(torch.tensor(self.theta, dtype=torch.float64), torch.linspace(0.0, 1.0, steps, dtype=torch.float64)).to(coords.device) * math.pi / 2.0
    freqs = (grid * 2.0 - 1.0).unsqueeze(-1) * base            # [B, P, n, steps]
    freqs = freqs.transpose(-1, -2).reshape(*freqs.shape[:2], -1)  # [B, P, steps * n]
    cos, sin = freqs.cos().float(), freqs.sin().float()
    if self.rope_type == "interleaved":
      cos, sin = cos.repeat_interleave(2, dim=-1), sin.repeat_interleave(2, dim=-1)
      pad = self.dim - cos.shape[-1]
      if pad > 0:
        cos = torch.cat([torch.ones_like(cos[..., :pad]), cos], dim=-1)
        sin = torch.cat([torch.zeros_like(sin[..., :pad]), sin], dim=-1)
      return cos, sin
    pad = self.dim // 2 - cos.shape[-1]
    if pad > 0:
      cos = torch.cat([torch.ones_like(cos[..., :pad]), cos], dim=-1)
      sin = torch.cat([torch.zeros_like(sin[..., :pad]), sin], dim=-1)
    B, P = cos.shape[:2]
    return (cos.reshape(B, P, self.heads, -1).permute(0, 2, 1, 3), sin.reshape(B, P, self.heads, -1).permute(0, 2, 1, 3))


class LTX2Attention(nn.Module):

  def __init__(self, query_dim: int, heads: int, dim_head: int, context_dim: Optional[int] = None, bias: bool = True,
               out_bias: bool = True, eps: float = 1e-6, rope_type: str = "interleaved", gated_attn: bool = False):
    super().__init__()
    self.heads, self.dim_head, self.inner_dim, self.rope_type = heads, dim_head, heads * dim_head, rope_type
    kv = context_dim if context_dim is not None else query_dim
    self.to_q = Linear(query_dim, self.inner_dim, bias=bias)
    self.to_k = Linear(kv, self.inner_dim, bias=bias)
    self.to_v = Linear(kv, self.inner_dim, bias=bias)
    self.norm_q, self.norm_k = RMSNorm(self.inner_dim, eps), RMSNorm(self.inner_dim, eps)
    self.to_out = nn.ModuleList([Linear(self.inner_dim, query_dim, bias=out_bias)])
    self.to_gate_logits = Linear(query_dim, heads, bias=True) if gated_attn else None

  def _norm(self, x, norm: RMSNorm):
    C = x.shape[-1]
    if C % 128 == 0:  # fused RMSNorm over the full row (the rotary tables are per channel: applied separately)
      return OF.rms_norm_rope(x, norm.weight, heads=C // 128, eps=norm.eps).reshape(x.shape)
    return norm(x)

  def compute_kv(self, context):
    return self._norm(self.to_k(context), self.norm_k), self.to_v(context)

  def forward(self, x, encoder_hidden_states=None, attention_mask=None, rotary_emb=None, k_rotary_emb=None,
              perturbation_mask=None, cached_kv=None):
    B, S, _ = x.shape
    q = self._norm(self.to_q(x), self.norm_q)
    if cached_kv is not None:
      k, v = cached_kv
    else:
      k, v = self.compute_kv(encoder_hidden_states if encoder_hidden_states is not None else x)
    rope = apply_split_rotary_emb if self.rope_type == "split" else apply_rotary_emb
    if rotary_emb is not None:
      q = rope(q, rotary_emb)
      if k_rotary_emb is not None:
        k = rope(k, k_rotary_emb)
      elif encoder_hidden_states is None:
        k = rope(k, rotary_emb)
    H, D = self.heads, self.dim_head
    q4, k4, v4 = q.view(B, S, H, D), k.view(B, k.shape[1], H, D), v.view(B, v.shape[1], H, D)
    if attention_mask is None:
      o = OF.attention(q4, k4, v4)
    elif attention_mask.dtype == torch.bool and attention_mask.dim() == 2:
      o = OF.attention(q4, k4, v4, keep_mask=attention_mask)  # kept keys are compacted for the flash kernel
    else:
      o = F.scaled_dot_product_attention(q4.transpose(1, 2), k4.transpose(1, 2), v4.transpose(1, 2),
                                         attn_mask=attention_mask[:, None, None, :]).transpose(1, 2)
    o = o.reshape(B, S, H * D)
    if perturbation_mask is not None:
      # spatio-temporal guidance: perturbed samples skip attention and pass the values through
      o = v + perturbation_mask.to(o.dtype) * (o - v)
    if self.to_gate_logits is not None:
      gates = 2.0 * torch.sigmoid(self.to_gate_logits(x).float())
      o = (o.view(B, S, H, D).float() * gates.unsqueeze(-1)).to(x.dtype).reshape(B, S, H * D)
    return self.to_out[0](o)
