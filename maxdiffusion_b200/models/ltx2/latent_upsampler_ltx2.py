"""LTX-2 latent up-sampler (second pass of multi-scale generation) and the latent post-filters.

Reference: src/maxdiffusion/models/ltx2/latent_upsampler_ltx2.py — `ResBlock` (conv, GroupNorm(32), SiLU; :34-66),
`PixelShuffleND` for 1 / 2 / 3 dims (:68-104), `BlurDownsample` (binomial 5-tap, depthwise, strided; :106-150),
`SpatialRationalResampler` (conv -> pixel shuffle by `num` -> blur-down by `den`; scales 0.75, 1.5, 2, 4; :152-177),
`LTX2LatentUpsamplerModel` (:179-330). Post-filters `adain_filter_latent` / `tone_map_latents`:
src/maxdiffusion/models/ltx2/ltx2_utils.py:838-858. Tensors are channels-first [B, C, F, H, W].
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..layers import GroupNorm

RATIONAL_RESAMPLER_SCALE_MAPPING = {0.75: (3, 4), 1.5: (3, 2), 2.0: (2, 1), 4.0: (4, 1)}


def _conv(dims, cin, cout):
  return (nn.Conv2d if dims == 2 else nn.Conv3d)(cin, cout, 3, padding=1)


class ResBlock(nn.Module):

  def __init__(self, channels: int, mid_channels: Optional[int] = None, dims: int = 3):
    super().__init__()
    mid = mid_channels or channels
    self.conv1, self.norm1 = _conv(dims, channels, mid), GroupNorm(32, mid)
    self.conv2, self.norm2 = _conv(dims, mid, channels), GroupNorm(32, channels)

  def forward(self, x):
    h = self.norm1(self.conv1(x), act=True)
    return F.silu(self.norm2(self.conv2(h)) + x)


def pixel_shuffle_nd(x, dims: int, factors: Sequence[int] = (2, 2, 2)):
  """Channels-first pixel shuffle; the channel index decomposes as (c, p1, p2, p3) with c slowest."""
  if dims == 3:
    p1, p2, p3 = factors[:3]
    B, Cp, D, H, W = x.shape
    C = Cp // (p1 * p2 * p3)
    return x.reshape(B, C, p1, p2, p3, D, H, W).permute(0, 1, 5, 2, 6, 3, 7, 4).reshape(B, C, D * p1, H * p2, W * p3)
  if dims == 2:
    p1, p2 = factors[:2]
    B, Cp, H, W = x.shape
    C = Cp // (p1 * p2)
    return x.reshape(B, C, p1, p2, H, W).permute(0, 1, 4, 2, 5, 3).reshape(B, C, H * p1, W * p2)
  p1 = factors[0]
  B, Cp, Fr, H, W = x.shape
  C = Cp // p1
  return x.reshape(B, C, p1, Fr, H, W).permute(0, 1, 3, 2, 4, 5).reshape(B, C, Fr * p1, H, W)


class BlurDownsample(nn.Module):

  def __init__(self, stride: int, kernel_size: int = 5):
    super().__init__()
    if kernel_size < 3 or kernel_size % 2 != 1:
      raise ValueError(f"`kernel_size` must be an odd number >= 3 but is {kernel_size}")
    self.stride, self.k = stride, kernel_size
    k = torch.tensor([math.comb(kernel_size - 1, i) for i in range(kernel_size)], dtype=torch.float32)
    k2 = torch.outer(k, k)
    self.register_buffer("kernel", k2 / k2.sum(), persistent=False)

  def forward(self, x):
    """x [N, C, H, W]."""
    if self.stride == 1:
      return x
    C = x.shape[1]
    return F.conv2d(x, self.kernel.to(x.dtype)[None, None].expand(C, 1, -1, -1), stride=self.stride, padding=self.k // 2, groups=C)


class SpatialRationalResampler(nn.Module):

  def __init__(self, mid_channels: int, scale: float):
    super().__init__()
    if scale not in RATIONAL_RESAMPLER_SCALE_MAPPING:
      raise ValueError(f"scale {scale} not supported.")
    self.num, den = RATIONAL_RESAMPLER_SCALE_MAPPING[scale]
    self.conv = nn.Conv2d(mid_channels, mid_channels * self.num ** 2, 3, padding=1)
    self.blur_down = BlurDownsample(den)

  def forward(self, x):
    return self.blur_down(pixel_shuffle_nd(self.conv(x), 2, (self.num, self.num)))


class LTX2LatentUpsamplerModel(nn.Module):

  def __init__(self, in_channels: int = 128, mid_channels: int = 1024, num_blocks_per_stage: int = 4, dims: int = 3,
               spatial_upsample: bool = True, temporal_upsample: bool = False, rational_spatial_scale: Optional[float] = 2.0):
    super().__init__()
    self.in_channels, self.mid_channels, self.dims = in_channels, mid_channels, dims
    self.spatial, self.temporal, self.rational = spatial_upsample, temporal_upsample, rational_spatial_scale
    self.initial_conv, self.initial_norm = _conv(dims, in_channels, mid_channels), GroupNorm(32, mid_channels)
    self.res_blocks = nn.ModuleList([ResBlock(mid_channels, dims=dims) for _ in range(num_blocks_per_stage)])
    self.upsampler = None
    if dims == 3 and spatial_upsample and temporal_upsample:
      self.upsampler = nn.ModuleList([nn.Conv3d(mid_channels, 8 * mid_channels, 3, padding=1)])
    elif dims == 3 and temporal_upsample:
      self.upsampler = nn.ModuleList([nn.Conv3d(mid_channels, 2 * mid_channels, 3, padding=1)])
    elif spatial_upsample:
      self.upsampler = SpatialRationalResampler(mid_channels, rational_spatial_scale) if rational_spatial_scale is not None \
          else nn.ModuleList([nn.Conv2d(mid_channels, 4 * mid_channels, 3, padding=1)])
    self.post_upsample_res_blocks = nn.ModuleList([ResBlock(mid_channels, dims=dims) for _ in range(num_blocks_per_stage)])
    self.final_conv = _conv(dims, mid_channels, in_channels)

  def _spatial(self, x2d):
    if isinstance(self.upsampler, SpatialRationalResampler):
      return self.upsampler(x2d)
    return pixel_shuffle_nd(self.upsampler[0](x2d), 2)

  def forward(self, x):
    """x [B, C, F, H, W] latents -> up-sampled latents."""
    B, C, Fr, H, W = x.shape
    frames = lambda t: t.permute(0, 2, 1, 3, 4).reshape(B * Fr, t.shape[1], t.shape[3], t.shape[4])
    video = lambda t: t.reshape(B, Fr, t.shape[1], t.shape[2], t.shape[3]).permute(0, 2, 1, 3, 4)
    if self.dims == 2:
      h = self.initial_norm(self.initial_conv(frames(x)), act=True)
      for blk in self.res_blocks:
        h = blk(h)
      if self.spatial:
        h = self._spatial(h)
      for blk in self.post_upsample_res_blocks:
        h = blk(h)
      return video(self.final_conv(h))
    h = self.initial_norm(self.initial_conv(x), act=True)
    for blk in self.res_blocks:
      h = blk(h)
    if self.spatial and self.temporal:
      h = pixel_shuffle_nd(self.upsampler[0](h), 3)[:, :, 1:]
    elif self.temporal:
      h = pixel_shuffle_nd(self.upsampler[0](h), 1)[:, :, 1:]
    elif self.spatial:
      h = video(self._spatial(frames(h)))
    for blk in self.post_upsample_res_blocks:
      h = blk(h)
    return self.final_conv(h)


def adain_filter_latent(latents: torch.Tensor, reference: torch.Tensor, factor: float = 1.0) -> torch.Tensor:
  """Match per-(sample, channel) mean / std of `latents` to `reference` and blend by `factor`."""
  dims = tuple(range(2, latents.dim()))
  lm, ls = latents.mean(dim=dims, keepdim=True), latents.std(dim=dims, keepdim=True, unbiased=False)
  rm, rs = reference.mean(dim=dims, keepdim=True), reference.std(dim=dims, keepdim=True, unbiased=False)
  matched = (latents - lm) / (ls + 1e-5) * rs + rm
  return torch.lerp(latents, matched, factor)


def tone_map_latents(latents: torch.Tensor, compression: float) -> torch.Tensor:
  """Sigmoid compression of large latent magnitudes (`compression` in [0, 1]; 0 = identity)."""
  scale_factor = compression * 0.75
  abs_latents = latents.abs()
  sigmoid_term = torch.sigmoid(4.0 * scale_factor * (abs_latents - 1.0))
  scales = 1.0 - 0.8 * scale_factor * sigmoid_term
  return latents * scales
