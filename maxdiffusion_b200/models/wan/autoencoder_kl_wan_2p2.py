"""Wan 2.2 VAE (TI2V-5B): 2x2 pixel patchify, z_dim 48, 16x spatial / 4x temporal compression, residual blocks with
parameter-free shortcut paths.

Reference: src/maxdiffusion/models/wan/autoencoder_kl_wan_2p2.py — `WanPatchify` / `WanUnpatchify` (:71-105),
`WanAvgDown3D` (space-time-to-channel then group mean, :579-636), `WanDupUp3D` (channel repeat then
channel-to-space-time, the first chunk drops its leading duplicate frame, :638-683), `WanDownBlock` / `WanUpBlock`
(:685-846: the resamplers keep the channel count, the shortcut is added to the block output), separate encoder
(160) and decoder (256) base widths, latent statistics (:1147-1258). The causal convolutions, RMS norms, resamplers,
mid block and the chunked cache loop are the Wan 2.1 ones.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .autoencoder_kl_wan import (DiagonalGaussian, FeatureCache, WanAttentionBlock, WanCausalConv3d, WanMidBlock,
                                 WanResample, WanResidualBlock, WanRMSNorm)

LATENTS_MEAN_2P2 = [-0.2289, -0.0052, -0.1323, -0.2339, -0.2799, 0.0174, 0.1838, 0.1557, -0.1382, 0.0542, 0.2813, 0.0891,
                    0.1570, -0.0098, 0.0375, -0.1825, -0.2246, -0.1207, -0.0698, 0.5109, 0.2665, -0.2108, -0.2158, 0.2502,
                    -0.2055, -0.0322, 0.1109, 0.1567, -0.0729, 0.0899, -0.2799, -0.1230, -0.0313, -0.1649, 0.0117, 0.0723,
                    -0.2839, -0.2083, -0.0520, 0.3748, 0.0152, 0.1957, 0.1433, -0.2944, 0.3573, -0.0548, -0.1681, -0.0667]
LATENTS_STD_2P2 = [0.4765, 1.0364, 0.4514, 1.1677, 0.5313, 0.4990, 0.4818, 0.5013, 0.8158, 1.0344, 0.5894, 1.0901, 0.6885,
                   0.6165, 0.8454, 0.4978, 0.5759, 0.3523, 0.7135, 0.6804, 0.5833, 1.4146, 0.8986, 0.5659, 0.7069, 0.5338,
                   0.4889, 0.4917, 0.4069, 0.4999, 0.6866, 0.4093, 0.5709, 0.6065, 0.6415, 0.4944, 0.5726, 1.2042, 0.5458,
                   1.6887, 0.3971, 1.0600, 0.3943, 0.5537, 0.5444, 0.4089, 0.7468, 0.7744]


@dataclass
class WanVAE2p2Config:
  base_dim: int = 160
  base_dec_dim: int = 256
  z_dim: int = 48
  dim_mult: Sequence[int] = (1, 2, 4, 4)
  num_res_blocks: int = 2
  attn_scales: Sequence[float] = ()
  temperal_downsample: Sequence[bool] = (False, True, True)
  dropout: float = 0.0
  patch_size: int = 2
  latents_mean: Sequence[float] = field(default_factory=lambda: list(LATENTS_MEAN_2P2))
  latents_std: Sequence[float] = field(default_factory=lambda: list(LATENTS_STD_2P2))

  @classmethod
  def from_dict(cls, d: dict) -> "WanVAE2p2Config":
    keys = cls.__dataclass_fields__.keys()
    return cls(**{k: v for k, v in d.items() if k in keys})


def patchify(x: torch.Tensor, p: int) -> torch.Tensor:
  """[B,C,T,H,W] -> [B, C*p*p, T, H/p, W/p]; channel index = c*p*p + w_in_patch*p + h_in_patch."""
  if p == 1:
    return x
  B, C, T, H, W = x.shape
  x = x.reshape(B, C, T, H // p, p, W // p, p).permute(0, 1, 6, 4, 2, 3, 5)
  return x.reshape(B, C * p * p, T, H // p, W // p)


def unpatchify(x: torch.Tensor, p: int) -> torch.Tensor:
  if p == 1:
    return x
  B, Ct, T, H, W = x.shape
  C = Ct // (p * p)
  x = x.reshape(B, C, p, p, T, H, W).permute(0, 1, 4, 5, 3, 6, 2)  # B, C, T, H, q, W, r
  return x.reshape(B, C, T, H * p, W * p)


class WanAvgDown3D(nn.Module):

  def __init__(self, cin, cout, factor_t, factor_s):
    super().__init__()
    self.ft, self.fs, self.cout = factor_t, factor_s, cout
    self.group = cin * factor_t * factor_s * factor_s // cout

  def forward(self, x):
    if self.ft == 1 and self.fs == 1 and self.group == 1:
      return x
    B, C, T, H, W = x.shape
    pad = (self.ft - T % self.ft) % self.ft
    if pad:
      x = F.pad(x, (0, 0, 0, 0, pad, 0))
      T += pad
    x = x.reshape(B, C, T // self.ft, self.ft, H // self.fs, self.fs, W // self.fs, self.fs)
    x = x.permute(0, 1, 3, 5, 7, 2, 4, 6).reshape(B, C * self.ft * self.fs * self.fs, T // self.ft, H // self.fs, W // self.fs)
    return x.reshape(B, self.cout, self.group, *x.shape[2:]).mean(dim=2)


class WanDupUp3D(nn.Module):

  def __init__(self, cin, cout, factor_t, factor_s):
    super().__init__()
    self.ft, self.fs, self.cout = factor_t, factor_s, cout
    self.repeats = cout * factor_t * factor_s * factor_s // cin

  def forward(self, x, first_chunk: bool):
    B, C, T, H, W = x.shape
    x = x.repeat_interleave(self.repeats, dim=1)
    x = x.reshape(B, self.cout, self.ft, self.fs, self.fs, T, H, W).permute(0, 1, 5, 2, 6, 3, 7, 4)
    x = x.reshape(B, self.cout, T * self.ft, H * self.fs, W * self.fs)
    return x[:, :, self.ft - 1:] if first_chunk else x


class _Resample2p2(WanResample):
  """The 2.2 resamplers keep the channel count."""

  def __init__(self, dim, mode):
    super().__init__(dim, mode, out_dim=dim)


class WanDownBlock2p2(nn.Module):

  def __init__(self, cin, cout, n, dropout, mode: Optional[str], down_flag: bool):
    super().__init__()
    self.avg_shortcut = WanAvgDown3D(cin, cout, 2 if mode == "downsample3d" else 1, 2 if down_flag else 1)
    layers, cur = [], cin
    for _ in range(n):
      layers.append(WanResidualBlock(cur, cout, dropout))
      cur = cout
    if mode is not None:
      layers.append(_Resample2p2(cout, mode))
    self.resnets = nn.ModuleList(layers)

  def forward(self, x, cache, first_chunk):
    h = x
    for layer in self.resnets:
      h = layer(h, cache, first_chunk) if isinstance(layer, WanResample) else layer(h, cache)
    return h + self.avg_shortcut(x)


class WanUpBlock2p2(nn.Module):

  def __init__(self, cin, cout, n, dropout, mode: Optional[str], up_flag: bool):
    super().__init__()
    self.avg_shortcut = WanDupUp3D(cin, cout, 2 if mode == "upsample3d" else 1, 2) if up_flag else None
    layers, cur = [], cin
    for _ in range(n + 1):
      layers.append(WanResidualBlock(cur, cout, dropout))
      cur = cout
    if mode is not None:
      layers.append(_Resample2p2(cout, mode))
    self.resnets = nn.ModuleList(layers)

  def forward(self, x, cache, first_chunk):
    h = x
    for layer in self.resnets:
      h = layer(h, cache, first_chunk) if isinstance(layer, WanResample) else layer(h, cache)
    return h + self.avg_shortcut(x, first_chunk) if self.avg_shortcut is not None else h


class WanEncoder3d2p2(nn.Module):

  def __init__(self, cfg: WanVAE2p2Config):
    super().__init__()
    dims = [cfg.base_dim * m for m in (1, *cfg.dim_mult)]
    n = len(cfg.dim_mult)
    self.conv_in = WanCausalConv3d(3 * cfg.patch_size ** 2, dims[0], 3, padding=1)
    self.down_blocks = nn.ModuleList([
        WanDownBlock2p2(din, dout, cfg.num_res_blocks, cfg.dropout,
                        ("downsample3d" if cfg.temperal_downsample[i] else "downsample2d") if i != n - 1 else None, i != n - 1)
        for i, (din, dout) in enumerate(zip(dims[:-1], dims[1:]))])
    self.mid_block = WanMidBlock(dims[-1], cfg.dropout)
    self.norm_out = WanRMSNorm(dims[-1], images=False)
    self.conv_out = WanCausalConv3d(dims[-1], cfg.z_dim * 2, 3, padding=1)

  def forward(self, x, cache=None, first_chunk=True):
    x = self.conv_in(x, cache)
    for blk in self.down_blocks:
      x = blk(x, cache, first_chunk)
    x = self.mid_block(x, cache)
    return self.conv_out(F.silu(self.norm_out(x)), cache)


class WanDecoder3d2p2(nn.Module):

  def __init__(self, cfg: WanVAE2p2Config):
    super().__init__()
    mult = list(cfg.dim_mult)
    dims = [cfg.base_dec_dim * m for m in (mult[-1], *mult[::-1])]
    up = list(cfg.temperal_downsample)[::-1]
    n = len(mult)
    self.conv_in = WanCausalConv3d(cfg.z_dim, dims[0], 3, padding=1)
    self.mid_block = WanMidBlock(dims[0], cfg.dropout)
    self.up_blocks = nn.ModuleList([
        WanUpBlock2p2(din, dout, cfg.num_res_blocks, cfg.dropout,
                      ("upsample3d" if up[i] else "upsample2d") if i != n - 1 else None, i != n - 1)
        for i, (din, dout) in enumerate(zip(dims[:-1], dims[1:]))])
    self.norm_out = WanRMSNorm(dims[-1], images=False)
    self.conv_out = WanCausalConv3d(dims[-1], 3 * cfg.patch_size ** 2, 3, padding=1)

  def forward(self, x, cache=None, first_chunk=True):
    x = self.mid_block(self.conv_in(x, cache), cache)
    for blk in self.up_blocks:
      x = blk(x, cache, first_chunk)
    return self.conv_out(F.silu(self.norm_out(x)), cache)


class AutoencoderKLWan2p2(nn.Module):

  def __init__(self, cfg: Optional[WanVAE2p2Config] = None):
    super().__init__()
    self.cfg = cfg or WanVAE2p2Config()
    self.encoder = WanEncoder3d2p2(self.cfg)
    self.quant_conv = WanCausalConv3d(self.cfg.z_dim * 2, self.cfg.z_dim * 2, 1)
    self.post_quant_conv = WanCausalConv3d(self.cfg.z_dim, self.cfg.z_dim, 1)
    self.decoder = WanDecoder3d2p2(self.cfg)

  def _stats(self, z):
    mean = torch.tensor(self.cfg.latents_mean, device=z.device, dtype=z.dtype).view(1, -1, 1, 1, 1)
    std = torch.tensor(self.cfg.latents_std, device=z.device, dtype=z.dtype).view(1, -1, 1, 1, 1)
    return mean, std

  def normalize_latents(self, z):
    mean, std = self._stats(z)
    return (z - mean) / std

  def denormalize_latents(self, z):
    mean, std = self._stats(z)
    return z * std + mean

  def _reset(self):
    for m in self.modules():
      if isinstance(m, WanResample):
        m.reset()

  def _run(self, net, x, chunk):
    self._reset()
    cache, outs, start, first = FeatureCache(), [], 0, True
    while start < x.shape[2]:
      n = 1 if first else min(chunk, x.shape[2] - start)
      cache.begin_pass()
      outs.append(net(x[:, :, start:start + n], cache, first_chunk=first))
      start, first = start + n, False
    return torch.cat(outs, dim=2)

  @torch.no_grad()
  def encode(self, x, chunk: int = 4) -> DiagonalGaussian:
    """x: [B,3,T,H,W] in [-1,1] with T = 1 + 4k and H, W multiples of 32."""
    return DiagonalGaussian(self.quant_conv(self._run(self.encoder, patchify(x, self.cfg.patch_size), chunk)))

  @torch.no_grad()
  def decode(self, z, chunk: int = 1):
    if z.is_cuda and z.dtype == torch.bfloat16 and self.cfg.z_dim % 16 == 0:
      # CUDA bf16 latents: channels-last on the implicit-GEMM convolution kernels (same modules and parameters)
      return self.channels_last_decoder().decode(z, chunk)
    out = self._run(self.decoder, self.post_quant_conv(z), chunk)
    return unpatchify(out, self.cfg.patch_size).clamp(-1.0, 1.0)

  def channels_last_decoder(self):
    """The kernel path of `decode` (`vae_channels_last.ChannelsLastDecoder`, created on first use)."""
    if getattr(self, "_cl_decoder", None) is None:
      from .vae_channels_last import ChannelsLastDecoder

      object.__setattr__(self, "_cl_decoder", ChannelsLastDecoder(self))
    return self._cl_decoder

  def encode_full(self, x):
    return DiagonalGaussian(self.quant_conv(self.encoder(patchify(x, self.cfg.patch_size), None, True)))

  def decode_full(self, z):
    return unpatchify(self.decoder(self.post_quant_conv(z), None, True), self.cfg.patch_size).clamp(-1.0, 1.0)
