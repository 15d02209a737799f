"""Wan 2.1 causal 3-D VAE (and the 2.2 variant's patchify / residual shortcuts) with chunked, cached decoding.

Parity target: the reference's `AutoencoderKLWan`
(src/maxdiffusion/models/wan/autoencoder_kl_wan.py:70-1340): `WanCausalConv3d` with a 2-frame feature cache
(`CACHE_T = 2`, :37,70-147), `WanRMS_norm` (:150), `WanResample` (nearest-2x + conv2d; `upsample3d` = time conv
C -> 2C then frame interleave, the first latent frame is not temporally up-sampled; `downsample3d` = strided
time conv, :245-389), `WanResidualBlock` (:392-484), single-head spatial `WanAttentionBlock` (:487-546),
encoder / decoder (:668-959), and the time-chunked encode / decode loops that carry the caches
(:1134-1327). Parameter names follow the diffusers checkpoint so that its safetensors load directly.

Two execution paths share the modules and parameters of this file. CUDA bf16 latents are decoded channels-last on
the implicit-GEMM convolution kernels of this repository (`vae_channels_last.ChannelsLastDecoder`). Everything else
(CPU, fp32, the encoder) runs the plain PyTorch forward below (`F.conv3d` / `F.conv2d`), which is also the oracle the
kernel path is tested against.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

CACHE_T = 2

LATENTS_MEAN = [-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508, 0.4134, -0.0715, 0.5517,
                -0.3632, -0.1922, -0.9497, 0.2503, -0.2921]
LATENTS_STD = [2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743, 3.2687, 2.1526, 2.8652, 1.5579,
               1.6382, 1.1253, 2.8251, 1.9160]


@dataclass
class WanVAEConfig:
  base_dim: int = 96
  z_dim: int = 16
  dim_mult: Sequence[int] = (1, 2, 4, 4)
  num_res_blocks: int = 2
  attn_scales: Sequence[float] = ()
  temperal_downsample: Sequence[bool] = (False, True, True)
  dropout: float = 0.0
  in_channels: int = 3
  out_channels: int = 3
  latents_mean: Sequence[float] = field(default_factory=lambda: list(LATENTS_MEAN))
  latents_std: Sequence[float] = field(default_factory=lambda: list(LATENTS_STD))

  @classmethod
  def from_dict(cls, d: dict) -> "WanVAEConfig":
    keys = cls.__dataclass_fields__.keys()
    return cls(**{k: v for k, v in d.items() if k in keys})


class FeatureCache:
  """Per-convolution history of the last CACHE_T input frames, addressed by call order within one pass."""

  def __init__(self):
    self.slots: List[Optional[torch.Tensor]] = []
    self.cursor = 0

  def begin_pass(self) -> None:
    self.cursor = 0

  def next(self) -> int:
    i = self.cursor
    self.cursor += 1
    if i >= len(self.slots):
      self.slots.append(None)
    return i


class WanCausalConv3d(nn.Conv3d):
  """3-D convolution that pads time only on the past side; the past comes from the cache when chunking."""

  def __init__(self, cin, cout, kernel_size, stride=1, padding=0):
    super().__init__(cin, cout, kernel_size, stride=stride, padding=0)
    k = (kernel_size,) * 3 if isinstance(kernel_size, int) else tuple(kernel_size)
    p = (padding,) * 3 if isinstance(padding, int) else tuple(padding)
    self.time_pad = 2 * p[0]
    self.space_pad = (p[2], p[2], p[1], p[1])
    self.kt = k[0]

  def forward(self, x, cache: Optional[FeatureCache] = None):
    hist = None
    slot = None
    if cache is not None and self.kt > 1:
      slot = cache.next()
      hist = cache.slots[slot]
      tail = x[:, :, -CACHE_T:]
      if tail.shape[2] < CACHE_T and hist is not None:
        tail = torch.cat([hist[:, :, -(CACHE_T - tail.shape[2]):], tail], dim=2)
      new_hist = tail
    pad_t = self.time_pad
    if hist is not None and pad_t > 0:
      use = hist[:, :, -pad_t:]
      x = torch.cat([use.to(x.dtype), x], dim=2)
      pad_t -= use.shape[2]
    x = F.pad(x, self.space_pad + (pad_t, 0))
    if slot is not None:
      cache.slots[slot] = new_hist
    return F.conv3d(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype), self.stride)


class WanRMSNorm(nn.Module):
  """x / max(||x||_2, eps) * sqrt(C) * gamma over the channel axis (reference: :150-183)."""

  def __init__(self, dim: int, channel_first: bool = True, images: bool = True, bias: bool = False):
    super().__init__()
    broad = (1, 1) if images else (1, 1, 1)
    shape = (dim, *broad) if channel_first else (dim,)
    self.channel_first = channel_first
    self.scale = dim ** 0.5
    self.gamma = nn.Parameter(torch.ones(shape))
    self.bias = nn.Parameter(torch.zeros(shape)) if bias else None

  def forward(self, x):
    y = F.normalize(x.float(), dim=(1 if self.channel_first else -1)) * self.scale * self.gamma.float()
    if self.bias is not None:
      y = y + self.bias.float()
    return y.to(x.dtype)


class WanResample(nn.Module):

  def __init__(self, dim: int, mode: str, out_dim: Optional[int] = None):
    super().__init__()
    self.dim, self.mode = dim, mode
    out_dim = out_dim if out_dim is not None else dim // 2
    if mode in ("upsample2d", "upsample3d"):
      self.resample = nn.Sequential(nn.Upsample(scale_factor=(2.0, 2.0), mode="nearest-exact"),
                                    nn.Conv2d(dim, out_dim, 3, padding=1))
      if mode == "upsample3d":
        self.time_conv = WanCausalConv3d(dim, dim * 2, (3, 1, 1), padding=(1, 0, 0))
    elif mode in ("downsample2d", "downsample3d"):
      self.resample = nn.Sequential(nn.ZeroPad2d((0, 1, 0, 1)), nn.Conv2d(dim, dim, 3, stride=(2, 2)))
      if mode == "downsample3d":
        self.time_conv = WanCausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0))
    else:
      self.resample = nn.Identity()
    self._started = False  # chunked mode: has the first chunk passed through this layer?

  def reset(self) -> None:
    self._started = False
    self._down_hist = None

  def forward(self, x, cache: Optional[FeatureCache] = None, first_chunk: bool = True):
    b, c, t, h, w = x.shape
    if self.mode == "upsample3d":
      if cache is None:
        # whole clip at once: the first frame is kept single, every later frame is doubled
        if t > 1:
          rest = self.time_conv(x[:, :, 1:])
          rest = rest.reshape(b, 2, c, t - 1, h, w).permute(0, 2, 3, 1, 4, 5).reshape(b, c, 2 * (t - 1), h, w)
          x = torch.cat([x[:, :, :1], rest], dim=2)
      elif first_chunk:
        cache.next()  # the first frame skips the time convolution but keeps the slot order of later chunks
      else:
        y = self.time_conv(x, cache)
        x = y.reshape(b, 2, c, t, h, w).permute(0, 2, 3, 1, 4, 5).reshape(b, c, 2 * t, h, w)
    t2 = x.shape[2]
    x = x.permute(0, 2, 1, 3, 4).reshape(b * t2, c, h, w)
    x = self.resample(x)
    x = x.reshape(b, t2, x.shape[1], x.shape[2], x.shape[3]).permute(0, 2, 1, 3, 4)
    if self.mode == "downsample3d":
      if cache is None:
        if x.shape[2] > 1:
          first, rest = x[:, :, :1], x[:, :, 1:]
          # strided time conv over [first | rest] without padding: frames (0,1,2) -> out 1, (2,3,4) -> out 2 ...
          rest = F.conv3d(torch.cat([first, rest], dim=2), self.time_conv.weight.to(x.dtype),
                          self.time_conv.bias.to(x.dtype), stride=(2, 1, 1))
          x = torch.cat([first, rest], dim=2)
      else:
        if first_chunk:
          self._down_hist = x[:, :, -1:].clone()
        else:
          inp = torch.cat([self._down_hist, x], dim=2)
          self._down_hist = x[:, :, -1:].clone()
          x = F.conv3d(inp, self.time_conv.weight.to(x.dtype), self.time_conv.bias.to(x.dtype), stride=(2, 1, 1))
    return x


class WanResidualBlock(nn.Module):

  def __init__(self, in_dim: int, out_dim: int, dropout: float = 0.0):
    super().__init__()
    self.norm1 = WanRMSNorm(in_dim, images=False)
    self.conv1 = WanCausalConv3d(in_dim, out_dim, 3, padding=1)
    self.norm2 = WanRMSNorm(out_dim, images=False)
    self.conv2 = WanCausalConv3d(out_dim, out_dim, 3, padding=1)
    self.conv_shortcut = WanCausalConv3d(in_dim, out_dim, 1) if in_dim != out_dim else None

  def forward(self, x, cache=None):
    h = self.conv_shortcut(x) if self.conv_shortcut is not None else x
    x = self.conv1(F.silu(self.norm1(x)), cache)
    x = self.conv2(F.silu(self.norm2(x)), cache)
    return x + h


class WanAttentionBlock(nn.Module):
  """Single-head self-attention over the H*W positions of every frame."""

  def __init__(self, dim: int):
    super().__init__()
    self.norm = WanRMSNorm(dim)
    self.to_qkv = nn.Conv2d(dim, dim * 3, 1)
    self.proj = nn.Conv2d(dim, dim, 1)

  def forward(self, x):
    b, c, t, h, w = x.shape
    y = x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w)
    y = self.norm(y)
    q, k, v = self.to_qkv(y).reshape(b * t, 1, 3 * c, h * w).permute(0, 1, 3, 2).chunk(3, dim=-1)
    y = F.scaled_dot_product_attention(q, k, v)
    y = y.squeeze(1).permute(0, 2, 1).reshape(b * t, c, h, w)
    y = self.proj(y).reshape(b, t, c, h, w).permute(0, 2, 1, 3, 4)
    return x + y


class WanMidBlock(nn.Module):

  def __init__(self, dim: int, dropout: float = 0.0):
    super().__init__()
    self.resnets = nn.ModuleList([WanResidualBlock(dim, dim, dropout), WanResidualBlock(dim, dim, dropout)])
    self.attentions = nn.ModuleList([WanAttentionBlock(dim)])

  def forward(self, x, cache=None):
    x = self.resnets[0](x, cache)
    x = self.attentions[0](x)
    return self.resnets[1](x, cache)


class WanEncoder3d(nn.Module):

  def __init__(self, cfg: WanVAEConfig):
    super().__init__()
    dims = [cfg.base_dim * m for m in (1, *cfg.dim_mult)]
    self.conv_in = WanCausalConv3d(cfg.in_channels, dims[0], 3, padding=1)
    blocks = []
    scale = 1.0
    for i, (din, dout) in enumerate(zip(dims[:-1], dims[1:])):
      for _ in range(cfg.num_res_blocks):
        blocks.append(WanResidualBlock(din, dout, cfg.dropout))
        if scale in cfg.attn_scales:
          blocks.append(WanAttentionBlock(dout))
        din = dout
      if i != len(cfg.dim_mult) - 1:
        blocks.append(WanResample(dout, "downsample3d" if cfg.temperal_downsample[i] else "downsample2d"))
        scale /= 2.0
    self.down_blocks = nn.ModuleList(blocks)
    self.mid_block = WanMidBlock(dims[-1], cfg.dropout)
    self.norm_out = WanRMSNorm(dims[-1], images=False)
    self.conv_out = WanCausalConv3d(dims[-1], cfg.z_dim * 2, 3, padding=1)

  def forward(self, x, cache=None, first_chunk=True):
    x = self.conv_in(x, cache)
    for blk in self.down_blocks:
      if isinstance(blk, WanResample):
        x = blk(x, cache, first_chunk)
      elif isinstance(blk, WanResidualBlock):
        x = blk(x, cache)
      else:
        x = blk(x)
    x = self.mid_block(x, cache)
    return self.conv_out(F.silu(self.norm_out(x)), cache)


class WanUpBlock(nn.Module):

  def __init__(self, in_dim, out_dim, num_res_blocks, dropout, upsample_mode):
    super().__init__()
    res, cur = [], in_dim
    for _ in range(num_res_blocks + 1):
      res.append(WanResidualBlock(cur, out_dim, dropout))
      cur = out_dim
    self.resnets = nn.ModuleList(res)
    self.upsamplers = nn.ModuleList([WanResample(out_dim, upsample_mode)]) if upsample_mode else None

  def forward(self, x, cache=None, first_chunk=True):
    for r in self.resnets:
      x = r(x, cache)
    if self.upsamplers is not None:
      x = self.upsamplers[0](x, cache, first_chunk)
    return x


class WanDecoder3d(nn.Module):

  def __init__(self, cfg: WanVAEConfig):
    super().__init__()
    mult = list(cfg.dim_mult)
    dims = [cfg.base_dim * m for m in (mult[-1], *mult[::-1])]
    temporal_up = list(cfg.temperal_downsample)[::-1]
    self.conv_in = WanCausalConv3d(cfg.z_dim, dims[0], 3, padding=1)
    self.mid_block = WanMidBlock(dims[0], cfg.dropout)
    ups = []
    for i, (din, dout) in enumerate(zip(dims[:-1], dims[1:])):
      if i > 0:
        din = din // 2
      mode = None
      if i != len(mult) - 1:
        mode = "upsample3d" if temporal_up[i] else "upsample2d"
      ups.append(WanUpBlock(din, dout, cfg.num_res_blocks, cfg.dropout, mode))
    self.up_blocks = nn.ModuleList(ups)
    self.norm_out = WanRMSNorm(dims[-1], images=False)
    self.conv_out = WanCausalConv3d(dims[-1], cfg.out_channels, 3, padding=1)

  def forward(self, x, cache=None, first_chunk=True):
    x = self.conv_in(x, cache)
    x = self.mid_block(x, cache)
    for up in self.up_blocks:
      x = up(x, cache, first_chunk)
    return self.conv_out(F.silu(self.norm_out(x)), cache)


class DiagonalGaussian:

  def __init__(self, moments: torch.Tensor):
    self.mean, self.logvar = moments.chunk(2, dim=1)
    self.logvar = self.logvar.clamp(-30.0, 20.0)

  def sample(self, generator=None):
    noise = torch.randn(self.mean.shape, generator=generator, device=self.mean.device, dtype=self.mean.dtype)
    return self.mean + torch.exp(0.5 * self.logvar) * noise

  def mode(self):
    return self.mean


class AutoencoderKLWan(nn.Module):

  def __init__(self, cfg: Optional[WanVAEConfig] = None):
    super().__init__()
    self.cfg = cfg or WanVAEConfig()
    self.encoder = WanEncoder3d(self.cfg)
    self.quant_conv = WanCausalConv3d(self.cfg.z_dim * 2, self.cfg.z_dim * 2, 1)
    self.post_quant_conv = WanCausalConv3d(self.cfg.z_dim, self.cfg.z_dim, 1)
    self.decoder = WanDecoder3d(self.cfg)

  # ---- latent statistics ------------------------------------------------------------------
  def normalize_latents(self, z):
    mean = torch.tensor(self.cfg.latents_mean, device=z.device, dtype=z.dtype).view(1, -1, 1, 1, 1)
    std = torch.tensor(self.cfg.latents_std, device=z.device, dtype=z.dtype).view(1, -1, 1, 1, 1)
    return (z - mean) / std

  def denormalize_latents(self, z):
    mean = torch.tensor(self.cfg.latents_mean, device=z.device, dtype=z.dtype).view(1, -1, 1, 1, 1)
    std = torch.tensor(self.cfg.latents_std, device=z.device, dtype=z.dtype).view(1, -1, 1, 1, 1)
    return z * std + mean

  def _reset(self):
    for m in self.modules():
      if isinstance(m, WanResample):
        m.reset()

  # ---- encode / decode ---------------------------------------------------------------------
  @torch.no_grad()
  def encode(self, x, chunk: int = 4) -> DiagonalGaussian:
    """x: [B,3,T,H,W] in [-1,1], T = 1 + 4k. Frames go through in chunks (first frame alone) with cached history."""
    if x.is_cuda and x.dtype == torch.bfloat16:
      # CUDA bf16 frames: channels-last on the implicit-GEMM convolution kernels (same modules and parameters)
      return DiagonalGaussian(self.channels_last_decoder().encode(x, chunk))
    self._reset()
    cache = FeatureCache()
    t = x.shape[2]
    outs = []
    start = 0
    first = True
    while start < t:
      n = 1 if first else min(chunk, t - start)
      cache.begin_pass()
      outs.append(self.encoder(x[:, :, start:start + n], cache, first_chunk=first))
      start += n
      first = False
    h = torch.cat(outs, dim=2)
    return DiagonalGaussian(self.quant_conv(h))

  @torch.no_grad()
  def decode(self, z, chunk: int = 1):
    """z: [B,16,T',H',W'] (de-normalised latents) -> video [B,3,1+4(T'-1),8H',8W'] clamped to [-1,1]."""
    if z.is_cuda and z.dtype == torch.bfloat16 and self.cfg.z_dim % 16 == 0:
      return self.channels_last_decoder().decode(z, chunk)
    self._reset()
    cache = FeatureCache()
    x = self.post_quant_conv(z)
    outs = []
    start = 0
    first = True
    t = x.shape[2]
    while start < t:
      n = 1 if first else min(chunk, t - start)
      cache.begin_pass()
      outs.append(self.decoder(x[:, :, start:start + n], cache, first_chunk=first))
      start += n
      first = False
    return torch.cat(outs, dim=2).clamp(-1.0, 1.0)

  def channels_last_decoder(self):
    """The kernel path of `decode` (created on first use; it re-packs a weight when the parameter changes)."""
    if getattr(self, "_cl_decoder", None) is None:
      from .vae_channels_last import ChannelsLastDecoder

      object.__setattr__(self, "_cl_decoder", ChannelsLastDecoder(self))
    return self._cl_decoder

  def decode_full(self, z):
    """Whole-clip decode without chunking (the oracle the chunked path is tested against)."""
    return self.decoder(self.post_quant_conv(z), None).clamp(-1.0, 1.0)

  def encode_full(self, x):
    return DiagonalGaussian(self.quant_conv(self.encoder(x, None)))


def postprocess_video(video: torch.Tensor) -> torch.Tensor:
  """[-1,1] float [B,C,T,H,W] -> uint8 [B,T,H,W,C] (reference: wan_pipeline.py:1379-1392)."""
  v = (video.float() / 2 + 0.5).clamp(0, 1) * 255.0
  return v.round().to(torch.uint8).permute(0, 2, 3, 4, 1).contiguous()
