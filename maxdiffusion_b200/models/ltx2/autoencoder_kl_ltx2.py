"""LTX-2 video VAE: 32x spatial / 8x temporal compression to 128 latent channels, with spatial and temporal tiling.

Reference: src/maxdiffusion/models/ltx2/autoencoder_kl_ltx2.py — `PerChannelRMSNorm` (:51), `LTX2VideoCausalConv3d`
(first-frame replication in time, causal or symmetric; :72-160), `LTX2VideoResnetBlock3d` (optional timestep
scale/shift table, :162-312), the space-time-to-channel down-sampler with a group-mean residual (:315-385) and the
channel-to-space-time up-sampler with a tiled residual (:388-455), down / mid / up blocks (:458-827), encoder (4x4
pixel patchify, :830-984), decoder (:987-1170), tiling with linear cross-fades (`blend_v/h/t`, `tiled_encode/decode`,
temporal tiling; :1292-1710). Tensors are channels-first [B, C, T, H, W]; parameter names follow the diffusers
`AutoencoderKLLTX2Video` checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..embeddings import TimestepEmbedding, Timesteps


def per_channel_rms_norm(x, eps: float = 1e-8):
  return x * torch.rsqrt(x.float().pow(2).mean(dim=1, keepdim=True) + eps).to(x.dtype)


class LTX2VideoCausalConv3d(nn.Module):

  def __init__(self, cin, cout, kernel_size=3, stride=1, spatial_padding_mode: str = "zeros"):
    super().__init__()
    k = (kernel_size,) * 3 if isinstance(kernel_size, int) else tuple(kernel_size)
    s = (stride,) * 3 if isinstance(stride, int) else tuple(stride)
    self.k = k
    self.mode = {"zeros": "constant", "constant": "constant", "reflect": "reflect", "replicate": "replicate"}[spatial_padding_mode]
    self.conv = nn.Conv3d(cin, cout, k, stride=s)

  def forward(self, x, causal: bool = True):
    kt = self.k[0]
    if causal and kt > 1:
      x = torch.cat([x[:, :, :1].expand(-1, -1, kt - 1, -1, -1), x], dim=2)
    elif kt > 1:
      p = (kt - 1) // 2
      x = torch.cat([x[:, :, :1].expand(-1, -1, p, -1, -1), x, x[:, :, -1:].expand(-1, -1, p, -1, -1)], dim=2)
    ph, pw = self.k[1] // 2, self.k[2] // 2
    if ph or pw:
      if self.mode == "constant":
        x = F.pad(x, (pw, pw, ph, ph))
      else:  # reflect / replicate pad the two spatial dims of every frame
        B, C, T, H, W = x.shape
        x = F.pad(x.reshape(B, C * T, H, W), (pw, pw, ph, ph), mode=self.mode).reshape(B, C, T, H + 2 * ph, W + 2 * pw)
    return self.conv(x)


class LTX2VideoResnetBlock3d(nn.Module):

  def __init__(self, cin, cout=None, inject_noise=False, timestep_conditioning=False, pad="zeros"):
    super().__init__()
    cout = cout or cin
    self.conv1 = LTX2VideoCausalConv3d(cin, cout, 3, spatial_padding_mode=pad)
    self.conv2 = LTX2VideoCausalConv3d(cout, cout, 3, spatial_padding_mode=pad)
    self.norm3 = nn.LayerNorm(cin, elementwise_affine=True) if cin != cout else None
    self.conv_shortcut = nn.Conv3d(cin, cout, 1) if cin != cout else None
    self.per_channel_scale1 = nn.Parameter(torch.zeros(cout, 1, 1)) if inject_noise else None
    self.per_channel_scale2 = nn.Parameter(torch.zeros(cout, 1, 1)) if inject_noise else None
    self.scale_shift_table = nn.Parameter(torch.randn(4, cin) / cin ** 0.5) if timestep_conditioning else None

  def _noise(self, h, scale, generator):
    if scale is None or generator is None:
      return h
    n = torch.randn(h.shape[-2:], generator=generator, device=h.device, dtype=h.dtype)
    return h + (n[None] * scale.to(h.dtype))[None, :, None]

  def forward(self, x, temb=None, causal=True, generator=None):
    h = per_channel_rms_norm(x)
    if self.scale_shift_table is not None:
      t = temb.reshape(x.shape[0], 4, -1) + self.scale_shift_table[None].to(temb.dtype)
      sh1, sc1, sh2, sc2 = (t[:, i, :, None, None, None] for i in range(4))
      h = h * (1 + sc1) + sh1
    h = self._noise(self.conv1(F.silu(h), causal), self.per_channel_scale1, generator)
    h = per_channel_rms_norm(h)
    if self.scale_shift_table is not None:
      h = h * (1 + sc2) + sh2
    h = self._noise(self.conv2(F.silu(h), causal), self.per_channel_scale2, generator)
    if self.norm3 is not None:
      x = self.norm3(x.movedim(1, -1)).movedim(-1, 1)
    if self.conv_shortcut is not None:
      x = self.conv_shortcut(x)
    return h + x


def _space_to_channel(x, s):
  """[B,C,T,H,W] -> [B, C*s0*s1*s2, T/s0, H/s1, W/s2]; channel index = c*(s0 s1 s2) + i0*(s1 s2) + i1*s2 + i2."""
  B, C, T, H, W = x.shape
  s0, s1, s2 = s
  x = x.reshape(B, C, T // s0, s0, H // s1, s1, W // s2, s2).permute(0, 1, 3, 5, 7, 2, 4, 6)
  return x.reshape(B, C * s0 * s1 * s2, T // s0, H // s1, W // s2)


def _channel_to_space(x, s):
  B, Ct, T, H, W = x.shape
  s0, s1, s2 = s
  C = Ct // (s0 * s1 * s2)
  x = x.reshape(B, C, s0, s1, s2, T, H, W).permute(0, 1, 5, 2, 6, 3, 7, 4)
  return x.reshape(B, C, T * s0, H * s1, W * s2)


class LTXVideoDownsampler3d(nn.Module):

  def __init__(self, cin, cout, stride, pad="zeros"):
    super().__init__()
    self.stride = tuple(stride)
    n = stride[0] * stride[1] * stride[2]
    self.group_size = cin * n // cout
    self.conv = LTX2VideoCausalConv3d(cin, cout // n, 3, spatial_padding_mode=pad)

  def forward(self, x, causal=True):
    if self.stride[0] > 1:
      x = torch.cat([x[:, :, :self.stride[0] - 1], x], dim=2)
    res = _space_to_channel(x, self.stride)
    B, C = res.shape[:2]
    res = res.reshape(B, C // self.group_size, self.group_size, *res.shape[2:]).mean(dim=2)
    return _space_to_channel(self.conv(x, causal), self.stride) + res


class LTXVideoUpsampler3d(nn.Module):

  def __init__(self, cin, stride, residual=False, upscale_factor=1, pad="zeros"):
    super().__init__()
    self.stride, self.residual, self.upscale_factor = tuple(stride), residual, upscale_factor
    n = stride[0] * stride[1] * stride[2]
    self.conv = LTX2VideoCausalConv3d(cin, cin * n // upscale_factor, 3, spatial_padding_mode=pad)

  def forward(self, x, causal=True):
    s0 = self.stride[0]
    n = self.stride[0] * self.stride[1] * self.stride[2]
    res = None
    if self.residual:
      res = _channel_to_space(x, self.stride)
      rep = n // self.upscale_factor
      if rep > 1:
        res = res.repeat(1, rep, 1, 1, 1)
      if s0 > 1:
        res = res[:, :, s0 - 1:]
    h = _channel_to_space(self.conv(x, causal), self.stride)
    if s0 > 1:
      h = h[:, :, s0 - 1:]
    return h + res if res is not None else h


_STRIDES = {"spatial": (1, 2, 2), "temporal": (2, 1, 1), "spatiotemporal": (2, 2, 2)}


class _TimeEmbedder(nn.Module):

  def __init__(self, dim):
    super().__init__()
    self.time_proj = Timesteps(256, flip_sin_to_cos=True, freq_shift=0.0)
    self.timestep_embedder = TimestepEmbedding(256, dim)

  def forward(self, t, dtype):
    return self.timestep_embedder(self.time_proj(t.flatten()).to(dtype))


class LTX2VideoDownBlock3D(nn.Module):

  def __init__(self, cin, cout, num_layers, scale: bool, downsample_type: str, pad):
    super().__init__()
    self.resnets = nn.ModuleList([LTX2VideoResnetBlock3d(cin, cin, pad=pad) for _ in range(num_layers)])
    self.downsamplers = None
    if scale:
      if downsample_type == "conv":
        self.downsamplers = nn.ModuleList([LTX2VideoCausalConv3d(cin, cin, 3, stride=(2, 2, 2), spatial_padding_mode=pad)])
      else:
        self.downsamplers = nn.ModuleList([LTXVideoDownsampler3d(cin, cout, _STRIDES[downsample_type], pad)])

  def forward(self, x, causal=True):
    for r in self.resnets:
      x = r(x, causal=causal)
    if self.downsamplers is not None:
      x = self.downsamplers[0](x, causal)
    return x


class LTX2VideoMidBlock3d(nn.Module):

  def __init__(self, cin, num_layers, inject_noise=False, timestep_conditioning=False, pad="zeros"):
    super().__init__()
    self.time_embedder = _TimeEmbedder(cin * 4) if timestep_conditioning else None
    self.resnets = nn.ModuleList([LTX2VideoResnetBlock3d(cin, cin, inject_noise, timestep_conditioning, pad) for _ in range(num_layers)])

  def forward(self, x, temb=None, causal=True, generator=None):
    if self.time_embedder is not None:
      temb = self.time_embedder(temb, x.dtype)
    for r in self.resnets:
      x = r(x, temb, causal, generator)
    return x


class LTX2VideoUpBlock3d(nn.Module):

  def __init__(self, cin, cout, num_layers, scale, inject_noise, timestep_conditioning, upsample_residual, upscale_factor,
               upsample_type, pad):
    super().__init__()
    self.time_embedder = _TimeEmbedder(cin * 4) if timestep_conditioning else None
    self.conv_in = LTX2VideoResnetBlock3d(cin, cout, inject_noise, timestep_conditioning, pad) if cin != cout else None
    self.upsamplers = nn.ModuleList([LTXVideoUpsampler3d(cout * upscale_factor, _STRIDES[upsample_type], upsample_residual,
                                                         upscale_factor, pad)]) if scale else None
    self.resnets = nn.ModuleList([LTX2VideoResnetBlock3d(cout, cout, inject_noise, timestep_conditioning, pad) for _ in range(num_layers)])

  def forward(self, x, temb=None, causal=True, generator=None):
    t = self.time_embedder(temb, x.dtype) if self.time_embedder is not None else None
    if self.conv_in is not None:
      x = self.conv_in(x, t, causal, generator)
    if self.upsamplers is not None:
      x = self.upsamplers[0](x, causal)
    for r in self.resnets:
      x = r(x, t, causal, generator)
    return x


@dataclass
class LTX2VAEConfig:
  in_channels: int = 3
  out_channels: int = 3
  latent_channels: int = 128
  block_out_channels: Sequence[int] = (256, 512, 1024, 2048)
  decoder_block_out_channels: Sequence[int] = (256, 512, 1024)
  layers_per_block: Sequence[int] = (4, 6, 6, 2, 2)
  decoder_layers_per_block: Sequence[int] = (5, 5, 5, 5)
  spatio_temporal_scaling: Sequence[bool] = (True, True, True, True)
  decoder_spatio_temporal_scaling: Sequence[bool] = (True, True, True)
  downsample_type: Sequence[str] = ("spatial", "temporal", "spatiotemporal", "spatiotemporal")
  upsample_type: Sequence[str] = ("spatiotemporal", "spatiotemporal", "spatiotemporal")
  decoder_inject_noise: Sequence[bool] = (False, False, False, False)
  upsample_residual: Sequence[bool] = (True, True, True)
  upsample_factor: Sequence[int] = (2, 2, 2)
  timestep_conditioning: bool = False
  patch_size: int = 4
  patch_size_t: int = 1
  encoder_causal: bool = True
  decoder_causal: bool = False
  encoder_spatial_padding_mode: str = "zeros"
  decoder_spatial_padding_mode: str = "reflect"
  scaling_factor: float = 1.0
  spatial_compression_ratio: int = 32
  temporal_compression_ratio: int = 8

  @classmethod
  def from_dict(cls, d):
    return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})


class LTX2VideoEncoder3d(nn.Module):

  def __init__(self, c: LTX2VAEConfig):
    super().__init__()
    self.p, self.pt, self.causal = c.patch_size, c.patch_size_t, c.encoder_causal
    pad = c.encoder_spatial_padding_mode
    ch = list(c.block_out_channels)
    self.conv_in = LTX2VideoCausalConv3d(c.in_channels * c.patch_size ** 2, c.latent_channels, 3, spatial_padding_mode=pad)
    self.down_blocks = nn.ModuleList([
        LTX2VideoDownBlock3D(c.latent_channels if i == 0 else ch[i - 1], ch[i], c.layers_per_block[i],
                             c.spatio_temporal_scaling[i], c.downsample_type[i], pad) for i in range(len(ch))])
    self.mid_block = LTX2VideoMidBlock3d(ch[-1], c.layers_per_block[-1], pad=pad)
    self.conv_out = LTX2VideoCausalConv3d(ch[-1], c.latent_channels + 1, 3, spatial_padding_mode=pad)

  def forward(self, x, causal: Optional[bool] = None):
    causal = self.causal if causal is None else causal
    B, C, T, H, W = x.shape
    p, pt = self.p, self.pt
    # channel index = c*(pt p p) + it*(p p) + iw*p + ih  (the reference transposes (7, 2, 6, 4))
    h = x.reshape(B, C, T // pt, pt, H // p, p, W // p, p).permute(0, 1, 3, 7, 5, 2, 4, 6).reshape(B, C * pt * p * p, T // pt, H // p, W // p)
    h = self.conv_in(h, causal)
    for blk in self.down_blocks:
      h = blk(h, causal)
    h = self.mid_block(h, causal=causal)
    h = self.conv_out(F.silu(per_channel_rms_norm(h)), causal)
    last = h[:, -1:]
    return torch.cat([h, last.expand(-1, h.shape[1] - 2, -1, -1, -1)], dim=1)  # mean | replicated log-variance


class LTX2VideoDecoder3d(nn.Module):

  def __init__(self, c: LTX2VAEConfig):
    super().__init__()
    self.p, self.pt, self.causal = c.patch_size, c.patch_size_t, c.decoder_causal
    pad = c.decoder_spatial_padding_mode
    ch = list(reversed(c.decoder_block_out_channels))
    scale = list(reversed(c.decoder_spatio_temporal_scaling))
    layers = list(reversed(c.decoder_layers_per_block))
    noise = list(reversed(c.decoder_inject_noise))
    ures, ufac, utype = list(reversed(c.upsample_residual)), list(reversed(c.upsample_factor)), list(reversed(c.upsample_type))
    out = ch[0]
    self.conv_in = LTX2VideoCausalConv3d(c.latent_channels, out, 3, spatial_padding_mode=pad)
    self.mid_block = LTX2VideoMidBlock3d(out, layers[0], noise[0], c.timestep_conditioning, pad)
    ups = []
    for i in range(len(ch)):
      cin, out = out // ufac[i], ch[i] // ufac[i]
      ups.append(LTX2VideoUpBlock3d(cin, out, layers[i + 1], scale[i], noise[i + 1], c.timestep_conditioning, ures[i], ufac[i], utype[i], pad))
    self.up_blocks = nn.ModuleList(ups)
    self.conv_out = LTX2VideoCausalConv3d(out, c.out_channels * c.patch_size ** 2, 3, spatial_padding_mode=pad)
    self.timestep_scale_multiplier = nn.Parameter(torch.tensor(1000.0)) if c.timestep_conditioning else None
    self.time_embedder = _TimeEmbedder(out * 2) if c.timestep_conditioning else None
    self.scale_shift_table = nn.Parameter(torch.randn(2, out) / out ** 0.5) if c.timestep_conditioning else None

  def forward(self, z, temb=None, causal: Optional[bool] = None, generator=None):
    causal = self.causal if causal is None else causal
    if self.timestep_scale_multiplier is not None and temb is not None:
      temb = temb * self.timestep_scale_multiplier
    h = self.mid_block(self.conv_in(z, causal), temb, causal, generator)
    for blk in self.up_blocks:
      h = blk(h, temb, causal, generator)
    h = per_channel_rms_norm(h)
    if self.time_embedder is not None and temb is not None:
      t = self.time_embedder(temb, h.dtype).reshape(h.shape[0], 2, -1) + self.scale_shift_table[None].to(h.dtype)
      h = h * (1 + t[:, 1, :, None, None, None]) + t[:, 0, :, None, None, None]
    h = self.conv_out(F.silu(h), causal)
    B, C, T, H, W = h.shape
    p, pt = self.p, self.pt
    co = C // (pt * p * p)
    # inverse of the encoder's patch order: (c, it, iw, ih)
    return h.reshape(B, co, pt, p, p, T, H, W).permute(0, 1, 5, 2, 6, 4, 7, 3).reshape(B, co, T * pt, H * p, W * p)


class LTX2VideoAutoencoderKL(nn.Module):

  def __init__(self, cfg: Optional[LTX2VAEConfig] = None):
    super().__init__()
    self.cfg = c = cfg or LTX2VAEConfig()
    self.encoder, self.decoder = LTX2VideoEncoder3d(c), LTX2VideoDecoder3d(c)
    self.register_buffer("latents_mean", torch.zeros(c.latent_channels))
    self.register_buffer("latents_std", torch.ones(c.latent_channels))
    self.use_tiling = self.use_framewise_decoding = False
    self.tile_sample_min_height = self.tile_sample_min_width = 512
    self.tile_sample_min_num_frames = 16
    self.tile_sample_stride_height = self.tile_sample_stride_width = 448
    self.tile_sample_stride_num_frames = 8

  def enable_tiling(self, **kw):
    self.use_tiling = True
    for k, v in kw.items():
      if v is not None and hasattr(self, k):
        setattr(self, k, v)

  # ---- latent statistics -------------------------------------------------------------------
  def normalize_latents(self, z):
    m, s = self.latents_mean.view(1, -1, 1, 1, 1).to(z), self.latents_std.view(1, -1, 1, 1, 1).to(z)
    return (z - m) * self.cfg.scaling_factor / s

  def denormalize_latents(self, z):
    m, s = self.latents_mean.view(1, -1, 1, 1, 1).to(z), self.latents_std.view(1, -1, 1, 1, 1).to(z)
    return z * s / self.cfg.scaling_factor + m

  # ---- blending ----------------------------------------------------------------------------
  @staticmethod
  def _blend(a, b, extent, dim):
    extent = min(a.shape[dim], b.shape[dim], extent)
    if extent <= 0:
      return b
    shape = [1] * b.dim()
    shape[dim] = extent
    w = (torch.arange(extent, device=b.device, dtype=torch.float32) / extent).reshape(shape).to(b.dtype)
    head = a.narrow(dim, a.shape[dim] - extent, extent) * (1 - w) + b.narrow(dim, 0, extent) * w
    return torch.cat([head, b.narrow(dim, extent, b.shape[dim] - extent)], dim=dim)

  def blend_v(self, a, b, extent):
    return self._blend(a, b, extent, 3)

  def blend_h(self, a, b, extent):
    return self._blend(a, b, extent, 4)

  def blend_t(self, a, b, extent):
    return self._blend(a, b, extent, 2)

  def _tiled(self, x, fn, min_h, min_w, stride_h, stride_w, out_stride_h, out_stride_w, blend_h, blend_w):
    rows = []
    for i in range(0, x.shape[3], stride_h):
      rows.append([fn(x[:, :, :, i:i + min_h, j:j + min_w]) for j in range(0, x.shape[4], stride_w)])
    out_rows = []
    for i, row in enumerate(rows):
      out = []
      for j, tile in enumerate(row):
        if i > 0:
          tile = self.blend_v(rows[i - 1][j], tile, blend_h)
        if j > 0:
          tile = self.blend_h(row[j - 1], tile, blend_w)
        row[j] = tile
        out.append(tile[:, :, :, :out_stride_h, :out_stride_w])
      out_rows.append(torch.cat(out, dim=4))
    return torch.cat(out_rows, dim=3)

  def tiled_encode(self, x, causal=None):
    r = self.cfg.spatial_compression_ratio
    return self._tiled(x, lambda t: self.encoder(t, causal), self.tile_sample_min_height, self.tile_sample_min_width,
                       self.tile_sample_stride_height, self.tile_sample_stride_width, self.tile_sample_stride_height // r,
                       self.tile_sample_stride_width // r, (self.tile_sample_min_height - self.tile_sample_stride_height) // r,
                       (self.tile_sample_min_width - self.tile_sample_stride_width) // r)

  def tiled_decode(self, z, temb=None, causal=None):
    r = self.cfg.spatial_compression_ratio
    return self._tiled(z, lambda t: self.decoder(t, temb, causal), self.tile_sample_min_height // r, self.tile_sample_min_width // r,
                       self.tile_sample_stride_height // r, self.tile_sample_stride_width // r, self.tile_sample_stride_height,
                       self.tile_sample_stride_width, self.tile_sample_min_height - self.tile_sample_stride_height,
                       self.tile_sample_min_width - self.tile_sample_stride_width)

  def _temporal_tiled_decode(self, z, temb=None, causal=None):
    tr = self.cfg.temporal_compression_ratio
    lat_min, lat_stride = self.tile_sample_min_num_frames // tr, self.tile_sample_stride_num_frames // tr
    blend = self.tile_sample_min_num_frames - self.tile_sample_stride_num_frames
    tiles = []
    for i in range(0, z.shape[2], lat_stride):
      tile = z[:, :, i:i + lat_min + 1]
      big = self.use_tiling and (tile.shape[3] * self.cfg.spatial_compression_ratio > self.tile_sample_min_height or
                                 tile.shape[4] * self.cfg.spatial_compression_ratio > self.tile_sample_min_width)
      dec = self.tiled_decode(tile, temb, causal) if big else self.decoder(tile, temb, causal)
      tiles.append(dec[:, :, :-1] if i > 0 else dec)
    out = []
    for i, tile in enumerate(tiles):
      if i > 0:
        tile = self.blend_t(tiles[i - 1], tile, blend)
        tiles[i] = tile
        out.append(tile[:, :, :self.tile_sample_stride_num_frames])
      else:
        out.append(tile[:, :, :self.tile_sample_stride_num_frames + 1])
    return torch.cat(out, dim=2)

  # ---- public ------------------------------------------------------------------------------
  @torch.no_grad()
  def encode(self, x, causal=None):
    """x [B,3,T,H,W] in [-1,1], T = 1 + 8k, H and W multiples of 32. Returns (mean, logvar) [B,128,T',H/32,W/32]."""
    big = self.use_tiling and (x.shape[3] > self.tile_sample_min_height or x.shape[4] > self.tile_sample_min_width)
    moments = self.tiled_encode(x, causal) if big else self.encoder(x, causal)
    return moments.chunk(2, dim=1)

  @torch.no_grad()
  def decode(self, z, temb=None, causal=None):
    r, tr = self.cfg.spatial_compression_ratio, self.cfg.temporal_compression_ratio
    if self.use_framewise_decoding and z.shape[2] > self.tile_sample_min_num_frames // tr:
      return self._temporal_tiled_decode(z, temb, causal)
    if self.use_tiling and (z.shape[3] > self.tile_sample_min_height // r or z.shape[4] > self.tile_sample_min_width // r):
      return self.tiled_decode(z, temb, causal)
    return self.decoder(z, temb, causal)
