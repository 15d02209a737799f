"""LTX-2 audio VAE over mel-spectrograms: [B, 2, time, mel] <-> latents [B, 8, time/4, mel/4].

Reference: src/maxdiffusion/models/ltx2/autoencoder_kl_ltx2_audio.py — causal 2-D convolution that pads only the past
along the causal axis (:58-113), pixel norm (:116-126), spatial attention block (:129-180), ResNet block (:183-302),
stride-2 down-sampler with causal padding (:305-348), nearest-2x up-sampler that drops the first row of the causal
axis (:351-402), patchifier `[B, T, F, C] <-> [B, T, C*F]` (:405-445), encoder / decoder (:448-734) and the wrapper
whose decode crops / pads to `time * 4 - 3` frames and `mel_bins` (:737-859). Tensors here are channels-first
[B, C, time, mel]: "height" causality = time.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as OF
from ..layers import GroupNorm


def _pads(axis: Optional[str], k: int, dilation: int = 1):
  """(top, bottom, left, right) zero padding of a k x k convolution for a causality axis."""
  p = (k - 1) * dilation
  if axis in (None, "none"):
    return p // 2, p - p // 2, p // 2, p - p // 2
  if axis in ("width", "width-compatibility"):
    return p // 2, p - p // 2, p, 0
  if axis == "height":
    return p, 0, p // 2, p - p // 2
  raise ValueError(f"Invalid causality_axis: {axis}")


class AudioCausalConv(nn.Module):

  def __init__(self, cin, cout, kernel_size=3, stride=1, dilation=1, causality_axis: Optional[str] = "height"):
    super().__init__()
    self.pad = _pads(causality_axis, kernel_size, dilation)
    self.conv = nn.Conv2d(cin, cout, kernel_size, stride=stride, dilation=dilation)

  def forward(self, x):
    t, b, l, r = self.pad
    return self.conv(F.pad(x, (l, r, t, b)))


class PixelNorm(nn.Module):

  def __init__(self, eps: float = 1e-8):
    super().__init__()
    self.eps = eps

  def forward(self, x, act: bool = False):
    y = x / torch.sqrt(x.float().pow(2).mean(dim=1, keepdim=True) + self.eps).to(x.dtype)
    return F.silu(y) if act else y


def _norm(kind: str, ch: int):
  if kind == "group":
    return GroupNorm(32, ch, eps=1e-6)
  if kind == "pixel":
    return PixelNorm()
  raise ValueError(f"Invalid normalization type: {kind}")


class AudioAttnBlock(nn.Module):

  def __init__(self, ch: int, norm_type: str):
    super().__init__()
    self.norm = _norm(norm_type, ch)
    self.q, self.k, self.v, self.proj_out = (nn.Conv2d(ch, ch, 1) for _ in range(4))

  def forward(self, x):
    B, C, H, W = x.shape
    h = self.norm(x)
    q, k, v = (f(h).reshape(B, C, H * W).transpose(1, 2).unsqueeze(2) for f in (self.q, self.k, self.v))
    o = OF.attention(q, k, v).squeeze(2).transpose(1, 2).reshape(B, C, H, W)
    return x + self.proj_out(o)


class AudioResnetBlock(nn.Module):

  def __init__(self, cin, cout=None, conv_shortcut=False, temb_channels=0, norm_type="pixel", causality_axis="height"):
    super().__init__()
    cout = cout or cin
    self.norm1, self.norm2 = _norm(norm_type, cin), _norm(norm_type, cout)
    self.conv1 = AudioCausalConv(cin, cout, 3, causality_axis=causality_axis)
    self.conv2 = AudioCausalConv(cout, cout, 3, causality_axis=causality_axis)
    self.temb_proj = nn.Linear(temb_channels, cout) if temb_channels > 0 else None
    self.conv_shortcut = AudioCausalConv(cin, cout, 3 if conv_shortcut else 1, causality_axis=causality_axis) if cin != cout else None

  def forward(self, x, temb=None):
    h = self.conv1(self.norm1(x, act=True))
    if temb is not None and self.temb_proj is not None:
      h = h + self.temb_proj(F.silu(temb))[:, :, None, None]
    h = self.conv2(self.norm2(h, act=True))
    return (self.conv_shortcut(x) if self.conv_shortcut is not None else x) + h


class AudioDownsample(nn.Module):

  def __init__(self, ch, with_conv=True, causality_axis="height"):
    super().__init__()
    self.axis = causality_axis
    self.conv = nn.Conv2d(ch, ch, 3, stride=2) if with_conv else None

  def forward(self, x):
    if self.conv is None:
      return F.avg_pool2d(x, 2, 2)
    pad = {"none": (0, 1, 0, 1), None: (0, 1, 0, 1), "width": (0, 1, 2, 0), "height": (2, 0, 0, 1),
           "width-compatibility": (0, 1, 1, 0)}[self.axis]  # (top, bottom, left, right)
    return self.conv(F.pad(x, (pad[2], pad[3], pad[0], pad[1])))


class AudioUpsample(nn.Module):

  def __init__(self, ch, with_conv=True, causality_axis="height"):
    super().__init__()
    self.axis = causality_axis
    self.conv = AudioCausalConv(ch, ch, 3, causality_axis=causality_axis) if with_conv else None

  def forward(self, x):
    x = F.interpolate(x, scale_factor=2.0, mode="nearest")
    if self.conv is not None:
      x = self.conv(x)
      if self.axis == "height":
        x = x[:, :, 1:]
      elif self.axis == "width":
        x = x[:, :, :, 1:]
    return x


@dataclass
class LTX2AudioVAEConfig:
  base_channels: int = 128
  output_channels: int = 2
  ch_mult: Sequence[int] = (1, 2, 4)
  num_res_blocks: int = 2
  attn_resolutions: Optional[Sequence[int]] = None
  in_channels: int = 2
  resolution: int = 256
  latent_channels: int = 8
  norm_type: str = "pixel"
  causality_axis: Optional[str] = "height"
  mid_block_add_attention: bool = False
  sample_rate: int = 16000
  mel_hop_length: int = 160
  is_causal: bool = True
  mel_bins: Optional[int] = 64
  double_z: bool = True

  @classmethod
  def from_dict(cls, d):
    return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})


class _Stage(nn.Module):

  def __init__(self, blocks, attns, resample, kind):
    super().__init__()
    self.block = nn.ModuleList(blocks)
    self.attn = nn.ModuleList(attns)
    setattr(self, kind, resample)
    self.kind = kind

  def forward(self, h):
    for i, b in enumerate(self.block):
      h = b(h)
      if len(self.attn) > i and not isinstance(self.attn[i], nn.Identity):
        h = self.attn[i](h)
    r = getattr(self, self.kind)
    return r(h) if r is not None else h


def _stages(c: LTX2AudioVAEConfig, decoder: bool):
  attn_res = set(c.attn_resolutions or ())
  n = len(c.ch_mult)
  stages = []
  if not decoder:
    res, cin = c.resolution, c.base_channels
    for level in range(n):
      cout = c.base_channels * c.ch_mult[level]
      blocks, attns = [], []
      for _ in range(c.num_res_blocks):
        blocks.append(AudioResnetBlock(cin, cout, norm_type=c.norm_type, causality_axis=c.causality_axis))
        cin = cout
        attns.append(AudioAttnBlock(cin, c.norm_type) if res in attn_res else nn.Identity())
      down = AudioDownsample(cin, True, c.causality_axis) if level != n - 1 else None
      res = res // 2 if down is not None else res
      stages.append(_Stage(blocks, attns, down, "downsample"))
    return stages, cin
  res, cin = c.resolution // 2 ** (n - 1), c.base_channels * c.ch_mult[-1]
  for level in reversed(range(n)):
    cout = c.base_channels * c.ch_mult[level]
    blocks, attns = [], []
    for _ in range(c.num_res_blocks + 1):
      blocks.append(AudioResnetBlock(cin, cout, norm_type=c.norm_type, causality_axis=c.causality_axis))
      cin = cout
      attns.append(AudioAttnBlock(cin, c.norm_type) if res in attn_res else nn.Identity())
    up = AudioUpsample(cin, True, c.causality_axis) if level != 0 else None
    res = res * 2 if up is not None else res
    stages.append(_Stage(blocks, attns, up, "upsample"))
  return stages, cin


class LTX2AudioEncoder(nn.Module):

  def __init__(self, c: LTX2AudioVAEConfig):
    super().__init__()
    self.conv_in = AudioCausalConv(c.in_channels, c.base_channels, 3, causality_axis=c.causality_axis)
    stages, ch = _stages(c, False)
    self.down = nn.ModuleList(stages)
    self.mid_block1 = AudioResnetBlock(ch, ch, norm_type=c.norm_type, causality_axis=c.causality_axis)
    self.mid_attn = AudioAttnBlock(ch, c.norm_type) if c.mid_block_add_attention else None
    self.mid_block2 = AudioResnetBlock(ch, ch, norm_type=c.norm_type, causality_axis=c.causality_axis)
    self.norm_out = _norm(c.norm_type, ch)
    self.conv_out = AudioCausalConv(ch, (2 if c.double_z else 1) * c.latent_channels, 3, causality_axis=c.causality_axis)

  def forward(self, x):
    h = self.conv_in(x)
    for st in self.down:
      h = st(h)
    h = self.mid_block1(h)
    if self.mid_attn is not None:
      h = self.mid_attn(h)
    return self.conv_out(self.norm_out(self.mid_block2(h), act=True))


class LTX2AudioDecoder(nn.Module):

  def __init__(self, c: LTX2AudioVAEConfig):
    super().__init__()
    self.out_ch = c.output_channels
    ch = c.base_channels * c.ch_mult[-1]
    self.conv_in = AudioCausalConv(c.latent_channels, ch, 3, causality_axis=c.causality_axis)
    self.mid_block1 = AudioResnetBlock(ch, ch, norm_type=c.norm_type, causality_axis=c.causality_axis)
    self.mid_attn = AudioAttnBlock(ch, c.norm_type) if c.mid_block_add_attention else None
    self.mid_block2 = AudioResnetBlock(ch, ch, norm_type=c.norm_type, causality_axis=c.causality_axis)
    stages, ch = _stages(c, True)
    self.up = nn.ModuleList(stages)
    self.norm_out = _norm(c.norm_type, ch)
    self.conv_out = AudioCausalConv(ch, c.output_channels, 3, causality_axis=c.causality_axis)

  def forward(self, z, target_frames=None, target_mel_bins=None):
    h = self.mid_block1(self.conv_in(z))
    if self.mid_attn is not None:
      h = self.mid_attn(h)
    h = self.mid_block2(h)
    for st in self.up:
      h = st(h)
    h = self.conv_out(self.norm_out(h, act=True))
    if target_frames is not None and target_mel_bins is not None:
      h = h[:, :self.out_ch, :min(h.shape[2], target_frames), :min(h.shape[3], target_mel_bins)]
      h = F.pad(h, (0, max(target_mel_bins - h.shape[3], 0), 0, max(target_frames - h.shape[2], 0)))
    return h


class AutoencoderKLLTX2Audio(nn.Module):

  def __init__(self, cfg: Optional[LTX2AudioVAEConfig] = None):
    super().__init__()
    self.cfg = c = cfg or LTX2AudioVAEConfig()
    self.encoder, self.decoder = LTX2AudioEncoder(c), LTX2AudioDecoder(c)
    self.latent_downsample_factor = 2 ** (len(c.ch_mult) - 1)
    # statistics of the packed tokens [B, T, latent_channels * mel/4] (128 values for the released model, which is
    # also its base_channels: the reference sizes them by base_channels)
    n = c.latent_channels * (c.mel_bins // self.latent_downsample_factor) if c.mel_bins else c.base_channels
    self.register_buffer("latents_mean", torch.zeros(n))
    self.register_buffer("latents_std", torch.ones(n))

  # patched latents are [B, time, C * F] with channel-major features (reference patchifier :421-445)
  @staticmethod
  def patchify(latents):
    B, C, T, Fq = latents.shape
    return latents.permute(0, 2, 1, 3).reshape(B, T, C * Fq)

  @staticmethod
  def unpatchify(tokens, channels: int, freq: int):
    B, T, _ = tokens.shape
    return tokens.reshape(B, T, channels, freq).permute(0, 2, 1, 3)

  def normalize_latents(self, tokens):
    return (tokens - self.latents_mean.to(tokens)) / self.latents_std.to(tokens)

  def denormalize_latents(self, tokens):
    return tokens * self.latents_std.to(tokens) + self.latents_mean.to(tokens)

  @torch.no_grad()
  def encode(self, x):
    """x: mel-spectrogram [B, 2, time, mel] -> (mean, logvar) [B, 8, time', mel/4]."""
    h = self.encoder(x)
    return h.chunk(2, dim=1) if self.cfg.double_z else (h, torch.zeros_like(h))

  @torch.no_grad()
  def decode(self, z):
    frames = z.shape[2] * self.latent_downsample_factor
    if self.cfg.causality_axis not in (None, "none"):
      frames = max(frames - (self.latent_downsample_factor - 1), 1)
    return self.decoder(z, frames, self.cfg.mel_bins)
