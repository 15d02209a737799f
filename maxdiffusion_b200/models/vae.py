"""AutoencoderKL for SD 1.x / 2.x / SDXL (4 latent channels) and Flux (16 channels, shift + scale).

Reference: `FlaxAutoencoderKL` and `FlaxDiagonalGaussianDistribution` (src/maxdiffusion/models/vae_flax.py:723-1020).
Module and parameter names follow the diffusers `AutoencoderKL` checkpoint. Convolutions run on the implicit-GEMM
kernels through `layers.Conv2d` (CUDA bf16; PyTorch elsewhere); the single-head mid-block attention uses
`ops.functional.attention`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from .layers import Conv2d, GroupNorm


@dataclass
class VAEConfig:
  in_channels: int = 3
  out_channels: int = 3
  block_out_channels: Sequence[int] = (128, 256, 512, 512)
  layers_per_block: int = 2
  latent_channels: int = 4
  norm_num_groups: int = 32
  scaling_factor: float = 0.18215
  shift_factor: float = 0.0
  use_quant_conv: bool = True
  use_post_quant_conv: bool = True

  @classmethod
  def from_dict(cls, d):
    return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})


VAE_PRESETS = {
    "sd": dict(),
    "sdxl": dict(scaling_factor=0.13025),
    "flux": dict(latent_channels=16, scaling_factor=0.3611, shift_factor=0.1159, use_quant_conv=False,
                 use_post_quant_conv=False),
    "tiny": dict(block_out_channels=(32, 32), layers_per_block=1, norm_num_groups=8),
}


class ResnetBlock2D(nn.Module):

  def __init__(self, cin, cout, groups=32, temb_channels: Optional[int] = None, eps=1e-6):
    super().__init__()
    self.norm1 = GroupNorm(groups, cin, eps=eps)
    self.conv1 = Conv2d(cin, cout, 3, padding=1)
    self.time_emb_proj = nn.Linear(temb_channels, cout) if temb_channels else None
    self.norm2 = GroupNorm(groups, cout, eps=eps)
    self.conv2 = Conv2d(cout, cout, 3, padding=1)
    self.conv_shortcut = Conv2d(cin, cout, 1) if cin != cout else None

  def forward(self, x, temb=None):
    h = self.conv1(self.norm1(x, act=True))
    if self.time_emb_proj is not None and temb is not None:
      h = h + self.time_emb_proj(F.silu(temb))[:, :, None, None]
    h = self.conv2(self.norm2(h, act=True))
    return (self.conv_shortcut(x) if self.conv_shortcut is not None else x) + h


class SpatialSelfAttention(nn.Module):

  def __init__(self, dim, groups=32, eps=1e-6):
    super().__init__()
    self.group_norm = GroupNorm(groups, dim, eps=eps)
    self.to_q, self.to_k, self.to_v = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
    self.to_out = nn.ModuleList([nn.Linear(dim, dim)])

  def forward(self, x):
    b, c, h, w = x.shape
    y = self.group_norm(x).reshape(b, c, h * w).transpose(1, 2)
    q, k, v = self.to_q(y), self.to_k(y), self.to_v(y)
    o = OF.attention(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2)).squeeze(2)
    o = self.to_out[0](o).transpose(1, 2).reshape(b, c, h, w)
    return x + o


class _Sampler(nn.Module):

  def __init__(self, dim, down: bool):
    super().__init__()
    self.down = down
    self.conv = Conv2d(dim, dim, 3, stride=2 if down else 1, padding="far" if down else 1)

  def forward(self, x):
    return self.conv(x) if self.down else self.conv(x, upsample=True)


class _Block(nn.Module):

  def __init__(self, cin, cout, n, groups, down=None):
    super().__init__()
    self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, groups) for i in range(n)])
    if down is True:
      self.downsamplers = nn.ModuleList([_Sampler(cout, True)])
    elif down is False:
      self.upsamplers = nn.ModuleList([_Sampler(cout, False)])

  def forward(self, x):
    for r in self.resnets:
      x = r(x)
    for name in ("downsamplers", "upsamplers"):
      if hasattr(self, name):
        x = getattr(self, name)[0](x)
    return x


class _Mid(nn.Module):

  def __init__(self, dim, groups):
    super().__init__()
    self.resnets = nn.ModuleList([ResnetBlock2D(dim, dim, groups), ResnetBlock2D(dim, dim, groups)])
    self.attentions = nn.ModuleList([SpatialSelfAttention(dim, groups)])

  def forward(self, x):
    return self.resnets[1](self.attentions[0](self.resnets[0](x)))


class Encoder(nn.Module):

  def __init__(self, cfg: VAEConfig):
    super().__init__()
    ch = list(cfg.block_out_channels)
    self.conv_in = Conv2d(cfg.in_channels, ch[0], 3, padding=1)
    self.down_blocks = nn.ModuleList([
        _Block(ch[max(i - 1, 0)], ch[i], cfg.layers_per_block, cfg.norm_num_groups, down=True if i < len(ch) - 1 else None)
        for i in range(len(ch))])
    self.mid_block = _Mid(ch[-1], cfg.norm_num_groups)
    self.conv_norm_out = GroupNorm(cfg.norm_num_groups, ch[-1], eps=1e-6)
    self.conv_out = Conv2d(ch[-1], 2 * cfg.latent_channels, 3, padding=1)

  def forward(self, x):
    x = self.conv_in(x)
    for b in self.down_blocks:
      x = b(x)
    return self.conv_out(self.conv_norm_out(self.mid_block(x), act=True))


class Decoder(nn.Module):

  def __init__(self, cfg: VAEConfig):
    super().__init__()
    ch = list(cfg.block_out_channels)[::-1]
    self.conv_in = Conv2d(cfg.latent_channels, ch[0], 3, padding=1)
    self.mid_block = _Mid(ch[0], cfg.norm_num_groups)
    self.up_blocks = nn.ModuleList([
        _Block(ch[max(i - 1, 0)], ch[i], cfg.layers_per_block + 1, cfg.norm_num_groups, down=False if i < len(ch) - 1 else None)
        for i in range(len(ch))])
    self.conv_norm_out = GroupNorm(cfg.norm_num_groups, ch[-1], eps=1e-6)
    self.conv_out = Conv2d(ch[-1], cfg.out_channels, 3, padding=1)

  def forward(self, z):
    x = self.mid_block(self.conv_in(z))
    for b in self.up_blocks:
      x = b(x)
    return self.conv_out(self.conv_norm_out(x, act=True))


class DiagonalGaussianDistribution:

  def __init__(self, moments):
    self.mean, logvar = moments.chunk(2, dim=1)
    self.logvar = logvar.clamp(-30.0, 20.0)
    self.std = torch.exp(0.5 * self.logvar)

  def sample(self, generator=None):
    return self.mean + self.std * torch.randn(self.mean.shape, generator=generator, device=self.mean.device, dtype=self.mean.dtype)

  def mode(self):
    return self.mean

  def kl(self):
    return 0.5 * torch.sum(self.mean.pow(2) + self.logvar.exp() - 1.0 - self.logvar, dim=[1, 2, 3])


class AutoencoderKL(nn.Module):

  def __init__(self, cfg: Optional[VAEConfig] = None):
    super().__init__()
    self.cfg = cfg or VAEConfig()
    self.encoder, self.decoder = Encoder(self.cfg), Decoder(self.cfg)
    lc = self.cfg.latent_channels
    self.quant_conv = Conv2d(2 * lc, 2 * lc, 1) if self.cfg.use_quant_conv else None
    self.post_quant_conv = Conv2d(lc, lc, 1) if self.cfg.use_post_quant_conv else None

  def encode(self, x) -> DiagonalGaussianDistribution:
    h = self.encoder(x)
    return DiagonalGaussianDistribution(self.quant_conv(h) if self.quant_conv is not None else h)

  def decode(self, z):
    return self.decoder(self.post_quant_conv(z) if self.post_quant_conv is not None else z)

  def scale_latents(self, z):
    return (z - self.cfg.shift_factor) * self.cfg.scaling_factor

  def unscale_latents(self, z):
    return z / self.cfg.scaling_factor + self.cfg.shift_factor
