"""Conditional 2-D UNet for SD 1.x / 2.x / SDXL (+ the hooks ControlNet needs).

Reference: `FlaxUNet2DConditionModel` (src/maxdiffusion/models/unet_2d_condition_flax.py:115-528), its blocks
(unet_2d_blocks_flax.py), ResNet / up- / down-sample layers (resnet_flax.py:37-186) and the SD transformer
(`FlaxTransformer2DModel`, `FlaxBasicTransformerBlock`, `FlaxGEGLU`, attention_flax.py:3047-3570). Module and
parameter names follow the diffusers `UNet2DConditionModel` checkpoint so that its safetensors load directly.

GEMMs (projections, GEGLU feed-forward, attention in/out) run on the tcgen05 GEMM through `ops.functional.linear`
for bf16 CUDA tensors; attention with head_dim 64 (SDXL) or 128 uses the flash kernels, other head sizes (40..160
for SD 1.x/2.x) go through `scaled_dot_product_attention`; convolutions (forward, input and weight gradients) run on the implicit-GEMM kernels through `layers.Conv2d` and keep
the activations in channels-last memory; GroupNorm(+SiLU) is the channels-last kernel of `ops.functional.group_norm`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from .layers import Conv2d, GroupNorm, LayerNorm, Linear, sinusoidal_embedding
from .vae import ResnetBlock2D


@dataclass
class UNetConfig:
  sample_size: int = 128
  in_channels: int = 4
  out_channels: int = 4
  down_block_types: Sequence[str] = ("DownBlock2D", "CrossAttnDownBlock2D", "CrossAttnDownBlock2D")
  up_block_types: Sequence[str] = ("CrossAttnUpBlock2D", "CrossAttnUpBlock2D", "UpBlock2D")
  block_out_channels: Sequence[int] = (320, 640, 1280)
  layers_per_block: int = 2
  transformer_layers_per_block: Union[int, Sequence[int]] = (1, 2, 10)
  attention_head_dim: Union[int, Sequence[int]] = (5, 10, 20)   # number of heads per stage (diffusers naming)
  cross_attention_dim: int = 2048
  use_linear_projection: bool = True
  addition_embed_type: Optional[str] = "text_time"
  addition_time_embed_dim: Optional[int] = 256
  projection_class_embeddings_input_dim: Optional[int] = 2816
  norm_num_groups: int = 32
  flip_sin_to_cos: bool = True
  freq_shift: float = 0.0

  @classmethod
  def from_dict(cls, d):
    return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

  def to_dict(self):
    return {k: (list(v) if isinstance(v, tuple) else v) for k, v in self.__dict__.items()}


UNET_PRESETS = {
    "sdxl": dict(),
    "sd15": dict(sample_size=64, down_block_types=("CrossAttnDownBlock2D",) * 3 + ("DownBlock2D",),
                 up_block_types=("UpBlock2D",) + ("CrossAttnUpBlock2D",) * 3, block_out_channels=(320, 640, 1280, 1280),
                 transformer_layers_per_block=1, attention_head_dim=8, cross_attention_dim=768, use_linear_projection=False,
                 addition_embed_type=None, addition_time_embed_dim=None, projection_class_embeddings_input_dim=None),
    "sd21": dict(sample_size=96, down_block_types=("CrossAttnDownBlock2D",) * 3 + ("DownBlock2D",),
                 up_block_types=("UpBlock2D",) + ("CrossAttnUpBlock2D",) * 3, block_out_channels=(320, 640, 1280, 1280),
                 transformer_layers_per_block=1, attention_head_dim=(5, 10, 20, 20), cross_attention_dim=1024,
                 use_linear_projection=True, addition_embed_type=None, addition_time_embed_dim=None,
                 projection_class_embeddings_input_dim=None),
    "tiny": dict(sample_size=16, block_out_channels=(32, 64), down_block_types=("DownBlock2D", "CrossAttnDownBlock2D"),
                 up_block_types=("CrossAttnUpBlock2D", "UpBlock2D"), layers_per_block=1, transformer_layers_per_block=(1, 1),
                 attention_head_dim=(2, 2), cross_attention_dim=32, addition_time_embed_dim=8,
                 projection_class_embeddings_input_dim=16 + 6 * 8, norm_num_groups=8),
    "tiny_sd": dict(sample_size=16, block_out_channels=(32, 64), down_block_types=("DownBlock2D", "CrossAttnDownBlock2D"),
                    up_block_types=("CrossAttnUpBlock2D", "UpBlock2D"), layers_per_block=1, transformer_layers_per_block=(1, 1),
                    attention_head_dim=(2, 2), cross_attention_dim=32, addition_embed_type=None, addition_time_embed_dim=None,
                    projection_class_embeddings_input_dim=None, norm_num_groups=8, use_linear_projection=False),
}


class Attention(nn.Module):

  def __init__(self, dim: int, heads: int, cross_dim: Optional[int] = None):
    super().__init__()
    self.heads = heads
    self.to_q = Linear(dim, dim, bias=False)
    self.to_k = Linear(cross_dim or dim, dim, bias=False)
    self.to_v = Linear(cross_dim or dim, dim, bias=False)
    self.to_out = nn.ModuleList([Linear(dim, dim)])

  def forward(self, x, context=None, residual=None):
    ctx = x if context is None else context
    B, S, C = x.shape
    q = self.to_q(x).view(B, S, self.heads, -1)
    k = self.to_k(ctx).view(B, ctx.shape[1], self.heads, -1)
    v = self.to_v(ctx).view(B, ctx.shape[1], self.heads, -1)
    return self.to_out[0](OF.attention(q, k, v).reshape(B, S, C), residual=residual)


class GEGLU(nn.Module):
  """lin * gelu(gate) with one projection dim -> 2 * inner (reference: `FlaxGEGLU`, attention_flax.py:3537-3570)."""

  def __init__(self, dim, inner):
    super().__init__()
    self.proj = Linear(dim, 2 * inner)

  def forward(self, x):
    return OF.geglu(self.proj(x))


class FeedForward(nn.Module):

  def __init__(self, dim, mult=4):
    super().__init__()
    self.net = nn.ModuleList([GEGLU(dim, dim * mult), nn.Identity(), Linear(dim * mult, dim)])

  def forward(self, x, residual=None):
    return self.net[2](self.net[0](x), residual=residual)


class BasicTransformerBlock(nn.Module):

  def __init__(self, dim, heads, cross_dim):
    super().__init__()
    self.norm1, self.norm2, self.norm3 = LayerNorm(dim), LayerNorm(dim), LayerNorm(dim)
    self.attn1, self.attn2 = Attention(dim, heads), Attention(dim, heads, cross_dim)
    self.ff = FeedForward(dim)

  def forward(self, x, context):
    # the three residual adds ride in the epilogues of the output projections
    x = self.attn1(self.norm1(x), residual=x)
    x = self.attn2(self.norm2(x), context, residual=x)
    return self.ff(self.norm3(x), residual=x)


class Transformer2DModel(nn.Module):

  def __init__(self, dim, heads, depth, cross_dim, groups, linear_proj):
    super().__init__()
    self.linear_proj = linear_proj
    self.norm = GroupNorm(groups, dim, eps=1e-6)
    self.proj_in = Linear(dim, dim) if linear_proj else Conv2d(dim, dim, 1)
    self.transformer_blocks = nn.ModuleList([BasicTransformerBlock(dim, heads, cross_dim) for _ in range(depth)])
    self.proj_out = Linear(dim, dim) if linear_proj else Conv2d(dim, dim, 1)

  def forward(self, x, context):
    b, c, h, w = x.shape
    res = x
    y = self.norm(x)
    if self.linear_proj:
      y = self.proj_in(y.permute(0, 2, 3, 1).reshape(b, h * w, c))
    else:
      y = self.proj_in(y).permute(0, 2, 3, 1).reshape(b, h * w, c)
    for blk in self.transformer_blocks:
      y = blk(y, context)
    if self.linear_proj:
      y = self.proj_out(y).reshape(b, h, w, c).permute(0, 3, 1, 2)
    else:
      y = self.proj_out(y.reshape(b, h, w, c).permute(0, 3, 1, 2))
    return y + res


class Downsample2D(nn.Module):

  def __init__(self, dim):
    super().__init__()
    self.conv = Conv2d(dim, dim, 3, stride=2, padding=1)

  def forward(self, x):
    return self.conv(x)


class Upsample2D(nn.Module):

  def __init__(self, dim):
    super().__init__()
    self.conv = Conv2d(dim, dim, 3, padding=1)

  def forward(self, x):
    return self.conv(x, upsample=True)  # nearest-2x folded into the convolution


class DownBlock(nn.Module):

  def __init__(self, cin, cout, temb, n, groups, attn=None, add_down=True):
    super().__init__()
    self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, groups, temb, eps=1e-5) for i in range(n)])
    self.attentions = nn.ModuleList([Transformer2DModel(cout, *attn) for _ in range(n)]) if attn else None
    self.downsamplers = nn.ModuleList([Downsample2D(cout)]) if add_down else None

  def forward(self, x, temb, context):
    outs = []
    for i, r in enumerate(self.resnets):
      x = r(x, temb)
      if self.attentions is not None:
        x = self.attentions[i](x, context)
      outs.append(x)
    if self.downsamplers is not None:
      x = self.downsamplers[0](x)
      outs.append(x)
    return x, outs


class UpBlock(nn.Module):

  def __init__(self, cin, cout, prev, temb, n, groups, attn=None, add_up=True):
    super().__init__()
    res = []
    for i in range(n):
      skip = cin if i == n - 1 else cout
      res.append(ResnetBlock2D((prev if i == 0 else cout) + skip, cout, groups, temb, eps=1e-5))
    self.resnets = nn.ModuleList(res)
    self.attentions = nn.ModuleList([Transformer2DModel(cout, *attn) for _ in range(n)]) if attn else None
    self.upsamplers = nn.ModuleList([Upsample2D(cout)]) if add_up else None

  def forward(self, x, skips, temb, context):
    for i, r in enumerate(self.resnets):
      x = r(torch.cat([x, skips.pop()], dim=1), temb)
      if self.attentions is not None:
        x = self.attentions[i](x, context)
    if self.upsamplers is not None:
      x = self.upsamplers[0](x)
    return x


class MidBlock(nn.Module):

  def __init__(self, dim, temb, groups, attn):
    super().__init__()
    self.resnets = nn.ModuleList([ResnetBlock2D(dim, dim, groups, temb, eps=1e-5) for _ in range(2)])
    self.attentions = nn.ModuleList([Transformer2DModel(dim, *attn)])

  def forward(self, x, temb, context):
    return self.resnets[1](self.attentions[0](self.resnets[0](x, temb), context), temb)


class _TimestepEmbedding(nn.Module):

  def __init__(self, cin, dim):
    super().__init__()
    self.linear_1, self.linear_2 = Linear(cin, dim), Linear(dim, dim)

  def forward(self, x):
    return self.linear_2(F.silu(self.linear_1(x)))


class UNet2DConditionModel(nn.Module):

  def __init__(self, cfg: Optional[UNetConfig] = None):
    super().__init__()
    self.cfg = cfg = cfg or UNetConfig()
    ch = list(cfg.block_out_channels)
    n = len(ch)
    depth = [cfg.transformer_layers_per_block] * n if isinstance(cfg.transformer_layers_per_block, int) else list(cfg.transformer_layers_per_block)
    heads = [cfg.attention_head_dim] * n if isinstance(cfg.attention_head_dim, int) else list(cfg.attention_head_dim)
    temb = ch[0] * 4
    g = cfg.norm_num_groups
    self.conv_in = Conv2d(cfg.in_channels, ch[0], 3, padding=1)
    self.time_embedding = _TimestepEmbedding(ch[0], temb)
    if cfg.addition_embed_type == "text_time":
      self.add_embedding = _TimestepEmbedding(cfg.projection_class_embeddings_input_dim, temb)
    attn = lambda i: (heads[i], depth[i], cfg.cross_attention_dim, g, cfg.use_linear_projection)
    downs, cin = [], ch[0]
    for i, kind in enumerate(cfg.down_block_types):
      downs.append(DownBlock(cin, ch[i], temb, cfg.layers_per_block, g, attn(i) if "CrossAttn" in kind else None, add_down=i < n - 1))
      cin = ch[i]
    self.down_blocks = nn.ModuleList(downs)
    self.mid_block = MidBlock(ch[-1], temb, g, attn(n - 1))
    ups, rev = [], ch[::-1]
    prev = rev[0]
    for i, kind in enumerate(cfg.up_block_types):
      cout, cin_skip = rev[i], rev[min(i + 1, n - 1)]
      j = n - 1 - i
      ups.append(UpBlock(cin_skip, cout, prev, temb, cfg.layers_per_block + 1, g, attn(j) if "CrossAttn" in kind else None, add_up=i < n - 1))
      prev = cout
    self.up_blocks = nn.ModuleList(ups)
    self.conv_norm_out = GroupNorm(g, ch[0], eps=1e-5)
    self.conv_out = Conv2d(ch[0], cfg.out_channels, 3, padding=1)

  def time_embed(self, timesteps, dtype, added_cond_kwargs=None):
    cfg = self.cfg
    t = sinusoidal_embedding(timesteps.reshape(-1), cfg.block_out_channels[0], cfg.flip_sin_to_cos, cfg.freq_shift).to(dtype)
    emb = self.time_embedding(t)
    if cfg.addition_embed_type == "text_time":
      text_embeds, time_ids = added_cond_kwargs["text_embeds"], added_cond_kwargs["time_ids"]
      tid = sinusoidal_embedding(time_ids.reshape(-1), cfg.addition_time_embed_dim, cfg.flip_sin_to_cos, cfg.freq_shift)
      add = torch.cat([text_embeds.to(dtype), tid.reshape(text_embeds.shape[0], -1).to(dtype)], dim=-1)
      emb = emb + self.add_embedding(add)
    return emb

  def forward(self, sample, timesteps, encoder_hidden_states, added_cond_kwargs=None,
              down_block_additional_residuals=None, mid_block_additional_residual=None):
    dtype = self.conv_in.weight.dtype
    if timesteps.dim() == 0:
      timesteps = timesteps.expand(sample.shape[0])
    emb = self.time_embed(timesteps, dtype, added_cond_kwargs)
    ctx = encoder_hidden_states.to(dtype)
    x = self.conv_in(sample.to(dtype))
    skips = [x]
    for blk in self.down_blocks:
      x, outs = blk(x, emb, ctx)
      skips.extend(outs)
    if down_block_additional_residuals is not None:  # ControlNet
      skips = [s + r for s, r in zip(skips, down_block_additional_residuals)]
    x = self.mid_block(x, emb, ctx)
    if mid_block_additional_residual is not None:
      x = x + mid_block_additional_residual
    for blk in self.up_blocks:
      x = blk(x, skips, emb, ctx)
    return self.conv_out(self.conv_norm_out(x, act=True))
