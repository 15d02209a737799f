"""ControlNet for SD / SDXL: a copy of the UNet encoder whose per-resolution outputs, passed through zero-initialised
1x1 convolutions, are added to the UNet's skip connections and mid block.

Reference: `FlaxControlNetModel` (src/maxdiffusion/models/controlnet_flax.py:447 lines) and its conditioning embedding.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .unet_2d_condition import DownBlock, MidBlock, UNetConfig, _TimestepEmbedding
from .layers import Conv2d, sinusoidal_embedding


class ControlNetConditioningEmbedding(nn.Module):
  """Image-space condition (e.g. canny edges) -> feature map at latent resolution (three stride-2 stages)."""

  def __init__(self, out_channels: int, in_channels: int = 3, block_out_channels=(16, 32, 96, 256)):
    super().__init__()
    self.conv_in = Conv2d(in_channels, block_out_channels[0], 3, padding=1)
    blocks = []
    for a, b in zip(block_out_channels[:-1], block_out_channels[1:]):
      blocks += [Conv2d(a, a, 3, padding=1), Conv2d(a, b, 3, padding=1, stride=2)]
    self.blocks = nn.ModuleList(blocks)
    self.conv_out = Conv2d(block_out_channels[-1], out_channels, 3, padding=1)
    nn.init.zeros_(self.conv_out.weight)
    nn.init.zeros_(self.conv_out.bias)

  def forward(self, x):
    x = F.silu(self.conv_in(x))
    for b in self.blocks:
      x = F.silu(b(x))
    return self.conv_out(x)


class ControlNetModel(nn.Module):

  def __init__(self, cfg: Optional[UNetConfig] = None, conditioning_channels: int = 3):
    super().__init__()
    self.cfg = cfg = cfg or UNetConfig()
    ch = list(cfg.block_out_channels)
    n = len(ch)
    depth = [cfg.transformer_layers_per_block] * n if isinstance(cfg.transformer_layers_per_block, int) else list(cfg.transformer_layers_per_block)
    heads = [cfg.attention_head_dim] * n if isinstance(cfg.attention_head_dim, int) else list(cfg.attention_head_dim)
    temb, g = ch[0] * 4, cfg.norm_num_groups
    self.conv_in = Conv2d(cfg.in_channels, ch[0], 3, padding=1)
    self.time_embedding = _TimestepEmbedding(ch[0], temb)
    if cfg.addition_embed_type == "text_time":
      self.add_embedding = _TimestepEmbedding(cfg.projection_class_embeddings_input_dim, temb)
    self.controlnet_cond_embedding = ControlNetConditioningEmbedding(ch[0], conditioning_channels)
    attn = lambda i: (heads[i], depth[i], cfg.cross_attention_dim, g, cfg.use_linear_projection)
    downs, zero, cin = [], [Conv2d(ch[0], ch[0], 1)], ch[0]
    for i, kind in enumerate(cfg.down_block_types):
      downs.append(DownBlock(cin, ch[i], temb, cfg.layers_per_block, g, attn(i) if "CrossAttn" in kind else None, add_down=i < n - 1))
      zero += [Conv2d(ch[i], ch[i], 1) for _ in range(cfg.layers_per_block + (1 if i < n - 1 else 0))]
      cin = ch[i]
    self.down_blocks, self.controlnet_down_blocks = nn.ModuleList(downs), nn.ModuleList(zero)
    self.mid_block = MidBlock(ch[-1], temb, g, attn(n - 1))
    self.controlnet_mid_block = Conv2d(ch[-1], ch[-1], 1)
    for z in list(self.controlnet_down_blocks) + [self.controlnet_mid_block]:
      nn.init.zeros_(z.weight)
      nn.init.zeros_(z.bias)

  def forward(self, sample, timesteps, encoder_hidden_states, controlnet_cond, conditioning_scale: float = 1.0,
              added_cond_kwargs=None):
    cfg = self.cfg
    dtype = self.conv_in.weight.dtype
    if timesteps.dim() == 0:
      timesteps = timesteps.expand(sample.shape[0])
    emb = self.time_embedding(sinusoidal_embedding(timesteps.reshape(-1), cfg.block_out_channels[0], cfg.flip_sin_to_cos, cfg.freq_shift).to(dtype))
    if cfg.addition_embed_type == "text_time":
      te, ti = added_cond_kwargs["text_embeds"], added_cond_kwargs["time_ids"]
      tid = sinusoidal_embedding(ti.reshape(-1), cfg.addition_time_embed_dim, cfg.flip_sin_to_cos, cfg.freq_shift)
      emb = emb + self.add_embedding(torch.cat([te.to(dtype), tid.reshape(te.shape[0], -1).to(dtype)], dim=-1))
    ctx = encoder_hidden_states.to(dtype)
    x = self.conv_in(sample.to(dtype)) + self.controlnet_cond_embedding(controlnet_cond.to(dtype))
    skips = [x]
    for blk in self.down_blocks:
      x, outs = blk(x, emb, ctx)
      skips.extend(outs)
    x = self.mid_block(x, emb, ctx)
    down = [z(s) * conditioning_scale for z, s in zip(self.controlnet_down_blocks, skips)]
    return down, self.controlnet_mid_block(x) * conditioning_scale
