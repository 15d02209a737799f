"""Embedding layers shared by the model families (reference: src/maxdiffusion/models/embeddings_flax.py).

  get_sinusoidal_embeddings / Timesteps        :28-62, :96
  TimestepEmbedding (Linear -> SiLU -> Linear) :65-93
  get_1d_rotary_pos_embed (real cos/sin or complex) :222-250
  WanImageEmbedding                            :253      (defined with the Wan transformer, re-exported here)
  PixArtAlphaTextProjection                    :332
  FluxPosEmbed                                 :437
  CombinedTimestepTextProjEmbeddings / CombinedTimestepGuidanceTextProjEmbeddings :514-652
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import Linear, sinusoidal_embedding

get_sinusoidal_embeddings = sinusoidal_embedding


class Timesteps(nn.Module):

  def __init__(self, dim: int = 32, flip_sin_to_cos: bool = False, freq_shift: float = 1.0, scale: float = 1.0):
    super().__init__()
    self.dim, self.flip, self.shift, self.scale = dim, flip_sin_to_cos, freq_shift, scale

  def forward(self, timesteps):
    return sinusoidal_embedding(timesteps, self.dim, self.flip, self.shift, scale=self.scale)


class TimestepEmbedding(nn.Module):

  def __init__(self, in_channels: int, time_embed_dim: int, out_dim: Optional[int] = None, act: str = "silu"):
    super().__init__()
    self.linear_1 = Linear(in_channels, time_embed_dim)
    self.linear_2 = Linear(time_embed_dim, out_dim or time_embed_dim)
    self.act = {"silu": F.silu, "gelu": F.gelu, "gelu_tanh": lambda x: F.gelu(x, approximate="tanh")}[act]

  def forward(self, x):
    return self.linear_2(self.act(self.linear_1(x)))


def get_1d_rotary_pos_embed(dim: int, pos, theta: float = 10000.0, use_real: bool = True, linear_factor: float = 1.0,
                            ntk_factor: float = 1.0, freqs_dtype=torch.float32):
  """Rotary tables for positions `pos` (int -> arange). Real: (cos, sin) [S, dim/2]; complex: exp(i * angle)."""
  if isinstance(pos, int):
    pos = torch.arange(pos)
  pos = torch.as_tensor(pos)
  inv = 1.0 / ((theta * ntk_factor) ** (torch.arange(0, dim, 2, dtype=freqs_dtype, device=pos.device)[: dim // 2] / dim)) / linear_factor
  ang = torch.outer(pos.to(freqs_dtype), inv)
  if use_real:
    return ang.cos().float(), ang.sin().float()
  return torch.polar(torch.ones_like(ang, dtype=torch.float32), ang.float())


class FluxPosEmbed(nn.Module):
  """Per-axis rotary tables concatenated along the feature axis: ids [S, n_axes] -> (cos, sin) [S, sum(axes)/2]."""

  def __init__(self, theta: float, axes_dim: Sequence[int]):
    super().__init__()
    self.theta, self.axes_dim = theta, tuple(axes_dim)

  def forward(self, ids: torch.Tensor):
    from .flux.transformer_flux import flux_rope_tables

    return flux_rope_tables(ids, self.axes_dim, self.theta)


class PixArtAlphaTextProjection(nn.Module):
  """Linear -> act -> Linear on caption / pooled-text features."""

  def __init__(self, in_features: int, hidden_size: int, out_features: Optional[int] = None, act_fn: str = "gelu_tanh"):
    super().__init__()
    self.linear_1 = Linear(in_features, hidden_size)
    self.linear_2 = Linear(hidden_size, out_features or hidden_size)
    self.act = {"gelu_tanh": lambda x: F.gelu(x, approximate="tanh"), "silu": F.silu, "gelu": F.gelu}[act_fn]

  def forward(self, caption):
    return self.linear_2(self.act(self.linear_1(caption)))


class CombinedTimestepTextProjEmbeddings(nn.Module):

  def __init__(self, embedding_dim: int, pooled_projection_dim: int):
    super().__init__()
    self.time_proj = Timesteps(256, flip_sin_to_cos=True, freq_shift=0.0)
    self.timestep_embedder = TimestepEmbedding(256, embedding_dim)
    self.text_embedder = PixArtAlphaTextProjection(pooled_projection_dim, embedding_dim, act_fn="silu")

  def forward(self, timestep, pooled_projection):
    t = self.timestep_embedder(self.time_proj(timestep).to(pooled_projection.dtype))
    return t + self.text_embedder(pooled_projection)


class CombinedTimestepGuidanceTextProjEmbeddings(nn.Module):

  def __init__(self, embedding_dim: int, pooled_projection_dim: int):
    super().__init__()
    self.time_proj = Timesteps(256, flip_sin_to_cos=True, freq_shift=0.0)
    self.timestep_embedder = TimestepEmbedding(256, embedding_dim)
    self.guidance_embedder = TimestepEmbedding(256, embedding_dim)
    self.text_embedder = PixArtAlphaTextProjection(pooled_projection_dim, embedding_dim, act_fn="silu")

  def forward(self, timestep, guidance, pooled_projection):
    dt = pooled_projection.dtype
    t = self.timestep_embedder(self.time_proj(timestep).to(dt)) + self.guidance_embedder(self.time_proj(guidance).to(dt))
    return t + self.text_embedder(pooled_projection)


def __getattr__(name):
  if name in ("WanImageEmbedding", "NNXWanImageEmbedding"):
    from .wan.transformer_wan import WanImageEmbedding

    return WanImageEmbedding
  raise AttributeError(name)
