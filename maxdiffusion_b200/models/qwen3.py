"""Qwen3 decoder used as a text encoder (Z-Image, Flux.2-Klein).

Architecture (reference: src/maxdiffusion/models/qwen3_flax.py:29-455): token embedding, N pre-norm decoder
layers with grouped-query attention (per-head RMSNorm on q and k, rotate-half RoPE with theta 1e6, causal +
padding mask) and a SwiGLU MLP, final RMSNorm. `forward` returns the last hidden state and the list
[embeddings, layer_1, ..., layer_N] like the reference (`all_hidden_states[-2]` conditions Z-Image).

Parameter names follow the Hugging Face checkpoint (`model.layers.N.self_attn.q_proj.weight`, ...), so the
safetensors shards load with `load_state_dict` (reference loader: src/maxdiffusion/models/qwen3_utils.py).
Projections run on the tcgen05 GEMM; the 512-token causal attention goes through
`scaled_dot_product_attention` (masked, short sequence: not a hot path).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import Linear, RMSNorm


@dataclass
class Qwen3Config:
  vocab_size: int = 151936
  hidden_size: int = 2560
  intermediate_size: int = 9728
  num_hidden_layers: int = 36
  num_attention_heads: int = 32
  num_key_value_heads: int = 8
  head_dim: int = 128
  rms_norm_eps: float = 1e-6
  rope_theta: float = 1000000.0
  max_position_embeddings: int = 40960

  @classmethod
  def from_dict(cls, d: dict) -> "Qwen3Config":
    names = {f.name for f in fields(cls)}
    return cls(**{k: v for k, v in d.items() if k in names})


QWEN3_PRESETS = {
    "qwen3-4b": Qwen3Config(),
    "qwen3-8b": Qwen3Config(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36),
    "tiny": Qwen3Config(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=64),
}


def qwen3_rope(head_dim: int, length: int, theta: float, device=None):
  """cos, sin [length, head_dim] for rotate-half RoPE (reference: qwen3_flax.py:130-144)."""
  inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
  ang = torch.outer(torch.arange(length, dtype=torch.float32, device=device), inv)
  emb = torch.cat([ang, ang], dim=-1)
  return emb.cos(), emb.sin()


def _rotate_half(x):
  h = x.shape[-1] // 2
  return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


class Qwen3Attention(nn.Module):

  def __init__(self, cfg: Qwen3Config):
    super().__init__()
    self.cfg = cfg
    H, KV, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    self.q_proj = Linear(cfg.hidden_size, H * D, bias=False)
    self.k_proj = Linear(cfg.hidden_size, KV * D, bias=False)
    self.v_proj = Linear(cfg.hidden_size, KV * D, bias=False)
    self.o_proj = Linear(H * D, cfg.hidden_size, bias=False)
    self.q_norm = RMSNorm(D, cfg.rms_norm_eps)
    self.k_norm = RMSNorm(D, cfg.rms_norm_eps)

  def forward(self, x, cos, sin, mask):
    B, S, _ = x.shape
    H, KV, D = self.cfg.num_attention_heads, self.cfg.num_key_value_heads, self.cfg.head_dim
    q = self.q_norm(self.q_proj(x).view(B, S, H, D))
    k = self.k_norm(self.k_proj(x).view(B, S, KV, D))
    v = self.v_proj(x).view(B, S, KV, D)
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    q = (q.float() * c + _rotate_half(q.float()) * s).to(x.dtype)
    k = (k.float() * c + _rotate_half(k.float()) * s).to(x.dtype)
    if KV != H:
      k = k.repeat_interleave(H // KV, dim=2)
      v = v.repeat_interleave(H // KV, dim=2)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask)
    return self.o_proj(o.transpose(1, 2).reshape(B, S, H * D))


class Qwen3MLP(nn.Module):

  def __init__(self, cfg: Qwen3Config):
    super().__init__()
    self.gate_proj = Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
    self.up_proj = Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
    self.down_proj = Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)

  def forward(self, x):
    return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class Qwen3DecoderLayer(nn.Module):

  def __init__(self, cfg: Qwen3Config):
    super().__init__()
    self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
    self.self_attn = Qwen3Attention(cfg)
    self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
    self.mlp = Qwen3MLP(cfg)

  def forward(self, x, cos, sin, mask):
    x = x + self.self_attn(self.input_layernorm(x), cos, sin, mask)
    return x + self.mlp(self.post_attention_layernorm(x))


class _Qwen3Body(nn.Module):

  def __init__(self, cfg: Qwen3Config):
    super().__init__()
    self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
    self.layers = nn.ModuleList([Qwen3DecoderLayer(cfg) for _ in range(cfg.num_hidden_layers)])
    self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)


class Qwen3Model(nn.Module):
  """`forward(input_ids, attention_mask)` -> (last_hidden_state, all_hidden_states)."""

  def __init__(self, cfg: Qwen3Config):
    super().__init__()
    self.cfg = cfg
    self.model = _Qwen3Body(cfg)

  @torch.no_grad()
  def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None):
    B, S = input_ids.shape
    x = self.model.embed_tokens(input_ids)
    cos, sin = qwen3_rope(self.cfg.head_dim, S, self.cfg.rope_theta, device=x.device)
    mask = torch.ones((S, S), dtype=torch.bool, device=x.device).tril()[None, None]
    if attention_mask is not None:
      mask = mask & attention_mask.bool()[:, None, None, :]
      # fully padded query rows still need one visible key to keep the softmax finite
      mask = mask | torch.eye(S, dtype=torch.bool, device=x.device)[None, None]
    hidden = [x]
    for layer in self.model.layers:
      x = layer(x, cos, sin, mask)
      hidden.append(x)
    return self.model.norm(x), hidden

  @classmethod
  def from_pretrained(cls, path: str, dtype=torch.bfloat16, device="cpu") -> "Qwen3Model":
    """Loads `config.json` + `*.safetensors` of a Hugging Face Qwen3 folder (lm_head is ignored)."""
    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json")) as f:
      cfg = Qwen3Config.from_dict(json.load(f))
    model = cls(cfg).to(dtype)
    state = {}
    for name in sorted(os.listdir(path)):
      if name.endswith(".safetensors"):
        state.update(load_file(os.path.join(path, name)))
    state = {k: v for k, v in state.items() if k.startswith("model.")}
    model.load_state_dict(state, strict=True)
    return model.to(device)
