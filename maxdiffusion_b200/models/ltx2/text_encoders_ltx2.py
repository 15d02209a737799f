"""LTX-2 text conditioning: Gemma-3 hidden states (all layers) -> feature extractor -> video / audio connectors.

Reference: src/maxdiffusion/models/ltx2/text_encoders/
  * `feature_extractor_ltx2.py:26-182`: stack the hidden states of every Gemma layer [B,T,D,L]; per sample and layer
    subtract the masked mean and divide by the masked range (x8), zero the (left) padding, flatten to D*L and project;
  * `embeddings_connector_ltx2.py:29-267`: a small 1-D transformer (LTX2Attention self-attention with 1-D RoPE over
    position / base_seq_len, GELU-tanh FFN, RMSNorm without affine) whose padded positions are replaced by learnable
    register tokens, tiled over the sequence, after the valid tokens were moved to the front;
  * `text_encoders_ltx2.py:32`: one feature extractor (or per-modality projections) feeding a video and an audio
    connector;
  * `torchax_text_encoder.py:52-82`: the Gemma-3 model itself is the Hugging Face PyTorch module; here it runs natively
    on the GPU through `transformers` (no interop layer needed).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..layers import Linear, RMSNorm
from .attention_ltx2 import LTX2Attention
from .transformer_ltx2 import FeedForward


def norm_and_concat_padded_batch(encoded_text: torch.Tensor, attention_mask: torch.Tensor) -> torch.Tensor:
  """[B,T,D,L] hidden states (left-padded) -> [B,T,D*L], normalised per sample and layer over the valid tokens."""
  b, t, d, l = encoded_text.shape
  x = encoded_text.float()
  lengths = attention_mask.sum(dim=-1)
  mask = (torch.arange(t, device=x.device)[None, :] >= (t - lengths[:, None]))[:, :, None, None]
  eps = 1e-6
  mean = torch.where(mask, x, 0.0).sum(dim=(1, 2), keepdim=True) / ((lengths * d).reshape(b, 1, 1, 1) + eps)
  x_min = torch.where(mask, x, float("inf")).amin(dim=(1, 2), keepdim=True)
  x_max = torch.where(mask, x, float("-inf")).amax(dim=(1, 2), keepdim=True)
  normed = (8.0 * (x - mean) / (x_max - x_min + eps)).reshape(b, t, d * l)
  return torch.where(mask[:, :, 0], normed, 0.0).to(encoded_text.dtype)


class LTX2GemmaFeatureExtractor(nn.Module):

  def __init__(self, input_dim: int, output_dim: int, per_modality_projections: bool = False, use_bias: bool = False,
               video_output_dim: Optional[int] = None, audio_output_dim: Optional[int] = None):
    super().__init__()
    self.per_modality = per_modality_projections
    if per_modality_projections:
      self.video_linear = Linear(input_dim, video_output_dim or output_dim, bias=use_bias)
      self.audio_linear = Linear(input_dim, audio_output_dim or output_dim, bias=use_bias)
    else:
      self.linear = Linear(input_dim, output_dim, bias=use_bias)

  def forward(self, hidden_states, attention_mask):
    x = torch.stack(list(hidden_states), dim=-1) if isinstance(hidden_states, (tuple, list)) else hidden_states
    x = norm_and_concat_padded_batch(x, attention_mask)
    w = self.video_linear.weight if self.per_modality else self.linear.weight
    x = x.to(w.dtype)
    return (self.video_linear(x), self.audio_linear(x)) if self.per_modality else self.linear(x)


class _Block1D(nn.Module):

  def __init__(self, dim, heads, dim_head, rope_type, gated_attn):
    super().__init__()
    self.attn1 = LTX2Attention(dim, heads, dim_head, rope_type=rope_type, gated_attn=gated_attn)
    self.ff = FeedForward(dim, "gelu_tanh")
    self.norm1 = RMSNorm(dim, 1e-6, elementwise_affine=False)
    self.norm2 = RMSNorm(dim, 1e-6, elementwise_affine=False)

  def forward(self, x, mask, rope):
    x = x + self.attn1(self.norm1(x), attention_mask=mask, rotary_emb=rope)
    return x + self.ff(self.norm2(x))


class Embeddings1DConnector(nn.Module):

  def __init__(self, input_dim: int, heads: int = 30, head_dim: int = 128, layers: int = 2, theta: float = 10000.0,
               num_learnable_registers: int = 128, rope_type: str = "interleaved", base_seq_len: int = 4096,
               gated_attn: bool = False):
    super().__init__()
    self.dim, self.heads, self.theta, self.rope_type, self.base_seq_len = input_dim, heads, theta, rope_type, base_seq_len
    self.num_registers = num_learnable_registers
    self.transformer_1d_blocks = nn.ModuleList([_Block1D(input_dim, heads, head_dim, rope_type, gated_attn) for _ in range(layers)])
    if num_learnable_registers > 0:
      self.learnable_registers = nn.Parameter(torch.rand(num_learnable_registers, input_dim) * 2.0 - 1.0)
    self.final_norm = RMSNorm(input_dim, 1e-6, elementwise_affine=False)

  def replace_padded_with_registers(self, x, attention_mask):
    """Valid tokens move to the front (order kept); the rest of the sequence holds the tiled register tokens."""
    b, t, d = x.shape
    if t % self.num_registers != 0:
      raise ValueError(f"Sequence length {t} must be divisible by {self.num_registers}")
    regs = self.learnable_registers.to(x.dtype).repeat(t // self.num_registers, 1)
    m = (attention_mask.reshape(b, t) > 0.5).long()
    n_valid = m.sum(dim=1, keepdim=True)
    target = torch.where(m == 1, m.cumsum(1) - 1, (1 - m).cumsum(1) - 1 + n_valid)
    shifted = torch.zeros_like(x).scatter(1, target[..., None].expand(-1, -1, d), x)
    shifted_mask = torch.zeros_like(m).scatter(1, target, m)
    out = torch.where(shifted_mask[..., None] == 1, shifted, regs[None])
    return out, torch.ones((b, t), dtype=torch.bool, device=x.device)

  def rope_1d(self, batch: int, seq_len: int, device):
    grid = (torch.arange(seq_len, dtype=torch.float64, device=device) / self.base_seq_len)[None].repeat(batch, 1)
    steps = self.dim // 2
    base = torch.pow(torch.tensor(self.theta, dtype=torch.float64), torch.linspace(0.0, 1.0, steps, dtype=torch.float64)).to(device) * math.pi / 2.0
    freqs = ((grid.unsqueeze(-1) * 2.0 - 1.0) * base).float()
    cos, sin = freqs.cos(), freqs.sin()
    if self.rope_type == "interleaved":
      cos, sin = cos.repeat_interleave(2, dim=-1), sin.repeat_interleave(2, dim=-1)
      pad = self.dim - cos.shape[-1]
      if pad > 0:
        cos = torch.cat([torch.ones_like(cos[..., :pad]), cos], dim=-1)
        sin = torch.cat([torch.zeros_like(sin[..., :pad]), sin], dim=-1)
      return cos, sin
    pad = self.dim // 2 - cos.shape[-1]
    if pad > 0:
      cos = torch.cat([torch.ones_like(cos[..., :pad]), cos], dim=-1)
      sin = torch.cat([torch.zeros_like(sin[..., :pad]), sin], dim=-1)
    b, t = cos.shape[:2]
    return cos.reshape(b, t, self.heads, -1).permute(0, 2, 1, 3), sin.reshape(b, t, self.heads, -1).permute(0, 2, 1, 3)

  def forward(self, x, attention_mask: Optional[torch.Tensor] = None):
    if self.num_registers > 0 and attention_mask is not None:
      x, attention_mask = self.replace_padded_with_registers(x, attention_mask)
    rope = self.rope_1d(x.shape[0], x.shape[1], x.device)
    mask = None if (attention_mask is None or bool(attention_mask.all())) else attention_mask.bool()
    for blk in self.transformer_1d_blocks:
      x = blk(x, mask, rope)
    return self.final_norm(x), attention_mask


class LTX2AudioVideoGemmaTextEncoder(nn.Module):
  """Gemma hidden states -> (video text embeddings, audio text embeddings, mask)."""

  def __init__(self, caption_channels: int = 3840, text_proj_in_factor: int = 49, gemma_dim: Optional[int] = None,
               video_connector_attention_head_dim: int = 128, video_connector_num_attention_heads: int = 30,
               video_connector_num_layers: int = 2, video_connector_num_learnable_registers: int = 128,
               audio_connector_attention_head_dim: int = 128, audio_connector_num_attention_heads: int = 30,
               audio_connector_num_layers: int = 2, audio_connector_num_learnable_registers: int = 128,
               connector_rope_base_seq_len: int = 4096, rope_theta: float = 10000.0, rope_type: str = "split",
               per_modality_projections: bool = False, proj_bias: bool = False, video_gated_attn: bool = False,
               audio_gated_attn: bool = False, video_hidden_dim: Optional[int] = None, audio_hidden_dim: Optional[int] = None):
    super().__init__()
    input_dim = (gemma_dim or caption_channels) * text_proj_in_factor
    v_dim, a_dim = video_hidden_dim or caption_channels, audio_hidden_dim or caption_channels
    self.feature_extractor = LTX2GemmaFeatureExtractor(input_dim, caption_channels, per_modality_projections, proj_bias, v_dim, a_dim)
    self.per_modality = per_modality_projections
    ck = dict(theta=rope_theta, rope_type=rope_type, base_seq_len=connector_rope_base_seq_len)
    self.video_embeddings_connector = Embeddings1DConnector(
        v_dim, video_connector_num_attention_heads, video_connector_attention_head_dim, video_connector_num_layers,
        num_learnable_registers=video_connector_num_learnable_registers, gated_attn=video_gated_attn, **ck)
    self.audio_embeddings_connector = Embeddings1DConnector(
        a_dim, audio_connector_num_attention_heads, audio_connector_attention_head_dim, audio_connector_num_layers,
        num_learnable_registers=audio_connector_num_learnable_registers, gated_attn=audio_gated_attn, **ck)

  def forward(self, hidden_states, attention_mask):
    feats = self.feature_extractor(hidden_states, attention_mask)
    v_in, a_in = feats if self.per_modality else (feats, feats)
    # the extractor works on left-padded text; the connectors move the valid tokens to the front
    video, mask = self.video_embeddings_connector(v_in, attention_mask)
    audio, _ = self.audio_embeddings_connector(a_in, attention_mask)
    return video, audio, mask


class GemmaTextEncoder:
  """Hugging Face Gemma-3 text model returning the hidden states of every layer (embeddings included)."""

  def __init__(self, path: str, device="cuda", dtype=torch.bfloat16):
    from transformers import AutoModel, AutoTokenizer

    self.tokenizer = AutoTokenizer.from_pretrained(path)
    self.tokenizer.padding_side = "left"
    self.model = AutoModel.from_pretrained(path, torch_dtype=dtype).to(device).eval()
    self.device = device

  @torch.no_grad()
  def __call__(self, prompts: Sequence[str], max_sequence_length: int = 1024) -> Tuple[torch.Tensor, torch.Tensor]:
    enc = self.tokenizer(list(prompts), padding="max_length", max_length=max_sequence_length, truncation=True, return_tensors="pt")
    ids, mask = enc["input_ids"].to(self.device), enc["attention_mask"].to(self.device)
    out = self.model(input_ids=ids, attention_mask=mask, output_hidden_states=True)
    return torch.stack(list(out.hidden_states), dim=-1), mask
