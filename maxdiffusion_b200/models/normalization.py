"""Adaptive normalisation layers (reference: src/maxdiffusion/models/normalization_flax.py:60-260). All of them are
one launch of the fused `layer_norm_mod` kernel (fp32 statistics, `(1 + scale) * x_hat + shift`, one rounding) after
a tiny fp32 GEMM on the conditioning vector.

  AdaLayerNormContinuous  : emb -> (scale, shift); LN without affine                     (:27-57)
  AdaLayerNormZero        : emb -> 6 vectors; returns (x_mod, gate_msa, shift_mlp, scale_mlp, gate_mlp)  (:60-110)
  AdaLayerNormZeroSingle  : emb -> 3 vectors; returns (x_mod, gate)                       (:113-157)
  FP32LayerNorm           : LayerNorm with fp32 statistics                                (:160-180)
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from .layers import FP32LayerNorm, Linear, RMSNorm  # noqa: F401  (re-exported)


def _mod(linear: Linear, emb: torch.Tensor, n: int):
  out = F.linear(F.silu(emb).float(), linear.weight.float(), None if linear.bias is None else linear.bias.float())
  return out.chunk(n, dim=-1)


class AdaLayerNormContinuous(nn.Module):

  def __init__(self, embedding_dim: int, conditioning_dim: int = 0, eps: float = 1e-6, bias: bool = True,
               scale_shift_order: str = "scale_shift"):
    super().__init__()
    self.linear = Linear(conditioning_dim or embedding_dim, 2 * embedding_dim, bias=bias)
    self.eps, self.order = eps, scale_shift_order

  def forward(self, x, emb):
    a, b = _mod(self.linear, emb, 2)
    scale, shift = (a, b) if self.order == "scale_shift" else (b, a)
    return OF.layer_norm_mod(x, scale=scale, shift=shift, eps=self.eps)


class AdaLayerNormZero(nn.Module):

  def __init__(self, embedding_dim: int, eps: float = 1e-6, bias: bool = True):
    super().__init__()
    self.linear = Linear(embedding_dim, 6 * embedding_dim, bias=bias)
    self.eps = eps

  def forward(self, x, emb):
    shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = _mod(self.linear, emb, 6)
    return OF.layer_norm_mod(x, scale=scale_msa, shift=shift_msa, eps=self.eps), gate_msa, shift_mlp, scale_mlp, gate_mlp


class AdaLayerNormZeroSingle(nn.Module):

  def __init__(self, embedding_dim: int, eps: float = 1e-6, bias: bool = True):
    super().__init__()
    self.linear = Linear(embedding_dim, 3 * embedding_dim, bias=bias)
    self.eps = eps

  def forward(self, x, emb):
    shift, scale, gate = _mod(self.linear, emb, 3)
    return OF.layer_norm_mod(x, scale=scale, shift=shift, eps=self.eps), gate
