"""Quantised linear layers: fp8 (e4m3) weights and activations with per-tensor absmax scales on the fp8 tensor-core
GEMM (`csrc/gemm_fp8.cu`).

The reference quantises through libraries around XLA dot_general: AQT int8 for the SD UNet
(src/maxdiffusion/models/quantizations.py:88-131) and qwix `int8` / `fp8` / `fp8_full` rules for Wan and LTX-2
(src/maxdiffusion/pipelines/wan/wan_pipeline.py:569-651; config keys `use_qwix_quantization`, `quantization`,
`*_quantization_calibration_method`). Here:

  fp8       weights are quantised once (static absmax), activations at every call (dynamic absmax, on the device,
            no host synchronisation); forward product in fp8; the backward pass (if any) runs in bf16
  fp8_full  as fp8, and the two backward products run in fp8 as well with e5m2 gradients
  int8      symmetric per-tensor int8 weights (static) and activations (dynamic) on the integer tensor-core path
            (tcgen05 kind::i8, exact int32 accumulation); the backward pass (if any) runs in bf16

`quantize_model(model, mode)` swaps the `Linear` layers of the transformer blocks in place and
`get_quantization_mode(config)` reads the reference's config keys.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import kernels as K
from .layers import Linear

FP8_MAX = {False: 448.0, True: 57344.0}


def fake_quantize(x: torch.Tensor, e5m2: bool = False) -> torch.Tensor:
  """Reference of the quantiser in plain PyTorch (CPU tests, numerics oracle)."""
  amax = x.detach().abs().max().float().clamp_min(1e-12)
  scale = amax / FP8_MAX[e5m2]
  dt = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
  return ((x.float() / scale).clamp(-FP8_MAX[e5m2], FP8_MAX[e5m2]).to(dt).float() * scale).to(x.dtype)


class _Fp8LinearFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x2, w, wq, w_scale, bias, full):
    xq, x_scale = K.quantize_fp8(x2)
    ctx.save_for_backward(x2, w)
    ctx.full, ctx.has_bias = full, bias is not None
    return K.gemm_fp8(xq, x_scale, wq, w_scale, bias)

  @staticmethod
  def backward(ctx, dy):
    x2, w = ctx.saved_tensors
    dy = dy.contiguous()
    if ctx.full and dy.shape[0] % 16 == 0 and dy.shape[1] % 16 == 0:
      # e5m2 gradients; the transposed operands are materialised because the fp8 kernel is K-major only
      dq, d_scale = K.quantize_fp8(dy, e5m2=True)
      wtq, wt_scale = K.quantize_fp8(w.t().contiguous())
      dx = K.gemm_fp8(dq, d_scale, wtq, wt_scale, a_e5m2=True)
      dtq, dt_scale = K.quantize_fp8(dy.t().contiguous(), e5m2=True)
      xtq, xt_scale = K.quantize_fp8(x2.t().contiguous())
      dw = K.gemm_fp8(dtq, dt_scale, xtq, xt_scale, a_e5m2=True)
    else:
      dx = K.gemm(dy, w, b_mn=True)
      dw = K.gemm(dy, x2, a_mn=True, b_mn=True)
    db = K.colsum(dy).to(torch.bfloat16) if ctx.has_bias else None
    return dx, dw, None, None, db, None


def fake_quantize_int8(x: torch.Tensor) -> torch.Tensor:
  """Plain-PyTorch reference of the int8 quantiser."""
  amax = x.detach().abs().max().float().clamp_min(1e-12)
  scale = amax / 127.0
  return ((x.float() / scale).round().clamp(-127, 127) * scale).to(x.dtype)


class _Int8LinearFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x2, w, wq, w_scale, bias):
    xq, x_scale = K.quantize_int8(x2)
    ctx.save_for_backward(x2, w)
    ctx.has_bias = bias is not None
    return K.gemm_int8(xq, x_scale, wq, w_scale, bias)

  @staticmethod
  def backward(ctx, dy):
    x2, w = ctx.saved_tensors
    dy = dy.contiguous()
    dx = K.gemm(dy, w, b_mn=True)
    dw = K.gemm(dy, x2, a_mn=True, b_mn=True)
    db = K.colsum(dy).to(torch.bfloat16) if ctx.has_bias else None
    return dx, dw, None, None, db


class Fp8Linear(nn.Module):
  """Drop-in for `layers.Linear` with the product in fp8. The bf16 master weight is kept (training, export); its
  quantised copy is refreshed by `requantize()` (after an optimizer step) or lazily when the weight changes."""

  int8 = False

  def __init__(self, base: Linear, full: bool = False):
    super().__init__()
    self.in_features, self.out_features, self.full = base.in_features, base.out_features, full
    self.weight, self.bias = base.weight, base.bias
    self._wq = self._w_scale = None
    self._version = -1

  def requantize(self) -> None:
    w = self.weight.detach()
    w = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
    self._wq, self._w_scale = (K.quantize_int8 if self.int8 else K.quantize_fp8)(w.contiguous())
    self._version = self.weight._version

  def forward(self, x, activation: Optional[str] = None):
    ok = (x.is_cuda and x.dtype == torch.bfloat16 and self.in_features % 16 == 0 and self.out_features % 8 == 0
          and (x.numel() // self.in_features) % 8 == 0)
    if not ok:
      fq = fake_quantize_int8 if self.int8 else fake_quantize
      y = F.linear(x, fq(self.weight.to(x.dtype)), None if self.bias is None else self.bias.to(x.dtype)) \
          if not x.is_cuda else F.linear(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))
    else:
      if self._wq is None or self._version != self.weight._version:
        self.requantize()
      bias = None if self.bias is None else self.bias.to(torch.bfloat16)
      x2 = x.reshape(-1, self.in_features)
      x2 = x2 if x2.is_contiguous() else x2.contiguous()
      if self.int8:
        y = _Int8LinearFn.apply(x2, self.weight, self._wq, self._w_scale, bias)
      else:
        y = _Fp8LinearFn.apply(x2, self.weight, self._wq, self._w_scale, bias, self.full)
      y = y.view(*x.shape[:-1], self.out_features)
    if activation == "gelu_tanh":
      y = F.gelu(y, approximate="tanh")
    elif activation == "silu":
      y = F.silu(y)
    return y


class Int8Linear(Fp8Linear):
  """Drop-in for `layers.Linear` with the product on the int8 tensor-core path (per-tensor symmetric scales)."""
  int8 = True


def get_quantization_mode(config) -> Optional[str]:
  """The reference's switches: `use_qwix_quantization: True` + `quantization: int8 | fp8 | fp8_full`."""
  if not config.get("use_qwix_quantization", False):
    return None
  mode = str(config.get("quantization", "") or "fp8").lower()
  if mode not in ("int8", "fp8", "fp8_full"):
    raise ValueError(f"quantization must be one of int8, fp8, fp8_full; got '{mode}'")
  return mode


def quantize_model(model: nn.Module, mode: str = "fp8", predicate: Optional[Callable[[str, nn.Module], bool]] = None) -> int:
  """Replaces `Linear` layers by `Fp8Linear` (`Int8Linear` for mode "int8") in place; returns how many were replaced. By default the layers inside
  transformer blocks are quantised and embedders / output heads keep bf16 (the reference's rules exclude the same
  small layers, wan_pipeline.py:600-640)."""
  if predicate is None:
    predicate = lambda name, m: "blocks." in name and m.in_features % 16 == 0 and m.out_features % 16 == 0
  full = mode == "fp8_full"
  count = 0
  for name, module in list(model.named_modules()):
    for child_name, child in list(module.named_children()):
      full_name = f"{name}.{child_name}" if name else child_name
      if type(child) is Linear and predicate(full_name, child):
        setattr(module, child_name, Int8Linear(child) if mode == "int8" else Fp8Linear(child, full))
        count += 1
  return count
