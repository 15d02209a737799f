"""Separable frequency-band filters over (H, W) written as two small real GEMMs.

The CFG-cache compensation of the Wan pipelines (src/maxdiffusion/pipelines/wan/wan_pipeline.py:1436-1510) takes
`rfft2` of cached tensors, scales a low band by w1 and the rest by w2, and transforms back. All of that is
linear, and the band is a product of a row band and a column band that are both symmetric in +/- frequency, so

    irfft2(weight * rfft2(x)) = w2 * x + (w1 - w2) * P_h x P_w

with P_n = the real projector onto the kept frequencies of a length-n axis,
P_n[i, j] = (1/n) * sum_{k in band} cos(2 pi k (i - j) / n). No complex arithmetic and no power-of-two sizes are
involved (Wan latents are 90 x 160 at 720p), and the work is two GEMMs with K = W and K = H.

On a GPU the GEMMs run on the tcgen05 bf16 kernel with fp32 output. To keep fp32-level accuracy both operands are
split into a bf16 head and a bf16 remainder, and the three significant products ride one GEMM by concatenating
them along K:  [x_hi | x_lo | x_hi] . [P_hi | P_hi | P_lo]^T.
"""
from __future__ import annotations

import functools
import math

import torch


def band_indices(n: int, cutoff: int, half_spectrum: bool) -> list[int]:
  """Signed frequencies kept by the reference's mask on an axis of length n.

  Full-spectrum axis (rows of rfft2): bins k < cutoff and k >= n - cutoff + 1, i.e. |f| < cutoff.
  Half-spectrum axis (last axis of rfft2): bins k < cutoff of n//2 + 1 bins; the mirrored negative
  frequencies are implied by the real inverse transform."""
  if half_spectrum:
    kept = [k for k in range(n // 2 + 1) if k < cutoff]
  else:
    kept = [k for k in range(n) if k < cutoff or k >= n - cutoff + 1]
    kept = [k if k <= n // 2 else k - n for k in kept]
  out = set()
  for k in kept:
    out.add(k)
    out.add(-k)
  if n % 2 == 0 and (n // 2 in out or -(n // 2) in out):  # the Nyquist bin is its own mirror image
    out.discard(-(n // 2))
    out.add(n // 2)
  return sorted(out)


@functools.lru_cache(maxsize=32)
def _projector_cpu(n: int, cutoff: int, half_spectrum: bool) -> torch.Tensor:
  d = torch.arange(n, dtype=torch.float64)
  diff = d[:, None] - d[None, :]
  p = torch.zeros(n, n, dtype=torch.float64)
  for k in band_indices(n, cutoff, half_spectrum):
    p += torch.cos(2.0 * math.pi * k * diff / n)
  return (p / n).float()


def band_projector(n: int, cutoff: int, half_spectrum: bool, device=None) -> torch.Tensor:
  """P_n (fp32 [n, n], symmetric): keeps the band of `band_indices` and removes every other frequency."""
  p = _projector_cpu(n, cutoff, half_spectrum)
  return p.to(device) if device is not None else p


def _pad_to(t: torch.Tensor, dim: int, multiple: int) -> torch.Tensor:
  extra = (-t.shape[dim]) % multiple
  if extra == 0:
    return t
  shape = list(t.shape)
  shape[dim] = extra
  return torch.cat([t, t.new_zeros(shape)], dim=dim)


def _split_bf16(t: torch.Tensor):
  hi = t.to(torch.bfloat16)
  lo = (t - hi.float()).to(torch.bfloat16)
  return hi, lo


def matmul_right(x2d: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
  """x2d [M, n] (fp32) times the symmetric p [n, n] (fp32) -> fp32 [M, n].

  CUDA: one tcgen05 GEMM over the three split-bf16 products. CPU: a plain fp32 matmul."""
  if not x2d.is_cuda:
    return x2d @ p
  from . import kernels as K
  n = p.shape[0]
  xp = _pad_to(x2d, 1, 8)  # 16-byte rows for the operand loads
  pp = _pad_to(_pad_to(p, 1, 8), 0, 8)  # [N_pad, K_pad]; the GEMM contracts over the last axis of both
  x_hi, x_lo = _split_bf16(xp)
  p_hi, p_lo = _split_bf16(pp)
  a = torch.cat([x_hi, x_lo, x_hi], dim=1).contiguous()
  b = torch.cat([p_hi, p_hi, p_lo], dim=1).contiguous()
  out = K.gemm(a, b, out_dtype=torch.float32)
  return out[:, :n]


def band_pass2d(x: torch.Tensor, cutoff_h: int, cutoff_w: int) -> torch.Tensor:
  """P_h x P_w over the last two axes of x (any leading axes); fp32 result."""
  h, w = x.shape[-2], x.shape[-1]
  lead = x.shape[:-2]
  xf = x.float()
  pw = band_projector(w, cutoff_w, True, x.device)
  ph = band_projector(h, cutoff_h, False, x.device)
  y = matmul_right(xf.reshape(-1, w), pw).reshape(*lead, h, w)
  yt = y.transpose(-1, -2).reshape(-1, h)
  z = matmul_right(yt, ph).reshape(*lead, w, h).transpose(-1, -2)
  return z


def band_weighted(x: torch.Tensor, w_low: float, w_high: float) -> torch.Tensor:
  """irfft2(weight * rfft2(x)) with weight = w_low on the lowest quarter of the frequencies of each axis
  (both axes low at once) and w_high elsewhere; fp32 result of x's shape."""
  h, w = x.shape[-2], x.shape[-1]
  # the reference sizes the band on the rfft2 output: h bins along rows, w//2+1 along columns
  ch, cw = max(1, h // 4), max(1, (w // 2 + 1) // 4)
  xf = x.float()
  if w_low == w_high:
    return xf * w_high
  return xf * w_high + (w_low - w_high) * band_pass2d(xf, ch, cw)
