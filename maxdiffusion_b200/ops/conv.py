"""Channels-last convolutions on the implicit-GEMM kernel (`csrc/conv_igemm.cu`) and the row norm that goes with them.

Tensors are channels-last bf16: video `[B, T, H, W, C]`, images `[B, H, W, C]`. A convolution is described to the
kernel as a table of taps (coordinate shifts + the K range of the tap in the packed weight matrix); this module builds
the tables and packs the weights:

  conv3d_causal      3x3x3 / (3,1,1) causal convolution with an optional 2-frame history tensor (the reference's
                     `WanCausalConv3d` and its feature cache, src/maxdiffusion/models/wan/autoencoder_kl_wan.py:70-147)
  conv2d             3x3 / 1x1, stride 1 or 2 (zero padding given per side; `WanResample` down-sampling pads right /
                     bottom only, the UNet pads all sides: :245-389, src/maxdiffusion/models/resnet_flax.py:37-95)
  upsample2x_conv2d  nearest-2x followed by a 3x3 convolution, computed at LOW resolution as four parity classes of
                     2x2 convolutions with pre-summed weights (2.25x fewer FLOPs, no up-sampled tensor)
  conv2d_dgrad       gradient of conv2d with respect to its input, as a convolution of dY with the transposed,
                     flipped weights (stride 2: parity classes of the input)
  rms_act            `WanRMS_norm` (+ SiLU) over the channel axis

CPU tensors and fp32 run the PyTorch reference (`F.conv3d` / `F.conv2d`), which is also the oracle of the tests.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from . import _lib


def _declare(L):
  c_void_p, c_int, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
  llp, ip = ctypes.POINTER(c_ll), ctypes.POINTER(c_int)
  L.mdb_conv_igemm.argtypes = [c_void_p] * 6 + [llp] * 4 + [ip, ip, c_int, c_int, c_ll, c_int, ip, ip, c_int, c_int,
                                                           llp, llp, c_int, c_void_p]
  L.mdb_conv_igemm.restype = c_int
  L.mdb_rms_act_cl.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int, ctypes.c_float, c_int,
                               c_int, c_int, c_void_p]
  L.mdb_rms_act_cl.restype = c_int
  L.mdb_conv_igemm_tune.argtypes = [c_int, c_int, c_int]
  L.mdb_conv_igemm_tune.restype = c_int
  L.mdb_conv_wgrad.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_int, llp, c_int, c_void_p]
  L.mdb_conv_wgrad.restype = c_int
  L.mdb_conv_wgrad_boxed.argtypes = [c_void_p] * 3 + [c_int] * 7 + [c_ll] * 6 + [c_int, c_int, ip, c_int, c_int, c_int, c_void_p]
  L.mdb_conv_wgrad_boxed.restype = c_int
  L.mdb_softmax_rows.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_ll, c_int, c_void_p]
  L.mdb_softmax_rows.restype = c_int
  L.mdb_gn_cl_sums.argtypes = [c_void_p] * 5 + [c_int] * 4 + [c_void_p]
  L.mdb_gn_cl_sums.restype = c_int
  L.mdb_gn_cl_apply.argtypes = [c_void_p] * 8 + [c_int] * 4 + [c_void_p]
  L.mdb_gn_cl_apply.restype = c_int
  c_float = ctypes.c_float
  L.mdb_gn_cl_fold_fwd.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_int] + [c_void_p] * 5
  L.mdb_gn_cl_fold_fwd.restype = c_int
  L.mdb_gn_cl_fold_bwd.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int] + [c_void_p] * 8
  L.mdb_gn_cl_fold_bwd.restype = c_int


_lib.register(_declare)


def tune(units_per_stage: int = 0, max_stages: int = 0, ctas_per_sm: int = 0) -> None:
  """Pins the launch shape of the implicit-GEMM convolution (0 = the launcher's own choice): (tap, channel block)
  units per pipeline stage, an upper limit on the stages, CTAs per SM (2 applies to tiles of at most 128 output
  channels). For the tile search and the benchmarks."""
  _lib.check(_lib.lib().mdb_conv_igemm_tune(int(units_per_stage), int(max_stages), int(ctas_per_sm)), "mdb_conv_igemm_tune")


def use_kernel(x: torch.Tensor) -> bool:
  return x.is_cuda and x.dtype == torch.bfloat16


def _round_up(v: int, m: int) -> int:
  return (v + m - 1) // m * m


@dataclass
class PackedConv:
  """Weights of one convolution in the kernel's layout, with its tap table."""
  w: torch.Tensor                 # [N_pad, n_taps * c_pad] bf16, K-major
  bias: Optional[torch.Tensor]    # [N_pad] bf16 or None
  taps: list                      # per class: list of (o0, o1, o2, o3, o4) ; koff is the running tap index * c_pad
  c_in: int                       # channels the activation must have (multiple of 16)
  c_pad: int                      # K span of a tap (multiple of 64)
  n_out: int                      # true output channels
  n_pad: int                      # multiple of 8
  kind: str
  src: tuple = ()                 # (weight, bias, stride, pad_top_left) as given: what the PyTorch reference path runs

  def tap_arrays(self, shift1: int = 0):
    """ctypes arrays of the tap table; `shift1` is added to every tap's offset along dim 1 (the width): an input
    that carries `shift1` halo columns on each side produces outputs for its interior columns only."""
    flat, begin, k = [], [0], 0
    for cls in self.taps:
      for t in cls:
        flat.extend([t[0], t[1] + shift1, t[2], t[3], t[4], k * self.c_pad])
        k += 1
      begin.append(k)
    return (ctypes.c_int * len(flat))(*flat), (ctypes.c_int * len(begin))(*begin), len(self.taps)


def _pack(w_taps: torch.Tensor, bias, taps, kind: str) -> PackedConv:
  """w_taps: [N, n_taps, C] (any float dtype) -> PackedConv with channels padded to 16 / 64 and N padded to 8."""
  n, n_taps, c = w_taps.shape
  c_in, c_pad, n_pad = _round_up(c, 16), _round_up(c, 64), _round_up(n, 8)
  w = torch.zeros((n_pad, n_taps, c_pad), dtype=torch.bfloat16, device=w_taps.device)
  w[:n, :, :c] = w_taps.to(torch.bfloat16)
  b = None
  if bias is not None:
    b = torch.zeros(n_pad, dtype=torch.bfloat16, device=w_taps.device)
    b[:n] = bias.to(torch.bfloat16)
  return PackedConv(w.reshape(n_pad, n_taps * c_pad), b, taps, c_in, c_pad, n, n_pad, kind)


def pack_conv3d(weight: torch.Tensor, bias=None) -> PackedConv:
  """weight [Co, Ci, kt, kh, kw] (causal in time, 'same' in space)."""
  co, ci, kt, kh, kw = weight.shape
  taps = [[(0, b - kw // 2, a - kh // 2, t - (kt - 1), 0) for t in range(kt) for a in range(kh) for b in range(kw)]]
  pk = _pack(weight.permute(0, 2, 3, 4, 1).reshape(co, kt * kh * kw, ci), bias, taps, "conv3d")
  pk.src = (weight, bias, 1, None)
  return pk


def pack_conv2d(weight: torch.Tensor, bias=None, stride: int = 1, pad_top_left: Optional[int] = None) -> PackedConv:
  """weight [Co, Ci, kh, kw]. `pad_top_left`: zero rows / columns before the image (default k // 2); the far side is
  padded with whatever the output size needs (out = in for stride 1, in / 2 for stride 2)."""
  co, ci, kh, kw = weight.shape
  p = kh // 2 if pad_top_left is None else pad_top_left
  w = weight.permute(0, 2, 3, 1).reshape(co, kh * kw, ci)
  if stride == 1:
    taps = [[(0, b - p, a - p, 0, 0) for a in range(kh) for b in range(kw)]]
    pk = _pack(w, bias, taps, "conv2d")
    pk.src = (weight, bias, 1, p)
    return pk
  assert stride == 2
  # activation seen as [B, H/2, 2, W/2, 2C]: input row 2*oh + a - p = 2*(oh + dh) + ph
  c16 = _round_up(ci, 16)
  taps = [[]]
  for a in range(kh):
    dh, ph = divmod(a - p, 2)
    for b in range(kw):
      dw, pw = divmod(b - p, 2)
      taps[0].append((pw * c16, dw, ph, dh, 0))
  pk = _pack(w, bias, taps, "conv2d_s2")
  pk.src = (weight, bias, 2, p)
  return pk


def _upsample_parity_taps():
  """For output parity r: which low-resolution shift each of the 3 kernel rows reads: floor((r + a - 1) / 2)."""
  return {r: [((r + a - 1) // 2) for a in range(3)] for r in (0, 1)}


def pack_upsample_conv2d(weight: torch.Tensor, bias=None) -> PackedConv:
  """nearest-2x + 3x3 'same' conv -> four classes (rh, rw) of 2x2 convolutions on the low-resolution input."""
  co, ci, kh, kw = weight.shape
  assert kh == 3 and kw == 3
  shift = _upsample_parity_taps()
  w32 = weight.float()
  mats, taps = [], []
  for rh in (0, 1):
    for rw in (0, 1):
      cls = []
      for dp in sorted(set(shift[rh])):
        for dq in sorted(set(shift[rw])):
          rows = [a for a in range(3) if shift[rh][a] == dp]
          cols = [b for b in range(3) if shift[rw][b] == dq]
          mats.append(w32[:, :, rows][:, :, :, cols].sum(dim=(2, 3)))  # [Co, Ci]
          cls.append((0, dq, dp, 0, 0))
      taps.append(cls)
  pk = _pack(torch.stack(mats, dim=1), bias, taps, "upsample_conv2d")
  pk.src = (weight, bias, 1, 1)
  return pk


def pack_conv2d_dgrad(weight: torch.Tensor, stride: int = 1, pad_top_left: Optional[int] = None) -> PackedConv:
  """Weights for dX = conv2d_dgrad(dY): contraction over Co, output channels Ci."""
  co, ci, kh, kw = weight.shape
  p = kh // 2 if pad_top_left is None else pad_top_left
  wt = weight.permute(1, 2, 3, 0)  # [Ci, kh, kw, Co]
  if stride == 1:
    # dX[i] = sum_a dY[i + p - a] W[a]
    taps = [[(0, p - b, p - a, 0, 0) for a in range(kh) for b in range(kw)]]
    pk = _pack(wt.reshape(ci, kh * kw, co), None, taps, "conv2d_dgrad_s1")
    pk.src = (weight, None, 1, p)
    return pk
  assert stride == 2
  # input row 2*u + r receives dY[u + (r + p - a) / 2] W[a] for the a with (r + p - a) even
  mats, taps = [], []
  for rh in (0, 1):
    for rw in (0, 1):
      cls = []
      for a in range(kh):
        if (rh + p - a) % 2:
          continue
        for b in range(kw):
          if (rw + p - b) % 2:
            continue
          mats.append(wt[:, a, b, :])
          cls.append((0, (rw + p - b) // 2, (rh + p - a) // 2, 0, 0))
      taps.append(cls)
  pk = _pack(torch.stack(mats, dim=1), None, taps, "conv2d_dgrad_s2")
  pk.src = (weight, None, 2, p)
  return pk


def _pick_box(e1: int, e2: int, e3: int, allow3: bool):
  """Tile (b1, b2, b3) with b1 * b2 * b3 = 128 that covers the e1 x e2 x e3 output positions with the least padding;
  among equals the widest along the fastest axis."""
  best, best_cost = None, None
  for l1 in range(8):
    for l2 in range(8 - l1):
      l3 = 7 - l1 - l2
      b1, b2, b3 = 1 << l1, 1 << l2, 1 << l3
      if b3 > 1 and not allow3:
        continue
      cost = _round_up(e1, b1) * _round_up(e2, b2) * _round_up(e3, b3)
      key = (cost, -b1, -b2)
      if best_cost is None or key < best_cost:
        best, best_cost = (b1, b2, b3), key
  return best


def _launch(x, x_alt, pk: PackedConv, dims, strides, alt_dims, alt_strides, box, ext, out, out_strides, class_off,
            residual, silu, alt_dim=-1, alt_shift=0, tap_shift1=0):
  taps, begin, n_classes = pk.tap_arrays(tap_shift1)
  LL, I = ctypes.c_longlong, ctypes.c_int
  arr = lambda T, v: (T * len(v))(*[int(i) for i in v])
  rc = _lib.lib().mdb_conv_igemm(
      _lib.ptr(x), _lib.ptr(x_alt), _lib.ptr(pk.w), _lib.ptr(out), _lib.ptr(pk.bias), _lib.ptr(residual),
      arr(LL, dims), arr(LL, strides), arr(LL, alt_dims if alt_dims else dims), arr(LL, alt_strides if alt_strides else strides),
      arr(I, box), arr(I, ext), pk.c_in, pk.n_pad, pk.w.shape[1], n_classes, begin, taps, alt_dim, alt_shift,
      arr(LL, out_strides), arr(LL, class_off), 1 if silu else 0, _lib.stream())
  _lib.check(rc, "mdb_conv_igemm")
  return out


def _check_cl(x: torch.Tensor, c_in: int):
  assert x.dtype == torch.bfloat16 and x.stride(-1) == 1, "channels-last bf16 expected"
  assert x.shape[-1] == c_in, f"activation has {x.shape[-1]} channels, the packed weights expect {c_in} (pad to 16)"
  assert all(s % 8 == 0 for s in x.stride()[:-1]) and x.data_ptr() % 16 == 0


def pad_channels(x: torch.Tensor, c: int) -> torch.Tensor:
  """Zero-pads the last (channel) axis up to c."""
  return x if x.shape[-1] == c else F.pad(x, (0, c - x.shape[-1]))


def conv3d_causal(x: torch.Tensor, pk: PackedConv, hist: Optional[torch.Tensor] = None,
                  residual: Optional[torch.Tensor] = None, silu: bool = False,
                  out: Optional[torch.Tensor] = None, halo: int = 0) -> torch.Tensor:
  """x [B, T, H, W, C] -> [B, T, H, W, N]. `hist` [B, 2, H, W, C]: the two frames before x (None: zeros). `out` may be
  a strided view (e.g. every second frame of a larger tensor) as long as its channels are dense. With `halo` = 1 the
  input (and `hist`) carry one extra column on each side of W (a width-sharded tensor with its neighbours' edge columns)
  and the output has W - 2 columns: the halo columns are read, not recomputed."""
  if not use_kernel(x):
    w, b = pk.src[0], pk.src[1]
    ci = w.shape[1]
    y = ref_conv3d_causal(x[..., :ci], w, b, hist=None if hist is None else hist[..., :ci], silu=silu)
    if halo:
      y = y[:, :, :, halo:-halo]
    y = (y + residual.float() if residual is not None else y).to(x.dtype)
    if out is not None:
      out.copy_(y)
      return out
    return y
  _check_cl(x, pk.c_in)
  B, T, H, Win, C = x.shape
  W = Win - 2 * halo  # output columns
  if out is None:
    out = torch.empty((B, T, H, W, pk.n_pad), dtype=x.dtype, device=x.device)
  else:
    assert out.shape == (B, T, H, W, pk.n_pad) and out.stride(-1) == 1 and out.dtype == x.dtype
    assert all(s % 8 == 0 for s in out.stride()[:-1]) and residual is None
  b1, b2, _ = _pick_box(W, H, 1, False)
  alt_dims = alt_strides = None
  if hist is not None:
    _check_cl(hist, pk.c_in)
    assert hist.shape == (B, 2, H, Win, C)
    alt_dims = [C, Win, H, 2, B]
    alt_strides = [hist.stride(3), hist.stride(2), hist.stride(1), hist.stride(0)]
  if residual is not None:
    assert residual.shape == out.shape and residual.is_contiguous()
  _launch(x, hist, pk, [C, Win, H, T, B], [x.stride(3), x.stride(2), x.stride(1), x.stride(0)], alt_dims, alt_strides,
          [b1, b2, 1], [W, H, T, B], out, [out.stride(3), out.stride(2), out.stride(1), out.stride(0)], [0], residual, silu,
          alt_dim=3, alt_shift=2, tap_shift1=halo)
  return out if pk.n_pad == pk.n_out else out[..., :pk.n_out]


def conv2d(x: torch.Tensor, pk: PackedConv, residual: Optional[torch.Tensor] = None, silu: bool = False) -> torch.Tensor:
  """x [B, H, W, C] -> [B, Ho, Wo, N] (Ho = H for stride 1, H / 2 for stride 2)."""
  if not use_kernel(x):
    w, b, stride, p = pk.src
    return ref_conv2d(x[..., :w.shape[1]], w, b, stride=stride, pad_top_left=p, residual=residual, silu=silu).to(x.dtype)
  _check_cl(x, pk.c_in)
  B, H, W, C = x.shape
  n = pk.n_pad
  if pk.kind in ("conv2d", "conv2d_dgrad_s1"):
    out = torch.empty((B, H, W, n), dtype=x.dtype, device=x.device)
    box = _pick_box(W, H, B, True)
    dims, strides = [C, W, H, B, 1], [x.stride(2), x.stride(1), x.stride(0), x.stride(0) * B]
    ext, os_ = [W, H, B, 1], [n, W * n, H * W * n, B * H * W * n]
  elif pk.kind == "conv2d_s2":
    assert H % 2 == 0 and W % 2 == 0 and x.stride(2) == C, "stride 2 needs even sizes and dense rows"
    Ho, Wo = H // 2, W // 2
    out = torch.empty((B, Ho, Wo, n), dtype=x.dtype, device=x.device)
    b1, b3, _ = _pick_box(Wo, Ho, 1, False)
    box = (b1, 1, b3)
    dims, strides = [2 * C, Wo, 2, Ho, B], [2 * C, x.stride(1), 2 * x.stride(1), x.stride(0)]
    ext, os_ = [Wo, 1, Ho, B], [n, 0, Wo * n, Ho * Wo * n]
  else:
    raise ValueError(f"conv2d cannot run weights packed as {pk.kind}")
  if residual is not None:
    assert residual.shape == out.shape and residual.is_contiguous()
  _launch(x, None, pk, dims, strides, None, None, box, ext, out, os_, [0], residual, silu)
  return out if pk.n_pad == pk.n_out else out[..., :pk.n_out]


def _parity_conv(x, pk, silu=False, halo: int = 0):
  """Shared by the fused up-sampling convolution and the stride-2 dgrad: x [B, H, W, C] -> [B, 2H, 2W, N], class
  (rh, rw) writes the output positions (2p + rh, 2q + rw). With `halo` the input carries that many extra columns on
  each side of W, which are read but produce no output."""
  _check_cl(x, pk.c_in)
  B, H, Win, C = x.shape
  W = Win - 2 * halo
  n = pk.n_pad
  out = torch.empty((B, 2 * H, 2 * W, n), dtype=x.dtype, device=x.device)
  box = _pick_box(W, H, B, True)
  class_off = [rh * 2 * W * n + rw * n for rh in (0, 1) for rw in (0, 1)]
  _launch(x, None, pk, [C, Win, H, B, 1], [x.stride(2), x.stride(1), x.stride(0), x.stride(0) * B], None, None, box,
          [W, H, B, 1], out, [2 * n, 4 * W * n, 4 * H * W * n, 4 * B * H * W * n], class_off, None, silu, tap_shift1=halo)
  return out if pk.n_pad == pk.n_out else out[..., :pk.n_out]


def upsample2x_conv2d(x: torch.Tensor, pk: PackedConv, halo: int = 0) -> torch.Tensor:
  assert pk.kind == "upsample_conv2d"
  if not use_kernel(x):
    y = ref_upsample2x_conv2d(x[..., :pk.src[0].shape[1]], pk.src[0], pk.src[1])
    return (y[:, :, 2 * halo:y.shape[2] - 2 * halo] if halo else y).to(x.dtype)
  return _parity_conv(x, pk, halo=halo)


def conv2d_dgrad(dy: torch.Tensor, pk: PackedConv) -> torch.Tensor:
  """dX for a conv2d whose weights were packed with `pack_conv2d_dgrad` (dy is [B, Ho, Wo, Co], channels-last)."""
  if not use_kernel(dy):
    w, _, stride, p = pk.src
    B, Ho, Wo, _ = dy.shape
    H, W = Ho * stride, Wo * stride
    far = max((Ho - 1) * stride + w.shape[2] - H - p, 0)
    g = torch.nn.grad.conv2d_input((B, w.shape[1], H + p + far, W + p + far), w.float(), dy.float().permute(0, 3, 1, 2)[..., :, :],
                                   stride=stride)
    return g[:, :, p:p + H, p:p + W].permute(0, 2, 3, 1).to(dy.dtype)
  if pk.kind == "conv2d_dgrad_s2":
    if any(len(c) == 0 for c in pk.taps):
      raise ValueError("a 1x1 stride-2 convolution leaves input parities without a tap; use the dense fallback")
    return _parity_conv(dy, pk)
  return conv2d(dy, pk)


def wgrad_plan(H: int, W: int, k: int, stride: int, pad: int):
  """How the weight gradient sees its operands: (planes, Hg, Wg, taps) with `planes` the (row parity, column parity)
  sub-grids of X that are stacked (one for stride 1), Hg x Wg the pixel grid shared by dY and every plane (bordered
  by one ring of zeros), and per kernel tap (plane index, row shift, column shift)."""
  if stride == 1:
    return [(0, 0)], H, W, [(0, a - pad, b - pad) for a in range(k) for b in range(k)]
  planes = [(ph, pw) for ph in (0, 1) for pw in (0, 1)]
  taps = []
  for a in range(k):
    dh, ph = divmod(a - pad, 2)
    for b in range(k):
      dw, pw = divmod(b - pad, 2)
      taps.append((planes.index((ph, pw)), dh, dw))
  return planes, H // 2, W // 2, taps


def wgrad_box(Ho: int, Wo: int) -> tuple:
  """(BW, BH) with BW * BH = 64: the box of output pixels that makes one K block, chosen for the fewest pixels of
  padding on a Ho x Wo grid (ties: the wider box, whose rows are longer contiguous runs)."""
  best = None
  for bw in (64, 32, 16, 8):
    bh = 64 // bw
    cost = -(-Wo // bw) * bw * -(-Ho // bh) * bh
    if best is None or cost < best[0]:
      best = (cost, bw, bh)
  return best[1], best[2]


def wgrad_splits(items: int, kb: int, out_elems: int, sms: int = 148) -> int:
  """K splits of the weight gradient: rounds of work items over the SMs times K blocks per item (0.27 us each), plus
  the write and read of one fp32 partial per split."""
  fold_us = out_elems * 8 / 5e6
  best, best_cost = 1, None
  for s in range(1, 65):
    per = -(-kb // s)
    if per < 8 and s > 1:
      break
    cost = -(-items * s // sms) * per * 0.27 + s * fold_us
    if best_cost is None or cost < best_cost * 0.97:
      best, best_cost = s, cost
  return best


def wgrad_taps_boxed(k: int, stride: int, pad: int) -> list:
  """Per kernel tap (column parity, column shift, row parity, row shift) on the grid the boxed kernel reads x
  through: the input pixel of output (ho, wo) is (stride * ho + a - pad, stride * wo + b - pad)."""
  taps = []
  for a in range(k):
    dh, ph = divmod(a - pad, stride) if stride == 2 else (a - pad, 0)
    for b in range(k):
      dw, pw = divmod(b - pad, stride) if stride == 2 else (b - pad, 0)
      taps.append((pw, dw, ph, dh))
  return taps


def _boxed_ok(x, dy, stride) -> bool:
  B, H, W, Ci = x.shape
  return (stride == 1 or (H % 2 == 0 and W % 2 == 0)) and x.stride(-1) == 1 and dy.stride(-1) == 1


def _conv2d_wgrad_boxed(x, dy, k, stride, pad):
  """No bordered copies: K blocks are boxes of output pixels read straight from x and dy (see csrc/conv_wgrad.cu)."""
  B, H, W, Ci = x.shape
  _, Ho, Wo, Co = dy.shape
  ci8, co8 = _round_up(Ci, 8), _round_up(Co, 8)
  x, dy = pad_channels(x, ci8), pad_channels(dy, co8)
  if stride == 2 and x.stride(2) != ci8:
    x = x.contiguous()
  if any(s % 8 for s in (*x.stride()[:3], *dy.stride()[:3])):
    x, dy = x.contiguous(), dy.contiguous()
  bw, bh = wgrad_box(Ho, Wo)
  taps = wgrad_taps_boxed(k, stride, pad)
  kb = B * -(-Ho // bh) * -(-Wo // bw)
  items = len(taps) * -(-co8 // 128) * max(1, -(-ci8 // 256))
  splits = wgrad_splits(items, kb, len(taps) * co8 * ci8)
  out = _wgrad_launch_boxed(dy, x, taps, (bw, bh), stride, splits)
  dw = (out.sum(dim=1) if splits > 1 else out[:, 0])[:, :Co, :Ci]
  return dw.reshape(k, k, Co, Ci).permute(2, 3, 0, 1)


def _wgrad_launch_boxed_kernel(dy, x, taps, box, stride, splits):
  """out[tap, split] = sum over the split's boxes of dy[box]^T x[box moved by the tap] (outside the image: zeros)."""
  B, Ho, Wo, M = dy.shape
  _, H, W, N = x.shape
  out = torch.empty((len(taps), splits, M, N), dtype=torch.float32, device=dy.device)
  flat = [v for t in taps for v in t]
  arr = (ctypes.c_int * len(flat))(*flat)
  rc = _lib.lib().mdb_conv_wgrad_boxed(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(out), B, Ho, Wo, H, W, M, N, dy.stride(0), dy.stride(1),
                                       dy.stride(2), x.stride(0), x.stride(1), x.stride(2), stride, len(taps), arr, box[0], box[1],
                                       splits, _lib.stream())
  _lib.check(rc, "mdb_conv_wgrad_boxed")
  return out


_wgrad_launch_boxed = _wgrad_launch_boxed_kernel


def conv2d_wgrad(x: torch.Tensor, dy: torch.Tensor, k: int = 3, stride: int = 1, pad: int = 1, boxed: Optional[bool] = None) -> torch.Tensor:
  """dW [Co, Ci, k, k] (fp32) of a conv2d from x [B, H, W, Ci] and dy [B, Ho, Wo, Co], both channels-last. `boxed`:
  None = the pad-free kernel form wherever it applies (stride 2 needs even H and W), False = the bordered form."""
  B, H, W, Ci = x.shape
  Co = dy.shape[-1]
  emulated = _wgrad_launch is not _wgrad_launch_kernel or _wgrad_launch_boxed is not _wgrad_launch_boxed_kernel
  if not use_kernel(x) and not emulated:
    xn = x.float().permute(0, 3, 1, 2)
    Ho, Wo = dy.shape[1:3]
    far_h, far_w = (Ho - 1) * stride + k - H - pad, (Wo - 1) * stride + k - W - pad
    xn = F.pad(xn, (pad, max(far_w, 0), pad, max(far_h, 0)))
    return torch.nn.grad.conv2d_weight(xn, (Co, Ci, k, k), dy.float().permute(0, 3, 1, 2), stride=stride)
  if (boxed is None or boxed) and _boxed_ok(x, dy, stride):
    return _conv2d_wgrad_boxed(x, dy, k, stride, pad)
  planes, Hg, Wg, taps = wgrad_plan(H, W, k, stride, pad)
  assert dy.shape[1:3] == (Hg, Wg), (dy.shape, Hg, Wg)
  ci8, co8 = _round_up(Ci, 8), _round_up(Co, 8)
  ring = lambda t: F.pad(t, (0, 0, 1, 1, 1, 1))  # one zero pixel around every image
  dyp = ring(pad_channels(dy, co8)).reshape(-1, co8)
  if stride == 1:
    xp = ring(pad_channels(x, ci8)).reshape(-1, ci8)
  else:
    xp = torch.stack([ring(pad_channels(x[:, ph::2, pw::2], ci8)) for ph, pw in planes]).reshape(-1, ci8)
  rows = dyp.shape[0]
  offs = [pl * rows + dh * (Wg + 2) + dw for pl, dh, dw in taps]
  kb = (rows + 63) // 64
  items = len(taps) * ((co8 + 127) // 128) * max(1, (ci8 + 255) // 256)
  splits = max(1, min(kb, (2 * 148 + items - 1) // items))
  out = _wgrad_launch(dyp, xp, offs, splits)
  dw = out.sum(dim=1)[:, :Co, :Ci]  # [taps, Co, Ci], splits added in a fixed order
  return dw.reshape(k, k, Co, Ci).permute(2, 3, 0, 1)


def _wgrad_launch_kernel(dyp, xp, offs, splits):
  """out[tap, split] = sum over the split's rows r of dyp[r, :]^T x xp[r + offs[tap], :] (rows outside xp are zeros)."""
  out = torch.empty((len(offs), splits, dyp.shape[1], xp.shape[1]), dtype=torch.float32, device=dyp.device)
  arr = (ctypes.c_longlong * len(offs))(*offs)
  rc = _lib.lib().mdb_conv_wgrad(_lib.ptr(dyp), _lib.ptr(xp), _lib.ptr(out), dyp.shape[0], xp.shape[0], dyp.shape[1],
                                 xp.shape[1], len(offs), arr, splits, _lib.stream())
  _lib.check(rc, "mdb_conv_wgrad")
  return out


_wgrad_launch = _wgrad_launch_kernel


def rms_act(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor] = None, silu: bool = True,
            eps: float = 1e-12, halo: int = 0) -> torch.Tensor:
  """y = act(x / max(||x||, eps) * sqrt(C) * gamma + beta) over the last axis of a channels-last tensor. With `halo`
  the result [..., W + 2 halo, C] has its interior columns written and its halo columns left for the caller (a
  width-sharded tensor that is about to receive its neighbours' edge columns)."""
  C = x.shape[-1]
  if not use_kernel(x):
    y = F.normalize(x.float(), dim=-1, eps=eps) * (C ** 0.5) * gamma.float().reshape(-1)
    if beta is not None:
      y = y + beta.float().reshape(-1)
    y = (F.silu(y) if silu else y).to(x.dtype)
    return F.pad(y, (0, 0, halo, halo)) if halo else y
  assert x.is_contiguous()
  W = x.shape[-2]
  y = torch.empty((*x.shape[:-2], W + 2 * halo, C), dtype=x.dtype, device=x.device)
  g = gamma.reshape(-1).float().contiguous()
  b = beta.reshape(-1).float().contiguous() if beta is not None else None
  rc = _lib.lib().mdb_rms_act_cl(_lib.ptr(x), C, _lib.ptr(y), C, _lib.ptr(g), _lib.ptr(b), x.numel() // C, C, float(eps),
                                 int(silu), W if halo else 0, halo, _lib.stream())
  _lib.check(rc, "mdb_rms_act_cl")
  return y


def softmax_rows(x: torch.Tensor) -> torch.Tensor:
  """Row softmax of a bf16 matrix (fp32 math), in place."""
  assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1
  rc = _lib.lib().mdb_softmax_rows(_lib.ptr(x), x.stride(0), _lib.ptr(x), x.stride(0), x.shape[0], x.shape[1], _lib.stream())
  _lib.check(rc, "mdb_softmax_rows")
  return x


def wide_head_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
  """Single-head attention for head sizes the flash kernels are not built for (q, k, v: [T, D], D a multiple of 8):
  scores on the tcgen05 GEMM, row softmax, P V on the GEMM. The score matrix is materialised in bf16 ([T, T]), which
  is fine for the few thousand positions of a latent frame."""
  from . import kernels as K

  T, D = q.shape
  scale = scale if scale is not None else D ** -0.5
  if not use_kernel(q) or T % 8 or D % 8 or T > 32768:
    p = torch.softmax((q.float() @ k.float().t()) * scale, dim=-1)
    return (p @ v.float()).to(q.dtype)
  scores = K.gemm(q.contiguous(), k.contiguous(), alpha=scale)         # [T, T] = scale * Q K^T
  softmax_rows(scores)
  return K.gemm(scores, v.contiguous(), b_mn=True)                     # [T, D] = P V   (V is [K = T, N = D])


# ---------------------------------------------------------------------------------------------
# GroupNorm (+ SiLU) on channels-last tensors [N, HW, C]: kernels for the two streaming passes, the fold between
# them (group statistics -> per-(n, c) coefficients) on [N, C]-sized arrays.
# ---------------------------------------------------------------------------------------------
def _gn_splits(n: int, hw: int) -> int:
  """Strips of pixels per image so that the sums pass fills the GPU (about 4 CTAs per SM) without tiny strips."""
  return max(1, min((4 * 148 + n - 1) // n, (hw + 63) // 64))


def _gn_partial(x3, dy3=None, act_a=None, act_b=None):
  """Per-channel partial sums fp32 [N, S, C, 2] over S strips of pixels (forward: x, x^2; backward: dy', dy' * x)."""
  N, HW, C = x3.shape
  S = _gn_splits(N, HW)
  partial = torch.empty((N, S, C, 2), device=x3.device, dtype=torch.float32)
  rc = _lib.lib().mdb_gn_cl_sums(_lib.ptr(x3), _lib.ptr(dy3), _lib.ptr(act_a), _lib.ptr(act_b), _lib.ptr(partial), N, HW, C, S,
                                 _lib.stream())
  _lib.check(rc, "mdb_gn_cl_sums")
  return partial


def _gn_apply(x3, dy3, ca, cb, cc, fa, fb, act):
  N, HW, C = x3.shape
  out = torch.empty_like(x3)
  rc = _lib.lib().mdb_gn_cl_apply(_lib.ptr(x3), _lib.ptr(dy3), _lib.ptr(out), _lib.ptr(ca), _lib.ptr(cb), _lib.ptr(cc),
                                  _lib.ptr(fa), _lib.ptr(fb), N, HW, C, int(act), _lib.stream())
  _lib.check(rc, "mdb_gn_cl_apply")
  return out


def _gn_params(gamma, beta):
  """(gamma, beta, is_bf16) in one dtype the fold kernels read: bf16 or fp32, contiguous."""
  ps = [p for p in (gamma, beta) if p is not None]
  if not ps:
    return None, None, 0
  bf16 = all(p.dtype == torch.bfloat16 for p in ps)
  conv = (lambda p: p.contiguous()) if bf16 else (lambda p: p.float().contiguous())
  return (None if gamma is None else conv(gamma)), (None if beta is None else conv(beta)), int(bf16)


def group_norm_cl_fwd(x3: torch.Tensor, groups: int, gamma, beta, eps: float, act: bool):
  """x3 [N, HW, C] bf16 contiguous -> (y, a, b, mean, rstd): y = act(x * a + b) with a, b fp32 [N, C]. Three launches:
  per-channel sums, the fold to coefficients (one CTA per sample), the apply pass."""
  N, HW, C = x3.shape
  partial = _gn_partial(x3)
  a = torch.empty((N, C), device=x3.device, dtype=torch.float32)
  b = torch.empty_like(a)
  mean = torch.empty((N, groups), device=x3.device, dtype=torch.float32)
  rstd = torch.empty_like(mean)
  g, bt, bf16 = _gn_params(gamma, beta)
  rc = _lib.lib().mdb_gn_cl_fold_fwd(_lib.ptr(partial), N, partial.shape[1], C, groups, float(HW * (C // groups)), float(eps),
                                     _lib.ptr(g), _lib.ptr(bt), bf16, _lib.ptr(a), _lib.ptr(b), _lib.ptr(mean), _lib.ptr(rstd),
                                     _lib.stream())
  _lib.check(rc, "mdb_gn_cl_fold_fwd")
  return _gn_apply(x3, None, a, b, None, None, None, act), a, b, mean, rstd


def group_norm_cl_bwd(dy3, x3, groups: int, gamma, a, b, mean, rstd, act: bool):
  """Returns (dx, dgamma fp32 [C], dbeta fp32 [C]) for y = act(groupnorm(x) * gamma + beta)."""
  N, HW, C = x3.shape
  partial = _gn_partial(x3, dy3, a if act else None, b if act else None)   # per channel: sum dy', sum dy' * x
  ca = torch.empty((N, C), device=x3.device, dtype=torch.float32)
  cb, cc, dg, db = (torch.empty_like(ca) for _ in range(4))
  g, _, bf16 = _gn_params(gamma, None)
  rc = _lib.lib().mdb_gn_cl_fold_bwd(_lib.ptr(partial), N, partial.shape[1], C, groups, float(HW * (C // groups)), _lib.ptr(g),
                                     bf16, _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(ca), _lib.ptr(cb), _lib.ptr(cc),
                                     _lib.ptr(dg), _lib.ptr(db), _lib.stream())
  _lib.check(rc, "mdb_gn_cl_fold_bwd")
  dx = _gn_apply(x3, dy3, ca, cb, cc, a if act else None, b if act else None, False)
  return dx, dg.sum(dim=0), db.sum(dim=0)


# ---------------------------------------------------------------------------------------------
# References (fp32, PyTorch) with the same channels-last signatures: the oracle of the tests and the CPU path.
# ---------------------------------------------------------------------------------------------
def ref_conv3d_causal(x, weight, bias=None, hist=None, residual=None, silu=False):
  xf = x.float().permute(0, 4, 1, 2, 3)
  kt, kh, kw = weight.shape[2:]
  if hist is not None and kt > 1:
    xf = torch.cat([hist.float().permute(0, 4, 1, 2, 3)[:, :, -(kt - 1):], xf], dim=2)
    xf = F.pad(xf, (kw // 2, kw // 2, kh // 2, kh // 2, 0, 0))
  else:
    xf = F.pad(xf, (kw // 2, kw // 2, kh // 2, kh // 2, kt - 1, 0))
  y = F.conv3d(xf, weight.float(), None if bias is None else bias.float())
  if silu:
    y = F.silu(y)
  y = y.permute(0, 2, 3, 4, 1)
  return y + residual.float() if residual is not None else y


def ref_conv2d(x, weight, bias=None, stride=1, pad_top_left=None, residual=None, silu=False):
  kh = weight.shape[2]
  p = kh // 2 if pad_top_left is None else pad_top_left
  xf = x.float().permute(0, 3, 1, 2)
  H, W = xf.shape[2:]
  Ho, Wo = (H, W) if stride == 1 else (H // 2, W // 2)
  far_h = (Ho - 1) * stride + kh - H - p
  far_w = (Wo - 1) * stride + kh - W - p
  xf = F.pad(xf, (p, max(far_w, 0), p, max(far_h, 0)))
  y = F.conv2d(xf, weight.float(), None if bias is None else bias.float(), stride=stride)[:, :, :Ho, :Wo]
  if silu:
    y = F.silu(y)
  y = y.permute(0, 2, 3, 1)
  return y + residual.float() if residual is not None else y


def ref_upsample2x_conv2d(x, weight, bias=None):
  xf = F.interpolate(x.float().permute(0, 3, 1, 2), scale_factor=2.0, mode="nearest")
  return F.conv2d(xf, weight.float(), None if bias is None else bias.float(), padding=1).permute(0, 2, 3, 1)
