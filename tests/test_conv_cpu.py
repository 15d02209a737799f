"""The tap tables, tensor views, weight packing and output addressing that `ops/conv.py` hands to the implicit-GEMM
kernel, checked on the CPU: an emulator executes the launch description literally (5-D array with zero fill outside,
box of output positions, per-tap coordinate shifts, K ranges of the packed weight matrix, strided output with class
offsets) and the result must equal PyTorch's convolution."""
import itertools

import pytest
import torch

from maxdiffusion_b200.ops import conv as OC


def _emulate(x, x_alt, pk, dims, strides, alt_dims, alt_strides, box, ext, out, out_strides, class_off, residual, silu,
             alt_dim=-1, alt_shift=0, tap_shift1=0):
  assert box[0] * box[1] * box[2] == 128

  def view5(t, d, s):
    return torch.as_strided(t, (d[4], d[3], d[2], d[1], d[0]), (s[3], s[2], s[1], s[0], 1), t.storage_offset()).float()

  main = view5(x, dims, strides)
  alt = view5(x_alt, alt_dims, alt_strides) if x_alt is not None else None
  C = pk.c_in
  w = pk.w.float()
  flat_out = torch.as_strided(out, (out.untyped_storage().nbytes() // 2,), (1,), 0)
  flat_res = None if residual is None else torch.as_strided(residual, (residual.untyped_storage().nbytes() // 2,), (1,), 0)
  e1, e2, e3, e4 = ext

  def fetch(arr, c4, c3, c2, c1, c0):
    d = arr.shape
    if not (0 <= c4 < d[0] and 0 <= c3 < d[1] and 0 <= c2 < d[2] and 0 <= c1 < d[3]):
      return torch.zeros(C)
    v = torch.zeros(C)
    lo, hi = max(c0, 0), min(c0 + C, d[4])
    if hi > lo:
      v[lo - c0:hi - c0] = arr[c4, c3, c2, c1, lo:hi]
    return v

  k = 0
  for cls, taps in enumerate(pk.taps):
    acc = torch.zeros(e4, e3, e2, e1, pk.n_pad)
    for (o0, o1, o2, o3, o4) in taps:
      wk = w[:, k * pk.c_pad:k * pk.c_pad + C]
      k += 1
      for p4, p3, p2, p1 in itertools.product(range(e4), range(e3), range(e2), range(e1)):
        c1, c2, c3, c4 = p1 + o1 + tap_shift1, p2 + o2, p3 + o3, p4 + o4
        arr = main
        if alt is not None and alt_dim == 3 and c3 < 0:
          # the kernel decides per TILE (box3 == 1 along the history axis), which is per position here
          c3 += alt_shift
          arr = alt
        acc[p4, p3, p2, p1] += wk @ fetch(arr, c4, c3, c2, c1, o0)
    if pk.bias is not None:
      acc += pk.bias.float()
    if silu:
      acc = torch.nn.functional.silu(acc)
    for p4, p3, p2, p1 in itertools.product(range(e4), range(e3), range(e2), range(e1)):
      off = p4 * out_strides[3] + p3 * out_strides[2] + p2 * out_strides[1] + p1 * out_strides[0] + class_off[cls]
      v = acc[p4, p3, p2, p1]
      if flat_res is not None:
        v = v + flat_res[off:off + pk.n_pad].float()
      flat_out[off:off + pk.n_pad] = v.to(out.dtype)
  return out


@pytest.fixture
def emulated(monkeypatch):
  monkeypatch.setattr(OC, "_launch", _emulate)
  monkeypatch.setattr(OC, "_check_cl", lambda x, c: None)
  monkeypatch.setattr(OC, "use_kernel", lambda x: True)  # CPU tensors take the kernel path, into the emulator


def _rand(shape, seed, scale=1.0):
  return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).to(torch.bfloat16)


def _close(got, want):
  assert got.shape == want.shape
  assert (got.float() - want.float()).abs().max() <= 2e-2 * (want.float().abs().max() + 1e-6)


@pytest.mark.parametrize("with_hist", [False, True])
def test_conv3d_description(emulated, with_hist):
  x = _rand((1, 2, 3, 5, 16), 1)
  w = _rand((8, 16, 3, 3, 3), 2, 0.1)
  b = _rand((8,), 3)
  hist = _rand((1, 2, 3, 5, 16), 4) if with_hist else None
  res = _rand((1, 2, 3, 5, 8), 5)
  _close(OC.conv3d_causal(x, OC.pack_conv3d(w, b), hist=hist, residual=res),
         OC.ref_conv3d_causal(x, w, b, hist=hist, residual=res))
  wt = _rand((8, 16, 3, 1, 1), 6, 0.2)
  _close(OC.conv3d_causal(x, OC.pack_conv3d(wt, None), hist=hist), OC.ref_conv3d_causal(x, wt, None, hist=hist))


def test_conv2d_descriptions(emulated):
  x = _rand((2, 4, 6, 16), 1)
  w = _rand((8, 16, 3, 3), 2, 0.1)
  b = _rand((8,), 3)
  _close(OC.conv2d(x, OC.pack_conv2d(w, b), silu=True), OC.ref_conv2d(x, w, b, silu=True))
  w1 = _rand((8, 16, 1, 1), 4, 0.3)
  _close(OC.conv2d(x, OC.pack_conv2d(w1, b)), OC.ref_conv2d(x, w1, b))
  for pad in (0, 1):
    got = OC.conv2d(x, OC.pack_conv2d(w, b, stride=2, pad_top_left=pad))
    _close(got, OC.ref_conv2d(x, w, b, stride=2, pad_top_left=pad))
  # channel counts that need padding: 12 input channels ride as 16, 3 output channels as 8
  x12 = _rand((1, 4, 4, 12), 5)
  w12 = _rand((3, 12, 3, 3), 6, 0.1)
  pk = OC.pack_conv2d(w12, None)
  assert pk.c_in == 16 and pk.n_pad == 8 and pk.n_out == 3
  _close(OC.conv2d(OC.pad_channels(x12, 16), pk), OC.ref_conv2d(x12, w12))


def test_upsample_conv_description(emulated):
  x = _rand((1, 3, 4, 16), 1)
  w = _rand((8, 16, 3, 3), 2, 0.1)
  b = _rand((8,), 3)
  _close(OC.upsample2x_conv2d(x, OC.pack_upsample_conv2d(w, b)), OC.ref_upsample2x_conv2d(x, w, b))


@pytest.mark.parametrize("stride,pad", [(1, 1), (2, 1), (2, 0)])
def test_dgrad_description(emulated, stride, pad):
  x = _rand((1, 6, 8, 16), 1).float().requires_grad_(True)
  w = _rand((8, 16, 3, 3), 2, 0.1)
  y = OC.ref_conv2d(x, w, None, stride=stride, pad_top_left=pad)
  dy = _rand(tuple(y.shape), 3)
  (y * dy.float()).sum().backward()
  _close(OC.conv2d_dgrad(dy, OC.pack_conv2d_dgrad(w, stride=stride, pad_top_left=pad)), x.grad)


def test_halo_columns_are_read_and_produce_no_output(emulated):
  """Width-sharded tensors: the middle shard of a wide tensor, extended by its neighbours' edge columns, gives exactly
  the middle columns of the unsharded convolution (causal conv3d with history, and the fused up-sampling conv)."""
  x = _rand((1, 2, 3, 9, 16), 1)
  hist = _rand((1, 2, 3, 9, 16), 2)
  w = _rand((8, 16, 3, 3, 3), 3, 0.1)
  pk = OC.pack_conv3d(w, None)
  whole = OC.ref_conv3d_causal(x, w, None, hist=hist)
  got = OC.conv3d_causal(x[:, :, :, 2:7].contiguous(), pk, hist=hist[:, :, :, 2:7].contiguous(), halo=1)
  _close(got, whole[:, :, :, 3:6])
  x2 = _rand((2, 3, 9, 16), 4)
  w2 = _rand((8, 16, 3, 3), 5, 0.1)
  whole2 = OC.ref_upsample2x_conv2d(x2, w2, None)
  got2 = OC.upsample2x_conv2d(x2[:, :, 2:7].contiguous(), OC.pack_upsample_conv2d(w2, None), halo=1)
  _close(got2, whole2[:, :, 6:12])


def test_box_choice_covers_with_least_padding():
  assert OC._pick_box(160, 90, 1, False) == (32, 4, 1)
  assert OC._pick_box(1280, 720, 1, False)[0] * OC._pick_box(1280, 720, 1, False)[1] == 128
  b = OC._pick_box(8, 8, 4, True)
  assert b == (8, 8, 2)
  assert OC._pick_box(8, 8, 4, False)[2] == 1


def _emulate_wgrad(dyp, xp, offs, splits):
  """The wgrad kernel's contract, literally: rows of xp outside [0, rows) are zeros; K is cut into `splits` ranges of
  64-row blocks."""
  rows = dyp.shape[0]
  kb = (rows + 63) // 64
  per = (kb + splits - 1) // splits
  out = torch.zeros((len(offs), splits, dyp.shape[1], xp.shape[1]))
  for t, off in enumerate(offs):
    idx = torch.arange(rows) + off
    ok = (idx >= 0) & (idx < xp.shape[0])
    shifted = torch.zeros((rows, xp.shape[1]))
    shifted[ok] = xp[idx[ok]].float()
    for s_ in range(splits):
      r0, r1 = min(rows, s_ * per * 64), min(rows, (s_ + 1) * per * 64)
      out[t, s_] = dyp[r0:r1].float().t() @ shifted[r0:r1]
  return out


def _emulate_wgrad_boxed(dy, x, taps, box, stride, splits):
  """The boxed kernel's contract, literally: K block kb is a BW x BH box of output pixels of one image; dy is read at
  the box, x at the box moved by the tap on its [B, H / s, s (row parity), W / s, s * C] view, out-of-range coordinates
  of either tensor read as zeros; K blocks are cut into `splits` consecutive ranges."""
  bw, bh = box
  B, Ho, Wo, M = dy.shape
  _, H, W, N = x.shape
  s = stride
  xv = x.float().reshape(B, H // s, s, W // s, s * N)
  n_wb, n_hb = -(-Wo // bw), -(-Ho // bh)
  kb_total = B * n_hb * n_wb
  per = -(-kb_total // splits)
  out = torch.zeros((len(taps), splits, M, N))
  for t, (pw, dw, ph, dh) in enumerate(taps):
    for kb in range(kb_total):
      wb, rest = kb % n_wb, kb // n_wb
      hb, img = rest % n_hb, rest // n_hb
      a = torch.zeros((bh, bw, M))
      b = torch.zeros((bh, bw, N))
      for i in range(bh):
        for j in range(bw):
          h, w = hb * bh + i, wb * bw + j
          if h < Ho and w < Wo:
            a[i, j] = dy[img, h, w].float()
          hx, wx = h + dh, w + dw
          if 0 <= hx < H // s and 0 <= wx < W // s:
            b[i, j] = xv[img, hx, ph, wx, pw * N:(pw + 1) * N]
      out[t, kb // per] += a.reshape(-1, M).t() @ b.reshape(-1, N)
  return out


@pytest.mark.parametrize("stride,pad", [(1, 1), (2, 1), (2, 0)])
@pytest.mark.parametrize("boxed", [False, True])
def test_wgrad_description(monkeypatch, stride, pad, boxed):
  monkeypatch.setattr(OC, "_wgrad_launch", _emulate_wgrad)
  monkeypatch.setattr(OC, "_wgrad_launch_boxed", _emulate_wgrad_boxed)
  monkeypatch.setattr(OC, "use_kernel", lambda x: True)
  x = _rand((2, 6, 8, 16), 1).float().requires_grad_(False)
  w = _rand((8, 16, 3, 3), 2, 0.1).float().requires_grad_(True)
  y = OC.ref_conv2d(x, w, None, stride=stride, pad_top_left=pad)
  dy = _rand(tuple(y.shape), 3)
  (y * dy.float()).sum().backward()
  got = OC.conv2d_wgrad(x.to(torch.bfloat16), dy, 3, stride, pad, boxed=boxed)
  assert got.shape == w.shape
  assert (got - w.grad).abs().max() <= 2e-2 * w.grad.abs().max()


def test_wgrad_box_and_split_choices():
  assert OC.wgrad_box(128, 128) == (64, 1) and OC.wgrad_box(32, 32) == (32, 2) and OC.wgrad_box(16, 16) == (16, 4)
  assert OC.wgrad_box(8, 8) == (8, 8) and OC.wgrad_box(20, 20)[0] in (32, 16, 8)
  # 1280 -> 1280 channels at 32^2, batch 8: 450 work items leave the last of 4 rounds a quarter full; splitting K evens it out
  assert OC.wgrad_splits(450, 128, 9 * 1280 * 1280) >= 1
  assert OC.wgrad_splits(135, 512, 9 * 640 * 640) == 1  # 135 items already fill 148 SMs to 91 %
  assert OC.wgrad_splits(27, 2048, 9 * 320 * 320) >= 4  # 27 items on 148 SMs: split K five ways
  assert OC.wgrad_taps_boxed(3, 1, 1)[0] == (0, -1, 0, -1) and OC.wgrad_taps_boxed(3, 2, 1)[0] == (1, -1, 1, -1)
  assert OC.wgrad_taps_boxed(3, 2, 0)[4] == (1, 0, 1, 0)


def test_cpu_reference_paths_of_the_conv_ops():
  """Without a GPU the ops run PyTorch convolutions; dgrad and wgrad must then equal autograd."""
  for stride, pad in ((1, 1), (2, 1), (2, 0)):
    x = _rand((1, 6, 8, 16), 1).float().requires_grad_(True)
    w = _rand((8, 16, 3, 3), 2, 0.1).float().requires_grad_(True)
    y = OC.ref_conv2d(x, w, None, stride=stride, pad_top_left=pad)
    dy = torch.randn(y.shape)
    (y * dy).sum().backward()
    _close(OC.conv2d_dgrad(dy, OC.pack_conv2d_dgrad(w.detach(), stride=stride, pad_top_left=pad)), x.grad)
    got = OC.conv2d_wgrad(x.detach(), dy, 3, stride, pad)
    assert (got - w.grad).abs().max() <= 1e-4 * (1 + w.grad.abs().max())
