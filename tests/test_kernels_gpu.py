"""Numerics of every hand-written CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

from maxdiffusion_b200.ops import _lib, kernels as K, ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
  a, b = a.float(), b.float()
  return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _report(name, out, want, rel_tol=6e-3, abs_frac=3e-2):
  rel = _rel(out, want)
  err = (out.float() - want.float()).abs()
  mx = err.max().item()
  scale = want.float().abs().max().item()
  bad = (err > abs_frac * scale).nonzero()
  msg = f"{name}: rel={rel:.3e} max_abs={mx:.3e} ref_max={scale:.3e} bad={bad.shape[0]} first_bad={bad[:4].tolist()}"
  print(msg)
  assert math.isfinite(rel) and rel < rel_tol and mx <= abs_frac * scale, msg
  _lib.raise_on_device_status()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,Kd", [(128, 256, 64), (256, 512, 256), (304, 264, 136), (1000, 1536, 1024)])
def test_gemm_layouts(M, N, Kd, a_mn, b_mn):
  torch.manual_seed(0)
  a = torch.randn((Kd, M) if a_mn else (M, Kd), device=DEV, dtype=torch.bfloat16)
  b = torch.randn((Kd, N) if b_mn else (N, Kd), device=DEV, dtype=torch.bfloat16)
  out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
  want = ref.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
  _report(f"gemm {M}x{N}x{Kd} a_mn={a_mn} b_mn={b_mn}", out, want)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,Kd", [(304, 264, 136), (1000, 1536, 1024), (4095, 5120, 512)])
def test_gemm_narrow_tile(M, N, Kd, a_mn, b_mn):
  """The optional 128-wide tile against fp32, all operand layouts."""
  torch.manual_seed(1)
  if a_mn:
    M -= M % 8  # a transposed A has leading dimension M, which the operand loads need as a multiple of 8
  a = torch.randn((Kd, M) if a_mn else (M, Kd), device=DEV, dtype=torch.bfloat16)
  b = torch.randn((Kd, N) if b_mn else (N, Kd), device=DEV, dtype=torch.bfloat16)
  want = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
  K.gemm_force_tile_n(128)
  try:
    out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
  finally:
    K.gemm_force_tile_n(0)
  _report(f"gemm narrow tile {M}x{N}x{Kd} a_mn={a_mn} b_mn={b_mn}", out, want)
  wide = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
  _report(f"gemm default tile {M}x{N}x{Kd}", wide, want)


@pytest.mark.parametrize("epi", ["none", "gelu_tanh", "silu", "gated_res", "add_res"])
@pytest.mark.parametrize("f32", [False, True])
def test_gemm_epilogues(epi, f32):
  torch.manual_seed(1)
  B, S, N, Kd = 2, 200, 520, 320
  M = B * S
  a = torch.randn((M, Kd), device=DEV, dtype=torch.bfloat16)
  b = torch.randn((N, Kd), device=DEV, dtype=torch.bfloat16) * 0.05
  bias = torch.randn((N,), device=DEV, dtype=torch.bfloat16)
  res = torch.randn((M, N), device=DEV, dtype=torch.bfloat16)
  gate = torch.randn((B, N), device=DEV, dtype=torch.float32)
  kw = dict(bias=bias, epi=epi, residual=res if epi in ("gated_res", "add_res") else None,
            gate=gate if epi == "gated_res" else None, rows_per_batch=S, alpha=0.5)
  out = K.gemm(a, b, out_dtype=torch.float32 if f32 else torch.bfloat16, **kw)
  want = ref.gemm(a, b, out_dtype=torch.float32, **kw)
  _report(f"gemm epi={epi} f32={f32}", out, want)


def test_gemm_large_persistent():
  torch.manual_seed(2)
  M, N, Kd = 4095, 5120, 5120
  a = torch.randn((M, Kd), device=DEV, dtype=torch.bfloat16)
  b = torch.randn((N, Kd), device=DEV, dtype=torch.bfloat16) * 0.02
  out = K.gemm(a, b)
  want = (a.float() @ b.float().t())
  _report("gemm 4095x5120x5120", out, want)


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("B,H,Sq,Skv", [(1, 2, 128, 128), (1, 2, 256, 384), (2, 3, 300, 200), (1, 4, 1000, 1111),
                                         (1, 2, 77, 512)])
def test_flash_fwd(B, H, Sq, Skv, D):
  torch.manual_seed(3)
  q = torch.randn((B, Sq, H, D), device=DEV, dtype=torch.bfloat16)
  k = torch.randn((B, Skv, H, D), device=DEV, dtype=torch.bfloat16)
  v = torch.randn((B, Skv, H, D), device=DEV, dtype=torch.bfloat16)
  out, lse = K.flash_fwd(q, k, v)
  want, want_lse = ref.attention(q, k, v, return_lse=True)
  _report(f"flash_fwd D{D} B{B} H{H} Sq{Sq} Skv{Skv}", out, want.float(), rel_tol=2e-2, abs_frac=5e-2)
  assert (lse - want_lse).abs().max().item() < 2e-2


def test_flash_fwd_segments_and_strided():
  """KV given as three segments (ring hops) inside a fused [B,S,3,H,D] projection buffer."""
  torch.manual_seed(4)
  B, H, Sq = 1, 4, 520
  qkv = torch.randn((B, Sq, 3, H, 128), device=DEV, dtype=torch.bfloat16)
  q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
  others = [torch.randn((B, Sq, 3, H, 128), device=DEV, dtype=torch.bfloat16) for _ in range(2)]
  k_list = [k] + [o[:, :333, 1] for o in others]
  v_list = [v] + [o[:, :333, 2] for o in others]
  out, lse = K.flash_fwd(q, k_list, v_list)
  want, want_lse = ref.attention(q, k_list, v_list, return_lse=True)
  _report("flash_fwd 3 segments strided", out, want.float(), rel_tol=2e-2, abs_frac=5e-2)
  assert (lse - want_lse).abs().max().item() < 2e-2


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("B,H,Sq,Skv", [(1, 4, 256, 384), (2, 3, 300, 200), (1, 4, 1000, 1111)])
def test_flash_fwd_fixed_m(B, H, Sq, Skv, D):
  """Fixed-exponent softmax on the eligible heads, running maximum on a head over the gate, in one launch: same
  output and log-sum-exp as the plain kernel and the fp32 reference; gradients flow through the saved lse."""
  from maxdiffusion_b200.ops import fixed_m as FM
  from maxdiffusion_b200.ops import functional as OF

  torch.manual_seed(13)
  q = torch.randn((B, Sq, H, D), device=DEV, dtype=torch.bfloat16)
  k = torch.randn((B, Skv, H, D), device=DEV, dtype=torch.bfloat16) + 0.25
  v = torch.randn((B, Skv, H, D), device=DEV, dtype=torch.bfloat16)
  q[:, :, H - 1] *= 40.0  # a "sink" head whose bound exceeds the gate
  ks = FM.smooth_keys(k)
  plan = FM.plan(q, ks)
  assert plan[1].tolist() == [1] * (H - 1) + [0]
  out, lse = K.flash_fwd(q, ks, v, fixed_m=plan)
  base, base_lse = K.flash_fwd(q, ks, v)
  # the oracle sees the same (bf16-rounded) smoothed keys: the sink head's huge logits would amplify the rounding
  # difference between k and k - mean(k); that smoothing leaves the softmax unchanged is checked in fp32 on the CPU
  want = ref.attention(q, ks, v)
  _report(f"flash_fwd fixed-m D{D} B{B} H{H} Sq{Sq} Skv{Skv}", out, want.float(), rel_tol=2e-2, abs_frac=5e-2)
  assert (out.float() - base.float()).abs().max().item() < 2e-2
  assert (lse - base_lse).abs().max().item() < 2e-2
  # two unsmoothed segments with the halved gate (the ring form)
  cut = Skv // 3
  plan2 = FM.plan(q, [k[:, :cut], k[:, cut:]], smoothed=False)
  out2, _ = K.flash_fwd(q, [k[:, :cut], k[:, cut:]], [v[:, :cut], v[:, cut:]], fixed_m=plan2)
  _report("flash_fwd fixed-m, two unsmoothed segments", out2, ref.attention(q, k, v).float(), rel_tol=2e-2,
          abs_frac=5e-2)
  # autograd through functional.attention: the backward kernels only need the true lse
  qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, ks, v))
  OF.attention(qg, kg, vg, fixed_m=plan).float().square().sum().backward()
  qb, kb, vb = (t.clone().requires_grad_(True) for t in (q, ks, v))
  OF.attention(qb, kb, vb).float().square().sum().backward()
  for a, b in ((qg, qb), (kg, kb), (vg, vb)):
    scale = b.grad.float().abs().max().item() + 1e-6
    assert (a.grad.float() - b.grad.float()).abs().max().item() <= 3e-2 * scale


@pytest.mark.parametrize("D", [128, 64])
def test_attention_keep_mask_compacts_keys_for_the_flash_kernel(D):
  """[B,Skv] keep-mask: prefix-, suffix- and scattered-dropped keys, one row fully kept; forward and gradients
  against fp32 masked softmax."""
  from maxdiffusion_b200.ops import functional as OF

  torch.manual_seed(17)
  B, H, Sq, Skv = 3, 4, 200, 333
  q, k, v = (torch.randn((B, S, H, D), device=DEV, dtype=torch.bfloat16, requires_grad=True) for S in (Sq, Skv, Skv))
  keep = torch.ones((B, Skv), device=DEV, dtype=torch.bool)
  keep[0, 250:] = False
  keep[0, :9] = False
  keep[1, ::3] = False
  out = OF.attention(q, k, v, keep_mask=keep)
  qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
  s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) / D ** 0.5
  s = s.masked_fill(~keep[:, None, None, :], float("-inf"))
  want = torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), vf)
  _report(f"attention keep-mask D{D}", out, want, rel_tol=2e-2, abs_frac=5e-2)
  g = torch.randn_like(out)
  out.backward(g)
  want.backward(g.float())
  for got, ref_t in ((q, qf), (k, kf), (v, vf)):
    scale = ref_t.grad.abs().max().item() + 1e-6
    assert (got.grad.float() - ref_t.grad).abs().max().item() <= 4e-2 * scale
  assert k.grad[0, 250:].abs().max().item() == 0.0  # dropped keys receive no gradient


@pytest.mark.parametrize("D", [40, 80, 96])
def test_attention_other_head_sizes_ride_the_padded_kernel(D):
  from maxdiffusion_b200.ops import functional as OF

  torch.manual_seed(19)
  B, H, Sq, Skv = 2, 5, 260, 77
  q, k, v = (torch.randn((B, S, H, D), device=DEV, dtype=torch.bfloat16, requires_grad=True) for S in (Sq, Skv, Skv))
  before = _lib.launch_count()
  out = OF.attention(q, k, v)
  assert _lib.launch_count() > before and out.shape == (B, Sq, H, D)
  want = ref.attention(q.detach(), k.detach(), v.detach())
  _report(f"attention head_dim {D} (padded)", out, want.float(), rel_tol=2e-2, abs_frac=5e-2)
  out.float().square().sum().backward()
  assert q.grad.shape == q.shape and torch.isfinite(q.grad.float()).all() and k.grad.abs().max() > 0


def test_flash_fwd_large_magnitude():
  """Scores with a large dynamic range exercise the lazy rescale path."""
  torch.manual_seed(5)
  B, H, S = 1, 2, 640
  q = torch.randn((B, S, H, 128), device=DEV, dtype=torch.bfloat16) * 4
  k = torch.randn((B, S, H, 128), device=DEV, dtype=torch.bfloat16) * 4
  k[:, 400:] *= 3
  v = torch.randn((B, S, H, 128), device=DEV, dtype=torch.bfloat16)
  out, _ = K.flash_fwd(q, k, v)
  want = ref.attention(q, k, v)
  _report("flash_fwd large magnitude", out, want.float(), rel_tol=2e-2, abs_frac=5e-2)


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("B,H,Sq,Skv", [(1, 2, 128, 128), (1, 2, 256, 192), (2, 3, 300, 200), (1, 2, 1000, 1111),
                                         (1, 2, 77, 512)])
def test_flash_bwd(B, H, Sq, Skv, D):
  torch.manual_seed(11)
  q = torch.randn((B, Sq, H, D), device=DEV, dtype=torch.bfloat16)
  k = torch.randn((B, Skv, H, D), device=DEV, dtype=torch.bfloat16)
  v = torch.randn((B, Skv, H, D), device=DEV, dtype=torch.bfloat16)
  d_o = torch.randn((B, Sq, H, D), device=DEV, dtype=torch.bfloat16)
  out, lse = K.flash_fwd(q, k, v)
  delta = K.flash_delta(out, d_o)
  _report("flash_delta", delta, (out.float() * d_o.float()).sum(-1).permute(0, 2, 1), rel_tol=1e-3)
  dk, dv = K.flash_bwd_dkv(q, d_o, k, v, lse, delta)
  dq = K.flash_bwd_dq(q, d_o, k, v, lse, delta)
  wq, wk, wv = ref.attention_bwd(q, k, v, out, d_o, lse)
  _report(f"flash_bwd dv {Sq}x{Skv}", dv, wv.float(), rel_tol=2e-2, abs_frac=5e-2)
  _report(f"flash_bwd dk {Sq}x{Skv}", dk, wk.float(), rel_tol=2e-2, abs_frac=5e-2)
  _report(f"flash_bwd dq {Sq}x{Skv}", dq, wq.float(), rel_tol=2e-2, abs_frac=5e-2)


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("B", [1, 2])
def test_flash_bwd_dkv_stacked_matches_per_segment_launches(B, D):
  """All stacked KV segments in one dK/dV launch: ring order -> owner order rotation, ragged last segment, outputs
  in slices with a foreign stride (as in a symmetric buffer), untouched rows beyond a segment's length."""
  torch.manual_seed(23)
  n, H, Sq, Skv = 3, 2, 200, 192
  lens = [192, 192, 77]
  q, d_o = (torch.randn((B, Sq, H, D), device=DEV, dtype=torch.bfloat16) for _ in range(2))
  kg = torch.randn((n, B, Skv, H, D), device=DEV, dtype=torch.bfloat16)
  vg = torch.randn((n, B, Skv, H, D), device=DEV, dtype=torch.bfloat16)
  ks = [kg[i][:, :lens[i]] for i in range(n)]
  vs = [vg[i][:, :lens[i]] for i in range(n)]
  out, lse = K.flash_fwd(q, ks, vs)
  delta = K.flash_delta(out, d_o)
  rot = 2
  cap = 2 * B * Skv * H * D + 64  # owner slices [dK | dV] with some slack between them
  buf = torch.full((n * cap,), 7.0, device=DEV, dtype=torch.bfloat16)
  both = buf.as_strided((n, 2, B, Skv, H, D), (cap, B * Skv * H * D, Skv * H * D, H * D, D, 1))
  step = n - 1  # a ring that turns backwards: segment i belongs to owner (rot - i) % n
  K.flash_bwd_dkv_stacked(q, d_o, kg, vg, lens, lse, delta, dk=both[:, 0], dv=both[:, 1], out_rot=rot, out_step=step)
  for i in range(n):
    dk, dv = K.flash_bwd_dkv(q, d_o, ks[i], vs[i], lse, delta)
    o = (rot - i) % n
    assert torch.equal(both[o, 0][:, :lens[i]], dk) and torch.equal(both[o, 1][:, :lens[i]], dv)
    if lens[i] < Skv:
      assert (both[o, 0][:, lens[i]:] == 7.0).all() and (both[o, 1][:, lens[i]:] == 7.0).all()
  # default outputs: allocated, contiguous
  dk2, dv2 = K.flash_bwd_dkv_stacked(q, d_o, kg, vg, lens, lse, delta)
  for i in range(n):  # default: segment i -> slice i
    assert torch.equal(dk2[i][:, :lens[i]], both[(rot - i) % n, 0][:, :lens[i]])


def test_flash_bwd_segments_match_concat():
  """dQ over three KV segments equals dQ over their concatenation; dK/dV per segment likewise."""
  torch.manual_seed(12)
  B, H, Sq = 1, 2, 320
  q = torch.randn((B, Sq, H, 128), device=DEV, dtype=torch.bfloat16)
  d_o = torch.randn((B, Sq, H, 128), device=DEV, dtype=torch.bfloat16)
  ks = [torch.randn((B, n, H, 128), device=DEV, dtype=torch.bfloat16) for n in (200, 200, 200)]
  vs = [torch.randn((B, n, H, 128), device=DEV, dtype=torch.bfloat16) for n in (200, 200, 200)]
  out, lse = K.flash_fwd(q, ks, vs)
  delta = K.flash_delta(out, d_o)
  dq = K.flash_bwd_dq(q, d_o, ks, vs, lse, delta)
  kc, vc = torch.cat(ks, 1), torch.cat(vs, 1)
  wq, wk, wv = ref.attention_bwd(q, kc, vc, out, d_o, lse)
  _report("flash_bwd dq segments", dq, wq.float(), rel_tol=2e-2, abs_frac=5e-2)
  dk1, dv1 = K.flash_bwd_dkv(q, d_o, ks[1], vs[1], lse, delta, out_dtype=torch.float32)
  _report("flash_bwd dk segment 1 (fp32 out)", dk1, wk[:, 200:400].float(), rel_tol=2e-2, abs_frac=5e-2)
  _report("flash_bwd dv segment 1 (fp32 out)", dv1, wv[:, 200:400].float(), rel_tol=2e-2, abs_frac=5e-2)


@pytest.mark.parametrize("C", [1536, 5120, 3072])
@pytest.mark.parametrize("mode", ["mod", "affine", "plain"])
def test_layer_norm_fwd_bwd(C, mode):
  torch.manual_seed(6)
  B, S = 2, 333
  x = torch.randn((B, S, C), device=DEV, dtype=torch.bfloat16) * 2 + 0.5
  gamma = torch.randn((C,), device=DEV, dtype=torch.bfloat16) if mode == "affine" else None
  beta = torch.randn((C,), device=DEV, dtype=torch.bfloat16) if mode == "affine" else None
  scale = torch.randn((B, C), device=DEV, dtype=torch.float32) * 0.3 if mode == "mod" else None
  shift = torch.randn((B, C), device=DEV, dtype=torch.float32) if mode == "mod" else None
  y, mean, rstd = K.ln_fwd(x, gamma, beta, scale, shift, save_stats=True)
  xr = x.float().requires_grad_(True)
  gr = gamma.float().requires_grad_(True) if gamma is not None else None
  br = beta.float().requires_grad_(True) if beta is not None else None
  sr = scale.clone().requires_grad_(True) if scale is not None else None
  hr = shift.clone().requires_grad_(True) if shift is not None else None
  want = ref.layer_norm_mod(xr, gr, br, sr, hr)
  _report(f"ln_fwd C={C} {mode}", y, want.detach(), rel_tol=5e-3)
  dy = torch.randn_like(x)
  want.backward(dy.float())
  dx, sums = K.ln_bwd(dy, x, mean, rstd, gamma, scale)
  _report(f"ln_bwd dx C={C} {mode}", dx, xr.grad, rel_tol=8e-3)
  if mode == "mod":
    _report("ln_bwd dscale", sums[:, 0], sr.grad, rel_tol=5e-3)
    _report("ln_bwd dshift", sums[:, 1], hr.grad, rel_tol=5e-3)
  if mode == "affine":
    _report("ln_bwd dgamma", sums[:, 0].sum(0), gr.grad, rel_tol=5e-3)
    _report("ln_bwd dbeta", sums[:, 1].sum(0), br.grad, rel_tol=5e-3)


@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("rope", [False, True])
def test_rms_rope_fwd_bwd(per_head, rope):
  torch.manual_seed(7)
  B, S, H = 2, 257, 12
  C = H * 128
  x = torch.randn((B, S, C), device=DEV, dtype=torch.bfloat16)
  w = (torch.randn((128 if per_head else C,), device=DEV) * 0.2 + 1).to(torch.bfloat16)
  ang = torch.rand((S, 64), device=DEV) * 6.28
  cos, sin = (ang.cos().contiguous(), ang.sin().contiguous()) if rope else (None, None)
  y, rstd = K.rms_rope_fwd(x, w, cos, sin, heads=H, per_head=per_head, save_stats=True)
  xr = x.float().requires_grad_(True)
  wr = w.float().requires_grad_(True)
  want = ref.rms_norm_rope(xr, wr, cos, sin, heads=H, per_head=per_head)
  _report(f"rms_rope_fwd per_head={per_head} rope={rope}", y, want.detach(), rel_tol=5e-3)
  dy = torch.randn_like(y)
  want.backward(dy.float())
  dx, dw = K.rms_rope_bwd(dy, x, rstd, w, cos, sin, per_head=per_head)
  _report("rms_rope_bwd dx", dx, xr.grad, rel_tol=8e-3)
  _report("rms_rope_bwd dw", dw, wr.grad, rel_tol=5e-3)


def test_gated_residual_gelu_colsum():
  torch.manual_seed(8)
  B, S, C = 2, 301, 1536
  res = torch.randn((B, S, C), device=DEV, dtype=torch.bfloat16)
  y = torch.randn((B, S, C), device=DEV, dtype=torch.bfloat16)
  gate = torch.randn((B, C), device=DEV, dtype=torch.float32)
  out = K.gated_res_fwd(res, y, gate)
  _report("gated_res_fwd", out, ref.gated_residual(res.float(), y.float(), gate), rel_tol=5e-3)
  dout = torch.randn_like(y)
  dy, dgate = K.gated_res_bwd(dout, y, gate)
  _report("gated_res_bwd dy", dy, dout.float() * gate[:, None, :], rel_tol=5e-3)
  _report("gated_res_bwd dgate", dgate, (dout.float() * y.float()).sum(1), rel_tol=5e-3)
  u = torch.randn((B, S, C), device=DEV, dtype=torch.bfloat16) * 2
  _report("gelu_fwd", K.gelu_fwd(u), ref.gelu_tanh(u.float()), rel_tol=5e-3)
  ur = u.float().requires_grad_(True)
  torch.nn.functional.gelu(ur, approximate="tanh").backward(dout.float())
  _report("gelu_bwd", K.gelu_bwd(dout, u), ur.grad, rel_tol=5e-3)
  _report("colsum", K.colsum(y.view(B * S, C)), y.float().view(B * S, C).sum(0), rel_tol=1e-4)


@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
def test_adamw_and_norms(state_dtype):
  torch.manual_seed(9)
  n = 1_000_003
  p = torch.randn((n,), device=DEV, dtype=torch.bfloat16)
  g = torch.randn((n,), device=DEV, dtype=torch.bfloat16)
  m = torch.zeros((n,), device=DEV, dtype=state_dtype)
  v = torch.zeros((n,), device=DEV, dtype=state_dtype)
  p2, m2, v2 = p.clone(), m.clone(), v.clone()
  hp = dict(lr=1e-2, b1=0.9, b2=0.999, eps=1e-8, wd=0.01)
  for step in (1, 2):
    K.adamw(p, g, m, v, step=step, stochastic=False, **hp)
    ref.adamw_step(p2, g, m2, v2, step=step, **hp)
  _report("adamw p", p, p2, rel_tol=1e-2, abs_frac=2e-2)
  _report("adamw m", m, m2, rel_tol=1e-2, abs_frac=2e-2)
  out = K.sumsq_maxabs(g)
  want = ref.sumsq_maxabs(g)
  assert abs(out[0].item() - want[0].item()) / want[0].item() < 1e-4 and out[1].item() == want[1].item()


def test_adamw_stochastic_rounding_is_unbiased():
  n = 1 << 20
  p = torch.ones((n,), device=DEV, dtype=torch.bfloat16)
  g = torch.ones((n,), device=DEV, dtype=torch.bfloat16)
  m = torch.zeros((n,), device=DEV, dtype=torch.float32)
  v = torch.zeros((n,), device=DEV, dtype=torch.float32)
  K.adamw(p, g, m, v, lr=1e-4, b1=0.9, b2=0.999, eps=1e-8, wd=0.0, step=1, seed=123, stochastic=True)
  # the exact update is 1 - 1e-4, far below the bf16 spacing (2^-8 below 1): the mean must still move by it
  assert abs((1.0 - p.float().mean().item()) - 1e-4) < 2e-5


def test_checkpoint_block_with_host_offload_matches_plain_autograd():
  from maxdiffusion_b200.ops import functional as OF

  torch.manual_seed(0)
  w = torch.randn((256, 256), device=DEV, dtype=torch.bfloat16, requires_grad=True)
  x = torch.randn((2, 128, 256), device=DEV, dtype=torch.bfloat16, requires_grad=True)
  fn = lambda t: OF.linear(t, w, None, "gelu_tanh")
  OF.checkpoint_block(fn, x, offload_input=True).float().sum().backward()
  gx, gw = x.grad.clone(), w.grad.clone()
  x.grad, w.grad = None, None
  fn(x).float().sum().backward()
  assert torch.equal(gx, x.grad) and torch.equal(gw, w.grad)


@pytest.mark.parametrize("M,N,Kd", [(128, 256, 128), (520, 264, 400), (1024, 1536, 2048)])
def test_gemm_fp8_matches_quantised_reference(M, N, Kd):
  torch.manual_seed(0)
  a = torch.randn((M, Kd), device=DEV, dtype=torch.bfloat16)
  b = torch.randn((N, Kd), device=DEV, dtype=torch.bfloat16) * 0.05
  bias = torch.randn((N,), device=DEV, dtype=torch.bfloat16)
  aq, sa = K.quantize_fp8(a)
  bq, sb = K.quantize_fp8(b)
  # the quantiser itself: bytes reinterpret as e4m3 and reproduce torch's rounding
  a_deq = aq.view(torch.float8_e4m3fn).float() * sa
  want_deq = (a.float() / sa).clamp(-448, 448).to(torch.float8_e4m3fn).float() * sa
  assert torch.equal(a_deq, want_deq) and abs(sa.item() - a.abs().max().item() / 448.0) < 1e-6
  out = K.gemm_fp8(aq, sa, bq, sb, bias)
  b_deq = bq.view(torch.float8_e4m3fn).float() * sb
  want = a_deq @ b_deq.t() + bias.float()
  _report(f"gemm_fp8 {M}x{N}x{Kd}", out, want)
  # against the unquantised product the error is the fp8 rounding error
  assert _rel(out, a.float() @ b.float().t() + bias.float()) < 8e-2


def test_fp8_linear_module_and_e5m2_backward():
  from maxdiffusion_b200.models.layers import Linear
  from maxdiffusion_b200.models.quantizations import Fp8Linear

  torch.manual_seed(0)
  base = Linear(256, 512).to(DEV, torch.bfloat16)
  x = torch.randn((4, 64, 256), device=DEV, dtype=torch.bfloat16, requires_grad=True)
  dy = torch.randn((4, 64, 512), device=DEV, dtype=torch.bfloat16)
  want = torch.nn.functional.linear(x.float(), base.weight.float(), base.bias.float())
  gx_want, gw_want = torch.autograd.grad(want, [x, base.weight], dy.float())
  for full in (False, True):
    q = Fp8Linear(base, full=full)
    y = q(x)
    gx, gw = torch.autograd.grad(y, [x, base.weight], dy)
    assert _rel(y, want) < 6e-2 and _rel(gx, gx_want) < (0.2 if full else 2e-2) and _rel(gw, gw_want) < (0.2 if full else 2e-2)
  _lib.raise_on_device_status()


def test_attention_head_dim_64_autograd_matches_reference():
  """The differentiable op on SDXL-shaped heads (d = 64) against fp32 autograd of the reference."""
  from maxdiffusion_b200.ops import functional as OF

  torch.manual_seed(21)
  B, S, H, D = 2, 1024, 10, 64
  q, k, v = (torch.randn((B, S, H, D), device=DEV, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
  g = torch.randn((B, S, H, D), device=DEV, dtype=torch.bfloat16)
  out = OF.attention(q, k, v)
  out.backward(g)
  qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
  want = ref.attention(qf, kf, vf)
  want.backward(g.float())
  _report("attention d64 out", out, want.float(), rel_tol=2e-2, abs_frac=5e-2)
  for name, a, b in (("dq", q.grad, qf.grad), ("dk", k.grad, kf.grad), ("dv", v.grad, vf.grad)):
    _report(f"attention d64 {name}", a, b, rel_tol=2e-2, abs_frac=5e-2)


def test_tile_search_choice_changes_the_launched_attention_variant():
  """A cached tile-search result for a shape makes `flash_fwd` launch that variant (K / V pipeline depth), other
  shapes keep the default, and every variant computes the same attention."""
  from maxdiffusion_b200.ops import ref

  torch.manual_seed(0)
  q = torch.randn(1, 512, 4, 128, device="cuda").to(torch.bfloat16)
  k = torch.randn(1, 640, 4, 128, device="cuda").to(torch.bfloat16)
  v = torch.randn(1, 640, 4, 128, device="cuda").to(torch.bfloat16)
  want = ref.attention(q, k, v).float()
  K._FLASH_TUNED.clear()
  K.flash_tune(0, 0)
  base, _ = K.flash_fwd(q, k, v)
  assert K.flash_last_variant()[0] == 4
  try:
    for stages in (2, 3, 5):
      K._FLASH_TUNED[K.flash_tuned_key(512, 128, 4, 1)] = (stages, 0)
      out, _ = K.flash_fwd(q, k, v)
      assert K.flash_last_variant()[0] == stages
      assert torch.equal(out, base)  # the pipeline depth does not change the arithmetic
      assert (out.float() - want).abs().max() < 2e-2
    K.flash_fwd(q[:, :256], k, v)  # no entry for this shape: back to the default variant
    assert K.flash_last_variant()[0] == 4
  finally:
    K._FLASH_TUNED.clear()
    K.flash_tune(0, 0)


@pytest.mark.parametrize("a_mn,b_mn", [(True, True), (False, False), (False, True)])
@pytest.mark.parametrize("M,N,Kd,splits", [(640, 640, 4096, 0), (320, 328, 2000, 3), (1280, 1280, 8192, 0), (136, 64, 1024, 16)])
def test_gemm_split_k_matches_fp32(a_mn, b_mn, M, N, Kd, splits):
  """The contraction cut into ranges with fp32 partials and an ordered fold (weight-gradient shapes: small output,
  long K), chosen automatically or forced, bf16 and fp32 outputs, ragged K; and bitwise equal run to run."""
  g = torch.Generator(device="cuda").manual_seed(0)
  a = (torch.randn((Kd, M) if a_mn else (M, Kd), device="cuda", generator=g) * 0.5).to(torch.bfloat16)
  b = (torch.randn((Kd, N) if b_mn else (N, Kd), device="cuda", generator=g) * 0.5).to(torch.bfloat16)
  want = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
  if splits == 0:
    assert K.split_k_for(M, N, Kd) > 1
  got = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, split_k=splits)
  got32 = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, split_k=splits, out_dtype=torch.float32)
  one = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, split_k=1, out_dtype=torch.float32)
  scale = want.abs().max().item()
  assert (got.float() - want).abs().max().item() <= 1e-2 * scale
  assert (got32 - want).abs().max().item() <= 2e-3 * scale
  assert (got32 - one).abs().max().item() <= 1e-3 * scale
  assert torch.equal(got, K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, split_k=splits))


@pytest.mark.parametrize("M,N,Kd", [(300, 328, 192), (4095, 1280, 640), (129, 8, 64), (1024, 2560, 320)])
@pytest.mark.parametrize("epi", ["none", "gelu_tanh", "add_res", "gated_res"])
@pytest.mark.parametrize("f32", [False, True])
def test_gemm_tma_store_epilogue_equals_direct_stores(M, N, Kd, epi, f32):
  """The epilogue that stages 128-byte slabs in shared memory and writes them with TMA stores against the one that
  stores from one thread per row: same values bit for bit, ragged edges in M and N, every epilogue, both output types."""
  g = torch.Generator(device="cuda").manual_seed(0)
  a = torch.randn((M, Kd), device="cuda", generator=g).to(torch.bfloat16)
  b = (torch.randn((N, Kd), device="cuda", generator=g) * 0.1).to(torch.bfloat16)
  bias = torch.randn((N,), device="cuda", generator=g).to(torch.bfloat16)
  kw = dict(bias=bias, epi=epi, out_dtype=torch.float32 if f32 else torch.bfloat16)
  if epi in ("add_res", "gated_res"):
    kw["residual"] = torch.randn((M, N), device="cuda", generator=g).to(torch.bfloat16)
  if epi == "gated_res":
    rows = 100 if M % 100 == 0 else M
    kw["gate"] = torch.randn((M // rows, N), device="cuda", generator=g)
    kw["rows_per_batch"] = rows
  try:
    K.gemm_epilogue_mode(direct=True)
    want = K.gemm(a, b, **kw)
  finally:
    K.gemm_epilogue_mode(direct=False)
  guard = torch.full((M + 2, N), 7.0, device="cuda", dtype=kw["out_dtype"])  # rows around the output stay untouched
  got = K.gemm(a, b, out=guard[1:-1], **{k: v for k, v in kw.items() if k != "out_dtype"})
  assert torch.equal(got, want)
  assert bool((guard[0] == 7).all()) and bool((guard[-1] == 7).all())
  ref32 = a.float() @ b.float().t() + bias.float()
  if epi == "none":
    assert (got.float() - ref32).abs().max() <= 2e-2 * ref32.abs().max()


@pytest.mark.parametrize("M,N,Kd", [(128, 256, 128), (520, 264, 400), (1024, 1536, 2048)])
def test_gemm_int8_is_exact_on_the_quantised_operands(M, N, Kd):
  """Integer tensor-core path: the quantiser rounds to nearest in [-127, 127]; the product of the int8 operands is
  accumulated exactly in int32, so against an int64 reference only the bf16 rounding of the output remains."""
  torch.manual_seed(0)
  a = torch.randn((M, Kd), device=DEV, dtype=torch.bfloat16)
  b = torch.randn((N, Kd), device=DEV, dtype=torch.bfloat16) * 0.05
  bias = torch.randn((N,), device=DEV, dtype=torch.bfloat16)
  aq, sa = K.quantize_int8(a)
  bq, sb = K.quantize_int8(b)
  assert aq.dtype == torch.int8 and abs(sa.item() - a.abs().max().item() / 127.0) < 1e-6
  # round to nearest of x * (127 / absmax); the reference divides by the scale instead, so exact ties may land one step apart
  assert (aq.int() - (a.float() / sa).round().clamp(-127, 127).int()).abs().max() <= 1
  assert aq.int().abs().max() == 127
  out = K.gemm_int8(aq, sa, bq, sb, bias)
  # integer products in float64 are exact at these sizes (|sum| <= 127^2 * K < 2^53)
  exact = (aq.double() @ bq.double().t()) * (sa.double() * sb.double()) + bias.double()
  assert (out.double() - exact).abs().max() <= 1e-2 * exact.abs().max()
  assert _rel(out, exact.float()) < 4e-3  # bf16 output rounding only
  assert _rel(out, a.float() @ b.float().t() + bias.float()) < 5e-2  # int8 rounding of the operands
  _lib.raise_on_device_status()


def test_int8_linear_module_forward_and_bf16_backward():
  from maxdiffusion_b200.models.layers import Linear
  from maxdiffusion_b200.models.quantizations import Int8Linear, quantize_model

  torch.manual_seed(0)
  base = Linear(256, 512).to(DEV, torch.bfloat16)
  x = torch.randn((4, 64, 256), device=DEV, dtype=torch.bfloat16, requires_grad=True)
  dy = torch.randn((4, 64, 512), device=DEV, dtype=torch.bfloat16)
  want = torch.nn.functional.linear(x.float(), base.weight.float(), base.bias.float())
  gx_want, gw_want = torch.autograd.grad(want, [x, base.weight], dy.float())
  q = Int8Linear(base)
  y = q(x)
  gx, gw = torch.autograd.grad(y, [x, base.weight], dy)
  assert _rel(y, want) < 4e-2 and _rel(gx, gx_want) < 2e-2 and _rel(gw, gw_want) < 2e-2
  holder = torch.nn.ModuleDict({"blocks": torch.nn.ModuleList([torch.nn.ModuleDict({"proj": Linear(64, 64)})])})
  assert quantize_model(holder, "int8") == 1 and isinstance(holder["blocks"][0]["proj"], Int8Linear)
  _lib.raise_on_device_status()


@pytest.mark.parametrize("C", [96, 320, 640, 1280, 2048, 2056])
@pytest.mark.parametrize("B,S", [(8, 100), (1, 1031)])
def test_affine_layer_norm_short_rows_forward_and_backward(C, B, S):
  """Plain affine LayerNorm on rows of at most 2048 channels runs a warp per row (UNet / DiT blocks); 2056 channels
  take the CTA-per-row kernels. Forward, input gradient and parameter gradients against fp32 autograd."""
  from maxdiffusion_b200.ops import functional as OF

  g = torch.Generator(device="cuda").manual_seed(C + S)
  x = (torch.randn((B, S, C), device="cuda", generator=g) * 2 + 0.5).to(torch.bfloat16).requires_grad_(True)
  gamma = (torch.rand((C,), device="cuda", generator=g) + 0.5).to(torch.bfloat16).requires_grad_(True)
  beta = (torch.randn((C,), device="cuda", generator=g) * 0.2).to(torch.bfloat16).requires_grad_(True)
  dy = torch.randn((B, S, C), device="cuda", generator=g).to(torch.bfloat16)
  y = OF.layer_norm_mod(x, gamma, beta, eps=1e-5)
  gx, gg, gb = torch.autograd.grad(y, (x, gamma, beta), dy)
  xf, gf, bf = (t.detach().float().requires_grad_(True) for t in (x, gamma, beta))
  want = torch.nn.functional.layer_norm(xf, (C,), gf, bf, 1e-5)
  wx, wg, wb = torch.autograd.grad(want, (xf, gf, bf), dy.float())
  assert _rel(y, want) < 1e-2 and _rel(gx, wx) < 1e-2
  assert _rel(gg, wg) < 2e-2 and _rel(gb, wb) < 2e-2
  y2 = OF.layer_norm_mod(x, gamma, beta, eps=1e-5)
  assert torch.equal(y, y2) and torch.equal(gx, torch.autograd.grad(y2, x, dy)[0])  # reproducible
