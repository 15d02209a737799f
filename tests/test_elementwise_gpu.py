"""GroupNorm(+SiLU) and the elementwise step kernels against plain PyTorch fp32 references."""
import pytest
import torch

from maxdiffusion_b200.ops import _lib, functional as F, kernels as K, ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(out, want, tol):
  err = (out.float() - want.float()).abs().max().item()
  scale = want.float().abs().max().item() + 1e-12
  assert err <= tol * scale, (err, scale)
  _lib.raise_on_device_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape,groups", [((2, 320, 32, 32), 32), ((1, 128, 96, 96), 32), ((2, 64, 5, 7), 8),
                                           ((1, 96, 3, 16, 16), 32)])
@pytest.mark.parametrize("act", [False, True])
def test_groupnorm_fwd_bwd(shape, groups, act, dtype):
  torch.manual_seed(0)
  C = shape[1]
  x = (torch.randn(shape, device=DEV) * 2 + 0.5).to(dtype).requires_grad_(True)
  gamma = (1 + 0.1 * torch.randn(C, device=DEV)).requires_grad_(True)
  beta = (0.1 * torch.randn(C, device=DEV)).requires_grad_(True)
  dy = torch.randn(shape, device=DEV).to(dtype)
  y = F.group_norm(x, groups, gamma, beta, 1e-5, act)
  y.backward(dy)
  got = (y.detach(), x.grad.clone(), gamma.grad.clone(), beta.grad.clone())
  x32 = x.detach().float().requires_grad_(True)
  g32, b32 = gamma.detach().clone().requires_grad_(True), beta.detach().clone().requires_grad_(True)
  yr = ref.group_norm(x32, groups, g32, b32, 1e-5, act)
  yr.backward(dy.float())
  tol = 2e-2 if dtype == torch.bfloat16 else 2e-4
  _close(got[0], yr.detach(), tol)
  _close(got[1], x32.grad, tol)
  _close(got[2], g32.grad, tol)
  _close(got[3], b32.grad, tol)


def test_lincomb_mixed_dtypes_and_sumsq():
  torch.manual_seed(1)
  a = torch.randn((2, 16, 21, 30, 52), device=DEV)
  b = torch.randn_like(a).to(torch.bfloat16)
  c = torch.randn_like(a)
  coefs = [[0.3, -1.25, 2.0], [1.0, 0.5, -0.75]]
  out, sq = K.lincomb([a, b, c], coefs, out_dtype=torch.float32, want_sumsq=True)
  want = ref.lincomb([a, b, c], coefs, torch.float32)
  _close(out, want, 1e-5)
  assert abs(sq.item() - (want ** 2).sum().item()) <= 1e-4 * (want ** 2).sum().item()
  out2 = K.lincomb([b, b], [5.0, -4.0])  # cfg combine, bf16 out
  _close(out2, b.float(), 1e-2)


def test_weighted_mse_loss_and_grad():
  torch.manual_seed(2)
  pred = torch.randn((2, 4096, 64), device=DEV, dtype=torch.bfloat16, requires_grad=True)
  target = torch.randn((2, 4096, 64), device=DEV)
  w = [0.7, 1.9]
  loss = F.weighted_mse(pred, target, w)
  loss.backward()
  p32 = pred.detach().float().requires_grad_(True)
  lr = ref.weighted_mse(p32, target, w)
  lr.backward()
  assert abs(loss.item() - lr.item()) <= 1e-4 * abs(lr.item())
  _close(pred.grad, p32.grad, 1e-2)


def test_channel_affine_uint8_blend():
  torch.manual_seed(3)
  x = torch.randn((1, 16, 5, 30, 52), device=DEV)
  mean, std = torch.randn(16), torch.rand(16) + 0.5
  y = K.channel_affine(x, mean, 1.0 / std, 1)
  _close(y, ref.channel_affine(x, mean, 1.0 / std, 1), 1e-5)
  z = K.channel_affine(y, mean, std, 1, denorm=True)
  _close(z, x, 1e-4)
  v = torch.randn((2, 3, 8, 64, 64), device=DEV, dtype=torch.bfloat16)
  u = K.to_uint8(v)
  assert (u.int() - ref.to_uint8(v).int()).abs().max().item() <= 1
  a = torch.randn((2, 4, 16, 32), device=DEV)
  b = torch.randn((2, 4, 16, 32), device=DEV)
  for dim in (2, 3):
    _close(K.blend_ramp(a, b, dim), ref.blend_ramp(a, b, dim), 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L", [50, 256, 1000])
def test_fused_antialiased_snake_matches_separable_path(L, dtype):
  from maxdiffusion_b200.models.ltx2.vocoder_ltx2 import AntiAliasAct1d, SnakeBeta

  torch.manual_seed(0)
  act = AntiAliasAct1d(SnakeBeta(6)).to(DEV)
  with torch.no_grad():
    act.act.alpha.copy_(torch.randn(6) * 0.3)
    act.act.beta.copy_(torch.randn(6) * 0.3)
  x = torch.randn((2, 6, L), device=DEV).to(dtype)
  got = act(x)
  want = act.downsample(act.act(act.upsample(x.float())))
  _close(got, want, 2e-2 if dtype == torch.bfloat16 else 2e-5)
  leaky = AntiAliasAct1d(torch.nn.LeakyReLU(0.1)).to(DEV)
  _close(leaky(x), leaky.downsample(leaky.act(leaky.upsample(x.float()))), 2e-2 if dtype == torch.bfloat16 else 2e-5)


@pytest.mark.parametrize("shape", [(1, 16, 5, 90, 160), (2, 4, 2, 45, 80), (1, 2, 1, 31, 53)])
def test_band_filter_gemms_on_the_tensor_cores_match_the_fft_form(shape):
  """CFG-cache compensation through the tcgen05 GEMM (split-bf16 operands) against torch.fft in fp32."""
  from maxdiffusion_b200.pipelines.wan import cache_policies as CP

  torch.manual_seed(0)
  a, b, c = (torch.randn(shape, device=DEV) for _ in range(3))
  for w1, w2 in ((1.2, 1.0), (1.0, 1.2)):
    got = CP.fft_compensate(a, b, c, w1, w2)
    want = CP.fft_compensate_reference(a, b, c, w1, w2)
    _close(got, want, 2e-4)


@pytest.mark.parametrize("rows,inner", [(37, 64), (4096, 2560), (3, 5120)])
def test_geglu_forward_and_backward_match_fp32(rows, inner):
  from maxdiffusion_b200.ops import functional as OF

  g = torch.Generator(device="cuda").manual_seed(0)
  u = torch.randn((2, rows, 2 * inner), device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True)
  dy = torch.randn((2, rows, inner), device="cuda", generator=g).to(torch.bfloat16)
  y = OF.geglu(u)
  (du,) = torch.autograd.grad(y, u, dy)
  uf = u.detach().float().requires_grad_(True)
  h, gate = uf.chunk(2, dim=-1)
  want = h * torch.nn.functional.gelu(gate)
  (dwant,) = torch.autograd.grad(want, uf, dy.float())
  assert (y.float() - want).abs().max() <= 2e-2 * (1 + want.abs().max())
  assert (du.float() - dwant).abs().max() <= 2e-2 * (1 + dwant.abs().max())


def test_linear_with_residual_in_the_epilogue_matches_fp32_forward_and_backward():
  from maxdiffusion_b200.ops import functional as OF

  g = torch.Generator(device="cuda").manual_seed(1)
  x = torch.randn((2, 300, 640), device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True)
  r = torch.randn((2, 300, 320), device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True)
  w = (torch.randn((320, 640), device="cuda", generator=g) * 0.04).to(torch.bfloat16).requires_grad_(True)
  b = torch.randn((320,), device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True)
  dy = torch.randn((2, 300, 320), device="cuda", generator=g).to(torch.bfloat16)
  y = OF.linear(x, w, b, residual=r)
  got = torch.autograd.grad(y, (x, r, w, b), dy)
  xf, rf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, r, w, b))
  want_y = rf + torch.nn.functional.linear(xf, wf, bf)
  want = torch.autograd.grad(want_y, (xf, rf, wf, bf), dy.float())
  assert (y.float() - want_y).abs().max() <= 2e-2 * (1 + want_y.abs().max())
  for a, e in zip(got, want):
    assert (a.float() - e).abs().max() <= 2e-2 * (1 + e.abs().max())
