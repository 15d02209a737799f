"""Implicit-GEMM convolutions (csrc/conv_igemm.cu) against fp32 PyTorch convolutions of the same bf16 inputs: ragged
sizes, channel counts that are not multiples of 64, the 2-frame history of the causal conv3d, stride 2 with either
padding convention, the fused nearest-2x + conv, input gradients, and the channels-last RMS norm + SiLU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(got, want, tol=2e-2):
  got, want = got.float(), want.float()
  err = (got - want).abs().max().item()
  scale = want.abs().max().item() + 1e-6
  assert err <= tol * scale, f"max err {err:.4g} vs scale {scale:.4g}"
  rel = ((got - want).norm() / (want.norm() + 1e-12)).item()
  assert rel < 1e-2, f"relative error {rel:.4g}"


def _rand(shape, seed, scale=1.0):
  g = torch.Generator(device="cuda").manual_seed(seed)
  return (torch.randn(shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("B,T,H,W,Ci,Co", [(1, 2, 8, 16, 16, 16), (1, 3, 9, 20, 96, 96), (2, 1, 12, 10, 192, 96),
                                          (1, 2, 6, 40, 384, 192), (1, 4, 5, 7, 16, 384), (1, 2, 16, 16, 96, 3)])
@pytest.mark.parametrize("with_hist", [False, True])
def test_conv3d_causal_matches_fp32(B, T, H, W, Ci, Co, with_hist):
  from maxdiffusion_b200.ops import conv as OC

  x = _rand((B, T, H, W, Ci), 1)
  w = _rand((Co, Ci, 3, 3, 3), 2, scale=(27 * Ci) ** -0.5)
  b = _rand((Co,), 3)
  hist = _rand((B, 2, H, W, Ci), 4) if with_hist else None
  res = _rand((B, T, H, W, (Co + 7) // 8 * 8), 5) if Co % 8 == 0 else None
  pk = OC.pack_conv3d(w, b)
  got = OC.conv3d_causal(x, pk, hist=hist, residual=res)
  want = OC.ref_conv3d_causal(x, w, b, hist=hist, residual=res)
  assert got.shape == want.shape
  _close(got, want)


def test_time_conv_3x1x1_and_view_inputs():
  from maxdiffusion_b200.ops import conv as OC

  full = _rand((1, 5, 6, 8, 96), 1)
  x = full[:, 1:]                      # a view along time: strides of the parent tensor
  w = _rand((192, 96, 3, 1, 1), 2, scale=0.06)
  b = _rand((192,), 3)
  pk = OC.pack_conv3d(w, b)
  hist = full[:, :1].repeat(1, 2, 1, 1, 1)
  _close(OC.conv3d_causal(x, pk, hist=hist), OC.ref_conv3d_causal(x, w, b, hist=hist))
  _close(OC.conv3d_causal(x, pk), OC.ref_conv3d_causal(x, w, b))


@pytest.mark.parametrize("B,H,W,Ci,Co,k", [(2, 8, 8, 32, 64, 3), (1, 33, 21, 96, 96, 3), (3, 16, 16, 320, 320, 3),
                                          (1, 12, 40, 128, 640, 3), (2, 10, 10, 64, 32, 1), (1, 64, 64, 16, 8, 3)])
def test_conv2d_stride1(B, H, W, Ci, Co, k):
  from maxdiffusion_b200.ops import conv as OC

  x = _rand((B, H, W, Ci), 1)
  w = _rand((Co, Ci, k, k), 2, scale=(k * k * Ci) ** -0.5)
  b = _rand((Co,), 3)
  res = _rand((B, H, W, Co), 4)
  pk = OC.pack_conv2d(w, b)
  _close(OC.conv2d(x, pk, residual=res), OC.ref_conv2d(x, w, b, residual=res))
  _close(OC.conv2d(x, pk, silu=True), OC.ref_conv2d(x, w, b, silu=True))


@pytest.mark.parametrize("pad", [0, 1])
@pytest.mark.parametrize("B,H,W,Ci,Co", [(1, 8, 8, 32, 32), (2, 18, 30, 96, 96), (1, 32, 32, 320, 320), (1, 6, 10, 192, 64)])
def test_conv2d_stride2_both_padding_conventions(B, H, W, Ci, Co, pad):
  from maxdiffusion_b200.ops import conv as OC

  x = _rand((B, H, W, Ci), 1)
  w = _rand((Co, Ci, 3, 3), 2, scale=(9 * Ci) ** -0.5)
  b = _rand((Co,), 3)
  pk = OC.pack_conv2d(w, b, stride=2, pad_top_left=pad)
  got = OC.conv2d(x, pk)
  want = OC.ref_conv2d(x, w, b, stride=2, pad_top_left=pad)
  assert got.shape == (B, H // 2, W // 2, Co)
  _close(got, want)


@pytest.mark.parametrize("B,H,W,Ci,Co", [(1, 4, 4, 32, 16), (2, 9, 15, 96, 48), (1, 20, 12, 384, 192)])
def test_upsample_conv_fused_matches_upsample_then_conv(B, H, W, Ci, Co):
  from maxdiffusion_b200.ops import conv as OC

  x = _rand((B, H, W, Ci), 1)
  w = _rand((Co, Ci, 3, 3), 2, scale=(9 * Ci) ** -0.5)
  b = _rand((Co,), 3)
  got = OC.upsample2x_conv2d(x, OC.pack_upsample_conv2d(w, b))
  want = OC.ref_upsample2x_conv2d(x, w, b)
  assert got.shape == (B, 2 * H, 2 * W, Co)
  _close(got, want)


@pytest.mark.parametrize("stride,pad", [(1, 1), (2, 1), (2, 0)])
def test_conv2d_dgrad_matches_autograd(stride, pad):
  from maxdiffusion_b200.ops import conv as OC

  B, H, W, Ci, Co = 2, 12, 20, 64, 96
  x = _rand((B, H, W, Ci), 1).float().requires_grad_(True)
  w = _rand((Co, Ci, 3, 3), 2, scale=(9 * Ci) ** -0.5)
  y = OC.ref_conv2d(x, w, None, stride=stride, pad_top_left=pad)
  dy = _rand(tuple(y.shape), 3)
  (y * dy.float()).sum().backward()
  got = OC.conv2d_dgrad(dy, OC.pack_conv2d_dgrad(w, stride=stride, pad_top_left=pad))
  assert got.shape == x.shape
  _close(got, x.grad)


@pytest.mark.parametrize("C", [96, 192, 384, 16, 1024, 8, 48, 112, 288, 320, 640, 1280])
@pytest.mark.parametrize("silu", [False, True])
def test_rms_act_channels_last(C, silu):
  """Every lane-group shape of the row kernel (exact factorisations of the row's vector count and the ragged
  fallback), and the variant that writes the interior of a tensor with halo columns."""
  from maxdiffusion_b200.ops import conv as OC

  x = _rand((3, 5, 7, C), 1, scale=3.0)
  gamma = torch.rand(C, device="cuda") + 0.5
  beta = torch.randn(C, device="cuda") * 0.1
  got = OC.rms_act(x, gamma, beta, silu=silu)
  want = OC.rms_act(x.cpu(), gamma.cpu(), beta.cpu(), silu=silu).cuda()
  _close(got, want)
  wide = OC.rms_act(x, gamma, beta, silu=silu, halo=1)
  assert wide.shape == (3, 5, 9, C) and torch.equal(wide[:, :, 1:-1], got)


def test_conv_results_are_bitwise_reproducible():
  from maxdiffusion_b200.ops import conv as OC

  x = _rand((1, 3, 20, 28, 96), 1)
  w = _rand((96, 96, 3, 3, 3), 2, scale=0.02)
  pk = OC.pack_conv3d(w, None)
  a = OC.conv3d_causal(x, pk)
  b = OC.conv3d_causal(x, pk)
  assert torch.equal(a, b)


def test_wan_vae_decode_on_the_conv_kernels_matches_the_pytorch_modules():
  """The channels-last decoder (conv3d with history tensors, fused up-sampling convs, GEMM 1x1s, row norm) against the
  fp32 PyTorch modules holding the same parameters, chunked frame by frame as the pipeline runs it."""
  from maxdiffusion_b200.models.wan.autoencoder_kl_wan import AutoencoderKLWan, WanVAEConfig

  torch.manual_seed(0)
  vae = AutoencoderKLWan(WanVAEConfig(base_dim=32)).cuda().eval()
  for n, p in vae.named_parameters():
    if p.dim() > 1:
      torch.nn.init.normal_(p, std=(p[0].numel()) ** -0.5)
  z = torch.randn(1, 16, 3, 8, 12, device="cuda")
  with torch.no_grad():
    want = vae.decode(z, chunk=1)                       # fp32 latents: the PyTorch path
    got = vae.decode(z.to(torch.bfloat16), chunk=1)     # bf16 latents: the kernel path
    got2 = vae.decode(z.to(torch.bfloat16), chunk=2)
  assert got.shape == want.shape == (1, 3, 9, 64, 96)
  for g in (got, got2):
    err = (g.float() - want).abs()
    assert err.max() < 0.08 and err.mean() < 0.01, (err.max().item(), err.mean().item())


@pytest.mark.parametrize("stride,pad", [(1, 1), (2, 1), (2, 0)])
@pytest.mark.parametrize("B,H,W,Ci,Co", [(2, 12, 20, 64, 96), (1, 34, 18, 320, 320), (3, 16, 16, 8, 640), (8, 32, 32, 256, 128),
                                        (2, 64, 64, 96, 64), (1, 8, 8, 72, 8)])
@pytest.mark.parametrize("boxed", [True, False])
def test_conv2d_wgrad_matches_autograd(B, H, W, Ci, Co, stride, pad, boxed):
  """Both forms of the weight gradient: boxes of output pixels read from the unpadded tensors (zero fill outside the
  image, parity coordinates for stride 2), and the bordered flat grid."""
  from maxdiffusion_b200.ops import conv as OC

  x = _rand((B, H, W, Ci), 1)
  w = _rand((Co, Ci, 3, 3), 2, scale=(9 * Ci) ** -0.5).float().requires_grad_(True)
  y = OC.ref_conv2d(x, w, None, stride=stride, pad_top_left=pad)
  dy = _rand(tuple(y.shape), 3)
  (y * dy.float()).sum().backward()
  got = OC.conv2d_wgrad(x, dy, 3, stride, pad, boxed=boxed)
  assert got.shape == w.shape
  _close(got, w.grad)
  assert torch.equal(got, OC.conv2d_wgrad(x, dy, 3, stride, pad, boxed=boxed))  # fixed summation order


@pytest.mark.parametrize("C,groups,HW", [(320, 32, (16, 24)), (64, 8, (9, 7)), (1280, 32, (8, 8)), (128, 32, (33, 5))])
@pytest.mark.parametrize("act", [False, True])
def test_group_norm_channels_last_fwd_bwd(C, groups, HW, act):
  from maxdiffusion_b200.ops import functional as OF

  H, W = HW
  torch.manual_seed(0)
  x = (torch.randn(3, C, H, W, device="cuda") * 2 + 0.5).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
  gamma = (torch.rand(C, device="cuda") + 0.5).to(torch.bfloat16)
  beta = (torch.randn(C, device="cuda") * 0.2).to(torch.bfloat16)
  xr = x.float().requires_grad_(True)
  gr, br = gamma.float().requires_grad_(True), beta.float().requires_grad_(True)
  want = torch.nn.functional.group_norm(xr, groups, gr, br, 1e-5)
  if act:
    want = torch.nn.functional.silu(want)
  dy = torch.randn_like(want).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
  want.backward(dy.float())
  xk = x.clone().requires_grad_(True)
  gk, bk = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
  got = OF.group_norm(xk, groups, gk, bk, 1e-5, act)
  assert got.is_contiguous(memory_format=torch.channels_last)
  got.backward(dy)
  _close(got, want)
  _close(xk.grad, xr.grad, tol=3e-2)
  _close(gk.grad, gr.grad, tol=3e-2)
  _close(bk.grad, br.grad, tol=3e-2)


def test_unet_on_the_conv_kernels_matches_fp32_modules_forward_and_backward():
  """The tiny SDXL-style UNet in bf16 on the kernel path (channels-last convolutions with dgrad / wgrad kernels,
  channels-last GroupNorm, flash attention) against the same parameters in fp32 through PyTorch convolutions."""
  from maxdiffusion_b200.models.unet_2d_condition import UNET_PRESETS, UNet2DConditionModel, UNetConfig

  torch.manual_seed(0)
  cfg = UNetConfig(**{**UNET_PRESETS["tiny"], "block_out_channels": (64, 128), "attention_head_dim": (1, 2), "norm_num_groups": 8})
  ref = UNet2DConditionModel(cfg).cuda().float()
  ker = UNet2DConditionModel(cfg).cuda().to(torch.bfloat16)
  ker.load_state_dict({k: v.to(torch.bfloat16) for k, v in ref.state_dict().items()})
  ref.load_state_dict({k: v.float() for k, v in ker.state_dict().items()})  # identical (bf16-representable) weights
  x = torch.randn(2, 4, 16, 16, device="cuda").to(torch.bfloat16)
  ctx = torch.randn(2, 7, 32, device="cuda").to(torch.bfloat16)
  add = {"text_embeds": torch.randn(2, 16, device="cuda").to(torch.bfloat16), "time_ids": torch.zeros(2, 6, device="cuda")}
  t = torch.tensor([10, 500], device="cuda")
  want = ref(x.float(), t, ctx.float(), {k: v.float() for k, v in add.items()})
  got = ker(x, t, ctx, add)
  _close(got, want, tol=6e-2)
  g = torch.randn_like(want)
  want.backward(g)
  got.backward(g.to(torch.bfloat16))
  checked = 0
  for (n, p), (_, q) in zip(ker.named_parameters(), ref.named_parameters()):
    if p.grad is None or q.grad is None or q.grad.abs().max() == 0:
      continue
    rel = ((p.grad.float() - q.grad).norm() / (q.grad.norm() + 1e-12)).item()
    assert rel < 0.12, (n, rel)
    checked += 1
  assert checked > 20


@pytest.mark.parametrize("T,D", [(96, 128), (1000, 384), (6240, 384)])
def test_wide_head_attention_matches_fp32(T, D):
  from maxdiffusion_b200.ops import conv as OC

  q, k, v = _rand((T, D), 1), _rand((T, D), 2), _rand((T, D), 3)
  got = OC.wide_head_attention(q, k, v)
  want = torch.softmax((q.float() @ k.float().t()) * D ** -0.5, dim=-1) @ v.float()
  _close(got, want, tol=3e-2)
  x = _rand((37, 2048), 4, scale=4.0)
  want_sm = torch.softmax(x.float(), dim=-1)
  assert (OC.softmax_rows(x.clone()).float() - want_sm).abs().max() < 2e-3


@pytest.mark.parametrize("W0,W1", [(3, 19), (0, 16), (8, 24)])
def test_halo_columns_are_read_and_produce_no_output(W0, W1):
  """A width shard extended by its neighbours' edge columns gives the same columns as the unsharded convolution (the
  first / last shard of a tensor pads its outer side with zeros, which is what the unsharded kernel reads there)."""
  from maxdiffusion_b200.ops import conv as OC

  x = _rand((1, 3, 10, 24, 96), 1)
  hist = _rand((1, 2, 10, 24, 96), 2)
  w = _rand((96, 96, 3, 3, 3), 3, scale=0.02)
  b = _rand((96,), 4)
  pk = OC.pack_conv3d(w, b)
  pad = lambda t: torch.nn.functional.pad(t, (0, 0, 1, 1))
  xs, hs = pad(x)[:, :, :, W0:W1 + 2].contiguous(), pad(hist)[:, :, :, W0:W1 + 2].contiguous()
  whole = OC.conv3d_causal(x, pk, hist=hist)
  got = OC.conv3d_causal(xs, pk, hist=hs, halo=1)
  assert torch.equal(got, whole[:, :, :, W0:W1])
  x2 = _rand((3, 10, 24, 96), 5)
  w2 = _rand((96, 96, 3, 3), 6, scale=0.03)
  pk2 = OC.pack_upsample_conv2d(w2, b)
  whole2 = OC.upsample2x_conv2d(x2, pk2)
  got2 = OC.upsample2x_conv2d(pad(x2)[:, :, W0:W1 + 2].contiguous(), pk2, halo=1)
  assert torch.equal(got2, whole2[:, :, 2 * W0:2 * W1])


def test_wan_2p2_vae_decode_on_the_conv_kernels_matches_the_pytorch_modules():
  """The Wan 2.2 VAE (resampler inside the up block, channel-duplicating shortcut, 2 x 2 pixel patches) on the
  channels-last kernel path against its fp32 PyTorch modules."""
  from maxdiffusion_b200.models.wan.autoencoder_kl_wan_2p2 import AutoencoderKLWan2p2, WanVAE2p2Config

  torch.manual_seed(0)
  cfg = WanVAE2p2Config(base_dim=32, base_dec_dim=32, z_dim=16, latents_mean=[0.0] * 16, latents_std=[1.0] * 16)
  vae = AutoencoderKLWan2p2(cfg).cuda().eval()
  for n, p in vae.named_parameters():
    if p.dim() > 1:
      torch.nn.init.normal_(p, std=(p[0].numel()) ** -0.5)
  z = torch.randn(1, 16, 3, 4, 6, device="cuda")
  with torch.no_grad():
    want = vae.decode(z, chunk=1)                       # fp32 latents: the PyTorch path
    got = vae.decode(z.to(torch.bfloat16), chunk=1)     # bf16 latents: the kernel path
  assert got.shape == want.shape == (1, 3, 9, 64, 96)
  err = (got.float() - want).abs()
  assert err.max() < 0.08 and err.mean() < 0.01, (err.max().item(), err.mean().item())


def test_wan_vae_encode_on_the_conv_kernels_matches_the_pytorch_modules():
  """The channels-last encoder (far-side padded stride-2 convolutions, the strided time convolution read off the causal
  one) against the fp32 PyTorch modules holding the same parameters."""
  from maxdiffusion_b200.models.wan.autoencoder_kl_wan import AutoencoderKLWan, WanVAEConfig

  torch.manual_seed(0)
  vae = AutoencoderKLWan(WanVAEConfig(base_dim=32)).cuda().eval()
  for n, p in vae.named_parameters():
    if p.dim() > 1:
      torch.nn.init.normal_(p, std=(p[0].numel()) ** -0.5)
  x = torch.randn(1, 3, 9, 32, 48, device="cuda").clamp(-1, 1)
  with torch.no_grad():
    want = vae.encode(x, chunk=4).mean                       # fp32 frames: the PyTorch path
    got = vae.encode(x.to(torch.bfloat16), chunk=4).mean     # bf16 frames: the kernel path
  assert got.shape == want.shape == (1, 16, 3, 4, 6)
  err = (got.float() - want).abs()
  assert err.max() < 0.08 * (1 + want.abs().max()) and err.mean() < 0.01 * (1 + want.abs().mean()), (err.max().item(), err.mean().item())
