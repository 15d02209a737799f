"""Model families on the GPU: bf16 forward passes through the hand-written kernels against the fp32 CPU path of
the same module (same weights), at head width 128 so that the tcgen05 GEMM / flash / fused norm kernels are used."""
import copy

import pytest
import torch

from maxdiffusion_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _rel(a, b):
  a, b = a.float().cpu(), b.float().cpu()
  return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _pair(model):
  ref = copy.deepcopy(model).float().eval()
  return ref, model.to("cuda", torch.bfloat16).eval()


def test_zimage_bf16_matches_fp32():
  from maxdiffusion_b200.models.z_image.transformer_z_image import ZImageConfig, ZImageTransformer2DModel

  torch.manual_seed(0)
  cfg = ZImageConfig(in_channels=16, dim=256, n_layers=2, n_refiner_layers=1, n_heads=2, cap_feat_dim=64,
                     axes_dims=(32, 48, 48), axes_lens=(512, 64, 64))
  ref, gpu = _pair(ZImageTransformer2DModel(cfg))
  x = [torch.randn(16, 1, 32, 32) for _ in range(2)]
  caps = [torch.randn(40, 64), torch.randn(40, 64)]
  t = torch.tensor([0.3, 0.6])
  n0 = _lib.launch_count()
  with torch.no_grad():
    want = ref(x, t, caps)
    got = gpu([v.cuda().bfloat16() for v in x], t.cuda(), [c.cuda().bfloat16() for c in caps])
  assert _lib.launch_count() > n0
  for g, w in zip(got, want):
    assert _rel(g, w) < 6e-2
  _lib.raise_on_device_status()


def test_flux2_klein_bf16_matches_fp32():
  from maxdiffusion_b200.models.flux.transformer_flux2_klein import Flux2KleinConfig, Flux2KleinTransformer2DModel
  from maxdiffusion_b200.pipelines.flux.flux2klein_pipeline import prepare_latent_image_ids, prepare_text_ids

  torch.manual_seed(0)
  cfg = Flux2KleinConfig(in_channels=128, num_layers=1, num_single_layers=2, num_attention_heads=2,
                         attention_head_dim=128, joint_attention_dim=96)
  ref, gpu = _pair(Flux2KleinTransformer2DModel(cfg))
  ids, tid = prepare_latent_image_ids(16, 16), prepare_text_ids(24)
  x, e, t = torch.randn(1, 256, 128), torch.randn(1, 24, 96), torch.tensor([0.7])
  with torch.no_grad():
    want = ref(x, e, t, ids, tid)
    got = gpu(x.cuda().bfloat16(), e.cuda().bfloat16(), t.cuda(), ids.cuda(), tid.cuda())
  assert _rel(got, want) < 6e-2
  _lib.raise_on_device_status()


def test_wan_vace_and_animate_bf16_match_fp32():
  from maxdiffusion_b200.models.wan.transformer_wan_animate import WanAnimateConfig, WanAnimateModel
  from maxdiffusion_b200.models.wan.transformer_wan_vace import WanVACEConfig, WanVACEModel

  torch.manual_seed(0)
  base = dict(num_attention_heads=2, attention_head_dim=128, ffn_dim=512, num_layers=2, text_dim=64, freq_dim=64)
  ref, gpu = _pair(WanVACEModel(WanVACEConfig(**base, vace_layers=(0, 1), vace_in_channels=96)))
  x, c = torch.randn(1, 16, 3, 16, 16), torch.randn(1, 96, 3, 16, 16)
  t, e = torch.tensor([500.0]), torch.randn(1, 12, 64)
  with torch.no_grad():
    want = ref(x, t, e, c)
    got = gpu(x.cuda().bfloat16(), t.cuda(), e.cuda().bfloat16(), c.cuda().bfloat16())
  assert _rel(got, want) < 6e-2
  acfg = WanAnimateConfig(**base, in_channels=36, image_dim=48, motion_encoder_size=16, motion_style_dim=16,
                          motion_dim=6, motion_encoder_dim=16, face_encoder_hidden_dim=16, face_encoder_num_heads=4,
                          inject_face_latents_blocks=1, motion_encoder_batch_size=4,
                          motion_encoder_channel_sizes={"4": 16, "8": 16, "16": 8})
  ref, gpu = _pair(WanAnimateModel(acfg))
  x, pose = torch.randn(1, 36, 3, 16, 16), torch.randn(1, 16, 2, 16, 16)
  face, img = torch.randn(1, 3, 8, 16, 16), torch.randn(1, 5, 48)
  with torch.no_grad():
    want = ref(x, t, e, img, pose_hidden_states=pose, face_pixel_values=face)
    # the face cross-attention has 5 key/value tokens per frame: the flash kernel's shortest segment
    got = gpu(x.cuda().bfloat16(), t.cuda(), e.cuda().bfloat16(), img.cuda().bfloat16(),
              pose_hidden_states=pose.cuda().bfloat16(), face_pixel_values=face.cuda().bfloat16())
  assert _rel(got, want) < 8e-2
  _lib.raise_on_device_status()


def test_sdxl_unet_groupnorm_path_bf16():
  from maxdiffusion_b200.models.unet_2d_condition import UNET_PRESETS, UNet2DConditionModel, UNetConfig

  torch.manual_seed(0)
  ref, gpu = _pair(UNet2DConditionModel(UNetConfig(**UNET_PRESETS["tiny"])))
  x, t, e = torch.randn(2, 4, 16, 16), torch.tensor([10.0, 500.0]), torch.randn(2, 7, 32)
  added = {"text_embeds": torch.randn(2, 16), "time_ids": torch.randn(2, 6)}
  with torch.no_grad():
    want = ref(x, t, e, added_cond_kwargs=added)
    got = gpu(x.cuda().bfloat16(), t.cuda(), e.cuda().bfloat16(),
              added_cond_kwargs={k: v.cuda().bfloat16() for k, v in added.items()})
  assert _rel(got, want) < 6e-2


def test_ltx2_transformer_bf16_matches_fp32():
  from maxdiffusion_b200.models.ltx2.transformer_ltx2 import LTX2Config, LTX2VideoTransformer3DModel

  torch.manual_seed(0)
  cfg = LTX2Config(in_channels=32, out_channels=32, num_attention_heads=2, attention_head_dim=128, cross_attention_dim=256,
                   audio_in_channels=16, audio_out_channels=16, audio_num_attention_heads=2, audio_attention_head_dim=64,
                   audio_cross_attention_dim=128, num_layers=2, caption_channels=48, gated_attn=True,
                   spatio_temporal_guidance_blocks=(1,))
  ref, gpu = _pair(LTX2VideoTransformer3DModel(cfg))
  B, Fr, H, W, Fa = 2, 2, 8, 8, 12
  x, a, txt = torch.randn(B, Fr * H * W, 32), torch.randn(B, Fa, 16), torch.randn(B, 16, 48)
  t = torch.tensor([400.0, 400.0])
  pm = torch.tensor([1.0, 0.0]).view(2, 1, 1)
  kw = dict(num_frames=Fr, height=H, width=W, audio_num_frames=Fa)
  with torch.no_grad():
    want, awant = ref(x, a, txt, txt, t, perturbation_mask=pm, **kw)
    got, agot = gpu(x.cuda().bfloat16(), a.cuda().bfloat16(), txt.cuda().bfloat16(), txt.cuda().bfloat16(), t.cuda(),
                    perturbation_mask=pm.cuda(), **kw)
  assert _rel(got, want) < 6e-2 and _rel(agot, awant) < 6e-2
  _lib.raise_on_device_status()


def test_cuda_graph_cache_captures_once_and_replays(tmp_path):
  from maxdiffusion_b200 import aot_cache
  from maxdiffusion_b200.ops import functional as OF

  w = torch.randn((256, 256), device="cuda", dtype=torch.bfloat16)

  @aot_cache.cached_graph(name="test_step")
  def step(x):
    return OF.linear(x, w, None, "gelu_tanh")

  aot_cache.install(str(tmp_path), revision="r")
  try:
    outs = []
    for i in range(3):
      x = torch.randn((128, 256), device="cuda", dtype=torch.bfloat16)
      outs.append((step(x).clone(), OF.linear(x, w, None, "gelu_tanh")))
    torch.cuda.synchronize()
    for got, want in outs:
      assert torch.equal(got, want)
    st = aot_cache.stats()["test_step"]
    assert st["captures"] == 1 and st["hits"] == 2
    step(torch.randn((64, 256), device="cuda", dtype=torch.bfloat16))  # a new shape is a new graph
    assert aot_cache.stats()["test_step"]["captures"] == 2
    assert len(step.known_signatures()) == 2  # recorded on disk for the next process
  finally:
    aot_cache.uninstall()


def test_flux_bf16_matches_fp32_forward_and_trains():
  """Flux at head width 128: the bf16 kernel path (modulations on the GEMM with fp32 output, fused q/k/v, gated
  residual epilogues) against the fp32 CPU path; then one backward through the same model (the modulation takes its
  differentiable form under autograd)."""
  from maxdiffusion_b200.models.flux.transformer_flux import FluxConfig, FluxTransformer2DModel, prepare_latent_image_ids

  torch.manual_seed(0)
  cfg = FluxConfig(num_layers=1, num_single_layers=2, num_attention_heads=2, attention_head_dim=128, joint_attention_dim=64,
                   pooled_projection_dim=32, axes_dims_rope=(16, 56, 56))
  ref, gpu = _pair(FluxTransformer2DModel(cfg))
  B, T = 2, 8
  x, txt, pooled = torch.randn(B, 64, 64), torch.randn(B, T, 64), torch.randn(B, 32)
  t, g = torch.tensor([0.25, 0.8]), torch.tensor([3.5, 2.0])
  img_ids, txt_ids = prepare_latent_image_ids(8, 8), torch.zeros(T, 3)
  with torch.no_grad():
    want = ref(x, txt, pooled, t, img_ids, txt_ids, g)
    got = gpu(x.cuda().bfloat16(), txt.cuda().bfloat16(), pooled.cuda().bfloat16(), t.cuda(), img_ids.cuda(), txt_ids.cuda(), g.cuda())
  assert _rel(got, want) < 6e-2
  out = gpu(x.cuda().bfloat16(), txt.cuda().bfloat16(), pooled.cuda().bfloat16(), t.cuda(), img_ids.cuda(), txt_ids.cuda(), g.cuda())
  out.float().pow(2).mean().backward()
  mod = gpu.transformer_blocks[0].norm1.weight.grad
  assert mod is not None and torch.isfinite(mod.float()).all() and mod.float().abs().sum() > 0
  _lib.raise_on_device_status()
