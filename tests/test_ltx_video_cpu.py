"""LTX-Video on CPU: fractional RoPE, skip-layer strategies, per-phase schedules and the two-pass pipeline."""
import pytest
import torch

from maxdiffusion_b200 import pyconfig
from maxdiffusion_b200.models.ltx_video.transformer3d import (LTXV_PRESETS, LTXVideoConfig, SkipLayerStrategy, Transformer3DModel,
                                                              fractional_rope)
from maxdiffusion_b200.pipelines.ltx_video.ltx_video_pipeline import _per_step


def test_fractional_rope_shape_and_padding():
  grid = torch.rand(2, 3, 10) * torch.tensor([5.0, 512, 512]).view(1, 3, 1)
  cos, sin = fractional_rope(grid, (20, 2048, 2048), 10000.0, 50)
  assert cos.shape == (2, 10, 50) and torch.all(cos[..., :2] == 1) and torch.all(sin[..., :2] == 0)  # 50 % 6 == 2
  assert torch.allclose(cos ** 2 + sin ** 2, torch.ones_like(cos), atol=1e-5)


def test_skip_layer_strategies_only_touch_the_masked_sample():
  torch.manual_seed(0)
  m = Transformer3DModel(LTXVideoConfig(**LTXV_PRESETS["tiny"])).eval()
  B, N = 2, 12
  x, txt, t = torch.randn(B, N, 8), torch.randn(B, 5, 16), torch.tensor([0.6, 0.6])
  grid = torch.rand(B, 3, N) * 100
  mask = m.create_skip_layer_mask(1, 2, 1, [1])
  assert mask.shape == (3, 2) and mask[1].tolist() == [1.0, 0.0]
  with torch.no_grad():
    base = m(x, grid, txt, t)
    for strat in SkipLayerStrategy:
      out = m(x, grid, txt, t, skip_layer_mask=mask, skip_layer_strategy=strat)
      assert torch.allclose(out[0], base[0], atol=1e-5) and (out[1] - base[1]).abs().max() > 1e-4, strat


def test_per_step_schedule_lookup():
  ts = [1.0, 0.99, 0.95, 0.7, 0.3]
  assert _per_step([1, 6, 8], [1.0, 0.9933, 0.6], ts) == [1, 6, 6, 8, 8]
  assert _per_step([3], None, ts) == [3] * 5 and _per_step(2.5, None, ts) == [2.5] * 5


def test_generate_ltx_video_multi_scale_tiny(tmp_path):
  from maxdiffusion_b200 import generate_ltx_video as G

  comps = ('{"vae": {"latent_channels": 8, "block_out_channels": [8, 16, 16, 32], "decoder_block_out_channels": [8, 16, 32], '
           '"layers_per_block": [1, 1, 1, 1, 1], "decoder_layers_per_block": [1, 1, 1, 1]}, '
           '"latent_upsampler": {"mid_channels": 32, "num_blocks_per_stage": 1}}')
  first = ('{"guidance_scale": [1, 3], "stg_scale": [0, 2], "rescaling_scale": [1, 0.5], "guidance_timesteps": [1.0, 0.9], '
           '"skip_block_list": [[], [1]], "num_inference_steps": 3, "skip_final_inference_steps": 1, '
           '"skip_initial_inference_steps": 0, "cfg_star_rescale": true}')
  second = ('{"guidance_scale": [1], "stg_scale": [1], "rescaling_scale": [1], "guidance_timesteps": [1.0], "skip_block_list": [1], '
            '"num_inference_steps": 3, "skip_initial_inference_steps": 1, "skip_final_inference_steps": 0, "cfg_star_rescale": true}')
  config = pyconfig.initialize(
      ["x", "maxdiffusion_b200/configs/ltx_video.yml", "random_init=True", "ltxv_preset=tiny", f"ltxv_component_overrides={comps}",
       f"first_pass={first}", f"second_pass={second}", "height=96", "width=96", "num_frames=9", "max_sequence_length=6",
       "downscale_factor=0.67", f"output_dir={tmp_path}", "log_config=false", "pretrained_model_name_or_path=/nonexistent"],
      unittest=True)
  video = G.run(config)
  assert video.shape == (1, 9, 96, 96, 3) and video.dtype == torch.uint8


def _tiny_pipe():
  from maxdiffusion_b200.models.ltx2.autoencoder_kl_ltx2 import LTX2VAEConfig, LTX2VideoAutoencoderKL
  from maxdiffusion_b200.pipelines.ltx_video.ltx_video_pipeline import LTXVideoPipeline

  torch.manual_seed(0)
  tr = Transformer3DModel(LTXVideoConfig(**LTXV_PRESETS["tiny"])).eval()
  vae = LTX2VideoAutoencoderKL(LTX2VAEConfig(latent_channels=8, block_out_channels=(8, 16, 16, 32), decoder_block_out_channels=(8, 16, 32),
                                             layers_per_block=(1, 1, 1, 1, 1), decoder_layers_per_block=(1, 1, 1, 1),
                                             timestep_conditioning=True, decoder_causal=True)).eval()
  return LTXVideoPipeline(tr, vae, device="cpu")


def test_conditioning_item_keeps_first_frame_latents():
  from maxdiffusion_b200.pipelines.ltx_video.ltx_video_pipeline import ConditioningItem

  pipe = _tiny_pipe()
  img = torch.rand(1, 3, 1, 64, 64) * 2 - 1
  kw = dict(height=64, width=64, num_frames=9, num_inference_steps=3, guidance_scale=1.0, output_type="latent",
            prompt_embeds=torch.randn(1, 6, 16), prompt_attention_mask=torch.ones(1, 6, dtype=torch.long))
  lat = pipe(conditioning_items=[ConditioningItem(img, 0, 1.0)], **kw)
  mean, _ = pipe.vae.encode(img)
  want = pipe.vae.normalize_latents(mean)
  assert lat.shape == (1, 8, 2, 2, 2)
  assert torch.allclose(lat[:, :, :1], want, atol=1e-5)  # strength 1: never denoised, never noised
  free = pipe(**kw)
  assert not torch.allclose(free[:, :, :1], want, atol=1e-2) and not torch.allclose(lat[:, :, 1:], free[:, :, 1:], atol=1e-4)
  # partial strength: blended start, denoised once t passes 1 - strength
  soft = pipe(conditioning_items=[ConditioningItem(img, 0, 0.5)], **kw)
  assert not torch.allclose(soft[:, :, :1], want, atol=1e-3)
  # per-token timesteps and hard-conditioning noise run and still pin nothing but change the rest
  noisy = pipe(conditioning_items=[ConditioningItem(img, 0, 1.0)], image_cond_noise_scale=0.15, per_token_timestep=True, **kw)
  assert torch.isfinite(noisy).all()


def test_conditioning_item_position_and_border_strip():
  from maxdiffusion_b200.pipelines.ltx_video.ltx_video_pipeline import ConditioningItem

  pipe = _tiny_pipe()
  z = torch.zeros(1, 8, 1, 3, 3)
  it = ConditioningItem(torch.zeros(1, 3, 1, 96, 96), 0, 1.0, media_x=32, media_y=0)
  out, lx, ly = pipe.latent_spatial_position(z, it, 128, 160)
  # left edge is interior (stripped, shifted by one latent), right edge (32+96=128 < 160) too; top touches the border
  assert out.shape[-2:] == (2, 1) and (lx, ly) == (2, 0)
  it2 = ConditioningItem(torch.zeros(1, 3, 1, 96, 96), 0, 1.0)
  out2, lx2, ly2 = pipe.latent_spatial_position(z, it2, 96, 96)
  assert out2.shape[-2:] == (3, 3) and (lx2, ly2) == (0, 0)


def test_prompt_enhancement_and_crf_identity():
  from maxdiffusion_b200.models.ltx_video.utils import prompt_enhance_utils as PE
  from maxdiffusion_b200.models.ltx_video.utils.diffusers_config_mapping import diffusers_to_native, native_to_diffusers
  from maxdiffusion_b200.pipelines.ltx_video import crf_compressor
  from maxdiffusion_b200.pipelines.ltx_video.ltx_video_pipeline import ConditioningItem

  class Tok:
    def apply_chat_template(self, msgs, tokenize, add_generation_prompt):
      return " | ".join(m["content"] for m in msgs)

    def __call__(self, texts, return_tensors, padding=False):
      self.texts = texts
      return {"input_ids": torch.zeros(len(texts), 3, dtype=torch.long)}

    def batch_decode(self, ids, skip_special_tokens):
      return [f"enhanced:{len(i)}" for i in ids]

  class LM:
    device = "cpu"

    def generate(self, input_ids, max_new_tokens):
      return torch.zeros(input_ids.shape[0], 3 + 4, dtype=torch.long)

  class Proc:
    def __call__(self, prompts, images, return_tensors):
      return {"input_ids": torch.zeros(len(images), 1, dtype=torch.long), "pixel_values": torch.zeros(len(images), 3, 2, 2)}

    def batch_decode(self, ids, skip_special_tokens):
      return ["a photo"] * len(ids)

  class Cap:
    device = "cpu"

    def generate(self, **kw):
      return torch.zeros(kw["input_ids"].shape[0], 2, dtype=torch.long)

  tok = Tok()
  assert PE.generate_cinematic_prompt(None, None, LM(), tok, "a cat") == ["enhanced:4"]
  assert "user_prompt: a cat" in tok.texts[0] and "image_caption" not in tok.texts[0]
  item = ConditioningItem(torch.zeros(1, 3, 1, 8, 8), 0, 1.0)
  assert PE.generate_cinematic_prompt(Cap(), Proc(), LM(), tok, ["a cat"], [item]) == ["enhanced:4"]
  assert "image_caption: a photo" in tok.texts[0]
  late = ConditioningItem(torch.zeros(1, 3, 1, 8, 8), 8, 1.0)
  assert PE.generate_cinematic_prompt(Cap(), Proc(), LM(), tok, ["a cat"], [late]) == ["a cat"]
  x = torch.rand(9, 9, 3)
  assert crf_compressor.compress(x, 0) is x
  d = {"_class_name": "LTXVideoTransformer3DModel", "num_layers": 48, "num_attention_heads": 32, "attention_head_dim": 128,
       "cross_attention_dim": 4096, "caption_channels": 4096, "in_channels": 128, "out_channels": 128}
  n = diffusers_to_native(d)
  assert n["num_layers"] == 48 and n["qk_norm"] == "rms_norm" and native_to_diffusers(n)["attention_head_dim"] == 128


def test_codec_noise_grows_with_the_rate_factor_and_follows_h264_quantisation():
  """The on-device model of an H.264 intra frame: the orthonormal core transform inverts itself, the step size doubles
  every 6 QP, a smooth picture survives better than noise, and the error grows monotonically with the rate factor."""
  from maxdiffusion_b200.pipelines.ltx_video import crf_compressor as cc

  assert torch.allclose(cc._CORE @ cc._CORE.t(), torch.eye(4), atol=1e-6)
  assert cc.qstep(0) == 0.625 and cc.qstep(28) == pytest.approx(16.0, rel=1e-6) and cc.qstep(34) == pytest.approx(2 * cc.qstep(28))
  assert [cc.chroma_qp(q) for q in (20, 29, 30, 40, 51)] == [20, 29, 29, 36, 39]
  g = torch.Generator().manual_seed(0)
  yy, xx = torch.meshgrid(torch.linspace(0, 1, 37), torch.linspace(0, 1, 50), indexing="ij")
  smooth = torch.stack([yy, xx, 0.5 * (yy + xx)], dim=-1)
  noisy = (smooth + 0.2 * torch.randn(smooth.shape, generator=g)).clamp(0, 1)

  def mse(img, crf):
    out = cc.compress(img, crf)
    assert out.shape == (36, 50, 3) and out.dtype == img.dtype and 0 <= out.min() and out.max() <= 1
    return ((out - img[:36, :50]) ** 2).mean().item()

  errs = [mse(noisy, c) for c in (10, 20, 29, 40, 51)]
  assert all(a < b for a, b in zip(errs, errs[1:])), errs
  assert mse(smooth, 29) < 0.1 * mse(noisy, 29)
  assert mse(smooth, 10) < 2e-4  # near-transparent at a low rate factor
