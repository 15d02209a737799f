"""LTX-Video on CPU: fractional RoPE, skip-layer strategies, per-phase schedules and the two-pass pipeline."""
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
