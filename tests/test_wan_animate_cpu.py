"""Wan-Animate on CPU: motion / face encoders, pose + face conditioning, and the segment loop of the pipeline."""
import os

import torch

from maxdiffusion_b200 import pyconfig
from maxdiffusion_b200.models.wan.transformer_wan_animate import (WAN_ANIMATE_PRESETS, WanAnimateConfig, WanAnimateModel,
                                                                   MotionConv2d)
from maxdiffusion_b200.pipelines.wan.wan_pipeline_animate import WanAnimatePipeline, pad_video_frames

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs",
                   "base_wan_animate.yml")


def test_pad_video_frames_reflects():
  v = torch.arange(1, 6).float().reshape(1, 1, 5, 1, 1)
  assert pad_video_frames(v, 10).flatten().tolist() == [1, 2, 3, 4, 5, 4, 3, 2, 1, 2]


def test_blur_downsample_conv_halves_resolution():
  conv = MotionConv2d(4, 6, 3, stride=2, padding=0, blur_kernel=(1, 3, 3, 1))
  assert conv(torch.randn(2, 4, 16, 16)).shape == (2, 6, 8, 8)
  skip = MotionConv2d(4, 6, 1, stride=2, padding=0, bias=False, blur_kernel=(1, 3, 3, 1), use_activation=False)
  assert skip(torch.randn(2, 4, 16, 16)).shape == (2, 6, 8, 8)


def test_model_conditioning_paths():
  torch.manual_seed(0)
  m = WanAnimateModel(WanAnimateConfig(**WAN_ANIMATE_PRESETS["tiny"])).eval()
  x, pose = torch.randn(1, 36, 3, 8, 8), torch.randn(1, 16, 2, 8, 8)
  face = torch.randn(1, 3, 8, 16, 16)
  t, e, img = torch.tensor([500.0]), torch.randn(1, 7, 32), torch.randn(1, 5, 24)
  with torch.no_grad():
    mv = m.encode_face_motion(face, 1)
    assert mv.shape == (1, 3, 3, 64) and float(mv[:, 0].abs().max()) == 0.0  # zero face latents for the reference frame
    a = m(x, t, e, img, pose_hidden_states=pose, face_motion_vec=mv)
    b = m(x, t, e, img, pose_hidden_states=pose, face_pixel_values=face)
    no_face = m(x, t, e, img, pose_hidden_states=pose)
    no_pose = m(x, t, e, img, face_motion_vec=mv)
  assert a.shape == (1, 16, 3, 8, 8) and torch.equal(a, b)
  assert (a - no_face).abs().max() > 1e-3 and (a - no_pose).abs().max() > 1e-3


def test_pipeline_two_segments(tmp_path):
  over = ('{"num_attention_heads": 2, "attention_head_dim": 32, "ffn_dim": 64, "num_layers": 2, "text_dim": 32, '
          '"freq_dim": 32, "image_dim": 24, "motion_encoder_size": 16, "motion_style_dim": 16, "motion_dim": 6, '
          '"motion_encoder_dim": 16, "face_encoder_hidden_dim": 16, "face_encoder_num_heads": 2, '
          '"inject_face_latents_blocks": 1, "motion_encoder_batch_size": 4, '
          '"motion_encoder_channel_sizes": {"4": 16, "8": 16, "16": 8}}')
  config = pyconfig.initialize(["t", CFG, "wan_preset=tiny", f"wan_config_overrides={over}", "random_init=True",
                                'vae_config_overrides={"base_dim": 8, "z_dim": 16}', "height=32", "width=32",
                                "num_inference_steps=2", "log_config=false", f"output_dir={tmp_path}"], unittest=True)
  pipe = WanAnimatePipeline.from_config(config, device="cpu")
  g = torch.Generator().manual_seed(0)
  image = torch.rand((1, 3, 32, 32), generator=g) * 2 - 1
  pose = torch.rand((1, 3, 13, 32, 32), generator=g) * 2 - 1
  face = torch.rand((1, 3, 13, 16, 16), generator=g) * 2 - 1
  kw = dict(prompt_embeds=torch.randn(1, 8, 32), negative_prompt_embeds=torch.randn(1, 8, 32),
            image_embeds=torch.randn(1, 5, 24), segment_frame_length=9, prev_segment_conditioning_frames=1,
            height=32, width=32, generator=g)
  video = pipe(image, pose, face, guidance_scale=2.0, **kw)          # 13 frames = 9 + 8 - 4 padded -> 2 segments
  assert video.shape == (1, 13, 32, 32, 3) and video.dtype == torch.uint8
  bg = torch.rand((1, 3, 13, 32, 32), generator=g) * 2 - 1
  mk = (torch.rand((1, 1, 13, 32, 32), generator=g) > 0.5).float()
  video2 = pipe(image, pose, face, background_video=bg, mask_video=mk, mode="replace", **kw)
  assert video2.shape == (1, 13, 32, 32, 3)


def test_check_inputs_rejects_what_the_segment_loop_cannot_run():
  import pytest

  pipe = WanAnimatePipeline.__new__(WanAnimatePipeline)
  img, pose, face = torch.zeros(1, 3, 32, 32), torch.zeros(1, 3, 9, 32, 32), torch.zeros(1, 3, 9, 16, 16)
  ok = dict(image=img, pose_video=pose, face_video=face, background_video=None, mask_video=None, prompt="a", negative_prompt=None,
            height=32, width=32)
  pipe.check_inputs(**ok)
  for change, match in (({"prompt_embeds": torch.zeros(1, 4, 8)}, "not both"), ({"image": None}, "provide `image`"),
                        ({"face_video": None}, "face_video"), ({"face_video": face[:, :, :5]}, "frames"),
                        ({"mode": "replace"}, "replace mode"), ({"mode": "swap"}, "mode must be"),
                        ({"height": 40}, "divisible by 16"), ({"prompt": 3}, "str or a list"),
                        ({"prev_segment_conditioning_frames": 3}, "1 or 5"),
                        ({"mode": "replace", "background_video": pose, "mask_video": pose[:, :1, :4]}, "mask_video")):
    with pytest.raises(ValueError, match=match):
      pipe.check_inputs(**{**ok, **change})
