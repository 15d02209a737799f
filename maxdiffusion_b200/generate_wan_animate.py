"""python -m maxdiffusion_b200.generate_wan_animate <config.yml> key=value ...

reference: src/maxdiffusion/generate_wan_animate.py. Inputs: `reference_image_path`, `pose_video_path`,
`face_video_path` (pre-processed driving videos) and, for `mode=replace`, `background_video_path` and
`mask_video_path`. With `random_init: True` and no paths, synthetic inputs of the configured size are used
(benchmarks)."""
import os
import sys
import time

import torch

from . import max_logging, pyconfig
from .parallel.mesh import init_distributed
from .pipelines.wan.wan_pipeline_animate import WanAnimatePipeline
from .utils.export_utils import export_to_video


def _load_video_tensor(path, height, width):
  from .video_processor import VideoProcessor
  from .utils.loading_utils import load_video

  return VideoProcessor().preprocess_video(load_video(path), height, width)


def run(config):
  t0 = time.perf_counter()
  pipe = WanAnimatePipeline.from_config(config) if config.get("random_init", False) else WanAnimatePipeline.from_pretrained(config)
  max_logging.log(f"load_time: {time.perf_counter() - t0:.1f}s")
  H, W, T = int(config.height), int(config.width), int(config.num_frames)
  face = pipe.transformer.cfg.motion_encoder_size
  mode = str(config.get("mode", "animate"))
  g = torch.Generator().manual_seed(int(config.seed))
  kw = {}
  if config.get("pose_video_path", "") and config.get("face_video_path", ""):
    from .image_processor import VaeImageProcessor
    from .utils.loading_utils import load_image

    image = VaeImageProcessor().preprocess(load_image(config.reference_image_path), H, W)
    pose = _load_video_tensor(config.pose_video_path, H, W)[:, :, :T]
    facev = _load_video_tensor(config.face_video_path, face, face)[:, :, :T]
    if mode == "replace":
      kw["background_video"] = _load_video_tensor(config.background_video_path, H, W)[:, :, :T]
      kw["mask_video"] = (_load_video_tensor(config.mask_video_path, H, W)[:, :1, :T] + 1) / 2
  elif config.get("random_init", False):
    image = torch.rand((1, 3, H, W), generator=g) * 2 - 1
    pose = torch.rand((1, 3, T, H, W), generator=g) * 2 - 1
    facev = torch.rand((1, 3, T, face, face), generator=g) * 2 - 1
  else:
    raise ValueError("Provide `reference_image_path`, `pose_video_path` and `face_video_path`.")
  if pipe.text_encoder is None:
    tdim = pipe.transformer.cfg.text_dim
    kw["prompt_embeds"] = torch.randn((1, int(config.max_sequence_length), tdim), generator=g)
    kw["negative_prompt_embeds"] = torch.randn((1, int(config.max_sequence_length), tdim), generator=g)
    if pipe.transformer.cfg.image_dim:
      kw["image_embeds"] = torch.randn((1, 257, pipe.transformer.cfg.image_dim), generator=g)
  t0 = time.perf_counter()
  video = pipe(image, pose, facev, prompt=config.get("prompt", ""), negative_prompt=config.get("negative_prompt", ""),
               height=H, width=W, segment_frame_length=int(config.get("segment_frame_length", 77)),
               prev_segment_conditioning_frames=int(config.get("prev_segment_conditioning_frames", 5)),
               num_inference_steps=int(config.num_inference_steps),
               guidance_scale=float(config.get("animate_guidance_scale", 1.0)), mode=mode, generator=g,
               motion_encode_batch_size=config.get("motion_encode_batch_size", None) or None, **kw)
  max_logging.log(f"generation_time: {time.perf_counter() - t0:.1f}s")
  if int(os.environ.get("RANK", "0")) == 0:
    out_dir = config.get("output_dir", ".") or "."
    os.makedirs(out_dir, exist_ok=True)
    for i in range(video.shape[0]):
      max_logging.log("wrote " + export_to_video(video[i].cpu().numpy(), os.path.join(out_dir, f"wan_animate_{config.seed}_{i}.mp4"),
                                                 fps=int(config.get("fps", 16))))
  return video


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
