"""Shared body of the image `generate_*` entry points: build or load the pipeline, warm up, time, write PNGs."""
import os
import time

import torch

from . import max_logging
from .utils.export_utils import export_to_png


def run_image_pipeline(config, pipe, call_kwargs: dict, prefix: str):
  t0 = time.perf_counter()
  pipe(**{**call_kwargs, "num_inference_steps": 2, "output_type": "latent"})
  warm = time.perf_counter() - t0
  t0 = time.perf_counter()
  images = pipe(**call_kwargs)
  if torch.cuda.is_available():
    torch.cuda.synchronize()
  gen = time.perf_counter() - t0
  max_logging.log(f"warm-up: {warm:.2f}s  generation: {gen:.2f}s  ({images.shape[0] / gen:.3f} images/s)")
  if int(os.environ.get("RANK", "0")) == 0 or config.get("write_all_ranks", False):
    out_dir = config.get("output_dir", ".") or "."
    os.makedirs(out_dir, exist_ok=True)
    for i in range(images.shape[0]):
      max_logging.log("wrote " + export_to_png(images[i].cpu().numpy(), os.path.join(out_dir, f"{prefix}_{config.seed}_{i}.png")))
  return images


def synthetic_text_conditioning(batch: int, seq: int, dim: int, pooled_dim: int, seed: int):
  g = torch.Generator().manual_seed(seed)
  return torch.randn((batch, seq, dim), generator=g), torch.randn((batch, pooled_dim), generator=g)
