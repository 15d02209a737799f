"""python -m maxdiffusion_b200.generate_flux_multi_res <config.yml> key=value ...

Flux over a list of `resolutions` with ONE pipeline (reference: src/maxdiffusion/generate_flux_multi_res.py, which
compiles one executable per resolution bucket). Every bucket is warmed up once (allocator, rotary tables, resolution
dependent time shift) and then timed; with `aot_cache_dir` set the denoising step of every bucket is replayed from a
CUDA graph."""
import os
import sys
import time

import torch

from . import max_logging, pyconfig
from ._generate_common import synthetic_text_conditioning
from .parallel.mesh import init_distributed
from .pipelines.flux.flux_pipeline import FluxPipeline
from .utils.export_utils import export_to_png


def run(config):
  if config.get("random_init", False):
    pipe = FluxPipeline.from_config(config)
  else:
    from .loaders.flux_loader import load_flux_pipeline

    pipe = load_flux_pipeline(config)
  if config.get("aot_cache_dir", ""):
    from . import aot_cache

    aot_cache.install(config.aot_cache_dir, revision=config.get("aot_build_revision", "") or None)
  kw = {}
  if pipe.t5 is None:
    cfg = pipe.transformer.cfg
    e, p = synthetic_text_conditioning(int(config.get("batch_size", 1)), int(config.max_sequence_length),
                                       cfg.joint_attention_dim, cfg.pooled_projection_dim, int(config.seed))
    kw = {"prompt_embeds": e, "pooled_prompt_embeds": p}
  prompts = list(config.get("prompts", []) or []) or [config.get("prompt", "")]
  results = {}
  for (h, w) in [tuple(r) for r in config.resolutions]:
    t0 = time.perf_counter()
    pipe(height=h, width=w, num_inference_steps=2, output_type="latent", **kw)
    warm = time.perf_counter() - t0
    for rep in range(int(config.get("num_reps", 1))):
      for pi, prompt in enumerate(prompts):
        t0 = time.perf_counter()
        call = dict(kw) if kw else {"prompt": prompt}
        images = pipe(height=h, width=w, **call)
        if torch.cuda.is_available():
          torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        results[(h, w, pi, rep)] = dt
        max_logging.log(f"{h}x{w} prompt {pi} rep {rep}: warm-up {warm:.2f}s generation {dt:.2f}s")
        if int(os.environ.get("RANK", "0")) == 0 and rep == 0:
          out_dir = config.get("output_dir", ".") or "."
          os.makedirs(out_dir, exist_ok=True)
          export_to_png(images[0].cpu().numpy(), os.path.join(out_dir, f"flux_{h}x{w}_{pi}.png"))
  return results


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
