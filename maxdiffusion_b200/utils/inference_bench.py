"""Inference benchmarks on random-initialised models of the real sizes: seconds per denoising step of Wan 2.1 14B
(720p x 81 frames by default, classifier-free guidance as a batch of two) and images per second of Flux-dev
(1024^2, 28 Euler steps). Text encoders and VAEs are left out: prompts are random embeddings, outputs stay latents,
so the numbers are those of the denoising loop (the part the reference's published figures are dominated by).

  python -m maxdiffusion_b200.utils.inference_bench wan  [--height 720 --width 1280 --frames 81 --steps 4 --attention flash]
  python -m maxdiffusion_b200.utils.inference_bench flux [--steps 28 --batch 1]
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m maxdiffusion_b200.utils.inference_bench wan --attention ulysses

One JSON line per run; the loop is timed on the device (synchronised wall clock around the whole loop, after one
untimed warm-up run), max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from .. import pyconfig
from ..parallel.mesh import create_device_mesh, init_distributed

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")


def _max_over_ranks(x: float) -> float:
  if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
  return x


def bench_wan(args) -> dict:
  from ..pipelines.wan.wan_pipeline import WanPipeline2_1

  config = pyconfig.initialize(
      ["bench", os.path.join(CFG, "base_wan_14b.yml"), "run_name=bench", "random_init=True", f"wan_preset={args.preset}",
       f"height={args.height}", f"width={args.width}", f"num_frames={args.frames}", f"num_inference_steps={args.steps}",
       f"attention={args.attention}", "guidance_scale=5.0", "log_config=false", "write_metrics=false"])
  mesh = create_device_mesh(config)
  pipe = WanPipeline2_1.from_config(config, load_vae=False, mesh=mesh)
  cfg = pipe.transformer.cfg
  g = torch.Generator().manual_seed(0)
  pe = torch.randn((1, 512, cfg.text_dim), generator=g).to(pipe.device, pipe.dtype)
  ne = torch.randn((1, 512, cfg.text_dim), generator=g).to(pipe.device, pipe.dtype)
  kw = dict(prompt_embeds=pe, negative_prompt_embeds=ne, output_type="latent", return_trace=True)
  with torch.no_grad():
    pipe(num_inference_steps=2, **kw)  # warm-up: kernels, graphs, allocator
    _, trace = pipe(**kw)
  sec = _max_over_ranks(trace["denoise_per_step"])
  tokens = ((args.frames - 1) // 4 + 1) * (args.height // 16) * (args.width // 16)
  return {"metric": "Wan 2.1 14B seconds per denoising step (CFG batch 2)", "value": sec, "unit": "s/step",
          "n_gpus": dist.get_world_size() if dist.is_initialized() else 1,
          "steps": args.steps, "higher_is_better": False, "dtype": "bf16", "data": "random prompt embeddings, random init",
          "config": {"video": f"{args.height}x{args.width}x{args.frames}", "tokens": tokens, "attention": args.attention,
                     "preset": args.preset}}


def bench_flux(args) -> dict:
  from ..pipelines.flux.flux_pipeline import FluxPipeline

  config = pyconfig.initialize(
      ["bench", os.path.join(CFG, "base_flux_dev.yml"), "run_name=bench", "random_init=True", f"flux_preset={args.preset}",
       f"resolution={args.resolution}", f"num_inference_steps={args.steps}", "log_config=false", "write_metrics=false"])
  pipe = FluxPipeline.from_config(config, load_vae=False)
  cfg = pipe.transformer.cfg
  B = args.batch
  g = torch.Generator().manual_seed(0)
  pe = torch.randn((B, 512, cfg.joint_attention_dim), generator=g).to(pipe.device, pipe.dtype)
  pooled = torch.randn((B, cfg.pooled_projection_dim), generator=g).to(pipe.device, pipe.dtype)
  kw = dict(prompt_embeds=pe, pooled_prompt_embeds=pooled, output_type="latent", return_trace=True)
  with torch.no_grad():
    pipe(num_inference_steps=2, **kw)
    _, trace = pipe(**kw)
  total = _max_over_ranks(trace["denoise_total"])
  world = dist.get_world_size() if dist.is_initialized() else 1
  return {"metric": "Flux-dev images per second (denoising loop)", "value": world * B / total, "unit": "images/s",
          "n_gpus": world, "steps": args.steps, "higher_is_better": True, "dtype": "bf16",
          "data": "random prompt embeddings, random init",
          "config": {"resolution": args.resolution, "batch_per_gpu": B, "seconds_per_image_batch": total, "preset": args.preset}}


def main(argv=None) -> int:
  ap = argparse.ArgumentParser()
  ap.add_argument("model", choices=["wan", "flux"])
  ap.add_argument("--height", type=int, default=720)
  ap.add_argument("--width", type=int, default=1280)
  ap.add_argument("--frames", type=int, default=81)
  ap.add_argument("--resolution", type=int, default=1024)
  ap.add_argument("--steps", type=int, default=None)
  ap.add_argument("--batch", type=int, default=1)
  ap.add_argument("--attention", default="flash")
  ap.add_argument("--preset", default=None)
  args = ap.parse_args(argv)
  if args.steps is None:
    args.steps = 4 if args.model == "wan" else 28
  if args.preset is None:
    args.preset = "wan2.1-t2v-14b" if args.model == "wan" else "flux-dev"
  rank, _, _ = init_distributed()
  out = bench_wan(args) if args.model == "wan" else bench_flux(args)
  if rank == 0:
    print(json.dumps(out), flush=True)
  return 0


if __name__ == "__main__":
  sys.exit(main())
