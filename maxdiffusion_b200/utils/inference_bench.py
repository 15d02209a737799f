"""The benchmark workloads besides the training headline, on random-initialised models of the real sizes:

  wan   seconds per denoising step of Wan 2.1 14B (720p x 81 frames by default, classifier-free guidance as a batch of
        two; on N > 1 GPUs 2-D Ulysses x ring context parallelism with U x R = N), optionally followed by the timed
        VAE decode of the result;
  flux  images per second of Flux-dev (1024^2, 28 Euler steps, one image per GPU);
  sdxl  seconds per SDXL UNet training step (batch 8 per GPU, 128^2 latents), with the step's counted FLOPs.

  python -m maxdiffusion_b200.utils.inference_bench wan  [--height 720 --width 1280 --frames 81 --steps 4 --decode]
  python -m maxdiffusion_b200.utils.inference_bench flux [--steps 28 --batch 1]
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m maxdiffusion_b200.utils.inference_bench wan

`bench.py --workload wan_infer | flux_infer | sdxl_train` calls the same functions. Each returns the dict that is
printed as ONE JSON line: `value` is timed on the device with CUDA events (max over ranks) after warm-up, `e2e` is the
same quantity through the public pipeline / trainer call including the host-to-device copy of its inputs from pinned
memory and the device-to-host read of its result. Text encoders are left out (prompts are random embeddings).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

from .. import pyconfig
from ..ops import _lib
from ..parallel.mesh import create_device_mesh, init_distributed

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")


def _world() -> int:
  return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _max_over_ranks(x: float) -> float:
  if _world() > 1:
    t = torch.tensor([x], device="cuda" if torch.cuda.is_available() else "cpu", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
  return x


def _barrier_sync() -> None:
  if _world() > 1:
    dist.barrier()
  if torch.cuda.is_available():
    torch.cuda.synchronize()


def _pinned(t: torch.Tensor) -> torch.Tensor:
  return t.pin_memory() if torch.cuda.is_available() else t


def _nbytes(*ts) -> int:
  return int(sum(t.numel() * t.element_size() for t in ts if torch.is_tensor(t)))


def usp_split(n: int, heads: int) -> int:
  """Ulysses shards U for n ranks (ring gets n / U): the largest U <= 4 that divides both n and the head count."""
  for u in (4, 2, 1):
    if n % u == 0 and heads % u == 0:
      return u
  return 1


def bench_wan(args) -> dict:
  from ..pipelines.wan.wan_pipeline import WanPipeline2_1

  n = _world()
  attention = args.attention or ("flash" if n == 1 else "ulysses_ring")
  ulysses = args.ulysses if args.ulysses > 0 else usp_split(n, 40)
  extra = [f"ulysses_shards={ulysses}"] if n > 1 else []
  config = pyconfig.initialize(
      ["bench", os.path.join(CFG, "base_wan_14b.yml"), "run_name=bench", "random_init=True", f"wan_preset={args.preset}",
       f"height={args.height}", f"width={args.width}", f"num_frames={args.frames}", f"num_inference_steps={args.steps}",
       f"attention={attention}", "guidance_scale=5.0", "log_config=false", "write_metrics=false", *extra])
  mesh = create_device_mesh(config)
  pipe = WanPipeline2_1.from_config(config, load_vae=bool(args.decode), mesh=mesh)
  cfg = pipe.transformer.cfg
  g = torch.Generator().manual_seed(0)
  pe = _pinned(torch.randn((1, 512, cfg.text_dim), generator=g).to(pipe.dtype))
  ne = _pinned(torch.randn((1, 512, cfg.text_dim), generator=g).to(pipe.dtype))
  kw = dict(output_type="latent", return_trace=True)

  def run(steps: int):
    """One public pipeline call: prompt embeddings host -> device, denoising loop, latents device -> host."""
    lat, trace = pipe(prompt_embeds=pe.to(pipe.device, non_blocking=True),
                      negative_prompt_embeds=ne.to(pipe.device, non_blocking=True), num_inference_steps=steps, **kw)
    return lat, lat.float().cpu(), trace

  with torch.no_grad():
    run(max(args.warmup, 1))  # warm-up: kernels, allocator, symmetric buffers
    _barrier_sync()
    l0 = _lib.launch_count()
    t0 = time.perf_counter()
    lat, host_lat, trace = run(args.steps)
    _barrier_sync()
    e2e = _max_over_ranks(time.perf_counter() - t0) / args.steps
    launches = _lib.launch_count() - l0
  sec = _max_over_ranks(trace["denoise_per_step"])
  tokens = ((args.frames - 1) // 4 + 1) * (args.height // 16) * (args.width // 16)
  out = {"metric": "Wan 2.1 14B seconds per denoising step (CFG batch 2)", "value": sec, "unit": "s/step", "n_gpus": n,
         "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": False,
         "scaling": "strong", "vs_baseline": sec / 2.65, "dtype": "bf16",
         "data": "random prompt embeddings, random init",
         "config": {"model": args.preset, "video": f"{args.height}x{args.width}x{args.frames}", "tokens": tokens,
                    "global_batch": 1, "seq_len": tokens, "attention": attention,
                    "parallelism": f"ulysses{ulysses} x ring{n // ulysses}" if n > 1 else "single GPU",
                    "l2": "inputs larger than L2 (every layer's activations and weights exceed 126 MB)",
                    "baseline_note": "reference: 2.6-2.7 s/step on TPU v7x-8 (end_to_end/tpu/run_wan_fast_inference.sh)"},
         "e2e": {"value": e2e, "unit": "s/step", "h2d_bytes_per_step": _nbytes(pe, ne) / args.steps,
                 "d2h_bytes_per_step": _nbytes(host_lat) / args.steps},
         "gpu_launches": launches, "impl": "ours"}
  if args.decode:
    with torch.no_grad():
      pipe.decode_latents(lat[:, :, :2])  # warm-up on two latent frames
      _barrier_sync()
      t0 = time.perf_counter()
      video = pipe.decode_latents(lat)
      _barrier_sync()
      out["config"]["vae_decode_seconds"] = time.perf_counter() - t0
      out["config"]["vae_decode_shape"] = list(video.shape)
  return out


def bench_flux(args) -> dict:
  from ..pipelines.flux.flux_pipeline import FluxPipeline

  n = _world()
  config = pyconfig.initialize(
      ["bench", os.path.join(CFG, "base_flux_dev.yml"), "run_name=bench", "random_init=True", f"flux_preset={args.preset}",
       f"resolution={args.resolution}", f"num_inference_steps={args.steps}", "log_config=false", "write_metrics=false",
       f"ici_data_parallelism={n}", "ici_fsdp_parallelism=1", "ici_context_parallelism=1"])
  pipe = FluxPipeline.from_config(config, load_vae=False)
  cfg = pipe.transformer.cfg
  B = args.batch
  g = torch.Generator().manual_seed(int(os.environ.get("RANK", "0")))
  pe = _pinned(torch.randn((B, 512, cfg.joint_attention_dim), generator=g).to(pipe.dtype))
  pooled = _pinned(torch.randn((B, cfg.pooled_projection_dim), generator=g).to(pipe.dtype))

  def run(steps):
    lat, trace = pipe(prompt_embeds=pe.to(pipe.device, non_blocking=True),
                      pooled_prompt_embeds=pooled.to(pipe.device, non_blocking=True), num_inference_steps=steps,
                      output_type="latent", return_trace=True)
    return lat.float().cpu(), trace

  with torch.no_grad():
    run(max(3, args.warmup))
    _barrier_sync()
    l0 = _lib.launch_count()
    t0 = time.perf_counter()
    host_lat, trace = run(args.steps)
    _barrier_sync()
    e2e_s = _max_over_ranks(time.perf_counter() - t0)
    launches = _lib.launch_count() - l0
  total = _max_over_ranks(trace["denoise_total"])
  value = n * B / total
  return {"metric": "Flux-dev images per second (denoising loop)", "value": value, "unit": "images/s", "n_gpus": n,
          "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": total * 1e3 / args.steps,
          "higher_is_better": True, "scaling": "weak", "vs_baseline": value / 0.73, "dtype": "bf16",
          "data": "random prompt embeddings, random init",
          "config": {"model": args.preset, "resolution": args.resolution, "global_batch": n * B, "seq_len": 512 + (args.resolution // 16) ** 2,
                     "parallelism": f"dp{n}" if n > 1 else "single GPU", "seconds_per_image_batch": total,
                     "l2": "inputs larger than L2 (24 GB of weights stream through every step)",
                     "baseline_note": "reference: 5.5 s for 4 images on TPU v6e-4 = 0.73 images/s"},
          "e2e": {"value": n * B / e2e_s, "unit": "images/s", "h2d_bytes_per_step": _nbytes(pe, pooled) / args.steps,
                  "d2h_bytes_per_step": _nbytes(host_lat) / args.steps},
          "gpu_launches": launches, "impl": "ours"}


def bench_sdxl(args) -> dict:
  from ..trainers.stable_diffusion_trainer import StableDiffusionXLTrainer

  n = _world()
  config = pyconfig.initialize(
      ["bench", os.path.join(CFG, "base_xl.yml"), "run_name=bench", f"per_device_batch_size={args.batch}",
       f"resolution={args.resolution}", "max_train_steps=1000000", "log_config=false", "write_metrics=false",
       "dataset_type=synthetic", f"unet_preset={args.preset}", f"ici_data_parallelism={n}", "ici_fsdp_parallelism=1",
       "ici_context_parallelism=1", f"cuda_graph_train_step={'false' if getattr(args, 'eager', False) else 'true'}"])
  tr = StableDiffusionXLTrainer(config, mesh=create_device_mesh(config))
  for _ in range(max(3, args.warmup)):
    float(tr.train_step(tr.synthetic_batch())["learning/loss"])
  dev = []
  for _ in range(args.steps):
    b = tr.synthetic_batch()
    dev.append({k: v.to(tr.device) for k, v in b.items()})
  _barrier_sync()
  l0 = _lib.launch_count()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for b in dev:
    m = tr.train_step(b)
  e1.record()
  _barrier_sync()
  launches = _lib.launch_count() - l0
  sec = _max_over_ranks(e0.elapsed_time(e1) / 1e3) / args.steps
  host = [tr.synthetic_batch() for _ in range(args.steps)]
  _barrier_sync()
  t0 = time.perf_counter()
  for b in host:
    loss = float(tr.train_step(b)["learning/loss"])
  _barrier_sync()
  e2e = _max_over_ranks(time.perf_counter() - t0) / args.steps
  # counted FLOPs: hooks on one forward pass at the benchmark's shapes
  counted = {"total": 0.0}
  import torch.nn as nn

  def conv_hook(mod, inp, out):
    counted["total"] += 2.0 * out.numel() * mod.weight.shape[1] * mod.weight.shape[2] * mod.weight.shape[3]

  def lin_hook(mod, inp, out):
    counted["total"] += 2.0 * out.numel() * mod.weight.shape[-1]

  from ..models.layers import Linear as KernelLinear

  hooks = []
  for mod in tr.unet.modules():
    if isinstance(mod, nn.Conv2d):
      hooks.append(mod.register_forward_hook(conv_hook))
    elif isinstance(mod, (nn.Linear, KernelLinear)):
      hooks.append(mod.register_forward_hook(lin_hook))
  with torch.no_grad():
    tr.loss({k: v.to(tr.device) for k, v in host[0].items()})
  for h in hooks:
    h.remove()
  flops = 3.0 * counted["total"]
  lat = args.resolution // 8
  images = n * args.batch
  return {"metric": "SDXL UNet training step seconds (batch 8 per GPU, 128^2 latents)", "value": sec, "unit": "s/step",
          "n_gpus": n, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": sec * 1e3, "higher_is_better": False,
          "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic latents and text embeddings",
          "config": {"model": f"SDXL UNet ({args.preset}), random init", "global_batch": images, "seq_len": lat * lat,
                     "parallelism": f"dp{n} (ZeRO-2 optimizer shards)" if n > 1 else "single GPU",
                     "flops_per_step_per_gpu": flops, "tflops_per_gpu": flops / sec / 1e12,
                     "note": "linear + convolution FLOPs counted by module hooks (3 x forward); attention products not included",
                     "l2": "inputs larger than L2 (activations of every stage exceed 126 MB at batch 8)"},
          "e2e": {"value": e2e, "unit": "s/step", "h2d_bytes_per_step": _nbytes(*host[0].values()), "d2h_bytes_per_step": 4},
          "gpu_launches": launches, "loss": loss, "impl": "ours"}


def add_arguments(ap: argparse.ArgumentParser) -> None:
  ap.add_argument("--height", type=int, default=720)
  ap.add_argument("--width", type=int, default=1280)
  ap.add_argument("--frames", type=int, default=81)
  ap.add_argument("--resolution", type=int, default=1024)
  ap.add_argument("--batch", type=int, default=None)
  ap.add_argument("--attention", default=None)
  ap.add_argument("--ulysses", type=int, default=-1, help="Ulysses shards of the 2-D context split (-1: chosen from the GPU count)")
  ap.add_argument("--decode", action="store_true", help="wan: also time the VAE decode of the result")
  ap.add_argument("--preset", default=None)
  ap.add_argument("--eager", action="store_true", help="sdxl: issue every kernel of the step instead of replaying a CUDA graph")


def run_workload(model: str, args) -> dict:
  defaults = {"wan": ("wan2.1-t2v-14b", 4, 1), "flux": ("flux-dev", 28, 1), "sdxl": ("sdxl", 3, 8)}[model]
  if args.preset is None:
    args.preset = defaults[0]
  if args.steps is None:
    args.steps = defaults[1]
  if args.batch is None:
    args.batch = defaults[2]
  if not hasattr(args, "warmup") or args.warmup is None:
    args.warmup = 1
  return {"wan": bench_wan, "flux": bench_flux, "sdxl": bench_sdxl}[model](args)


def main(argv=None) -> int:
  ap = argparse.ArgumentParser()
  ap.add_argument("model", choices=["wan", "flux", "sdxl"])
  ap.add_argument("--steps", type=int, default=None)
  ap.add_argument("--warmup", type=int, default=1)
  add_arguments(ap)
  args = ap.parse_args(argv)
  rank, _, _ = init_distributed()
  out = run_workload(args.model, args)
  if rank == 0:
    print(json.dumps(out), flush=True)
  if _world() > 1:
    dist.destroy_process_group()
  return 0


if __name__ == "__main__":
  sys.exit(main())
