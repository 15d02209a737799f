"""Headline benchmark: Wan2.1-14B text-to-video TRAINING tokens/s (480x832x81 frames = 32 760 tokens).

  python bench.py --gpus 1 --steps 3 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W

One sample per step (global batch 1, strong scaling): on N GPUs the sequence is context-parallel over all N ranks
(ring schedule) and the weights + AdamW moments are sharded over the same ranks. bf16 compute, random-init weights
of the real 40-layer architecture, synthetic latents / text embeddings of the named shape, remat per block, AdamW
step inside the timed region. Prints ONE JSON line (rank 0).

Two timed regions of K steps each, both after W warm-up steps:
  * `value`: CUDA events around K steps with the batch already on the device (max over ranks);
  * `e2e`: the public `WanTrainer.train_step(host_batch)` path — pinned host batch -> device copy every step and a
    device -> host read of the loss every step — timed by the host clock between barriers + synchronize.

Other arms and workloads:
  --impl reference   the unmodified reference (prints its `unavailable` line: JAX is not installed here);
  --impl library     a yardstick, NOT the reference: the same model, trainer and sharding with every kernel of this
                     repository switched off (`F.linear` = cuBLAS, PyTorch SDPA, eager norms, NCCL all-gather /
                     reduce-scatter, eager AdamW), so that a same-box end-to-end ratio exists;
  --workload wan_infer | flux_infer | sdxl_train   the other metrics of the baseline (Wan 720p seconds per denoising
                     step, Flux-dev images per second, SDXL UNet training step), see `utils/inference_bench.py`.
  --keep-blocks K    fixes the remat policy (K blocks keep their activations) so that runs at different GPU counts do
                     the same work; the default keeps as many blocks as memory allows.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

BASELINE_TOKENS_PER_S = 2100.0  # reference README: 36.0 s/step at 75 600 tokens on TPU v5p-8 (4 chips)


def reference_arm():
  print(json.dumps({"impl": "reference",
                    "unavailable": "reference needs jax/flax/orbax and the hatchling build backend; none is in the "
                                   "image or the offline wheelhouse (pip install --no-index failed: No module named 'hatchling')"}))
  return 0


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

  def __init__(self, index: int):
    self.index = index
    self.samples, self.max_mhz, self.reasons = [], None, set()
    self._stop = threading.Event()
    self.thread = threading.Thread(target=self._run, daemon=True)

  def _run(self):
    q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    while not self._stop.is_set():
      try:
        out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                             capture_output=True, text=True, timeout=5).stdout.strip().splitlines()[0]
        f = [x.strip() for x in out.split(",")]
        self.samples.append(float(f[0]))
        self.max_mhz = float(f[1])
        for n, v in zip(names, f[2:6]):
          if v.lower().startswith("active"):
            self.reasons.add(n)
      except Exception:
        pass
      self._stop.wait(0.2)

  def start(self):
    self.thread.start()

  def stop(self) -> dict:
    self._stop.set()
    self.thread.join(timeout=10)
    return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons), "samples": len(self.samples)}


def wan_step_flops(cfg, tokens: int, text_len: int, recomputed_blocks: int) -> dict:
  """FLOPs of one training step of one sample. `algorithmic`: forward + backward of every product (linear layers
  3 x forward; attention forward + 2.5 x forward for its backward, which recomputes S). `executed` adds what
  rematerialisation runs again: the linear layers and the cross-attention of the recomputed blocks (the self-attention
  output is saved, not recomputed)."""
  d, f, L = cfg.dim, cfg.ffn_dim, cfg.num_layers
  lin = 2 * tokens * (4 * d * d + 2 * d * d + 2 * d * f) + 2 * text_len * 2 * d * d  # self qkvo, cross q/o, ffn, cross k/v
  self_attn = 4 * tokens * tokens * d
  cross_attn = 4 * tokens * text_len * d
  algorithmic = L * (3 * lin + 3.5 * (self_attn + cross_attn))
  executed = algorithmic + recomputed_blocks * (lin + cross_attn)
  return {"algorithmic": float(algorithmic), "executed": float(executed)}


def kept_block_bytes(cfg, tokens: int, ranks: int = 1) -> int:
  """Activation bytes a Wan block holds for its backward when it is not rematerialised (bf16): the residual stream
  and its three modulated norms, q / k / v before and after RMSNorm + RoPE, the attention output and its projection,
  the cross-attention query, output and projection, the two FFN hidden tensors, plus fp32 softmax statistics."""
  d, f = cfg.dim, cfg.ffn_dim
  per_token = 2 * (4 * d + 3 * d + 3 * d + 2 * d + 3 * d + 2 * f) + 16 * cfg.num_attention_heads
  if ranks > 1:  # ring attention keeps the gathered K and V of all ranks for its backward
    per_token += 2 * 2 * ranks * d
  return int(1.15 * per_token * tokens)


def other_workload(args) -> int:
  """The baseline's other metrics (`utils/inference_bench.py`), printed with the same JSON contract."""
  import torch
  import torch.distributed as dist

  here = os.path.dirname(os.path.abspath(__file__))
  sys.path.insert(0, here)
  from maxdiffusion_b200.parallel.mesh import init_distributed
  from maxdiffusion_b200.utils import inference_bench as IB

  if args.impl == "library":
    from maxdiffusion_b200.ops import functional as OF

    OF.set_library_mode(True)
  rank, world, local_rank = init_distributed()
  model = {"wan_infer": "wan", "flux_infer": "flux", "sdxl_train": "sdxl"}[args.workload]
  if args.workload == "wan_infer" and (args.height, args.width) == (480, 832):
    args.height, args.width = 720, 1280  # the inference metric is quoted at 720p; --height / --width override it
  args.preset = None if args.preset == "wan2.1-t2v-14b" and model != "wan" else args.preset
  args.attention = None if args.attention == "tokamax_ring" else args.attention
  sampler = ClockSampler(local_rank)
  sampler.start()
  out = IB.run_workload(model, args)
  out["clocks"] = sampler.stop()
  out["impl"] = args.impl
  if rank == 0:
    print(json.dumps(out))
  if world > 1:
    dist.destroy_process_group()
  return 0


def main() -> int:
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=None, help="timed steps (default 3; flux_infer: 28 Euler steps, wan_infer: 4)")
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="ours")
  ap.add_argument("--remat", default="SAVE_ATTENTION", help="FULL | SAVE_ATTENTION")
  ap.add_argument("--keep-blocks", type=int, default=-1,
                  help="blocks that keep their activations instead of recomputing them (-1: as many as the memory of the GPU allows)")
  ap.add_argument("--preset", default="wan2.1-t2v-14b", help="model preset (anything but the default is a smoke run)")
  ap.add_argument("--height", type=int, default=480)
  ap.add_argument("--width", type=int, default=832)
  ap.add_argument("--frames", type=int, default=81)
  ap.add_argument("--attention", default="tokamax_ring")
  ap.add_argument("--ring-kv-transport", default=None, choices=["sm", "dma"],
                  help="wan_train: how ring attention stages remote K/V (default: the configuration's `ring_kv_transport`)")
  ap.add_argument("--workload", default="wan_train", choices=["wan_train", "wan_infer", "flux_infer", "sdxl_train"])
  ap.add_argument("--resolution", type=int, default=1024)
  ap.add_argument("--batch", type=int, default=None)
  ap.add_argument("--ulysses", type=int, default=-1)
  ap.add_argument("--decode", action="store_true", help="wan_infer: also time the VAE decode")
  ap.add_argument("--eager", action="store_true", help="sdxl_train: issue every kernel instead of replaying a CUDA graph")
  args = ap.parse_args()
  if args.impl == "reference":
    return reference_arm()
  if args.impl not in ("ours", "library"):
    print(f"unknown --impl {args.impl}", file=sys.stderr)
    return 2
  if args.warmup < 3:
    args.warmup = 3
  if args.workload != "wan_train":
    return other_workload(args)
  if args.steps is None:
    args.steps = 3

  import torch
  import torch.distributed as dist

  here = os.path.dirname(os.path.abspath(__file__))
  sys.path.insert(0, here)
  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.ops import _lib
  from maxdiffusion_b200.parallel.mesh import create_device_mesh, init_distributed
  from maxdiffusion_b200.trainers.wan_trainer import WanTrainer

  if args.impl == "library":
    from maxdiffusion_b200.ops import functional as OF

    OF.set_library_mode(True)
  rank, world, local_rank = init_distributed()
  if world != args.gpus:
    if rank == 0:
      print(f"warning: --gpus {args.gpus} but WORLD_SIZE is {world}; using {world}", file=sys.stderr)
  n = world
  config = pyconfig.initialize(
      ["bench", os.path.join(here, "maxdiffusion_b200", "configs", "base_wan_14b.yml"), "run_name=bench",
       f"height={args.height}", f"width={args.width}", f"num_frames={args.frames}", "dataset_type=synthetic",
       f"per_device_batch_size={1.0 / n}", f"attention={args.attention}", f"remat_policy={args.remat}",
       f"remat_keep_blocks={max(0, args.keep_blocks)}",
       f"wan_preset={args.preset}", "warmup_steps_fraction=0.0", "max_train_steps=1000000", "log_config=false",
       "write_metrics=false", "flow_shift=5.0",
       f"peer_memory_transport={'false' if args.impl == 'library' else 'true'}"]
      + ([f"ring_kv_transport={args.ring_kv_transport}"] if args.ring_kv_transport else []))
  mesh = create_device_mesh(config)
  trainer = WanTrainer(config, mesh=mesh)
  data = trainer.load_dataset()
  seq_len = trainer.seq_len()

  def barrier_sync():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  # ---- how many blocks may keep their activations: one probing step with full remat, then the memory that is left
  # over (minus a reserve) is divided by what a kept block holds. Every rank takes the minimum.
  keep = max(0, args.keep_blocks)
  if args.keep_blocks < 0:
    m = trainer.train_step(next(data))
    float(m["learning/loss"])
    torch.cuda.synchronize()
    free, total = torch.cuda.mem_get_info()
    peak = torch.cuda.max_memory_reserved()
    per_block = kept_block_bytes(trainer.model.cfg, -(-seq_len // n), n) * (2 if args.impl == "library" else 1)
    room = total - peak - int(0.08 * total)
    keep_t = torch.tensor([max(0, min(len(trainer.model.blocks), room // per_block))], device="cuda")
    if world > 1:
      dist.all_reduce(keep_t, op=dist.ReduceOp.MIN)
    keep = int(keep_t.item())
    trainer.model.remat_keep_blocks = keep

  # ---- warm-up (through the public path)
  for _ in range(args.warmup):
    m = trainer.train_step(next(data))
    float(m["learning/loss"])
  if args.impl == "ours":
    _lib.raise_on_device_status()

  # ---- region 1: device-timed, inputs resident on the device
  dev_batches = [trainer.to_device(next(data)) for _ in range(args.steps)]
  sampler = ClockSampler(local_rank)
  barrier_sync()
  sampler.start()
  launches0 = _lib.launch_count()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for b in dev_batches:
    m = trainer.train_step(b, host_inputs=False)
  e1.record()
  barrier_sync()
  clocks = sampler.stop()
  launches = _lib.launch_count() - launches0
  ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
  if world > 1:
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
  ms_per_step = ms.item() / args.steps
  last_loss = float(m["learning/loss"])
  if args.impl == "ours":
    _lib.raise_on_device_status()

  # ---- region 2: end to end through the public API (H2D of the batch and D2H of the loss every step)
  host_batches = [next(data) for _ in range(args.steps)]
  h2d = sum(t.numel() * t.element_size() for t in host_batches[0].values() if torch.is_tensor(t))
  barrier_sync()
  t0 = time.perf_counter()
  for b in host_batches:
    m = trainer.train_step(b)
    last_loss = float(m["learning/loss"])  # device -> host read of the step's result
  barrier_sync()
  e2e_s = torch.tensor([time.perf_counter() - t0], device="cuda")
  if world > 1:
    dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
  e2e_tokens_per_s = seq_len * args.steps / e2e_s.item()

  value = seq_len * 1000.0 / ms_per_step
  n_blocks = len(trainer.model.blocks)
  flops = wan_step_flops(trainer.model.cfg, seq_len, 512, 0 if args.remat == "NONE" else n_blocks - keep)
  official = args.preset == "wan2.1-t2v-14b" and (args.height, args.width, args.frames) == (480, 832, 81)
  if rank == 0:
    print(json.dumps({
        "metric": "Wan-14B train tokens/s" if official else f"{args.preset} train tokens/s (smoke, not the headline config)",
        "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": value / BASELINE_TOKENS_PER_S, "dtype": "bf16", "data": "synthetic",
        "config": {"model": "Wan2.1-T2V-14B (40 layers, dim 5120, 40 heads, ffn 13824), random init" if official else args.preset,
                   "global_batch": 1, "seq_len": seq_len,
                   "parallelism": f"cp{n} ring x fsdp over the same {n} ranks" if n > 1 else "single GPU",
                   "ring_kv_transport": str(config.get("ring_kv_transport", "dma")) if n > 1 else None,
                   "video": f"{args.height}x{args.width}x{args.frames}",
                   "remat": f"per block ({args.remat}); the last {keep} of {len(trainer.model.blocks)} blocks keep their activations "
                            f"(peak {torch.cuda.max_memory_reserved() / 2**30:.0f} GiB reserved)",
                   "optimizer": "AdamW, bf16 moments, stochastic rounding, step inside the timed region",
                   "l2": "inputs larger than L2 (activations and weights of every block exceed 126 MB)",
                   "baseline_note": "published reference figure: 2100 tokens/s on TPU v5p-8 at 720p (75 600 tokens)"},
        "clocks": clocks,
        "e2e": {"value": e2e_tokens_per_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                "seconds_per_step": e2e_s.item() / args.steps},
        "flops_per_step": flops["algorithmic"], "executed_flops_per_step": flops["executed"],
        "tflops_per_gpu": flops["algorithmic"] / (ms_per_step * 1e-3) / n / 1e12,
        "executed_tflops_per_gpu": flops["executed"] / (ms_per_step * 1e-3) / n / 1e12,
        "gpu_launches": launches, "loss": last_loss, "impl": args.impl}))
  if world > 1:
    dist.destroy_process_group()
  return 0


if __name__ == "__main__":
  sys.exit(main())
