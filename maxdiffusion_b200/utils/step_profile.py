"""Where a training step's time goes: device time per kernel family and host issue time, for one rank.

    python -m maxdiffusion_b200.utils.step_profile sdxl_train
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m maxdiffusion_b200.utils.step_profile wan_train --layers 8 --keep-blocks 8

Two measurements of the same warmed-up trainer:
  * host issue time: wall clock of `train_step` calls without any synchronisation inside, against the wall clock
    until the device has finished them; a step whose issue time equals its total time is bound by the host;
  * device time per kernel family from `torch.profiler` (CUPTI activity records) over `--steps` steps. A number taken
    under the profiler is a SHARE, not a benchmark: kernels are a little slower and the host much slower than in a
    plain run, so the table is normalised to the profiled device total.

The reference's counterpart is the JAX profiler switch of its trainers (`enable_profiler`, `profiler_steps`:
src/maxdiffusion/max_utils.py:95-140, trainers/wan_trainer.py:420-470), which writes an XPlane trace for TensorBoard;
this tool prints the table such a trace is usually opened for.
"""
from __future__ import annotations

import argparse
import os
import re
import sys
import time
from collections import defaultdict

import torch

from .. import pyconfig
from ..parallel.mesh import create_device_mesh, init_distributed

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")

# kernel name pattern -> family (first match wins)
FAMILIES = [
    (r"flash_fwd|attn_fwd", "attention forward"), (r"dkv", "attention backward dK/dV"), (r"flash_bwd.*dq|dq_kernel", "attention backward dQ"),
    (r"flash_delta|flash_bwd", "attention backward (other)"), (r"conv_wgrad", "conv weight gradient"), (r"conv_igemm", "conv forward / input gradient"),
    (r"gemm_tcgen05|gemm_kernel|mdb::gemm", "GEMM (tcgen05)"), (r"gn_cl|group_norm", "group norm"), (r"rms_rope", "RMSNorm + RoPE"),
    (r"rms_act|softmax_rows", "VAE row kernels"), (r"ln_mod|layer_norm|ln_fwd|ln_bwd", "layer norm (+ modulation)"), (r"adamw", "AdamW"),
    (r"pull_gather|pull_reduce|peer_copy|pull_a2a|small_allreduce", "peer-memory collectives"), (r"wait_flags|signal_peers|set_flag", "flag kernels"),
    (r"nccl", "NCCL"), (r"colsum|sumsq|lincomb|gelu|silu|gate", "other row kernels of this repository"),
    (r"cutlass|cublas|cudnn|sm\d+_xmma|nvjet|gemv|fmha", "library kernels (cuBLAS / cuDNN)"), (r"at::native|elementwise|vectorized|reduce_kernel|CatArray|index", "PyTorch elementwise / copies"),
    (r"Memcpy|Memset|memcpy|memset", "memcpy / memset"),
]


def family(name: str) -> str:
  for pat, fam in FAMILIES:
    if re.search(pat, name):
      return fam
  return "other"


def summarise(events, steps: int) -> list[tuple[str, int, float]]:
  """[(family, launches per step, device ms per step)] sorted by time, from profiler key averages."""
  acc = defaultdict(lambda: [0, 0.0])
  for e in events:
    dev_us = getattr(e, "device_time_total", None)
    if dev_us is None:
      dev_us = getattr(e, "cuda_time_total", 0.0)
    if getattr(e, "device_type", None) is not None and "CUDA" not in str(e.device_type):
      continue
    if dev_us <= 0:
      continue
    a = acc[family(e.key)]
    a[0] += e.count
    a[1] += dev_us / 1e3
  return sorted(((k, v[0] // steps, v[1] / steps) for k, v in acc.items()), key=lambda r: -r[2])


def _sdxl(args):
  from ..trainers.stable_diffusion_trainer import StableDiffusionXLTrainer

  n = int(os.environ.get("WORLD_SIZE", "1"))
  config = pyconfig.initialize(
      ["profile", os.path.join(CFG, "base_xl.yml"), "run_name=profile", f"per_device_batch_size={args.batch or 8}",
       f"resolution={args.resolution}", "max_train_steps=1000000", "log_config=false", "write_metrics=false",
       "dataset_type=synthetic", f"unet_preset={args.preset or 'sdxl'}", f"ici_data_parallelism={n}", "ici_fsdp_parallelism=1",
       "ici_context_parallelism=1", f"cuda_graph_train_step={'true' if args.graph else 'false'}"])
  tr = StableDiffusionXLTrainer(config, mesh=create_device_mesh(config))
  batches = [{k: v.to(tr.device) for k, v in tr.synthetic_batch().items()} for _ in range(args.steps)]
  return tr, (lambda b: tr.train_step(b)), batches


def _wan(args):
  from ..trainers.wan_trainer import WanTrainer

  n = int(os.environ.get("WORLD_SIZE", "1"))
  over = [f'wan_config_overrides={{"num_layers": {args.layers}}}'] if args.layers > 0 else []
  config = pyconfig.initialize(
      ["profile", os.path.join(CFG, "base_wan_14b.yml"), "run_name=profile", f"height={args.height}", f"width={args.width}",
       f"num_frames={args.frames}", "dataset_type=synthetic", f"per_device_batch_size={1.0 / n}", f"attention={args.attention}",
       "remat_policy=SAVE_ATTENTION", f"remat_keep_blocks={max(0, args.keep_blocks)}", f"wan_preset={args.preset or 'wan2.1-t2v-14b'}",
       "warmup_steps_fraction=0.0", "max_train_steps=1000000", "log_config=false", "write_metrics=false", "flow_shift=5.0", *over])
  tr = WanTrainer(config, mesh=create_device_mesh(config))
  data = tr.load_dataset()
  batches = [tr.to_device(next(data)) for _ in range(args.steps)]
  return tr, (lambda b: tr.train_step(b, host_inputs=False)), batches


def main(argv=None) -> int:
  ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
  ap.add_argument("workload", choices=["wan_train", "sdxl_train"])
  ap.add_argument("--steps", type=int, default=2)
  ap.add_argument("--layers", type=int, default=0, help="wan_train: number of blocks (0 = the preset's)")
  ap.add_argument("--keep-blocks", type=int, default=0)
  ap.add_argument("--height", type=int, default=480)
  ap.add_argument("--width", type=int, default=832)
  ap.add_argument("--frames", type=int, default=81)
  ap.add_argument("--attention", default="tokamax_ring")
  ap.add_argument("--preset", default=None)
  ap.add_argument("--resolution", type=int, default=1024)
  ap.add_argument("--batch", type=int, default=None)
  ap.add_argument("--graph", action="store_true", help="sdxl_train: replay the step from a CUDA graph")
  ap.add_argument("--rows", type=int, default=25, help="kernel names listed under the family table")
  args = ap.parse_args(argv)
  rank, world, _ = init_distributed()
  tr, step, batches = (_sdxl if args.workload == "sdxl_train" else _wan)(args)
  for b in batches[:1] * 3:  # warm-up: allocator, packed weights, tuned variants
    float(step(b)["learning/loss"])
  torch.cuda.synchronize()
  t0 = time.perf_counter()
  for b in batches:
    m = step(b)
  issued = time.perf_counter() - t0
  torch.cuda.synchronize()
  total = time.perf_counter() - t0
  from torch.profiler import ProfilerActivity, profile

  with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
    for b in batches:
      m = step(b)
    torch.cuda.synchronize()
  events = prof.key_averages()
  rows = summarise(events, len(batches))
  if rank == 0:
    dev_total = sum(r[2] for r in rows)
    print(f"{args.workload}: {world} rank(s), {len(batches)} step(s) after 3 warm-up steps")
    print(f"plain run : host issue {issued / len(batches) * 1e3:9.1f} ms/step   until the device is done {total / len(batches) * 1e3:9.1f} ms/step")
    print(f"profiled  : device busy {dev_total:9.1f} ms/step (sum over kernels, rank 0)")
    print(f"{'family':48s} {'launches':>9s} {'ms/step':>10s} {'share':>7s}")
    for fam, cnt, ms in rows:
      print(f"{fam:48s} {cnt:9d} {ms:10.2f} {ms / max(dev_total, 1e-9):7.1%}")
    print()
    print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=args.rows, max_name_column_width=90))
  if world > 1:
    import torch.distributed as dist

    dist.barrier()
    dist.destroy_process_group()
  return 0


if __name__ == "__main__":
  sys.exit(main())
