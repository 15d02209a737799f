"""Run-time utilities: profiler, mesh construction, optimizer / schedule factories, model-FLOP counting.

Counterpart of the reference's `max_utils.py` (src/maxdiffusion/max_utils.py): `Profiler` (:143-211),
`create_device_mesh` (:453-506), `create_learning_rate_schedule` (:658-680), `create_optimizer` (:683-696),
`get_flash_block_sizes` (:717-818), `calculate_model_tflops` (:851-900), memory report (:825-846).
"""
from __future__ import annotations

import contextlib
import os
from typing import Optional

import torch

from . import max_logging
from .parallel.fsdp import AdamWConfig, lr_schedule
from .parallel.mesh import create_device_mesh, fill_unspecified_mesh_axes, init_distributed  # noqa: F401 (re-export)


class Profiler:
  """torch.profiler trace (Chrome / TensorBoard format) over a window of steps, with NVTX ranges.

  `maybe_start(step)` / `maybe_stop(step)` implement the reference's window: start after
  `skip_first_n_steps_for_profiler`, stop `profiler_steps` later. `profiler: nsys` only emits NVTX ranges so an
  external Nsight Systems capture sees the steps (reference: trainers/flux_trainer.py:432-438).
  """

  def __init__(self, config, output_dir: Optional[str] = None):
    self.enabled = bool(config.get("enable_profiler", False))
    self.mode = str(config.get("profiler", "") or "")
    self.first = int(config.get("skip_first_n_steps_for_profiler", 5))
    self.steps = int(config.get("profiler_steps", 10))
    self.dir = output_dir or os.path.join(config.get("tensorboard_dir", "") or ".", "profile")
    self._prof = None
    self.active = False

  def start(self) -> None:
    if not self.enabled or self.active:
      return
    self.active = True
    if self.mode == "nsys":
      return
    os.makedirs(self.dir, exist_ok=True)
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
      acts.append(torch.profiler.ProfilerActivity.CUDA)
    self._prof = torch.profiler.profile(activities=acts, record_shapes=False)
    self._prof.__enter__()

  def stop(self) -> None:
    if not self.active:
      return
    self.active = False
    if self._prof is not None:
      self._prof.__exit__(None, None, None)
      path = os.path.join(self.dir, f"trace_rank{os.environ.get('RANK', '0')}.json")
      self._prof.export_chrome_trace(path)
      max_logging.log(f"profiler trace written to {path}")
      self._prof = None

  def maybe_start(self, step: int) -> None:
    if self.enabled and step == self.first:
      self.start()

  def maybe_stop(self, step: int) -> None:
    if self.active and step >= self.first + self.steps - 1:
      self.stop()

  def __enter__(self):
    self.start()
    return self

  def __exit__(self, *exc):
    self.stop()


@contextlib.contextmanager
def named_scope(name: str, enabled: bool = True):
  """NVTX range (the reference's `jax.named_scope`, gated by `enable_jax_named_scopes`)."""
  if enabled and torch.cuda.is_available():
    torch.cuda.nvtx.range_push(name)
    try:
      yield
    finally:
      torch.cuda.nvtx.range_pop()
  else:
    yield


def create_learning_rate_schedule(learning_rate: float, schedule_steps: int, warmup_steps_fraction: float):
  return lambda step: lr_schedule(step, learning_rate, schedule_steps, warmup_steps_fraction)


def create_optimizer(config) -> AdamWConfig:
  """AdamW (+ value clip, + global-norm clip; applied in the order clip(value) -> clip_by_global_norm -> adamw)."""
  return AdamWConfig(
      lr=float(config.learning_rate), b1=float(config.adam_b1), b2=float(config.adam_b2), eps=float(config.adam_eps),
      weight_decay=float(config.adam_weight_decay),
      clip_value=float(config.max_grad_value) if config.get("opt_enable_grad_clipping", False) else 0.0,
      clip_global_norm=float(config.max_grad_norm) if config.get("opt_enable_grad_global_norm_clipping", False) else 0.0,
      state_dtype=config.get("opt_state_dtype", torch.bfloat16))


def get_flash_block_sizes(config) -> Optional[dict]:
  """`flash_block_sizes` from the config (empty dict -> kernel defaults). Keys kept: block_q, block_kv, ... ."""
  sizes = config.get("flash_block_sizes", None)
  return dict(sizes) if sizes else None


def calculate_model_tflops(module: torch.nn.Module, *example_inputs, train: bool = False, **example_kwargs) -> float:
  """TFLOPs of one forward (x3 for training) counted by running the module under FlopCounterMode on meta-free CPU
  or CUDA inputs; falls back to a traversal of Linear / Conv weights when the counter is unavailable."""
  try:
    from torch.utils.flop_counter import FlopCounterMode

    with FlopCounterMode(display=False) as counter, torch.no_grad():
      module(*example_inputs, **example_kwargs)
    flops = counter.get_total_flops()
  except Exception:
    flops = 0
    for m in module.modules():
      w = getattr(m, "weight", None)
      if w is not None and w.dim() >= 2:
        flops += 2 * w.numel()
  return (3 if train else 1) * flops / 1e12


def get_memory_allocations() -> dict:
  if not torch.cuda.is_available():
    return {}
  free, total = torch.cuda.mem_get_info()
  stats = {"allocated_gb": torch.cuda.memory_allocated() / 2**30, "reserved_gb": torch.cuda.memory_reserved() / 2**30,
           "free_gb": free / 2**30, "total_gb": total / 2**30}
  max_logging.log("memory: " + ", ".join(f"{k}={v:.2f}" for k, v in stats.items()))
  return stats
