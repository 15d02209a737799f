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


@contextlib.contextmanager
def _count_kernel_path_flops(total: list):
  """While active, the products that this package runs on its own CUDA kernels add their FLOPs to `total[0]`.

  Those kernels are called through ctypes and never reach PyTorch's dispatcher, so `FlopCounterMode` cannot see them.
  The entry points of `ops.functional` are wrapped for the duration; a call that falls back to PyTorch operators
  (CPU tensors, other dtypes) is left to `FlopCounterMode`, so nothing is counted twice."""
  from .ops import functional as OF

  saved = {name: getattr(OF, name) for name in ("linear", "linear_gated_residual", "attention", "conv2d")}

  def rows_of(x):
    return x.numel() // x.shape[-1]

  def linear(x, weight, *a, **k):
    if OF._fast(x) and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0:
      total[0] += 2 * rows_of(x) * weight.shape[0] * weight.shape[1]
    return saved["linear"](x, weight, *a, **k)

  def linear_gated_residual(x, weight, *a, **k):
    if OF._fast(x):
      total[0] += 2 * rows_of(x) * weight.shape[0] * weight.shape[1]
    return saved["linear_gated_residual"](x, weight, *a, **k)

  def attention(q, k, v, *a, **kw):
    if OF._fast(q) and q.shape[-1] % 8 == 0:
      ks = list(k) if isinstance(k, (list, tuple)) else [k]
      keys = sum(t.shape[1] for t in ks)
      B, Sq, H, D = q.shape
      total[0] += 4 * B * H * Sq * keys * D  # q.k and p.v
    return saved["attention"](q, k, v, *a, **kw)

  def conv2d(x, weight, bias=None, stride=1, padding=1, upsample=False):
    y = saved["conv2d"](x, weight, bias, stride, padding, upsample)
    kk = weight.shape[-1]
    if OF._fast(x) and kk == 3:
      # the 1x1 form goes through `linear` above; everything that is not the 3x3 kernel path is torch.conv2d
      even = x.shape[2] % 2 == 0 and x.shape[3] % 2 == 0
      pad = 0 if padding == "far" else int(padding)
      if stride in (1, 2) and (stride == 1 or even) and ((stride == 1 and pad == 1) or (stride == 2 and pad in (0, 1))):
        total[0] += 2 * y.shape[0] * y.shape[2] * y.shape[3] * weight.shape[0] * weight.shape[1] * kk * kk
    return y

  wrappers = {"linear": linear, "linear_gated_residual": linear_gated_residual, "attention": attention, "conv2d": conv2d}
  try:
    for name, fn in wrappers.items():
      setattr(OF, name, fn)
    yield
  finally:
    for name, fn in saved.items():
      setattr(OF, name, fn)


def _sdpa_cpu_flops(query_shape, key_shape, value_shape, *args, out_shape=None, **kwargs) -> int:
  """q.k and p.v of the CPU flash kernel behind `scaled_dot_product_attention`; `FlopCounterMode` hands a formula the
  SHAPES of the operands ([B, H, S, D])."""
  B, H, Sq, D = query_shape
  return 2 * B * H * Sq * key_shape[2] * D + 2 * B * H * Sq * key_shape[2] * value_shape[3]


def calculate_model_tflops(module: torch.nn.Module, *example_inputs, train: bool = False, **example_kwargs) -> float:
  """TFLOPs of one forward (x3 for training: the backward runs two products per forward product), counted by running
  the module once. PyTorch operators are counted by `FlopCounterMode` (with the CPU attention kernel added to its
  table); the products that run on this package's own kernels are counted at their entry points. Falls back to a
  traversal of Linear / Conv weights when the counter is unavailable.
  Reference: src/maxdiffusion/max_utils.py:851-900 (`calculate_model_tflops`)."""
  own = [0]
  try:
    from torch.utils.flop_counter import FlopCounterMode

    table = {}
    cpu_sdpa = getattr(torch.ops.aten, "_scaled_dot_product_flash_attention_for_cpu", None)
    if cpu_sdpa is not None:
      table[cpu_sdpa] = _sdpa_cpu_flops
    with FlopCounterMode(display=False, custom_mapping=table) as counter, torch.no_grad(), _count_kernel_path_flops(own):
      module(*example_inputs, **example_kwargs)
    flops = counter.get_total_flops() + own[0]
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


# ---- small helpers that scripts written for the reference import from this module --------------------------------------
def _leaves(tree):
  """Tensors of a nested dict / list / tuple (or of a module's parameters), depth first."""
  if isinstance(tree, torch.nn.Module):
    yield from tree.parameters()
  elif torch.is_tensor(tree):
    yield tree
  elif isinstance(tree, dict):
    for v in tree.values():
      yield from _leaves(v)
  elif isinstance(tree, (list, tuple)):
    for v in tree:
      yield from _leaves(v)
  elif tree is not None and hasattr(tree, "__array__"):
    yield torch.as_tensor(tree.__array__())


def l2norm_pytree(tree) -> float:
  """sqrt of the sum of squares over every tensor of a nested structure (reference: src/maxdiffusion/max_utils.py:138-140)."""
  total = 0.0
  for t in _leaves(tree):
    total += float(t.detach().double().pow(2).sum())
  return total ** 0.5


def calculate_num_params_from_pytree(params) -> int:
  return sum(int(t.numel()) for t in _leaves(params))


def get_global_batch_size(per_device_batch_size: float) -> float:
  """Samples per step over all ranks of the job (one rank drives one GPU)."""
  import torch.distributed as dist

  world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else int(os.environ.get("WORLD_SIZE", "1"))
  return per_device_batch_size * world


def get_precision(config) -> str:
  """`precision` of the configuration as the name `torch.set_float32_matmul_precision` takes: DEFAULT -> "high" (TF32
  products for fp32 operands), HIGH -> "high", HIGHEST -> "highest". bf16 operands are unaffected."""
  return {"HIGHEST": "highest"}.get(str(config.get("precision", "DEFAULT")).upper(), "high")


def safe_getattr(obj, name: str, default):
  return getattr(obj, name, default) if obj is not None else default


def profiler_enabled(config) -> bool:
  return bool(config.get("enable_profiler", False))


def is_gpu_backend(raw_keys) -> bool:
  """Always a GPU backend here; a `hardware` key that says otherwise only steers the reference's runtime."""
  return True


def get_git_commit_hash() -> Optional[str]:
  """Current commit of the working directory's repository, for run provenance; None outside a repository."""
  import subprocess

  try:
    return subprocess.check_output(["git", "rev-parse", "HEAD"], stderr=subprocess.DEVNULL).strip().decode("utf-8")
  except (subprocess.CalledProcessError, FileNotFoundError):
    max_logging.log("Warning: could not read a git commit hash (no repository, or no git).")
    return None


def parse_gcs_bucket_and_prefix(destination_gcs_name: str) -> tuple:
  parts = destination_gcs_name.replace("gs://", "").split("/")
  return parts[0], "/".join(parts[1:])


def _no_object_store(what: str):
  raise EnvironmentError(f"{what}: object-store paths (gs://...) need network access, which this installation does not "
                         "use; write to a local or mounted directory and copy from there")


def upload_blob(destination_gcs_name: str, source_file_name: str):
  _no_object_store(f"upload of {source_file_name} to {destination_gcs_name}")


def download_blobs(source_gcs_folder: str, local_destination: str):
  _no_object_store(f"download of {source_gcs_folder}")


def delete_file(file_path: str) -> None:
  try:
    os.remove(file_path)
  except FileNotFoundError:
    max_logging.log(f"File not found: {file_path}")
  except OSError as e:
    max_logging.log(f"Error deleting file {file_path}: {e}")


def save_images(config, images) -> list:
  """Writes every image (PIL images or uint8 arrays) next to `output_file` (default `<run_name>_output_<seed>.png`),
  numbering them when there are several (reference: src/maxdiffusion/max_utils.py:330-344)."""
  import numpy as np
  from PIL import Image

  if str(config.get("output_dir", "") or "").startswith("gs://"):
    _no_object_store("save_images")
  stem, ext = os.path.splitext(str(config.get("output_file", "") or f"{config.get('run_name', 'run')}_output_{config.get('seed', 0)}.png"))
  paths = []
  for i, image in enumerate(images):
    path = f"{stem}{ext}" if len(images) == 1 else f"{stem}_{i}{ext}"
    if os.path.dirname(path):
      os.makedirs(os.path.dirname(path), exist_ok=True)
    if not isinstance(image, Image.Image):
      arr = image.detach().cpu().numpy() if torch.is_tensor(image) else np.asarray(image)
      image = Image.fromarray(arr.astype(np.uint8))
    image.save(path)
    paths.append(path)
  max_logging.log(f"Saved {len(paths)} image(s), first: {paths[0]}")
  return paths


def write_metrics_locally(metrics: dict, step: int, config, file) -> None:
  """One JSON line per step with the scalars, the step and the run name; the file is emptied at step 0 and closed
  after the last step (reference: src/maxdiffusion/max_utils.py:223-242)."""
  import json

  if step == 0:
    file.seek(0)
    file.truncate(0)
  line = {k: float(v) for k, v in metrics.get("scalar", metrics).items()}
  line.update(step=float(step), run_name=str(config.get("run_name", "")))
  file.write(json.dumps(line) + "\n")
  if step == int(config.get("max_train_steps", 0)) - 1:
    file.close()


def initialize_summary_writer(config):
  """TensorBoard writer on rank 0 (None elsewhere, or when TensorBoard is not installed)."""
  if int(os.environ.get("RANK", "0")) != 0:
    return None
  try:
    from torch.utils.tensorboard import SummaryWriter
  except Exception:
    return None
  return SummaryWriter(str(config.get("tensorboard_dir", "") or os.path.join(str(config.get("output_dir", ".")), "tensorboard")))


def close_summary_writer(summary_writer) -> None:
  if summary_writer is not None:
    summary_writer.close()
