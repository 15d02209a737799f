"""The training loop shared by the Stable Diffusion / SDXL / Dreambooth and Flux trainers: resume from the latest
checkpoint, data prefetch on a host thread, encoded-batch caching, metrics, periodic and final checkpoints, periodic
evaluation, and the once-per-step device status check.

Reference: `BaseStableDiffusionTrainer.start_training` / `training_loop`
(src/maxdiffusion/trainers/base_stable_diffusion_trainer.py:115-197, sdxl_trainer.py:178-291) and the same skeleton in
`FluxTrainer` (flux_trainer.py:355-468): load or restore state, build the (cached) dataset, loop over steps writing
metrics, save every `checkpoint_every` steps and at the end.
"""
from __future__ import annotations

import os
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Callable, Iterator, Optional

import torch
import torch.distributed as dist

from .. import max_logging
from ..ops import _lib
from ..train_utils import MetricsWriter, load_next_batch


class EncodedBatchCache:
  """Keeps the encoded form of every batch of a FINITE dataset on the host, so that the frozen VAE / text encoders run
  once per sample and later epochs replay their outputs (the reference caches latents and text-encoder outputs in the
  dataset itself: `cache_latents_text_encoder_outputs`, input_pipeline_interface.py:60-140)."""

  def __init__(self, source: Iterator[dict], encode: Callable[[dict], dict], max_batches: int = 4096):
    self.source, self.encode, self.max_batches = source, encode, max_batches
    self.store: list = []
    self.replay = False
    self.pos = 0

  def __iter__(self):
    return self

  def __next__(self) -> dict:
    if self.replay:
      if not self.store:
        raise StopIteration
      b = self.store[self.pos % len(self.store)]
      self.pos += 1
      return b
    try:
      raw = next(self.source)
    except StopIteration:
      self.replay, self.pos = True, 0
      return next(self)
    enc = {k: (v.detach().to("cpu") if torch.is_tensor(v) else v) for k, v in self.encode(raw).items()
           if k not in ("pixel_values", "captions", "input_ids", "input_ids_2")}
    if len(self.store) < self.max_batches:
      self.store.append(enc)
    return enc


def _health_monitor(config, mesh):
  """Heartbeats through the rendezvous store for multi-rank runs (`parallel.health`): a rank that raised or fell
  silent is seen by the others BEFORE their next launch, so they leave with an exception instead of waiting in a
  collective. Together with a launcher that restarts the ranks (`torch.distributed.run --max-restarts`,
  `gpu_multi_process_run.sh`) and the restore at the top of this loop, that is the recovery path: fail, tear down,
  start again from the last checkpoint."""
  if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1 and config.get("health_monitor", True)):
    return None
  from ..parallel.health import HealthMonitor

  # one key space per incarnation of the job: a restarted run must not read the failure that ended the previous one
  incarnation = os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")
  return HealthMonitor(timeout_s=float(config.get("health_timeout_s", 120.0)), prefix=f"mdb_health/{incarnation}").start()


def _maybe_inject_failure(config, trainer) -> None:
  """Host-side fault injection for the recovery tests: the configured rank raises before the configured step, in
  the first incarnation of the job only (a launcher that restarts the ranks counts incarnations in
  TORCHELASTIC_RESTART_COUNT). Nothing on the device is touched."""
  at = int(config.get("inject_failure_at_step", -1))
  if at < 0 or trainer.step != at or int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")) != 0:
    return
  if trainer.mesh.rank == int(config.get("inject_failure_rank", 0)):
    raise RuntimeError(f"injected host failure on rank {trainer.mesh.rank} before step {at}")


class PhaseTimer:
  """Wall-clock duration of the phases around the steps (restore, data set, the loop itself, the final save), written
  as "Starting: ..." / "Finished: ... - Duration: ... seconds" lines: into `timing_metrics_file` when
  `write_timing_metrics` is set and the file is named, else into the log; rank 0 only
  (reference: src/maxdiffusion/trainers/base_stable_diffusion_trainer.py:84-103, `_time_and_log_call`)."""

  def __init__(self, config, rank: int = 0):
    self.file = str(config.get("timing_metrics_file", "") or "") if config.get("write_timing_metrics", False) else ""
    self.rank = rank
    self.durations: dict = {}

  def _emit(self, line: str) -> None:
    if self.rank != 0:
      return
    if self.file:
      os.makedirs(os.path.dirname(os.path.abspath(self.file)), exist_ok=True)
      with open(self.file, "a", encoding="utf-8") as f:
        f.write(line + "\n")
    else:
      max_logging.log(line)

  def __call__(self, description: str, fn: Callable, *args, **kwargs):
    self._emit(f"Starting: {description}...")
    t0 = time.perf_counter()
    out = fn(*args, **kwargs)
    self.durations[description] = time.perf_counter() - t0
    self._emit(f"Finished: {description} - Duration: {self.durations[description]:.4f} seconds")
    return out


def run_training_loop(trainer, data, checkpointer=None, evaluate: Optional[Callable[[int], dict]] = None):
  """Drives `trainer.train_step` until `max_train_steps`. `trainer` provides `config`, `mesh`, `step` and `train_step`;
  `checkpointer` provides `maybe_restore(trainer)` and `save(step, trainer)`. `data` is an iterator of batches or a
  function that builds one; the function is called AFTER the restore, so that it can start at the restored step."""
  from ..parallel.health import guarded_step

  config = trainer.config
  max_steps = int(config.max_train_steps)
  every = int(config.get("checkpoint_every", -1))
  eval_every = int(config.get("eval_every", -1))
  timed = PhaseTimer(config, trainer.mesh.rank)
  trainer.phase_timer = timed
  if checkpointer is not None:
    restored = timed("restore checkpoint", checkpointer.maybe_restore, trainer)
    if restored is not None:
      trainer.step = int(restored)
  if callable(data) and not hasattr(data, "__next__"):
    data = iter(timed("load dataset", data))
  # sources that can save their position (grain) continue where the checkpoint left them
  source = getattr(data, "source", data)
  if checkpointer is not None and hasattr(source, "set_state") and hasattr(checkpointer, "restore_iterator"):
    checkpointer.restore_iterator(source)
  writer = MetricsWriter(config, trainer.mesh.rank)
  monitor = _health_monitor(config, trainer.mesh)
  step_barrier = bool(config.get("health_step_barrier", True))
  pool = ThreadPoolExecutor(max_workers=1)
  reuse = {"batch": None}   # `reuse_example_batch`: the first batch is served for every step

  def fetch():
    reuse["batch"] = load_next_batch(data, reuse["batch"], config)
    return reuse["batch"]

  nxt = pool.submit(fetch)
  timed._emit("Starting: training loop...")
  loop_t0 = time.perf_counter()
  try:
    while trainer.step < max_steps:
      batch = nxt.result()
      nxt = pool.submit(fetch)
      t0 = time.perf_counter()
      with guarded_step(monitor, trainer.step):  # peers checked first; this rank's exception is announced to them
        _maybe_inject_failure(config, trainer)
        if monitor is not None and step_barrier:
          # every rank has reached this step alive (or its failure report is seen here) before any rank enters the
          # step's collectives: a few store round trips per step against a collective that would wait out its timeout
          monitor.barrier(timeout_s=float(config.get("health_timeout_s", 120.0)))
        m = trainer.train_step(batch)
        scalars = {k: float(v) for k, v in m.items()}  # device -> host: ends the step
        _lib.raise_on_device_status_if_loaded()
      scalars["perf/step_time_seconds"] = time.perf_counter() - t0
      writer.write(trainer.step, scalars)
      if evaluate is not None and eval_every > 0 and trainer.step % eval_every == 0:
        writer.write(trainer.step, {f"eval/{k}": float(v) for k, v in evaluate(trainer.step).items()})
      if checkpointer is not None and every > 0 and trainer.step % every == 0:
        _save(checkpointer, trainer, source)
    timed.durations["training loop"] = time.perf_counter() - loop_t0
    timed._emit(f"Finished: training loop - Duration: {timed.durations['training loop']:.4f} seconds")
    if checkpointer is not None and config.get("save_final_checkpoint", False) and (every <= 0 or trainer.step % every != 0):
      timed("final checkpoint", _save, checkpointer, trainer, source)
  finally:
    writer.close()
    if monitor is not None:
      monitor.stop()
    pool.shutdown(wait=False, cancel_futures=True)
    if checkpointer is not None and getattr(checkpointer, "manager", None) is not None:
      checkpointer.manager.wait_until_finished()
  return trainer


def _save(checkpointer, trainer, source=None) -> None:
  _lib.raise_on_device_status_if_loaded()
  if source is not None and hasattr(source, "get_state"):
    # note: the loop prefetches one batch, so the saved position is one batch ahead of the step; a resumed run skips
    # that batch instead of seeing it twice
    checkpointer.save(trainer.step, trainer, data_iterator=source)
  else:
    checkpointer.save(trainer.step, trainer)
  if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
    dist.barrier()  # saving is rank-asymmetric host work: start the next step together
