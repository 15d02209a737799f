"""Training-side utilities: config validation, metric names, and the metrics writer.

The writer keeps the reference's behaviour (src/maxdiffusion/train_utils.py:106-209): scalars are pushed to a
queue drained by a writer thread (TensorBoard when `torch.utils.tensorboard` is importable, plus an optional
JSONL `metrics_file` consumed by `end_to_end/eval_assert.py`), and a console line
`completed step: N, seconds: ..., TFLOP/s/device: ..., loss: ...` is printed by rank 0.
"""
from __future__ import annotations

import contextlib
import json
import os
import queue
import threading
from typing import Optional

import torch

from . import max_logging


def validate_train_config(config) -> None:
  """Fail early on settings that cannot train (reference: train_utils.py:38-76)."""
  if not config.get("run_name", ""):
    raise ValueError("run_name must be set for training (it names the output sub-directories)")
  if int(config.get("max_train_steps", 0)) <= 0 and int(config.get("num_train_epochs", 0)) <= 0:
    raise ValueError("max_train_steps or num_train_epochs must be positive")
  if str(config.get("dataset_type", "")) not in ("tfrecord", "hf", "tf", "grain", "synthetic"):
    raise ValueError(f"unknown dataset_type {config.get('dataset_type')}")


def compute_snr(alphas_cumprod: torch.Tensor, timesteps: torch.Tensor) -> torch.Tensor:
  """SNR(t) = alpha_bar / (1 - alpha_bar) (reference: train_utils.py:217)."""
  a = alphas_cumprod.to(timesteps.device)[timesteps.long()]
  return a / (1.0 - a)


def generate_timestep_weights(config, num_timesteps: int) -> torch.Tensor:
  """Sampling weights over timesteps for `timestep_bias` strategies later/earlier/range/none."""
  bias = config.get("timestep_bias", {"strategy": "none"}) or {"strategy": "none"}
  w = torch.ones(num_timesteps)
  strategy = bias.get("strategy", "none")
  if strategy == "none":
    return w / w.sum()
  n_bias = int(float(bias.get("portion", 0.25)) * num_timesteps)
  mult = float(bias.get("multiplier", 1.0))
  if strategy == "later":
    w[-n_bias:] *= mult
  elif strategy == "earlier":
    w[:n_bias] *= mult
  elif strategy == "range":
    w[int(bias.get("begin", 0)):int(bias.get("end", num_timesteps))] *= mult
  else:
    raise ValueError(f"unknown timestep_bias strategy {strategy}")
  return w / w.sum()


# metric name in the scalars of a step -> short name used by dashboards (reference: src/maxdiffusion/train_utils.py:86-103)
METRICS_TO_MANAGED = {
    "learning/loss": "loss", "learning/current_learning_rate": "learning_rate", "learning/grad_norm": "gradient_norm",
    "learning/total_weights": "total_weights", "perf/step_time_seconds": "step_time",
    "perf/per_device_tflops_per_sec": "tflops",
}


def get_first_step(state) -> int:
  """Step a restored state resumes from (`state.step`, an engine's `step_count`, or a plain number)."""
  for name in ("step", "step_count"):
    if hasattr(state, name):
      return int(getattr(state, name))
  return int(state)


def load_next_batch(train_iter, example_batch, config):
  """The next batch, or -- with `reuse_example_batch` -- the first one again and again: steps then time the model
  without the input pipeline (reference: src/maxdiffusion/train_utils.py:30-35)."""
  if config.get("reuse_example_batch", False) and example_batch is not None:
    return example_batch
  return next(train_iter)


def record_scalar_metrics(metrics: dict, step_time_delta, per_device_tflops: float, lr: float, total_weights=None) -> None:
  """Adds the per-step performance scalars to `metrics["scalar"]`; `step_time_delta` is seconds or a timedelta."""
  seconds = step_time_delta.total_seconds() if hasattr(step_time_delta, "total_seconds") else float(step_time_delta)
  metrics.setdefault("scalar", {}).update({
      "perf/step_time_seconds": seconds, "perf/per_device_tflops": per_device_tflops,
      "perf/per_device_tflops_per_sec": per_device_tflops / seconds, "learning/current_learning_rate": lr})
  if total_weights is not None:
    metrics["scalar"]["learning/total_weights"] = float(total_weights)


def get_params_to_save(params):
  """Host copies of every tensor of a nested structure (what a checkpoint writes)."""
  if torch.is_tensor(params):
    return params.detach().to("cpu")
  if isinstance(params, dict):
    return {k: get_params_to_save(v) for k, v in params.items()}
  if isinstance(params, (list, tuple)):
    return type(params)(get_params_to_save(v) for v in params)
  return params


class MetricsWriter:

  def __init__(self, config, rank: int = 0):
    self.config = config
    self.rank = rank
    self.queue: "queue.Queue" = queue.Queue()
    self.tb = None
    self.file = None
    if rank == 0:
      tb_dir = config.get("tensorboard_dir", "")
      if tb_dir and config.get("write_metrics", True):
        try:
          from torch.utils.tensorboard import SummaryWriter

          os.makedirs(tb_dir, exist_ok=True)
          self.tb = SummaryWriter(tb_dir)
        except Exception as e:  # tensorboard is optional
          max_logging.log(f"TensorBoard writer unavailable ({e}); metrics go to the console / metrics_file only")
      path = config.get("metrics_file", "")
      if path:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self.file = open(path, "a", encoding="utf-8")
    self.thread = threading.Thread(target=self._worker, daemon=True)
    self.thread.start()

  def _worker(self) -> None:
    while True:
      item = self.queue.get()
      if item is None:
        break
      step, scalars = item
      if self.rank != 0:
        continue
      max_logging.log("completed step: {}, seconds: {:.3f}, TFLOP/s/device: {:.3f}, loss: {:.3f}".format(
          step, scalars.get("perf/step_time_seconds", 0.0), scalars.get("perf/per_device_tflops_per_sec", 0.0),
          scalars.get("learning/loss", float("nan"))))
      if self.tb is not None:
        for k, v in scalars.items():
          self.tb.add_scalar(k, v, step)
        if step % max(1, int(self.config.get("log_period", 100))) == 0:
          self.tb.flush()
      if self.file is not None:
        self.file.write(json.dumps({"step": step, **scalars}) + "\n")
        self.file.flush()

  def write(self, step: int, scalars: dict) -> None:
    self.queue.put((step, dict(scalars)))

  def close(self) -> None:
    self.queue.put(None)
    self.thread.join(timeout=30)
    if self.tb is not None:
      self.tb.close()
    if self.file is not None:
      self.file.close()


def write_metrics(writer: "MetricsWriter", metrics: dict, step: int, config=None) -> None:
  """Function form of `MetricsWriter.write` with the reference's argument shape (`metrics["scalar"]` holds the values;
  the writer thread does the file and TensorBoard work one step behind the loop)."""
  writer.write(int(step), {k: float(v) for k, v in metrics.get("scalar", metrics).items()})


@contextlib.contextmanager
def transformer_engine_context():
  """Present for scripts that wrap their training call in it: the reference uses it to tell TransformerEngine about
  its mesh; nothing here depends on that library, so the block simply runs."""
  yield


def structural_similarity(a, b, data_range: float = 255.0, win_size: int = 7) -> float:
  """Mean structural similarity of two arrays [*spatial, C] (an image [H, W, C] or a clip [T, H, W, C]) with a uniform
  `win_size` window over ALL spatial axes, sample covariances and the border of half a window left out: what
  `skimage.metrics.structural_similarity(..., channel_axis=-1, data_range=...)` computes with its defaults, which is how
  the reference scores a clip generated after training against one generated before
  (src/maxdiffusion/trainers/base_wan_trainer.py:65-81)."""
  import torch.nn.functional as F

  x = torch.as_tensor(a).double()
  y = torch.as_tensor(b).double()
  if x.shape != y.shape or x.dim() not in (3, 4):
    raise ValueError(f"expected two arrays of one shape [H, W, C] or [T, H, W, C], got {tuple(x.shape)} and {tuple(y.shape)}")
  nd = x.dim() - 1
  if min(x.shape[:-1]) < win_size:
    raise ValueError(f"every spatial axis must be at least win_size = {win_size} long, got {tuple(x.shape[:-1])}")
  pool = F.avg_pool2d if nd == 2 else F.avg_pool3d
  mean = lambda t: pool(t.movedim(-1, 0).unsqueeze(0), win_size, stride=1)[0]      # [C, *valid]
  n = float(win_size ** nd)
  cov_norm = n / (n - 1.0)
  ux, uy = mean(x), mean(y)
  vx = cov_norm * (mean(x * x) - ux * ux)
  vy = cov_norm * (mean(y * y) - uy * uy)
  vxy = cov_norm * (mean(x * y) - ux * uy)
  c1, c2 = (0.01 * data_range) ** 2, (0.03 * data_range) ** 2
  s = ((2 * ux * uy + c1) * (2 * vxy + c2)) / ((ux * ux + uy * uy + c1) * (vx + vy + c2))
  return float(s.flatten(1).mean(dim=1).mean())


def print_ssim(pretrained_video, posttrained_video) -> float:
  """Logs and returns the SSIM of two clips given as uint8 arrays [T, H, W, C] or as paths of video files."""
  def frames(v):
    if isinstance(v, (str, os.PathLike)):
      from .utils.loading_utils import load_video

      import numpy as np

      return np.stack([np.asarray(f) for f in load_video(os.fspath(v))])
    return v

  score = structural_similarity(frames(pretrained_video), frames(posttrained_video), data_range=255.0)
  max_logging.log(f"SSIM score after training is {score}")
  return score
