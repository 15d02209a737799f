"""Rectified-flow multistep scheduler of LTX-Video: uniform / linear-quadratic / constant-shift timesteps, the SD3 and
SimpleDiffusion resolution-dependent shifts, Euler update x <- x - dt * v, optional stochastic sampling, per-token
timesteps for conditioning frames.

Reference: src/maxdiffusion/schedulers/scheduling_rectified_flow.py (samplers :34-55,205-216, shifts :85-137, step
:283-329). The trajectories stored with the reference's scheduler test
(src/maxdiffusion/tests/legacy_hf_tests/schedulers/rf_scheduler_test_ref/) are reproduced in tests/test_schedulers_cpu.py.
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass
from typing import Optional

import torch

from .configuration_utils import SchedulerConfigMixin


@dataclass
class RectifiedFlowSchedulerState:
  timesteps: Optional[torch.Tensor] = None
  num_inference_steps: int = 0

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


def time_shift(mu: float, sigma: float, t: torch.Tensor) -> torch.Tensor:
  return math.exp(mu) / (math.exp(mu) + (1 / t - 1) ** sigma)


def resolution_dependent_shift(n_tokens: int, t: torch.Tensor, min_tokens=1024, max_tokens=4096, base=0.95, top=2.05):
  m = (top - base) / (max_tokens - min_tokens)
  return time_shift(m * n_tokens + (base - m * min_tokens), 1.0, t)


def linear_quadratic_schedule(num_steps: int, threshold_noise: float = 0.025, linear_steps: Optional[int] = None) -> torch.Tensor:
  """Timesteps 1 - sigma with sigma rising linearly to `threshold_noise` over the first half of the steps and
  quadratically (value- and slope-continuous at the joint) to 1 over the second."""
  if num_steps == 1:
    return torch.ones(1)
  linear_steps = num_steps // 2 if linear_steps is None else linear_steps
  i = torch.arange(linear_steps, dtype=torch.float32)
  linear = i * threshold_noise / linear_steps
  diff = linear_steps - threshold_noise * num_steps
  quad_steps = num_steps - linear_steps
  a = diff / (linear_steps * quad_steps ** 2)
  b = threshold_noise / linear_steps - 2 * diff / quad_steps ** 2
  c = a * linear_steps ** 2
  j = torch.arange(linear_steps, num_steps, dtype=torch.float32)
  return 1.0 - torch.cat([linear, a * j ** 2 + b * j + c])


class RectifiedFlowMultistepScheduler(SchedulerConfigMixin):

  def __init__(self, num_train_timesteps: int = 1000, shifting: Optional[str] = None, base_resolution: int = 32 ** 2,
               target_shift_terminal: Optional[float] = None, sampler: str = "Uniform", shift: Optional[float] = None):
    self.register_to_config(num_train_timesteps=num_train_timesteps, shifting=shifting, base_resolution=base_resolution,
                            target_shift_terminal=target_shift_terminal, sampler=sampler, shift=shift)

  def create_state(self):
    return RectifiedFlowSchedulerState()

  def set_timesteps(self, state, num_inference_steps: int, samples_shape=None, timesteps=None, device=None):
    c = self.config
    if timesteps is None:
      num_inference_steps = min(int(c.num_train_timesteps), int(num_inference_steps))
      uniform = torch.linspace(1.0, 1.0 / num_inference_steps, num_inference_steps)
      if c.sampler == "Uniform":
        ts = uniform
      elif c.sampler == "LinearQuadratic":
        ts = linear_quadratic_schedule(num_inference_steps)
      elif c.sampler == "Constant":
        if c.shift is None:
          raise ValueError("the Constant sampler needs `shift`")
        ts = time_shift(float(c.shift), 1.0, uniform)
      else:
        raise ValueError(f"sampler {c.sampler!r} is not supported (Uniform, LinearQuadratic, Constant)")
      if samples_shape is not None and c.shifting in ("SD3", "SimpleDiffusion"):
        if len(samples_shape) not in (3, 4, 5):
          raise ValueError("samples must have shape (b, t, c), (b, c, h, w) or (b, c, f, h, w)")
        m = samples_shape[1] if len(samples_shape) == 3 else math.prod(samples_shape[2:])
        if c.shifting == "SD3":
          ts = resolution_dependent_shift(m, ts)
          if c.target_shift_terminal is not None:  # stretch so that the last timestep equals the terminal value
            if not 0.0 < c.target_shift_terminal < 1.0:
              raise ValueError("the terminal value must be between 0 and 1 (exclusive)")
            one_minus = 1 - ts
            ts = 1 - one_minus / (one_minus[-1] / (1 - c.target_shift_terminal))
        else:
          # log-SNR shifted by the ratio of the actual to the base token count: sigmoid(logit(t) + log(m / n))
          n = c.base_resolution if c.base_resolution else 32 ** 2
          ts = torch.sigmoid(torch.logit(ts.clamp(1e-8, 1 - 1e-8)) + math.log(m / n))
    else:
      ts = torch.as_tensor(timesteps, dtype=torch.float32)
    return state.replace(timesteps=ts.to(device), num_inference_steps=len(ts))

  def scale_model_input(self, state, sample, timestep=None):
    return sample

  def step(self, state, model_output, timestep, sample, stochastic_sampling: bool = False, generator=None):
    """timestep: scalar or per-token tensor broadcastable to sample[..., 0]; tokens whose timestep is already below the
    next global timestep (conditioning tokens) are left untouched."""
    ts = state.timesteps
    t = torch.as_tensor(timestep, dtype=torch.float32, device=sample.device)
    cur = float(t.max())
    idx = int((ts - cur).abs().argmin())
    nxt = float(ts[idx + 1]) if idx + 1 < len(ts) else 0.0
    dt = (t - nxt).clamp_min(0.0)
    while dt.dim() < sample.dim():
      dt = dt.unsqueeze(-1)
    if stochastic_sampling:
      x0 = sample - t.reshape(dt.shape) * model_output
      noise = torch.randn(sample.shape, generator=generator, device=sample.device, dtype=sample.dtype)
      return (1 - nxt) * x0 + nxt * noise, state
    return sample - dt * model_output, state

  def add_noise(self, state, original, noise, timesteps):
    t = torch.as_tensor(timesteps, dtype=original.dtype, device=original.device)
    while t.dim() < original.dim():
      t = t.unsqueeze(-1)
    return (1 - t) * original + t * noise
