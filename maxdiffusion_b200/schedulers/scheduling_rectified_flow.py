"""Rectified-flow multistep scheduler of LTX-Video: uniform / resolution-shifted timesteps, Euler update
x <- x - dt * v, optional stochastic sampling, per-token timesteps for conditioning frames.

Reference: src/maxdiffusion/schedulers/scheduling_rectified_flow.py (330 lines).
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
      ts = torch.linspace(1.0, 1.0 / num_inference_steps, num_inference_steps)
      if c.shifting == "SD3" and samples_shape is not None:
        ts = resolution_dependent_shift(math.prod(samples_shape[2:]) if len(samples_shape) > 3 else samples_shape[1], ts)
      elif c.shifting == "SimpleDiffusion" and samples_shape is not None:
        n = math.prod(samples_shape[2:])
        snr = ts / (1 - ts).clamp_min(1e-8)
        # shift the log-SNR by the ratio of the base and the actual resolution
        ts = torch.sigmoid(torch.log(snr.clamp_min(1e-8)) + 2 * math.log(c.base_resolution ** 0.5 / n ** 0.5))
      if c.target_shift_terminal is not None:  # stretch so that the last timestep equals the terminal value
        one_minus = 1 - ts
        ts = 1 - one_minus / (one_minus[-1] / (1 - c.target_shift_terminal))
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
