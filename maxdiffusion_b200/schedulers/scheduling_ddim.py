"""DDIM scheduler (deterministic for eta = 0). Reference: src/maxdiffusion/schedulers/scheduling_ddim_flax.py."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .configuration_utils import SchedulerConfigMixin
from .scheduling_utils import CommonSchedulerState, add_noise_common, get_velocity_common


@dataclass
class DDIMSchedulerState:
  common: CommonSchedulerState
  final_alpha_cumprod: float = 1.0
  init_noise_sigma: float = 1.0
  timesteps: Optional[torch.Tensor] = None
  num_inference_steps: int = 0

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


class DDIMScheduler(SchedulerConfigMixin):

  def __init__(self, num_train_timesteps: int = 1000, beta_start: float = 0.0001, beta_end: float = 0.02,
               beta_schedule: str = "linear", trained_betas=None, clip_sample: bool = True,
               clip_sample_range: float = 1.0, set_alpha_to_one: bool = True, steps_offset: int = 0,
               prediction_type: str = "epsilon", timestep_spacing: str = "leading",
               rescale_zero_terminal_snr: bool = False, dtype: torch.dtype = torch.float32):
    self.register_to_config(num_train_timesteps=num_train_timesteps, beta_start=beta_start, beta_end=beta_end,
                            beta_schedule=beta_schedule, trained_betas=trained_betas, clip_sample=clip_sample,
                            clip_sample_range=clip_sample_range, set_alpha_to_one=set_alpha_to_one,
                            steps_offset=steps_offset, prediction_type=prediction_type,
                            timestep_spacing=timestep_spacing, rescale_zero_terminal_snr=rescale_zero_terminal_snr)
    self.dtype = dtype

  def create_state(self, common: Optional[CommonSchedulerState] = None) -> DDIMSchedulerState:
    common = common or CommonSchedulerState.create(self.config)
    final = 1.0 if self.config.set_alpha_to_one else float(common.alphas_cumprod[0])
    n = self.config.num_train_timesteps
    return DDIMSchedulerState(common=common, final_alpha_cumprod=final, timesteps=torch.arange(n - 1, -1, -1),
                              num_inference_steps=n)

  def set_timesteps(self, state, num_inference_steps: int, shape=None, device=None):
    c = self.config
    n = c.num_train_timesteps
    if c.timestep_spacing == "leading":
      ts = (np.arange(0, num_inference_steps) * (n // num_inference_steps)).round()[::-1] + c.steps_offset
    elif c.timestep_spacing == "trailing":
      ts = np.round(np.arange(n, 0, -n / num_inference_steps)) - 1
    elif c.timestep_spacing == "linspace":
      ts = np.linspace(0, n - 1, num_inference_steps).round()[::-1]
    else:
      raise ValueError(c.timestep_spacing)
    return state.replace(timesteps=torch.as_tensor(ts.copy(), dtype=torch.long, device=device),
                         num_inference_steps=num_inference_steps)

  def scale_model_input(self, state, sample, timestep=None):
    return sample

  def step(self, state, model_output, timestep, sample, eta: float = 0.0, generator: Optional[torch.Generator] = None):
    c = self.config
    t = int(timestep)
    prev_t = t - c.num_train_timesteps // state.num_inference_steps
    a = state.common.alphas_cumprod
    a_t = float(a[t])
    a_prev = float(a[prev_t]) if prev_t >= 0 else state.final_alpha_cumprod
    b_t = 1 - a_t
    if c.prediction_type == "epsilon":
      x0 = (sample - b_t ** 0.5 * model_output) / a_t ** 0.5
      eps = model_output
    elif c.prediction_type == "sample":
      x0 = model_output
      eps = (sample - a_t ** 0.5 * x0) / b_t ** 0.5
    elif c.prediction_type == "v_prediction":
      x0 = a_t ** 0.5 * sample - b_t ** 0.5 * model_output
      eps = a_t ** 0.5 * model_output + b_t ** 0.5 * sample
    else:
      raise ValueError(c.prediction_type)
    if c.clip_sample:
      x0 = x0.clamp(-c.clip_sample_range, c.clip_sample_range)
    var = (1 - a_prev) / (1 - a_t) * (1 - a_t / a_prev)
    std = eta * max(var, 0.0) ** 0.5
    direction = max(1 - a_prev - std ** 2, 0.0) ** 0.5 * eps
    prev = a_prev ** 0.5 * x0 + direction
    if eta > 0:
      prev = prev + std * torch.randn(sample.shape, generator=generator, device=sample.device, dtype=sample.dtype)
    return prev, state

  def add_noise(self, state, original, noise, timesteps):
    return add_noise_common(state.common, original, noise, timesteps)

  def get_velocity(self, state, sample, noise, timesteps):
    return get_velocity_common(state.common, sample, noise, timesteps)
