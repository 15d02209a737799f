"""DDPM scheduler: training noising (`add_noise`, `get_velocity`) and ancestral sampling step.

Reference: src/maxdiffusion/schedulers/scheduling_ddpm_flax.py. The SD / SDXL trainers use it as the noise
scheduler (src/maxdiffusion/trainers/sdxl_trainer.py:294-391).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .configuration_utils import SchedulerConfigMixin
from .scheduling_utils import CommonSchedulerState, add_noise_common, get_velocity_common


@dataclass
class DDPMSchedulerState:
  common: CommonSchedulerState
  init_noise_sigma: float = 1.0
  timesteps: Optional[torch.Tensor] = None
  num_inference_steps: int = 0

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


class DDPMScheduler(SchedulerConfigMixin):

  def __init__(self, num_train_timesteps: int = 1000, beta_start: float = 0.0001, beta_end: float = 0.02,
               beta_schedule: str = "linear", trained_betas=None, variance_type: str = "fixed_small",
               clip_sample: bool = True, prediction_type: str = "epsilon", rescale_zero_terminal_snr: bool = False,
               timestep_spacing: str = "leading", steps_offset: int = 0, dtype: torch.dtype = torch.float32):
    self.register_to_config(num_train_timesteps=num_train_timesteps, beta_start=beta_start, beta_end=beta_end,
                            beta_schedule=beta_schedule, trained_betas=trained_betas, variance_type=variance_type,
                            clip_sample=clip_sample, prediction_type=prediction_type,
                            rescale_zero_terminal_snr=rescale_zero_terminal_snr, timestep_spacing=timestep_spacing,
                            steps_offset=steps_offset)
    self.dtype = dtype

  def create_state(self, common: Optional[CommonSchedulerState] = None) -> DDPMSchedulerState:
    common = common or CommonSchedulerState.create(self.config)
    n = self.config.num_train_timesteps
    return DDPMSchedulerState(common=common, timesteps=torch.arange(n - 1, -1, -1), num_inference_steps=n)

  def set_timesteps(self, state, num_inference_steps: int, shape=None, device=None):
    ratio = self.config.num_train_timesteps // num_inference_steps
    ts = (np.arange(0, num_inference_steps) * ratio).round()[::-1].copy()
    return state.replace(timesteps=torch.as_tensor(ts, dtype=torch.long, device=device),
                         num_inference_steps=num_inference_steps)

  def scale_model_input(self, state, sample, timestep=None):
    return sample

  def _variance(self, state, t: int, prev_t: int) -> float:
    a = state.common.alphas_cumprod
    a_t = float(a[t])
    a_prev = float(a[prev_t]) if prev_t >= 0 else 1.0
    beta_t = 1 - a_t / a_prev
    var = (1 - a_prev) / (1 - a_t) * beta_t
    vt = self.config.variance_type
    if vt == "fixed_small":
      return max(var, 1e-20)
    if vt == "fixed_large":
      return beta_t
    raise NotImplementedError(f"variance_type {vt}")

  def step(self, state, model_output, timestep, sample, generator: Optional[torch.Generator] = None):
    c = self.config
    t = int(timestep)
    prev_t = t - c.num_train_timesteps // state.num_inference_steps
    a = state.common.alphas_cumprod
    a_t = float(a[t])
    a_prev = float(a[prev_t]) if prev_t >= 0 else 1.0
    beta_prod_t, beta_prod_prev = 1 - a_t, 1 - a_prev
    cur_alpha = a_t / a_prev
    cur_beta = 1 - cur_alpha
    if c.prediction_type == "epsilon":
      x0 = (sample - beta_prod_t ** 0.5 * model_output) / a_t ** 0.5
    elif c.prediction_type == "sample":
      x0 = model_output
    elif c.prediction_type == "v_prediction":
      x0 = a_t ** 0.5 * sample - beta_prod_t ** 0.5 * model_output
    else:
      raise ValueError(c.prediction_type)
    if c.clip_sample:
      x0 = x0.clamp(-1, 1)
    coef_x0 = a_prev ** 0.5 * cur_beta / beta_prod_t
    coef_xt = cur_alpha ** 0.5 * beta_prod_prev / beta_prod_t
    prev = coef_x0 * x0 + coef_xt * sample
    if t > 0:
      noise = torch.randn(sample.shape, generator=generator, device=sample.device, dtype=sample.dtype)
      prev = prev + self._variance(state, t, prev_t) ** 0.5 * noise
    return prev, state

  def add_noise(self, state, original, noise, timesteps):
    return add_noise_common(state.common, original, noise, timesteps)

  def get_velocity(self, state, sample, noise, timesteps):
    return get_velocity_common(state.common, sample, noise, timesteps)
