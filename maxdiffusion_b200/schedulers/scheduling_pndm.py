"""PNDM (pseudo linear multistep, `skip_prk_steps` form used by Stable Diffusion).

Reference: src/maxdiffusion/schedulers/scheduling_pndm_flax.py.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np
import torch

from .configuration_utils import SchedulerConfigMixin
from .scheduling_utils import CommonSchedulerState, add_noise_common


@dataclass
class PNDMSchedulerState:
  common: CommonSchedulerState
  final_alpha_cumprod: float = 1.0
  init_noise_sigma: float = 1.0
  timesteps: Optional[torch.Tensor] = None
  num_inference_steps: int = 0
  ets: List[torch.Tensor] = field(default_factory=list)
  counter: int = 0
  cur_sample: Optional[torch.Tensor] = None

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


class PNDMScheduler(SchedulerConfigMixin):

  def __init__(self, num_train_timesteps=1000, beta_start=0.0001, beta_end=0.02, beta_schedule="linear", trained_betas=None,
               skip_prk_steps=True, set_alpha_to_one=False, steps_offset=0, prediction_type="epsilon", dtype=torch.float32):
    self.register_to_config(num_train_timesteps=num_train_timesteps, beta_start=beta_start, beta_end=beta_end,
                            beta_schedule=beta_schedule, trained_betas=trained_betas, skip_prk_steps=skip_prk_steps,
                            set_alpha_to_one=set_alpha_to_one, steps_offset=steps_offset, prediction_type=prediction_type)
    if not skip_prk_steps:
      raise NotImplementedError("Runge-Kutta warm-up steps are not implemented (Stable Diffusion skips them)")

  def create_state(self, common=None):
    common = common or CommonSchedulerState.create(self.config)
    final = 1.0 if self.config.set_alpha_to_one else float(common.alphas_cumprod[0])
    return PNDMSchedulerState(common=common, final_alpha_cumprod=final)

  def set_timesteps(self, state, num_inference_steps, shape=None, device=None):
    ratio = self.config.num_train_timesteps // num_inference_steps
    base = (np.arange(0, num_inference_steps) * ratio).round() + self.config.steps_offset
    ts = np.concatenate([base[:-1], base[-2:-1], base[-1:]])[::-1].copy()  # the second step is taken twice
    return state.replace(timesteps=torch.as_tensor(ts, dtype=torch.long, device=device), num_inference_steps=num_inference_steps,
                         ets=[], counter=0, cur_sample=None)

  def scale_model_input(self, state, sample, timestep=None):
    return sample

  def _prev_sample(self, state, sample, t, prev_t, eps):
    a = state.common.alphas_cumprod
    a_t = float(a[t])
    a_p = float(a[prev_t]) if prev_t >= 0 else state.final_alpha_cumprod
    b_t, b_p = 1 - a_t, 1 - a_p
    if self.config.prediction_type == "v_prediction":
      eps = a_t ** 0.5 * eps + b_t ** 0.5 * sample
    coeff = (a_p / a_t) ** 0.5
    denom = a_t * b_p ** 0.5 + (a_t * b_t * a_p) ** 0.5
    return coeff * sample - (a_p - a_t) * eps / denom

  def step(self, state, model_output, timestep, sample):
    t = int(timestep)
    prev_t = t - self.config.num_train_timesteps // state.num_inference_steps
    ets, counter, cur = list(state.ets), state.counter, state.cur_sample
    if counter != 1:
      ets = ets[-3:] + [model_output]
    else:
      prev_t, t = t, t + self.config.num_train_timesteps // state.num_inference_steps
    if len(ets) == 1 and counter == 0:
      eps, cur = model_output, sample
    elif len(ets) == 1 and counter == 1:
      eps, sample, cur = (model_output + ets[-1]) / 2, cur, None
    elif len(ets) == 2:
      eps = (3 * ets[-1] - ets[-2]) / 2
    elif len(ets) == 3:
      eps = (23 * ets[-1] - 16 * ets[-2] + 5 * ets[-3]) / 12
    else:
      eps = (55 * ets[-1] - 59 * ets[-2] + 37 * ets[-3] - 9 * ets[-4]) / 24
    prev = self._prev_sample(state, sample, t, prev_t, eps)
    return prev, state.replace(ets=ets, counter=counter + 1, cur_sample=cur)

  def add_noise(self, state, original, noise, timesteps):
    return add_noise_common(state.common, original, noise, timesteps)
