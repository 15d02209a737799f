"""PNDM: pseudo linear multistep steps, started either by a repeated first step (`skip_prk_steps`, the form Stable
Diffusion uses) or by three Runge-Kutta steps of four model evaluations each.

Reference: src/maxdiffusion/schedulers/scheduling_pndm_flax.py (`step_prk`, `step_plms`, `_get_prev_sample`). The full-loop
values of the reference's scheduler tests (src/maxdiffusion/tests/legacy_hf_tests/schedulers/test_scheduler_flax.py:
903-939) are reproduced in tests/test_schedulers_cpu.py.
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
  cur_model_output: Optional[torch.Tensor] = None   # running Runge-Kutta combination of a warm-up step
  prk_timesteps: Optional[torch.Tensor] = None
  plms_timesteps: Optional[torch.Tensor] = None

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


class PNDMScheduler(SchedulerConfigMixin):

  def __init__(self, num_train_timesteps=1000, beta_start=0.0001, beta_end=0.02, beta_schedule="linear", trained_betas=None,
               skip_prk_steps=True, set_alpha_to_one=False, steps_offset=0, prediction_type="epsilon", dtype=torch.float32):
    self.register_to_config(num_train_timesteps=num_train_timesteps, beta_start=beta_start, beta_end=beta_end,
                            beta_schedule=beta_schedule, trained_betas=trained_betas, skip_prk_steps=skip_prk_steps,
                            set_alpha_to_one=set_alpha_to_one, steps_offset=steps_offset, prediction_type=prediction_type)
    self.pndm_order = 4

  def create_state(self, common=None):
    common = common or CommonSchedulerState.create(self.config)
    final = 1.0 if self.config.set_alpha_to_one else float(common.alphas_cumprod[0])
    return PNDMSchedulerState(common=common, final_alpha_cumprod=final)

  def set_timesteps(self, state, num_inference_steps, shape=None, device=None):
    ratio = self.config.num_train_timesteps // num_inference_steps
    base = (np.arange(0, num_inference_steps) * ratio).round() + self.config.steps_offset
    if self.config.skip_prk_steps:
      prk = np.array([], dtype=np.int64)
      plms = np.concatenate([base[:-1], base[-2:-1], base[-1:]])[::-1].copy()  # the second step is taken twice
    else:
      # every one of the last `pndm_order` steps is evaluated at t, t + ratio/2 (twice) and t + ratio: the four stages
      # of a Runge-Kutta step from t + ratio down to t; the linear multistep steps take over below them
      k = self.pndm_order
      stages = base[-k:].repeat(2) + np.tile(np.array([0, ratio // 2]), k)
      prk = stages[:-1].repeat(2)[1:-1][::-1].copy()
      plms = base[:-3][::-1].copy()
    ts = np.concatenate([prk, plms]).astype(np.int64)
    as_t = lambda a: torch.as_tensor(a.astype(np.int64), dtype=torch.long, device=device)
    return state.replace(timesteps=as_t(ts), prk_timesteps=as_t(prk), plms_timesteps=as_t(plms),
                         num_inference_steps=num_inference_steps, ets=[], counter=0, cur_sample=None, cur_model_output=None)

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
    if state.prk_timesteps is not None and state.counter < len(state.prk_timesteps):
      return self.step_prk(state, model_output, timestep, sample)
    return self.step_plms(state, model_output, timestep, sample)

  def step_prk(self, state, model_output, timestep, sample):
    """One of the four stages of a Runge-Kutta step: the stage outputs are combined with weights 1/6, 1/3, 1/3, 1/6
    and every stage moves the sample the step STARTED from (kept in the state) to the stage's evaluation point."""
    half = self.config.num_train_timesteps // state.num_inference_steps // 2
    t_stage = int(timestep)
    prev_t = t_stage - (0 if state.counter % 2 else half)
    t = int(state.prk_timesteps[state.counter // 4 * 4])
    ets, acc, cur = list(state.ets), state.cur_model_output, state.cur_sample
    acc = torch.zeros_like(model_output) if acc is None else acc
    stage = state.counter % 4
    if stage == 0:
      acc, ets, cur = acc + model_output / 6, ets + [model_output], sample
    elif stage in (1, 2):
      acc = acc + model_output / 3
    else:
      model_output, acc = acc + model_output / 6, None
    cur = sample if cur is None else cur
    prev = self._prev_sample(state, cur, t, prev_t, model_output)
    return prev, state.replace(ets=ets, counter=state.counter + 1, cur_sample=cur, cur_model_output=acc)

  def step_plms(self, state, model_output, timestep, sample):
    if not self.config.skip_prk_steps and len(state.ets) < 3:
      raise ValueError("the linear multistep steps need three earlier model outputs: run the Runge-Kutta warm-up steps "
                       "first (`step_prk`), or build the scheduler with skip_prk_steps=True")
    t = int(timestep)
    # the step below timestep 0 lands on timestep 0 (as in the reference, scheduling_pndm_flax.py:382-383), so the last
    # step of a schedule that ends at 0 leaves the sample as it is and `set_alpha_to_one` only matters with an offset
    prev_t = max(0, t - self.config.num_train_timesteps // state.num_inference_steps)
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
