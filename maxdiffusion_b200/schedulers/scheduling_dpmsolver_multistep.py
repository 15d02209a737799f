"""DPM-Solver++ multistep (orders 1-2, `dpmsolver++` / midpoint) in the epsilon / v / sample parametrisations.

Reference: src/maxdiffusion/schedulers/scheduling_dpmsolver_multistep_flax.py (627 lines).
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np
import torch

from .configuration_utils import SchedulerConfigMixin
from .scheduling_utils import CommonSchedulerState, add_noise_common


@dataclass
class DPMSolverMultistepSchedulerState:
  common: CommonSchedulerState
  init_noise_sigma: float = 1.0
  timesteps: Optional[torch.Tensor] = None
  num_inference_steps: int = 0
  model_outputs: List[Optional[torch.Tensor]] = field(default_factory=list)
  lower_order_nums: int = 0
  step_index: int = 0
  prev_timestep: Optional[int] = None

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


class DPMSolverMultistepScheduler(SchedulerConfigMixin):

  def __init__(self, num_train_timesteps=1000, beta_start=0.0001, beta_end=0.02, beta_schedule="linear", trained_betas=None,
               solver_order=2, prediction_type="epsilon", algorithm_type="dpmsolver++", solver_type="midpoint",
               lower_order_final=True, timestep_spacing="linspace", steps_offset=0, rescale_zero_terminal_snr=False,
               dtype=torch.float32):
    self.register_to_config(num_train_timesteps=num_train_timesteps, beta_start=beta_start, beta_end=beta_end,
                            beta_schedule=beta_schedule, trained_betas=trained_betas, solver_order=solver_order,
                            prediction_type=prediction_type, algorithm_type=algorithm_type, solver_type=solver_type,
                            lower_order_final=lower_order_final, timestep_spacing=timestep_spacing,
                            steps_offset=steps_offset, rescale_zero_terminal_snr=rescale_zero_terminal_snr)
    if algorithm_type != "dpmsolver++" or solver_order > 2:
      raise NotImplementedError("only dpmsolver++ of order <= 2 is implemented")

  def create_state(self, common=None):
    return DPMSolverMultistepSchedulerState(common=common or CommonSchedulerState.create(self.config))

  def set_timesteps(self, state, num_inference_steps, shape=None, device=None):
    n = self.config.num_train_timesteps
    ts = np.linspace(0, n - 1, num_inference_steps + 1).round()[::-1][:-1].astype(np.int64)
    return state.replace(timesteps=torch.as_tensor(ts.copy(), device=device), num_inference_steps=num_inference_steps,
                         model_outputs=[None] * self.config.solver_order, lower_order_nums=0, step_index=0)

  def scale_model_input(self, state, sample, timestep=None):
    return sample

  def _abl(self, state, t):
    a = float(state.common.alphas_cumprod[int(t)]) if t >= 0 else 1.0
    alpha, sigma = math.sqrt(a), math.sqrt(max(1 - a, 1e-20))
    return alpha, sigma, math.log(alpha) - math.log(sigma)

  def _x0(self, state, model_output, t, sample):
    alpha, sigma, _ = self._abl(state, t)
    p = self.config.prediction_type
    if p == "epsilon":
      return (sample - sigma * model_output) / alpha
    if p == "sample":
      return model_output
    if p == "v_prediction":
      return alpha * sample - sigma * model_output
    raise ValueError(p)

  def step(self, state, model_output, timestep, sample):
    i = state.step_index
    t = int(timestep)
    ts = state.timesteps.tolist()
    prev_t = int(ts[i + 1]) if i + 1 < len(ts) else -1
    x0 = self._x0(state, model_output.float(), t, sample.float())
    outputs = list(state.model_outputs[1:]) + [x0]
    final = i == len(ts) - 1
    order = 1 if (state.lower_order_nums < 1 or (self.config.lower_order_final and final and len(ts) < 15) or self.config.solver_order == 1) else 2
    a_t, s_t, l_t = self._abl(state, prev_t)
    a_s, s_s, l_s = self._abl(state, t)
    h = l_t - l_s
    if prev_t < 0:
      prev = x0
    elif order == 1:
      prev = (s_t / s_s) * sample - a_t * math.expm1(-h) * x0
    else:
      t_prev2 = int(ts[i - 1])
      _, _, l_s1 = self._abl(state, t_prev2)
      h0 = l_s - l_s1
      r0 = h0 / h
      d0, d1 = x0, (1.0 / r0) * (x0 - outputs[-2])
      prev = (s_t / s_s) * sample - a_t * math.expm1(-h) * d0 - 0.5 * a_t * math.expm1(-h) * d1
    return prev, state.replace(model_outputs=outputs, lower_order_nums=min(state.lower_order_nums + 1, self.config.solver_order),
                               step_index=i + 1)

  def add_noise(self, state, original, noise, timesteps):
    return add_noise_common(state.common, original, noise, timesteps)
