"""Euler discrete scheduler (Karras et al. 2022, alg. 2 without churn) incl. the `flux` timestep spacing.

Reference: src/maxdiffusion/schedulers/scheduling_euler_discrete_flax.py:146-270.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .configuration_utils import SchedulerConfigMixin
from .scheduling_utils import CommonSchedulerState, _bcast


@dataclass
class EulerDiscreteSchedulerState:
  common: CommonSchedulerState
  init_noise_sigma: float = 1.0
  timesteps: Optional[torch.Tensor] = None
  sigmas: Optional[torch.Tensor] = None
  num_inference_steps: int = 0

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


class EulerDiscreteScheduler(SchedulerConfigMixin):

  def __init__(self, num_train_timesteps: int = 1000, beta_start: float = 0.0001, beta_end: float = 0.02,
               beta_schedule: str = "linear", trained_betas=None, prediction_type: str = "epsilon",
               timestep_spacing: str = "linspace", steps_offset: int = 0, rescale_zero_terminal_snr: bool = False,
               dtype: torch.dtype = torch.float32):
    self.register_to_config(num_train_timesteps=num_train_timesteps, beta_start=beta_start, beta_end=beta_end,
                            beta_schedule=beta_schedule, trained_betas=trained_betas, prediction_type=prediction_type,
                            timestep_spacing=timestep_spacing, steps_offset=steps_offset,
                            rescale_zero_terminal_snr=rescale_zero_terminal_snr)
    self.dtype = dtype

  def create_state(self, common: Optional[CommonSchedulerState] = None) -> EulerDiscreteSchedulerState:
    common = common or CommonSchedulerState.create(self.config)
    sig = ((1 - common.alphas_cumprod) / common.alphas_cumprod).sqrt()
    init = float(sig.max()) if self.config.timestep_spacing in ("linspace", "trailing") else float((sig.max() ** 2 + 1).sqrt())
    return EulerDiscreteSchedulerState(common=common, init_noise_sigma=init)

  def set_timesteps(self, state, num_inference_steps: int, shape=None, timestep_shift: Optional[float] = None, device=None):
    c = self.config
    n = c.num_train_timesteps
    if c.timestep_spacing == "flux":
      # flow sigmas 1 -> 0 with the resolution-dependent exponential shift mu
      t = np.linspace(1.0, 0.0, num_inference_steps + 1)
      if timestep_shift is not None:
        with np.errstate(divide="ignore"):
          t = np.where(t > 0, np.exp(timestep_shift) / (np.exp(timestep_shift) + (1.0 / np.maximum(t, 1e-12) - 1.0)), 0.0)
      sigmas = torch.as_tensor(t, dtype=torch.float32, device=device)
      return state.replace(timesteps=sigmas[:-1] * n, sigmas=sigmas, num_inference_steps=num_inference_steps,
                           init_noise_sigma=1.0)
    if c.timestep_spacing == "linspace":
      ts = np.linspace(n - 1, 0, num_inference_steps)
    elif c.timestep_spacing == "leading":
      ts = (np.arange(0, num_inference_steps) * (n // num_inference_steps)).round()[::-1].astype(np.float64) + c.steps_offset
    elif c.timestep_spacing == "trailing":
      ts = np.arange(n, 0, -n / num_inference_steps).round() - 1
    else:
      raise ValueError(f"timestep_spacing {c.timestep_spacing}")
    a = state.common.alphas_cumprod.double().cpu().numpy()
    all_sig = ((1 - a) / a) ** 0.5
    sig = np.interp(ts, np.arange(len(all_sig)), all_sig)
    sig = np.concatenate([sig, [0.0]])
    init = float(sig.max()) if c.timestep_spacing in ("linspace", "trailing") else float((sig.max() ** 2 + 1) ** 0.5)
    return state.replace(timesteps=torch.as_tensor(ts, dtype=torch.float32, device=device),
                         sigmas=torch.as_tensor(sig, dtype=torch.float32, device=device),
                         num_inference_steps=num_inference_steps, init_noise_sigma=init)

  def _index(self, state, timestep) -> int:
    return int((state.timesteps - float(timestep)).abs().argmin())

  def scale_model_input(self, state, sample, timestep):
    if self.config.timestep_spacing == "flux":
      return sample
    sigma = state.sigmas[self._index(state, timestep)]
    return sample / (sigma ** 2 + 1).sqrt()

  def step(self, state, model_output, timestep, sample, step_index: Optional[int] = None):
    i = step_index if step_index is not None else self._index(state, timestep)
    sigma, sigma_next = state.sigmas[i], state.sigmas[i + 1]
    c = self.config
    if c.timestep_spacing == "flux":
      return sample + (sigma_next - sigma).to(sample.dtype) * model_output, state
    if c.prediction_type == "epsilon":
      x0 = sample - sigma * model_output
    elif c.prediction_type == "v_prediction":
      x0 = model_output * (-sigma / (sigma ** 2 + 1).sqrt()) + sample / (sigma ** 2 + 1)
    elif c.prediction_type == "sample":
      x0 = model_output
    else:
      raise ValueError(c.prediction_type)
    derivative = (sample - x0) / sigma
    return sample + derivative * (sigma_next - sigma), state

  def add_noise(self, state, original, noise, timesteps, flux: bool = False):
    if flux:
      t = _bcast(torch.as_tensor(timesteps, dtype=torch.float32), original)
      return t * noise + (1.0 - t) * original
    idx = torch.as_tensor([self._index(state, t) for t in torch.as_tensor(timesteps).reshape(-1)])
    sigma = _bcast(state.sigmas[idx], original)
    return original + noise * sigma
