"""Linear multistep (LMS) scheduler on the Karras sigma parametrisation.

Reference: src/maxdiffusion/schedulers/scheduling_lms_discrete_flax.py.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np
import torch

from .configuration_utils import SchedulerConfigMixin
from .scheduling_utils import CommonSchedulerState


@dataclass
class LMSDiscreteSchedulerState:
  common: CommonSchedulerState
  init_noise_sigma: float = 1.0
  timesteps: Optional[torch.Tensor] = None
  sigmas: Optional[np.ndarray] = None
  num_inference_steps: int = 0
  derivatives: List[torch.Tensor] = field(default_factory=list)

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


class LMSDiscreteScheduler(SchedulerConfigMixin):

  def __init__(self, num_train_timesteps=1000, beta_start=0.0001, beta_end=0.02, beta_schedule="linear", trained_betas=None,
               prediction_type="epsilon", dtype=torch.float32):
    self.register_to_config(num_train_timesteps=num_train_timesteps, beta_start=beta_start, beta_end=beta_end,
                            beta_schedule=beta_schedule, trained_betas=trained_betas, prediction_type=prediction_type)

  def create_state(self, common=None):
    common = common or CommonSchedulerState.create(self.config)
    sig = ((1 - common.alphas_cumprod) / common.alphas_cumprod).sqrt()
    return LMSDiscreteSchedulerState(common=common, init_noise_sigma=float(sig.max()))

  def set_timesteps(self, state, num_inference_steps, shape=None, device=None):
    n = self.config.num_train_timesteps
    ts = np.linspace(n - 1, 0, num_inference_steps)
    a = state.common.alphas_cumprod.double().cpu().numpy()
    all_sig = ((1 - a) / a) ** 0.5
    sig = np.concatenate([np.interp(ts, np.arange(len(all_sig)), all_sig), [0.0]])
    return state.replace(timesteps=torch.as_tensor(ts, dtype=torch.float32, device=device), sigmas=sig,
                         num_inference_steps=num_inference_steps, derivatives=[], init_noise_sigma=float(sig.max()))

  def _index(self, state, t):
    return int((state.timesteps - float(t)).abs().argmin())

  def scale_model_input(self, state, sample, timestep):
    s = state.sigmas[self._index(state, timestep)]
    return sample / (s * s + 1) ** 0.5

  @staticmethod
  def _lms_coeff(sigmas, order, t, cur):
    """Integral over [sigma_t, sigma_{t+1}] of the Lagrange basis polynomial of derivative `cur`."""
    xs = np.linspace(sigmas[t], sigmas[t + 1], 129)
    prod = np.ones_like(xs)
    for k in range(order):
      if k != cur:
        prod *= (xs - sigmas[t - k]) / (sigmas[t - cur] - sigmas[t - k])
    return float(np.trapezoid(prod, xs))

  def step(self, state, model_output, timestep, sample, order: int = 4):
    i = self._index(state, timestep)
    sigma = float(state.sigmas[i])
    p = self.config.prediction_type
    if p == "epsilon":
      x0 = sample - sigma * model_output
    elif p == "v_prediction":
      x0 = model_output * (-sigma / (sigma ** 2 + 1) ** 0.5) + sample / (sigma ** 2 + 1)
    else:
      raise ValueError(p)
    derivs = (list(state.derivatives) + [(sample - x0) / sigma])[-order:]
    o = min(i + 1, order, len(derivs))
    coeffs = [self._lms_coeff(state.sigmas, o, i, c) for c in range(o)]
    prev = sample + sum(c * d for c, d in zip(coeffs, reversed(derivs)))
    return prev, state.replace(derivatives=derivs)

  def add_noise(self, state, original, noise, timesteps):
    idx = [self._index(state, t) for t in torch.as_tensor(timesteps).reshape(-1)]
    sig = torch.as_tensor([state.sigmas[j] for j in idx], dtype=original.dtype, device=original.device)
    return original + noise * sig.reshape((-1,) + (1,) * (original.dim() - 1))
