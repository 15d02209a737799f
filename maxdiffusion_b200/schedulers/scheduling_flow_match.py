"""Flow-matching scheduler: shifted sigma schedule, training noising/target/weights, Euler sampling step.

Functional API with an explicit state object, like the reference's `FlaxFlowMatchScheduler`
(src/maxdiffusion/schedulers/scheduling_flow_match_flax.py:70-354): `create_state`, `set_timesteps`,
`sample_timesteps`, `apply_flow_match`, `step`, `add_noise`.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Optional

import torch

from .configuration_utils import SchedulerConfigMixin


@dataclass
class FlowMatchSchedulerState:
  sigmas: Optional[torch.Tensor] = None
  timesteps: Optional[torch.Tensor] = None
  linear_timesteps_weights: Optional[torch.Tensor] = None
  training: bool = False
  num_inference_steps: int = 0

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


class FlowMatchScheduler(SchedulerConfigMixin):
  config_name = "scheduler_config.json"

  def __init__(self, num_train_timesteps: int = 1000, shift: float = 3.0, sigma_max: float = 1.0,
               sigma_min: float = 0.003 / 1.002, inverse_timesteps: bool = False, extra_one_step: bool = False,
               reverse_sigmas: bool = False, use_dynamic_shifting: bool = False, time_shift_type: str = "linear",
               shift_terminal: Optional[float] = None, dtype: torch.dtype = torch.float32):
    self.register_to_config(num_train_timesteps=num_train_timesteps, shift=shift, sigma_max=sigma_max,
                            sigma_min=sigma_min, inverse_timesteps=inverse_timesteps, extra_one_step=extra_one_step,
                            reverse_sigmas=reverse_sigmas, use_dynamic_shifting=use_dynamic_shifting,
                            time_shift_type=time_shift_type, shift_terminal=shift_terminal)
    self.dtype = dtype

  def create_state(self) -> FlowMatchSchedulerState:
    return FlowMatchSchedulerState()

  def set_timesteps(self, state, num_inference_steps: int = 100, shape=None, denoising_strength: float = 1.0,
                    training: bool = False, shift: Optional[float] = None, device=None):
    c = self.config
    s = shift if shift is not None else c.shift
    start = c.sigma_min + (c.sigma_max - c.sigma_min) * denoising_strength
    if c.extra_one_step:
      sigmas = torch.linspace(start, c.sigma_min, num_inference_steps + 1, dtype=torch.float64)[:-1]
    else:
      sigmas = torch.linspace(start, c.sigma_min, num_inference_steps, dtype=torch.float64)
    if c.inverse_timesteps:
      sigmas = sigmas.flip(0)
    if c.use_dynamic_shifting and c.time_shift_type == "exponential":
      e = torch.exp(torch.tensor(float(s), dtype=torch.float64))
      sigmas = e / (e + (1.0 / sigmas.clamp(1e-7, 1.0) - 1.0))
    else:
      sigmas = s * sigmas / (1 + (s - 1) * sigmas)
    if c.reverse_sigmas:
      sigmas = 1 - sigmas
    sigmas = sigmas.to(self.dtype)
    timesteps = sigmas * c.num_train_timesteps
    weights = self._training_weights(timesteps, num_inference_steps) if training else None
    if device is not None:
      sigmas, timesteps = sigmas.to(device), timesteps.to(device)
      weights = weights.to(device) if weights is not None else None
    return state.replace(sigmas=sigmas, timesteps=timesteps, linear_timesteps_weights=weights, training=training,
                         num_inference_steps=num_inference_steps)

  def set_timesteps_ltx2(self, state, num_inference_steps: int = 100, shape=None, denoising_strength: float = 1.0,
                         training: bool = False, shift: Optional[float] = None, timesteps=None, sigmas=None, device=None):
    """Schedule with caller-provided sigmas / timesteps, exponential dynamic shifting (`shift` is mu) and the
    terminal stretch `sigma -> 1 - (1 - sigma) * (1 - shift_terminal) / (1 - sigma_last)` (LTX-2, Flux.2-Klein).

    reference: src/maxdiffusion/schedulers/scheduling_flow_match_flax.py:172-236."""
    c = self.config
    s = float(shift if shift is not None else c.shift)
    given_t = timesteps is not None
    if sigmas is None:
      if timesteps is None:
        start = c.sigma_min + (c.sigma_max - c.sigma_min) * denoising_strength
        n = num_inference_steps + 1 if c.extra_one_step else num_inference_steps
        sigmas = torch.linspace(start, c.sigma_min, n, dtype=torch.float64)
        sigmas = sigmas[:-1] if c.extra_one_step else sigmas
      else:
        sigmas = torch.as_tensor(timesteps, dtype=torch.float64) / c.num_train_timesteps
    sigmas = torch.as_tensor(sigmas, dtype=torch.float64)
    if c.inverse_timesteps:
      sigmas = sigmas.flip(0)
    if c.use_dynamic_shifting and c.time_shift_type == "exponential":
      e = torch.exp(torch.tensor(s, dtype=torch.float64))
      sigmas = e / (e + (1.0 / sigmas.clamp(1e-7, 1.0) - 1.0))
    else:
      sigmas = s * sigmas / (1 + (s - 1) * sigmas)
    if c.reverse_sigmas:
      sigmas = 1 - sigmas
    if c.get("shift_terminal", None) is not None:
      omz = 1 - sigmas
      sigmas = 1 - omz / (omz[-1] / (1 - c.shift_terminal))
    sigmas = sigmas.to(self.dtype)
    ts = torch.as_tensor(timesteps, dtype=self.dtype) if given_t else sigmas * c.num_train_timesteps
    weights = self._training_weights(ts, len(ts)) if training else None
    if device is not None:
      sigmas, ts = sigmas.to(device), ts.to(device)
    return state.replace(sigmas=sigmas, timesteps=ts, linear_timesteps_weights=weights, training=training,
                         num_inference_steps=len(ts))

  @staticmethod
  def _training_weights(timesteps: torch.Tensor, n: int) -> torch.Tensor:
    """Gaussian bump over the timestep axis, normalised to mean 1 over the grid it was computed on."""
    y = torch.exp(-2 * ((timesteps - n / 2) / n) ** 2)
    y = y - y.min()
    return y * (n / y.sum())

  def sample_timesteps(self, batch_size: int, generator: Optional[torch.Generator] = None, device=None):
    """Uniform t in [0,1), shifted by `shift`, scaled to [0, num_train_timesteps)."""
    t = torch.rand((batch_size,), generator=generator, device=generator.device if generator is not None else device)
    s = self.config.shift
    t = (t * s) / (1 + (s - 1) * t)
    return (t * self.config.num_train_timesteps).to(device) if device is not None else t * self.config.num_train_timesteps

  def apply_flow_match(self, noise, batch, timesteps, state: Optional[FlowMatchSchedulerState] = None):
    """(noisy, target, weights): x_t = (1-sigma) x + sigma eps, target = eps - x, weight from the bump.

    The weight of a sample is read from the bump normalised over the whole training grid (`state`, as built by
    `set_timesteps(training=True)`). The reference normalises over the timesteps of the batch instead
    (scheduling_flow_match_flax.py:259-282), which is undefined (0/0) for a batch of one sample.
    """
    c = self.config
    t = timesteps.float() / c.num_train_timesteps
    t = t.reshape((-1,) + (1,) * (batch.dim() - 1))
    sigma = (1 - t) * c.sigma_min + t * c.sigma_max
    noisy = (1 - sigma) * batch + sigma * noise
    target = noise - batch
    if state is not None and state.linear_timesteps_weights is not None:
      idx = self._find_timestep_id(state, timesteps.to(state.timesteps.device).reshape(-1))
      weights = state.linear_timesteps_weights[idx].to(batch.device)
    elif timesteps.numel() > 1:
      weights = self._training_weights(timesteps.float(), c.num_train_timesteps)
    else:
      weights = torch.ones_like(timesteps, dtype=torch.float32)
    return noisy, target, weights

  def add_noise(self, state, original, noise, timestep):
    idx = self._find_timestep_id(state, timestep)
    sigma = state.sigmas[idx].reshape((-1,) + (1,) * (original.dim() - 1)) if torch.as_tensor(timestep).dim() else state.sigmas[idx]
    return (1 - sigma) * original + sigma * noise

  @staticmethod
  def _find_timestep_id(state, timestep):
    ts = torch.as_tensor(timestep, dtype=state.timesteps.dtype, device=state.timesteps.device)
    if ts.dim() == 0:
      return torch.argmin((state.timesteps - ts).abs())
    return torch.argmin((state.timesteps[None, :] - ts[:, None]).abs(), dim=1)

  def step(self, state, model_output, timestep, sample, to_final: bool = False, step_index: Optional[int] = None):
    """Euler step x <- x + v * (sigma_next - sigma). Returns (prev_sample, state)."""
    idx = step_index if step_index is not None else int(self._find_timestep_id(state, timestep))
    sigma = state.sigmas[idx]
    last = to_final or idx + 1 >= state.timesteps.shape[0]
    if last:
      final = 1.0 if (self.config.inverse_timesteps or self.config.reverse_sigmas) else 0.0
      sigma_next = torch.full_like(sigma, final)
    else:
      sigma_next = state.sigmas[idx + 1]
    prev = sample + model_output * (sigma_next - sigma).to(model_output.dtype)
    return prev, state


def compute_empirical_mu(image_seq_len: int, num_steps: int) -> float:
  """Resolution- and step-count-dependent time shift of the Flux family
  (reference: src/maxdiffusion/schedulers/scheduling_flow_match_flax.py:422-437)."""
  a1, b1 = 8.73809524e-05, 1.89833333
  a2, b2 = 0.00016927, 0.45666666
  if image_seq_len > 4300:
    return float(a2 * image_seq_len + b2)
  m_200 = a2 * image_seq_len + b2
  m_10 = a1 * image_seq_len + b1
  a = (m_200 - m_10) / 190.0
  return float(a * num_steps + (m_200 - 200.0 * a))
