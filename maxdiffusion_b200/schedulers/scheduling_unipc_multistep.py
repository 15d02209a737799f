"""UniPC multistep scheduler (predictor UniP + corrector UniC, B(h) variants bh1 / bh2), flow-sigma capable.

Functional API with an explicit state, as the reference's `FlaxUniPCMultistepScheduler`
(src/maxdiffusion/schedulers/scheduling_unipc_multistep_flax.py:152-777): `create_state`, `set_timesteps`,
`step`, `add_noise`. It is the default Wan sampler (flow_prediction, use_flow_sigmas, flow_shift).

Every coefficient of a step depends only on the sigma schedule and the step index, so they are computed on the
host in float64 once per step (`_coefficients`) and the device work of a step is a short chain of AXPYs over the
latent — the form the CUDA-graph-captured denoising loop wants. Karras / exponential / beta sigmas are not
implemented (the reference raises NotImplementedError for them as well, :228-239).
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np
import torch

from .configuration_utils import SchedulerConfigMixin
from .scheduling_utils import betas_for_config


@dataclass
class UniPCMultistepSchedulerState:
  timesteps: Optional[torch.Tensor] = None
  sigmas: Optional[np.ndarray] = None         # host float64, length steps + 1
  model_outputs: List[Optional[torch.Tensor]] = field(default_factory=list)
  lower_order_nums: int = 0
  step_index: Optional[int] = None
  last_sample: Optional[torch.Tensor] = None
  this_order: int = 0
  num_inference_steps: int = 0
  alphas_cumprod: Optional[np.ndarray] = None

  def replace(self, **kw):
    return dataclasses.replace(self, **kw)


class UniPCMultistepScheduler(SchedulerConfigMixin):

  def __init__(self, num_train_timesteps: int = 1000, beta_start: float = 0.0001, beta_end: float = 0.02,
               beta_schedule: str = "linear", solver_order: int = 2, prediction_type: str = "flow_prediction",
               thresholding: bool = False, predict_x0: bool = True, solver_type: str = "bh2",
               lower_order_final: bool = True, disable_corrector=(), use_karras_sigmas: bool = False,
               use_exponential_sigmas: bool = False, use_beta_sigmas: bool = False, use_flow_sigmas: bool = True,
               flow_shift: float = 1.0, timestep_spacing: str = "linspace", steps_offset: int = 0,
               final_sigmas_type: str = "zero", dtype: torch.dtype = torch.float32):
    if solver_type not in ("bh1", "bh2"):
      raise NotImplementedError(f"solver_type {solver_type}")
    self.register_to_config(num_train_timesteps=num_train_timesteps, beta_start=beta_start, beta_end=beta_end,
                            beta_schedule=beta_schedule, solver_order=solver_order, prediction_type=prediction_type,
                            thresholding=thresholding, predict_x0=predict_x0, solver_type=solver_type,
                            lower_order_final=lower_order_final, disable_corrector=list(disable_corrector),
                            use_karras_sigmas=use_karras_sigmas, use_exponential_sigmas=use_exponential_sigmas,
                            use_beta_sigmas=use_beta_sigmas, use_flow_sigmas=use_flow_sigmas, flow_shift=flow_shift,
                            timestep_spacing=timestep_spacing, steps_offset=steps_offset,
                            final_sigmas_type=final_sigmas_type)
    self.dtype = dtype

  # ------------------------------------------------------------------ schedule
  def create_state(self) -> UniPCMultistepSchedulerState:
    betas = betas_for_config(self.config)
    return UniPCMultistepSchedulerState(alphas_cumprod=np.cumprod(1.0 - betas))

  def set_timesteps(self, state, num_inference_steps: int, shape=None, device=None):
    c = self.config
    if c.use_karras_sigmas or c.use_exponential_sigmas or c.use_beta_sigmas:
      raise NotImplementedError("karras / exponential / beta sigmas are not implemented")
    n_train = c.num_train_timesteps
    if c.use_flow_sigmas:
      sig = np.linspace(1.0, 1.0 / n_train, num_inference_steps + 1)[:-1]
      sig = c.flow_shift * sig / (1 + (c.flow_shift - 1) * sig)
      if abs(sig[0] - 1.0) < 1e-6:
        sig[0] -= 1e-6
      timesteps = (sig * n_train).astype(np.int64)
      last = sig[-1] if c.final_sigmas_type == "sigma_min" else 0.0
    else:
      if c.timestep_spacing == "linspace":
        timesteps = np.linspace(0, n_train - 1, num_inference_steps + 1).round()[::-1][:-1].astype(np.int64)
      elif c.timestep_spacing == "leading":
        ratio = n_train // (num_inference_steps + 1)
        timesteps = (np.arange(0, num_inference_steps + 1) * ratio).round()[::-1][:-1].astype(np.int64) + c.steps_offset
      elif c.timestep_spacing == "trailing":
        timesteps = np.arange(n_train, 0, -n_train / num_inference_steps).round().astype(np.int64) - 1
      else:
        raise ValueError(f"timestep_spacing {c.timestep_spacing} is not supported")
      all_sig = ((1 - state.alphas_cumprod) / state.alphas_cumprod) ** 0.5
      sig = np.interp(timesteps, np.arange(len(all_sig)), all_sig)
      last = all_sig[0] if c.final_sigmas_type == "sigma_min" else 0.0
    if c.final_sigmas_type not in ("zero", "sigma_min"):
      raise ValueError("final_sigmas_type must be 'zero' or 'sigma_min'")
    sigmas = np.concatenate([sig, [last]]).astype(np.float64)
    return state.replace(timesteps=torch.as_tensor(timesteps, device=device), sigmas=sigmas,
                         model_outputs=[None] * c.solver_order, lower_order_nums=0, step_index=None, last_sample=None,
                         this_order=0, num_inference_steps=num_inference_steps)

  def _alpha_sigma(self, sigma: float):
    if self.config.use_flow_sigmas:
      return 1.0 - sigma, sigma
    alpha = 1.0 / math.sqrt(sigma * sigma + 1.0)
    return alpha, sigma * alpha

  @staticmethod
  def _lambda(alpha: float, sigma: float) -> float:
    if sigma <= 0.0:
      return math.inf
    return math.log(alpha) - math.log(sigma)

  # ------------------------------------------------------------------ model output conversion
  def convert_model_output(self, state, model_output, sample):
    c = self.config
    sigma = float(state.sigmas[state.step_index])
    alpha_t, sigma_t = self._alpha_sigma(sigma)
    if c.predict_x0:
      if c.prediction_type == "epsilon":
        x0 = (sample - sigma_t * model_output) / alpha_t
      elif c.prediction_type == "sample":
        x0 = model_output
      elif c.prediction_type == "v_prediction":
        x0 = alpha_t * sample - sigma_t * model_output
      elif c.prediction_type == "flow_prediction":
        x0 = sample - sigma_t * model_output
      else:
        raise ValueError(f"prediction_type {c.prediction_type}")
      if c.thresholding:
        raise NotImplementedError("dynamic thresholding")
      return x0
    if c.prediction_type == "epsilon":
      return model_output
    if c.prediction_type == "sample":
      return (sample - alpha_t * model_output) / sigma_t
    if c.prediction_type == "v_prediction":
      return alpha_t * model_output + sigma_t * sample
    raise ValueError(f"prediction_type {c.prediction_type}")

  # ------------------------------------------------------------------ coefficients (host, float64)
  def _coefficients(self, sigmas: np.ndarray, i_s0: int, i_t: int, history: List[int], order: int, corrector: bool):
    """Returns (c_x, c_m0, B_coef, rhos): x_t = c_x * x + c_m0 * m0 + B_coef * (sum_k rho_k D1_k [+ rho_last D1_t]).

    `history[k]` is the schedule index of the (k+1)-th older model output relative to s0.
    """
    c = self.config
    a_t, s_t = self._alpha_sigma(float(sigmas[i_t]))
    a_s0, s_s0 = self._alpha_sigma(float(sigmas[i_s0]))
    lam_t, lam_s0 = self._lambda(a_t, s_t), self._lambda(a_s0, s_s0)
    h = lam_t - lam_s0
    rks = []
    for k in range(order - 1):
      a_k, s_k = self._alpha_sigma(float(sigmas[history[k]]))
      rks.append((self._lambda(a_k, s_k) - lam_s0) / h)
    rks.append(1.0)
    hh = -h if c.predict_x0 else h
    h_phi_1 = math.expm1(hh) if math.isfinite(hh) else -1.0
    h_phi_k = (h_phi_1 / hh - 1.0) if math.isfinite(hh) else -1.0
    B_h = hh if c.solver_type == "bh1" else h_phi_1
    R, b = [], []
    fact = 1.0
    for i in range(1, order + 1):
      R.append([rk ** (i - 1) for rk in rks])
      b.append(h_phi_k * fact / B_h)
      fact *= i + 1
      h_phi_k = (h_phi_k / hh - 1.0 / fact) if math.isfinite(hh) else -1.0 / fact
    R, b = np.array(R, dtype=np.float64), np.array(b, dtype=np.float64)
    if corrector:
      rhos = np.array([0.5]) if order == 1 else np.linalg.solve(R, b)
    else:
      if order == 1:
        rhos = np.zeros(0)
      elif order == 2:
        rhos = np.array([0.5])
      else:
        rhos = np.linalg.solve(R[:-1, :-1], b[:-1])
    if c.predict_x0:
      c_x, c_m0, B_coef = s_t / s_s0, -a_t * h_phi_1, -a_t * B_h
    else:
      c_x, c_m0, B_coef = a_t / a_s0, -s_t * h_phi_1, -s_t * B_h
    return c_x, c_m0, B_coef, rhos, rks

  def _predict(self, state, sample, order: int):
    i = state.step_index
    hist = [i - k for k in range(1, order)]
    c_x, c_m0, B_coef, rhos, rks = self._coefficients(state.sigmas, i, i + 1, hist, order, corrector=False)
    m0 = state.model_outputs[-1]
    x = c_x * sample + c_m0 * m0
    for k in range(order - 1):
      mk = state.model_outputs[-(k + 2)]
      x = x + (B_coef * rhos[k] / rks[k]) * (mk - m0)
    return x

  def _correct(self, state, this_model_output, last_sample, order: int):
    i = state.step_index
    hist = [i - 1 - k for k in range(1, order)]
    c_x, c_m0, B_coef, rhos, rks = self._coefficients(state.sigmas, i - 1, i, hist, order, corrector=True)
    m0 = state.model_outputs[-1]
    x = c_x * last_sample + c_m0 * m0
    for k in range(order - 1):
      mk = state.model_outputs[-(k + 2)]
      x = x + (B_coef * rhos[k] / rks[k]) * (mk - m0)
    return x + (B_coef * rhos[-1]) * (this_model_output - m0)

  # ------------------------------------------------------------------ step
  def step(self, state, model_output, timestep, sample):
    """One denoising step. Returns (prev_sample, new_state)."""
    c = self.config
    if state.step_index is None:
      # a loop may start in the middle of the schedule (image-to-image: noise added at `timesteps[k]`, then steps from
      # k on): the first step's position is where its timestep sits in the schedule, the last position if it is absent
      match = (state.timesteps.to(torch.float64) == float(timestep)).nonzero()
      state = state.replace(step_index=int(match[0]) if match.numel() else len(state.timesteps) - 1)
    i = state.step_index
    work_dtype = torch.float32
    sample = sample.to(work_dtype)
    x0 = self.convert_model_output(state, model_output.to(work_dtype), sample)
    use_corrector = i > 0 and (i - 1) not in c.disable_corrector and state.last_sample is not None
    if use_corrector:
      sample = self._correct(state, x0, state.last_sample, state.this_order)
    outputs = list(state.model_outputs[1:]) + [x0]
    n_steps = len(state.sigmas) - 1
    this_order = min(c.solver_order, n_steps - i) if c.lower_order_final else c.solver_order
    this_order = max(1, min(this_order, state.lower_order_nums + 1))
    state = state.replace(model_outputs=outputs, this_order=this_order, last_sample=sample)
    prev = self._predict(state, sample, this_order)
    lower = state.lower_order_nums + 1 if state.lower_order_nums < c.solver_order else state.lower_order_nums
    state = state.replace(lower_order_nums=lower, step_index=i + 1)
    return prev, state

  def scale_model_input(self, state, sample, timestep=None):
    return sample

  def add_noise(self, state, original, noise, timesteps):
    idx = [int((state.timesteps == t).nonzero()[0]) for t in torch.as_tensor(timesteps).reshape(-1)]
    sig = torch.as_tensor([state.sigmas[j] for j in idx], dtype=original.dtype, device=original.device)
    sig = sig.reshape((-1,) + (1,) * (original.dim() - 1))
    if self.config.use_flow_sigmas:
      return (1 - sig) * original + sig * noise
    alpha = 1.0 / (sig * sig + 1).sqrt()
    return alpha * original + sig * alpha * noise
