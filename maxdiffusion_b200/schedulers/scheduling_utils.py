"""Shared scheduler pieces: beta schedules, the common (alphas, betas) state, add_noise / velocity helpers.

Reference: src/maxdiffusion/schedulers/scheduling_utils_flax.py (`CommonSchedulerState`, `betas_for_alpha_bar`,
`add_noise_common`, `get_velocity_common`, :249-315).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch


def betas_for_alpha_bar(num_steps: int, max_beta: float = 0.999) -> np.ndarray:
  def alpha_bar(t):
    return math.cos((t + 0.008) / 1.008 * math.pi / 2) ** 2

  return np.array([min(1 - alpha_bar((i + 1) / num_steps) / alpha_bar(i / num_steps), max_beta) for i in range(num_steps)],
                  dtype=np.float64)


def rescale_zero_terminal_snr(betas: np.ndarray) -> np.ndarray:
  """Rescales betas so that the last timestep has zero SNR (arXiv 2305.08891, alg. 1)."""
  alphas_bar_sqrt = np.sqrt(np.cumprod(1.0 - betas))
  first, last = alphas_bar_sqrt[0], alphas_bar_sqrt[-1]
  alphas_bar_sqrt = (alphas_bar_sqrt - last) * first / (first - last)
  alphas_bar = alphas_bar_sqrt ** 2
  alphas = np.concatenate([alphas_bar[:1], alphas_bar[1:] / alphas_bar[:-1]])
  return 1.0 - alphas


def betas_for_config(config) -> np.ndarray:
  n = config.num_train_timesteps
  kind = config.get("beta_schedule", "linear")
  if config.get("trained_betas", None) is not None:
    betas = np.asarray(config.trained_betas, dtype=np.float64)
  elif kind == "linear":
    betas = np.linspace(config.beta_start, config.beta_end, n, dtype=np.float64)
  elif kind == "scaled_linear":
    betas = np.linspace(config.beta_start ** 0.5, config.beta_end ** 0.5, n, dtype=np.float64) ** 2
  elif kind == "squaredcos_cap_v2":
    betas = betas_for_alpha_bar(n)
  else:
    raise NotImplementedError(f"beta_schedule {kind}")
  if config.get("rescale_zero_terminal_snr", False):
    betas = rescale_zero_terminal_snr(betas)
  return betas


@dataclass
class CommonSchedulerState:
  alphas: torch.Tensor
  betas: torch.Tensor
  alphas_cumprod: torch.Tensor

  @classmethod
  def create(cls, config, device=None) -> "CommonSchedulerState":
    betas = torch.as_tensor(betas_for_config(config), dtype=torch.float64, device=device)
    alphas = 1.0 - betas
    return cls(alphas=alphas.float(), betas=betas.float(), alphas_cumprod=torch.cumprod(alphas, 0).float())


def _bcast(v: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
  return v.reshape((-1,) + (1,) * (like.dim() - 1)).to(like.device, like.dtype)


def add_noise_common(common: CommonSchedulerState, original, noise, timesteps):
  a = common.alphas_cumprod.to(original.device)[timesteps.long()]
  return _bcast(a.sqrt(), original) * original + _bcast((1 - a).sqrt(), original) * noise


def get_velocity_common(common: CommonSchedulerState, sample, noise, timesteps):
  a = common.alphas_cumprod.to(sample.device)[timesteps.long()]
  return _bcast(a.sqrt(), sample) * noise - _bcast((1 - a).sqrt(), sample) * sample
