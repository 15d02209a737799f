"""Step-skipping policies for Wan sampling: CFG-cache (FasterCache), MagCache, SenCache.

All schedules depend only on host-side quantities, so they are computed before (MagCache, CFG-cache) or between
(SenCache) steps on the host and the device never branches.

Reference: CFG-cache schedule src/maxdiffusion/pipelines/wan/wan_pipeline_2_1.py:269-311 and FFT compensation
src/maxdiffusion/pipelines/wan/wan_pipeline.py:1436-1510; MagCache :1513-1644; SenCache
src/maxdiffusion/pipelines/wan/wan_pipeline_2_2.py:474-609.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------- CFG-cache
def cfg_cache_schedule(num_steps: int, height: int) -> List[bool]:
  """True for the steps that run the cond branch only and reconstruct the uncond one from the cache.

  Cache steps lie in [steps/3, end) with (s - start) % 5 != 0, end = 0.9*steps at >= 720p else steps - 2;
  a cache step always follows at least one full step.
  """
  start = max(1, num_steps // 3)
  end = int(num_steps * 0.9) if height >= 720 else num_steps - 2
  return [start <= s < end and (s - start) % 5 != 0 for s in range(num_steps)]


def cfg_cache_schedule_two_experts(num_steps: int, height: int, step_uses_high: Sequence[bool]) -> List[bool]:
  """CFG-cache schedule of the two-expert models (Wan 2.2): a step of the high-noise expert is never a cache step, the
  first low-noise step is always a full step (it fills the cache: the experts' outputs do not carry over), and the
  window ends one step later than for one expert at below 720p (steps - 1 instead of steps - 2)
  (reference: src/maxdiffusion/pipelines/wan/wan_pipeline_2_2.py, `run_inference_2_2`)."""
  start = int(num_steps / 3)
  end = int(num_steps * 0.9) if height >= 720 else num_steps - 1
  out, full_seen = [], False
  for s in range(num_steps):
    cache = (not step_uses_high[s]) and full_seen and start <= s < end and (s - start) % 5 != 0
    out.append(cache)
    if not step_uses_high[s] and not cache:
      full_seen = True
  return out


def cfg_cache_weights(step: int, num_steps: int, alpha: float = 0.2) -> tuple[float, float]:
  """(w1, w2): boost the low-frequency correction before the midpoint step, the high-frequency one after."""
  return (1.0 + alpha, 1.0) if step < num_steps // 2 else (1.0, 1.0 + alpha)


def fft_compensate(noise_cond, cached_cond, cached_uncond, w1: float, w2: float):
  """uncond ≈ irfft2(rfft2(cond_new) + (low*w1 + high*w2) ⊙ (rfft2(uncond_cached) − rfft2(cond_cached))) over (H, W);
  the low band is the lowest quarter of the frequencies of each axis (wrap-around rows included).

  The transform pair is linear and the band separable, so this is cond_new plus a band-weighted copy of the
  cached difference, computed by `ops.dft.band_weighted` as two real GEMMs (no FFT library, any H and W)."""
  from ...ops import dft
  delta = cached_uncond.float() - cached_cond.float()
  approx = noise_cond.float() + dft.band_weighted(delta, w1, w2)
  return approx.to(noise_cond.dtype)


def fft_compensate_reference(noise_cond, cached_cond, cached_uncond, w1: float, w2: float):
  """The same quantity through `torch.fft`, kept as the oracle of the tests."""
  fc = torch.fft.rfft2(cached_cond.float())
  fu = torch.fft.rfft2(cached_uncond.float())
  bias = fu - fc
  h, w = bias.shape[-2], bias.shape[-1]
  ch, cw = max(1, h // 4), max(1, w // 4)
  fh = torch.arange(h, device=bias.device)
  fw = torch.arange(w, device=bias.device)
  low = ((fh < ch) | (fh >= h - ch + 1))[:, None] & (fw < cw)[None, :]
  weight = torch.where(low, torch.tensor(w1, device=bias.device), torch.tensor(w2, device=bias.device))
  approx = torch.fft.irfft2(torch.fft.rfft2(noise_cond.float()) + bias * weight, s=noise_cond.shape[-2:])
  return approx.to(noise_cond.dtype)


# ---------------------------------------------------------------------------------------------- MagCache
def nearest_interp(src: np.ndarray, target_len: int) -> np.ndarray:
  if target_len == 1:
    return np.array([src[-1]])
  idx = np.round(np.linspace(0, len(src) - 1, target_len)).astype(np.int32)
  return src[idx]


def magcache_forced_steps(num_steps: int, retention_ratio: float, step_uses_high: Optional[Sequence[bool]] = None) -> List[bool]:
  """True for the steps that always run the transformer. One expert: the first `retention_ratio * steps` steps. Two
  experts (`step_uses_high` per step): the first `retention_ratio` fraction of EACH expert's phase, and the step at
  which the expert changes (its residual does not carry over)
  (reference: src/maxdiffusion/pipelines/wan/wan_pipeline_2_2.py, MagCache branch of `run_inference_2_2`)."""
  if step_uses_high is None:
    return [s < int(num_steps * retention_ratio) for s in range(num_steps)]
  high = sum(bool(h) for h in step_uses_high)
  high_end = int(high * retention_ratio)
  low_end = high + int((num_steps - high) * retention_ratio)
  return [s < high_end or high <= s < low_end or (s > 0 and bool(step_uses_high[s]) != bool(step_uses_high[s - 1]))
          for s in range(num_steps)]


def magcache_schedule(num_steps: int, mag_ratios_base: Sequence[float], thresh: float, K: int,
                      retention_ratio: float, step_uses_high: Optional[Sequence[bool]] = None) -> List[bool]:
  """True for the steps whose transformer blocks are skipped (output = input + cached residual).

  `mag_ratios_base` interleaves (cond, uncond) magnitude ratios per calibrated step and is resampled to
  `num_steps`; it is indexed by the global step for both experts. A step is skipped while the accumulated error
  |1 - prod ratios| stays below `thresh` for both branches and fewer than K consecutive steps have been skipped; the
  steps of `magcache_forced_steps` always run and restart the accumulation.
  """
  base = np.asarray(mag_ratios_base, dtype=np.float64)
  if len(base) != 2 * num_steps:
    cond, uncond = nearest_interp(base[0::2], num_steps), nearest_interp(base[1::2], num_steps)
    ratios = np.stack([cond, uncond], axis=1).reshape(-1)
  else:
    ratios = base
  forced = magcache_forced_steps(num_steps, retention_ratio, step_uses_high)
  rc = ru = 1.0
  ec = eu = 0.0
  nc = nu = 0
  out = []
  for s in range(num_steps):
    skip = False
    if forced[s]:
      rc = ru = 1.0
      ec = eu = 0.0
      nc = nu = 0
    else:
      new_c, new_u = rc * ratios[2 * s], ru * ratios[2 * s + 1]
      dc, du = abs(1.0 - new_c), abs(1.0 - new_u)
      if ec + dc < thresh and nc < K and eu + du < thresh and nu < K:
        skip = True
        rc, ru, ec, eu, nc, nu = new_c, new_u, ec + dc, eu + du, nc + 1, nu + 1
      else:
        rc = ru = 1.0
        ec = eu = 0.0
        nc = nu = 0
    out.append(skip)
  # the very first executed step has no residual to reuse
  if out and out[0]:
    out[0] = False
  return out


# ---------------------------------------------------------------------------------------------- SenCache
@dataclass
class SenCacheState:
  score: float = 0.0
  reuse_count: int = 0
  x_ref: Optional[torch.Tensor] = None
  t_ref: float = 0.0
  cached_pred: Optional[torch.Tensor] = None


class SenCache:
  """Reuses the guided noise prediction while the accumulated sensitivity score stays small.

  score += alpha_x * rms(x - x_ref) + alpha_t * |t - t_ref| / N_train since the last full compute; reuse iff
  score <= threshold and fewer than `max_reuse` consecutive reuses. Forced full compute on step 0, during the
  first 30 % and last 10 % of the steps and at the high -> low noise expert boundary.
  """

  def __init__(self, num_steps: int, threshold: float = 0.1, max_reuse: int = 3, alpha_x: float = 1.0,
               alpha_t: float = 1.0, num_train_timesteps: int = 1000, warmup: float = 0.3, tail: float = 0.1):
    self.n, self.threshold, self.max_reuse = num_steps, threshold, max_reuse
    self.alpha_x, self.alpha_t, self.n_train = alpha_x, alpha_t, num_train_timesteps
    self.first_free = int(num_steps * warmup)
    self.last_free = int(num_steps * (1.0 - tail))
    self.state = SenCacheState()

  def forced(self, step: int, at_boundary: bool = False) -> bool:
    """Steps that always run the model whatever the score: the first, the first 30 %, the last 10 %, an expert change."""
    return step == 0 or step < self.first_free or step >= self.last_free or at_boundary

  def should_reuse(self, step: int, latents: torch.Tensor, t: float, at_boundary: bool) -> bool:
    st = self.state
    if self.forced(step, at_boundary) or st.cached_pred is None:
      return False
    dx = float((latents.float() - st.x_ref.float()).pow(2).mean().sqrt())  # one device -> host scalar per step
    st.score += self.alpha_x * dx + self.alpha_t * abs(t - st.t_ref) / self.n_train
    st.x_ref, st.t_ref = latents, t
    return st.score <= self.threshold and st.reuse_count < self.max_reuse

  def record_full(self, latents: torch.Tensor, t: float, pred: torch.Tensor) -> None:
    self.state = SenCacheState(score=0.0, reuse_count=0, x_ref=latents, t_ref=t, cached_pred=pred)

  def record_reuse(self) -> torch.Tensor:
    self.state.reuse_count += 1
    return self.state.cached_pred
