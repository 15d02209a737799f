"""Scheduler trajectories: every sampler must integrate a known linear model to the analytic answer."""
import math

import pytest
import torch

from maxdiffusion_b200.schedulers import (DDIMScheduler, DDPMScheduler, DPMSolverMultistepScheduler, EulerDiscreteScheduler,
                                          FlowMatchScheduler, LMSDiscreteScheduler, PNDMScheduler,
                                          RectifiedFlowMultistepScheduler, UniPCMultistepScheduler)


def test_unipc_flow_recovers_x0_for_exact_velocity():
  """With the exact flow velocity v = eps - x0 of a fixed (x0, eps) pair every order of UniPC lands on x0."""
  torch.manual_seed(0)
  x0, eps = torch.randn(2, 4, 3, 8, 8), torch.randn(2, 4, 3, 8, 8)
  for order in (1, 2, 3):
    s = UniPCMultistepScheduler(solver_order=order, flow_shift=5.0)
    st = s.set_timesteps(s.create_state(), 12, x0.shape)
    assert st.timesteps[0] > st.timesteps[-1] and len(st.sigmas) == 13 and st.sigmas[-1] == 0
    x = (1 - st.sigmas[0]) * x0 + st.sigmas[0] * eps
    for t in st.timesteps.tolist():
      x, st = s.step(st, eps - x0, t, x)
    assert torch.allclose(x, x0, atol=1e-4), order


def test_unipc_matches_euler_limit_and_order_ramp():
  s = UniPCMultistepScheduler(solver_order=2, flow_shift=3.0)
  st = s.set_timesteps(s.create_state(), 8, (1,))
  orders = []
  x = torch.ones(1)
  for t in st.timesteps.tolist():
    x, st = s.step(st, torch.zeros(1), t, x)
    orders.append(st.this_order)
  assert orders[0] == 1 and orders[1] == 2 and orders[-1] == 1   # warm-up and lower_order_final


def test_flow_match_schedule_and_euler_step():
  s = FlowMatchScheduler(shift=5.0)
  st = s.set_timesteps(s.create_state(), 10)
  sig = torch.linspace(1.0, 0.003 / 1.002, 10, dtype=torch.float64)
  assert torch.allclose(st.sigmas.double(), 5 * sig / (1 + 4 * sig), atol=1e-6)
  x0, eps = torch.randn(3, 4), torch.randn(3, 4)
  x = (1 - st.sigmas[0]) * x0 + st.sigmas[0] * eps
  for i, t in enumerate(st.timesteps):
    x, st = s.step(st, eps - x0, t, x, step_index=i)
  assert torch.allclose(x, x0, atol=1e-5)
  noisy, target, w = s.apply_flow_match(eps, x0, torch.tensor([500.0, 100.0, 900.0]), s.set_timesteps(s.create_state(), 1000, training=True))
  assert torch.allclose(target, eps - x0) and w.shape == (3,) and (w >= 0).all()


@pytest.mark.parametrize("cls,kw", [(DDIMScheduler, {}), (EulerDiscreteScheduler, {}), (DPMSolverMultistepScheduler, {}),
                                    (PNDMScheduler, {}), (LMSDiscreteScheduler, {})])
def test_epsilon_samplers_denoise_a_point_mass(cls, kw):
  """Data distribution = a single point x*; the optimal epsilon-predictor is (x - sqrt(a) x*) / sqrt(1 - a)."""
  torch.manual_seed(1)
  s = cls(beta_start=0.00085, beta_end=0.012, beta_schedule="scaled_linear", **kw)
  st = s.set_timesteps(s.create_state(), 30)
  target = torch.tensor([[0.7, -0.3, 0.2, 0.5]])
  x = torch.randn(1, 4) * getattr(st, "init_noise_sigma", 1.0)
  acp = st.common.alphas_cumprod.double()
  for t in st.timesteps.tolist():
    xin = s.scale_model_input(st, x, t)
    ti = int(round(t))
    a = float(acp[ti])
    eps = (xin - math.sqrt(a) * target) / math.sqrt(1 - a)
    x, st = s.step(st, eps, t, x)
  assert torch.allclose(x, target, atol=5e-2), (cls.__name__, x)


def test_ddpm_add_noise_velocity_and_rectified_flow():
  s = DDPMScheduler(beta_schedule="scaled_linear", beta_start=0.00085, beta_end=0.012)
  st = s.create_state()
  x0, n = torch.randn(2, 3), torch.randn(2, 3)
  t = torch.tensor([10, 900])
  a = st.common.alphas_cumprod[t][:, None]
  assert torch.allclose(s.add_noise(st, x0, n, t), a.sqrt() * x0 + (1 - a).sqrt() * n, atol=1e-6)
  assert torch.allclose(s.get_velocity(st, x0, n, t), a.sqrt() * n - (1 - a).sqrt() * x0, atol=1e-6)
  rf = RectifiedFlowMultistepScheduler()
  rs = rf.set_timesteps(rf.create_state(), 10)
  x = rf.add_noise(rs, x0, n, torch.tensor([1.0, 1.0]))
  for tt in rs.timesteps.tolist():
    x, rs = rf.step(rs, n - x0, tt, x)
  assert torch.allclose(x, x0, atol=1e-5)


def test_euler_flux_spacing():
  s = EulerDiscreteScheduler(timestep_spacing="flux")
  st = s.set_timesteps(s.create_state(), 4, timestep_shift=1.15)
  assert st.sigmas[0] == 1.0 and st.sigmas[-1] == 0.0 and len(st.sigmas) == 5
