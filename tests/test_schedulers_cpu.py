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


# ---------------------------------------------------------------------------------------------------------------
# An oracle that owes nothing to any sampler: for Gaussian data x0 ~ N(0, s^2) the optimal denoiser is linear,
#   E[x0 | x_t] = alpha s^2 / (alpha^2 s^2 + sigma^2) * x_t,
# and the probability-flow ODE has the closed-form solution  x_t = x_T * std_t / std_T  with
# std_t^2 = alpha_t^2 s^2 + sigma_t^2. A sampler of order p, fed this denoiser, must land on the closed form with an
# error that falls like (step size)^p.
# ---------------------------------------------------------------------------------------------------------------
S_DATA = 0.6


def _gaussian_eps(x, a):
  """Optimal epsilon prediction at alphas_cumprod = a."""
  alpha, sigma = math.sqrt(a), math.sqrt(1 - a)
  x0 = alpha * S_DATA ** 2 / (alpha ** 2 * S_DATA ** 2 + sigma ** 2) * x
  return (x - alpha * x0) / sigma


def _run_epsilon_sampler(cls, steps, kw=None):
  """Relative error against the closed form at the first timestep <= 250. The comparison stops there on purpose: the
  final step of several samplers is by construction a plain denoising jump to t = 0, and on the integer timestep grid
  the last steps (3 -> 2 -> 1 -> 0) keep a fixed size in log-SNR however many steps are taken, so the end point does
  not show a solver's order."""
  kw = dict(kw or {})
  if cls is DDIMScheduler:
    kw.setdefault("clip_sample", False)  # clipping x0 to [-1, 1] is not part of the ODE
  s = cls(beta_start=0.00085, beta_end=0.012, beta_schedule="scaled_linear", **kw)
  st = s.set_timesteps(s.create_state(), steps)
  acp = st.common.alphas_cumprod.double()
  ve = cls in (EulerDiscreteScheduler, LMSDiscreteScheduler)  # these integrate x / alpha (variance-exploding form)
  torch.manual_seed(3)
  z = torch.randn(1, 64, dtype=torch.float64)

  def closed_form(t):
    a = float(acp[int(round(float(t)))])
    x = z * math.sqrt(a * S_DATA ** 2 + (1 - a))
    return x / math.sqrt(a) if ve else x

  ts = st.timesteps.tolist()
  stop = next(i for i, t in enumerate(ts) if t <= 250)
  x = closed_form(ts[0])
  for t in ts[:stop]:
    xin = s.scale_model_input(st, x.float(), t).double()
    a = float(acp[int(round(t))])
    x, st = s.step(st, _gaussian_eps(xin, a).float(), t, x.float())
    x = x.double()
  want = closed_form(ts[stop])
  return ((x - want).norm() / want.norm()).item()


@pytest.mark.parametrize("cls,min_order", [(DDIMScheduler, 0.8), (EulerDiscreteScheduler, 0.8), (DPMSolverMultistepScheduler, 1.6),
                                           (PNDMScheduler, 1.5), (LMSDiscreteScheduler, 0.4)])
def test_samplers_converge_to_the_closed_form_with_their_order(cls, min_order):
  e1, e2 = _run_epsilon_sampler(cls, 25), _run_epsilon_sampler(cls, 50)
  assert e2 < 0.05, (cls.__name__, e1, e2)
  assert e2 < 1e-4 or math.log2(e1 / e2) > min_order, (cls.__name__, e1, e2, math.log2(e1 / e2))


def _run_flow_sampler(make, steps, stop_sigma=0.3):
  """Flow matching: alpha = 1 - sigma; the model predicts v = eps - x0 with the optimal (linear) denoiser. The error is
  taken where sigma first falls to `stop_sigma` (the last step to sigma = 0 is a first-order jump by design)."""
  s = make()
  st = s.set_timesteps(s.create_state(), steps, (1, 64))
  torch.manual_seed(4)
  z = torch.randn(1, 64, dtype=torch.float64)
  closed = lambda sig: z * math.sqrt((1 - sig) ** 2 * S_DATA ** 2 + sig ** 2)
  sigmas = [float(v) for v in st.sigmas]
  stop = next(i for i, sg in enumerate(sigmas) if sg <= stop_sigma)
  x = closed(sigmas[0])
  for i, t in enumerate(st.timesteps.tolist()[:stop]):
    sig = sigmas[i]
    alpha = 1 - sig
    x0 = alpha * S_DATA ** 2 / (alpha ** 2 * S_DATA ** 2 + sig ** 2) * x
    eps = (x - alpha * x0) / sig
    x, st = s.step(st, (eps - x0).float(), t, x.float())
    x = x.double()
  want = closed(sigmas[stop])
  return ((x - want).norm() / want.norm()).item()


@pytest.mark.parametrize("order,min_rate", [(1, 1.2), (2, 2.2), (3, 2.2)])
def test_unipc_flow_trajectory_matches_the_closed_form_and_its_order(order, min_rate):
  """UniP-p with the UniC-p corrector converges at order p + 1 (the final order-1 step is left out, see above)."""
  make = lambda: UniPCMultistepScheduler(solver_order=order, flow_shift=3.0)
  e1, e2 = _run_flow_sampler(make, 24), _run_flow_sampler(make, 48)
  assert e2 < (1e-2 if order == 1 else 1e-3), (order, e1, e2)
  assert math.log2(e1 / e2) > min_rate, (order, e1, e2)
  if order > 1:  # a higher order is more accurate at the same number of steps
    assert e2 < _run_flow_sampler(lambda: UniPCMultistepScheduler(solver_order=1, flow_shift=3.0), 48)
