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


# Entries 17 + 2731 k (k = 0..11) of the flattened [1, 256, 128] sample after each of the five steps, then its mean and
# mean absolute value: read from the trajectories stored with the reference's scheduler test
# (src/maxdiffusion/tests/legacy_hf_tests/schedulers/rf_scheduler_test_ref/step_01..05.npy), which were produced by the
# original PyTorch scheduler of LTX-Video. Procedure of that test: torch.Generator seeded with 42 draws the sample and then
# one "model output" per step; sampler LinearQuadratic, no shifting, 5 steps.
_RF_GOLDEN = (
    ([-0.175802, 1.459738, -1.672742, -0.964861, -0.964565, -1.910584, -0.73948, 0.875368, -1.86244, 0.401301, -0.481901, -1.324342], 0.0030629, 0.801981),
    ([-0.184602, 1.460864, -1.678226, -0.956433, -0.976795, -1.927391, -0.729426, 0.87471, -1.865385, 0.391484, -0.495163, -1.336622], 0.0029942, 0.802161),
    ([-0.378744, 1.623711, -1.907421, -0.847355, -1.149233, -1.85593, -0.821218, 0.864833, -2.015669, 0.416599, -0.427006, -1.442634], 0.0035431, 0.808093),
    ([0.386029, 1.70213, -1.655608, -1.16029, -1.218508, -1.766913, -0.563438, 0.828621, -2.053754, -0.07025, -0.451482, -1.080794], 0.0015037, 0.849606),
    ([0.458059, 0.971902, -1.366318, -1.079545, -1.289791, -0.756919, -0.886947, 0.711523, -1.528732, -0.300032, -0.87654, -0.912497], 0.0054846, 0.95287),
)


def test_rectified_flow_reproduces_the_stored_trajectory_of_the_original_scheduler():
  from maxdiffusion_b200.schedulers.scheduling_rectified_flow import RectifiedFlowMultistepScheduler, linear_quadratic_schedule

  shape = (1, 256, 128)
  g = torch.Generator().manual_seed(42)
  sch = RectifiedFlowMultistepScheduler(num_train_timesteps=1000, shifting=None, base_resolution=None, sampler="LinearQuadratic")
  state = sch.set_timesteps(sch.create_state(), 5, shape)
  assert torch.allclose(state.timesteps, torch.tensor([1.0, 0.9875, 0.975, 0.858333, 0.533333]), atol=1e-5)
  x = torch.randn(shape, generator=g)
  idx = [17 + 2731 * k for k in range(12)]
  for t, (vals, mean, mean_abs) in zip(state.timesteps, _RF_GOLDEN):
    x, state = sch.step(state, torch.randn(shape, generator=g), t, x)
    flat = x.reshape(-1).double()
    assert torch.allclose(flat[idx], torch.tensor(vals, dtype=torch.float64), atol=2e-6)
    assert abs(float(flat.mean()) - mean) < 1e-6 and abs(float(flat.abs().mean()) - mean_abs) < 2e-6
  # the schedule is 1 - sigma, ends one step short of 0, and is a single value for one step
  assert linear_quadratic_schedule(1).tolist() == [1.0]
  lq = linear_quadratic_schedule(40)
  assert lq[0] == 1.0 and bool((lq[1:] < lq[:-1]).all()) and abs(float(lq[20]) - 0.975) < 1e-6


def test_rectified_flow_samplers_and_resolution_shifts():
  from maxdiffusion_b200.schedulers.scheduling_rectified_flow import RectifiedFlowMultistepScheduler, time_shift

  uni = torch.linspace(1.0, 0.25, 4)
  const = RectifiedFlowMultistepScheduler(sampler="Constant", shift=1.5)
  assert torch.allclose(const.set_timesteps(const.create_state(), 4).timesteps, time_shift(1.5, 1.0, uni))
  with pytest.raises(ValueError, match="shift"):
    RectifiedFlowMultistepScheduler(sampler="Constant").set_timesteps(RectifiedFlowMultistepScheduler().create_state(), 4)
  with pytest.raises(ValueError, match="not supported"):
    RectifiedFlowMultistepScheduler(sampler="Cosine").set_timesteps(RectifiedFlowMultistepScheduler().create_state(), 4)
  # SimpleDiffusion: logit(t) + log(tokens / base): more tokens than the base resolution push every timestep up
  sd = RectifiedFlowMultistepScheduler(shifting="SimpleDiffusion", base_resolution=32 * 32)
  ts = sd.set_timesteps(sd.create_state(), 4, (1, 8, 4, 32, 32)).timesteps
  want = torch.sigmoid(torch.logit(uni.clamp(max=1 - 1e-8)) + math.log(4 * 32 * 32 / (32 * 32)))
  assert torch.allclose(ts[1:], want[1:], atol=1e-6) and bool((ts[1:] > uni[1:]).all())
  same = sd.set_timesteps(sd.create_state(), 4, (1, 8, 1, 32, 32)).timesteps
  assert torch.allclose(same[1:], uni[1:], atol=1e-6)
  # SD3 with a terminal value: the last timestep lands on it; without SD3 shifting the terminal is not applied
  sd3 = RectifiedFlowMultistepScheduler(shifting="SD3", target_shift_terminal=0.1)
  assert abs(float(sd3.set_timesteps(sd3.create_state(), 6, (1, 2048, 64)).timesteps[-1]) - 0.1) < 1e-6
  plain = RectifiedFlowMultistepScheduler(target_shift_terminal=0.1)
  assert torch.allclose(plain.set_timesteps(plain.create_state(), 4, (1, 2048, 64)).timesteps, uni)


# Full-loop values asserted by the reference's scheduler tests (src/maxdiffusion/tests/legacy_hf_tests/schedulers/
# test_scheduler_flax.py:607-643,903-939 and test_scheduler_unipc.py:445-465,500-531), which go back to the PyTorch
# implementations the reference was ported from. Procedure there: the sample is arange(768) / 768 laid out as
# [3, 8, 8, 4] and moved to [4, 3, 8, 8]; the "model" is x * t / (t + 1); 10 inference steps on the linear beta schedule.
def _deterministic_sample(reverse=False):
  n = 4 * 3 * 8 * 8
  base = torch.arange(n, dtype=torch.float32)
  return ((base.flip(-1) if reverse else base).reshape(3, 8, 8, 4) / n).permute(3, 0, 1, 2).contiguous()


def _full_loop(sch, start=0, noise=None):
  state = sch.set_timesteps(sch.create_state(), 10, (4, 3, 8, 8))
  x = _deterministic_sample()
  ts = state.timesteps[start:]
  if noise is not None:
    x = sch.add_noise(state, x, noise, ts[:1])
  for t in ts:
    x, state = sch.step(state, x * t / (t + 1), t, x)
  return float(x.abs().sum()), float(x.abs().mean())


@pytest.mark.parametrize("kw,want_sum,want_mean", [({}, 172.0067, 0.223967),
                                                   ({"set_alpha_to_one": True, "beta_start": 0.01}, 149.8295, 0.1951),
                                                   ({"set_alpha_to_one": False, "beta_start": 0.01}, 149.0784, 0.1941)])
def test_ddim_full_loop_matches_the_reference_values(kw, want_sum, want_mean):
  cfg = dict(num_train_timesteps=1000, beta_start=0.0001, beta_end=0.02, beta_schedule="linear")
  got_sum, got_mean = _full_loop(DDIMScheduler(**{**cfg, **kw}))
  assert abs(got_sum - want_sum) < 1e-2 and abs(got_mean - want_mean) < 1e-3


@pytest.mark.parametrize("kw,want_sum,want_mean", [({}, 198.1318, 0.2580),
                                                   ({"set_alpha_to_one": True, "beta_start": 0.01}, 186.9466, 0.24342),
                                                   ({"set_alpha_to_one": False, "beta_start": 0.01}, 186.9482, 0.2434)])
def test_pndm_with_runge_kutta_warm_up_matches_the_reference_values(kw, want_sum, want_mean):
  cfg = dict(num_train_timesteps=1000, beta_start=0.0001, beta_end=0.02, beta_schedule="linear", skip_prk_steps=False)
  sch = PNDMScheduler(**{**cfg, **kw})
  state = sch.set_timesteps(sch.create_state(), 10, (4, 3, 8, 8))
  assert state.prk_timesteps.tolist() == [900, 850, 850, 800, 800, 750, 750, 700, 700, 650, 650, 600]
  assert state.plms_timesteps.tolist() == [600, 500, 400, 300, 200, 100, 0]
  got_sum, got_mean = _full_loop(sch)
  assert abs(got_sum - want_sum) < 1e-2 and abs(got_mean - want_mean) < 1e-3
  with pytest.raises(ValueError, match="three earlier model outputs"):
    sch.step_plms(state, torch.zeros(1), 100, torch.zeros(1))


def test_unipc_on_the_beta_schedule_matches_the_reference_values():
  cfg = dict(num_train_timesteps=1000, beta_start=0.0001, beta_end=0.02, beta_schedule="linear", solver_order=2,
             solver_type="bh2", final_sigmas_type="sigma_min", use_flow_sigmas=False)
  assert abs(_full_loop(UniPCMultistepScheduler(prediction_type="epsilon", **cfg))[1] - 0.2464) < 1e-3
  assert abs(_full_loop(UniPCMultistepScheduler(prediction_type="v_prediction", **cfg))[1] - 0.1014) < 1e-3
  # image-to-image: noise is added at the 9th timestep and the loop runs from there -- the first step has to find its
  # place in the schedule from its timestep
  got_sum, got_mean = _full_loop(UniPCMultistepScheduler(prediction_type="epsilon", **cfg), start=8,
                                 noise=_deterministic_sample(reverse=True))
  assert abs(got_sum - 315.5757) < 1e-2 and abs(got_mean - 0.4109) < 1e-3


def test_ddpm_variance_matches_the_reference_values():
  sch = DDPMScheduler()
  state = sch.create_state()
  for t, want in ((0, 0.0), (487, 0.00979), (999, 0.02)):
    assert abs(float(sch._variance(state, t, t - 1)) - want) < 1e-5
