"""Failure detection and tensor parallelism on gloo ranks (CPU). Failures are made on the host: a rank that raises,
a rank that stops sending heartbeats, a rank that never reaches a barrier."""
import time

import pytest
import torch

from tests.dist_utils import run_ranks


def _announced_failure(rank, world):
  from maxdiffusion_b200.parallel.health import HealthMonitor, RankFailure, guarded_step

  mon = HealthMonitor(timeout_s=30.0).start()
  mon.barrier(timeout_s=30.0)
  out = "none"
  try:
    with guarded_step(mon, 0):
      if rank == 1:
        raise ValueError("loss is NaN")
  except ValueError:
    out = "raised"
  except RankFailure as e:
    # rank 1 may announce its exception before rank 0 has even entered step 0: then this check already sees it
    out = f"detected {e.ranks} {e.reasons[1]}"
  if rank == 0 and out == "none":
    deadline = time.time() + 20
    while time.time() < deadline:
      try:
        with guarded_step(mon, 1):
          pass
      except RankFailure as e:
        out = f"detected {e.ranks} {e.reasons[1]}"
        break
      time.sleep(0.05)
  mon.stop()
  return out


def test_peer_exception_is_seen_before_the_next_step():
  res = run_ranks(_announced_failure, 2)
  assert res[1] == "raised"
  assert res[0].startswith("detected [1]") and "loss is NaN" in res[0]


def _stale_heartbeat(rank, world):
  from maxdiffusion_b200.parallel.health import HealthMonitor, RankFailure

  mon = HealthMonitor(timeout_s=1.0, interval_s=0.2)
  mon.beat(0)
  mon.barrier(timeout_s=30.0)
  if rank == 1:
    time.sleep(4.0)  # alive but silent: no heartbeat thread was started
    return "silent"
  mon.start()
  deadline = time.time() + 3.5
  while time.time() < deadline:
    try:
      mon.check()
    except RankFailure as e:
      mon.stop()
      return f"stale {e.ranks}"
    time.sleep(0.1)
  mon.stop()
  return "missed"


def test_silent_rank_is_reported_stale():
  res = run_ranks(_stale_heartbeat, 2)
  assert res[0] == "stale [1]"


def _barrier_timeout(rank, world):
  from maxdiffusion_b200.parallel.health import HealthMonitor

  mon = HealthMonitor(timeout_s=30.0)
  mon.beat(0)
  if rank == 1:
    time.sleep(2.5)  # never joins the first barrier in time
    return "late"
  try:
    mon.barrier(timeout_s=1.0)
  except TimeoutError as e:
    return "timeout " + str(e)[-20:]
  return "passed"


def test_barrier_gives_up_instead_of_hanging():
  res = run_ranks(_barrier_timeout, 2)
  assert res[0].startswith("timeout") and "1/2" in res[0]


def _tp_matches_dense(rank, world):
  import torch.distributed as dist

  from maxdiffusion_b200.parallel.tensor import parallel_attention_projections, parallel_mlp

  torch.manual_seed(0)
  dim, hidden = 16, 48
  w_up, b_up = torch.randn(hidden, dim), torch.randn(hidden)
  w_dn, b_dn = torch.randn(dim, hidden), torch.randn(dim)
  x = torch.randn(3, 5, dim, requires_grad=True)
  up, down = parallel_mlp(dim, hidden, group=dist.group.WORLD)
  up.load_full(w_up, b_up)
  down.load_full(w_dn, b_dn)
  y = down(torch.nn.functional.gelu(up(x)))
  y.sum().backward()
  xr = x.detach().clone().requires_grad_(True)
  yr = torch.nn.functional.linear(torch.nn.functional.gelu(torch.nn.functional.linear(xr, w_up, b_up)), w_dn, b_dn)
  yr.sum().backward()
  qkv, out = parallel_attention_projections(dim, group=dist.group.WORLD)
  w_qkv = torch.arange(3 * dim * dim, dtype=torch.float32).reshape(3 * dim, dim)
  qkv.load_full(w_qkv)
  per = dim // world
  want_rows = torch.cat([w_qkv[c * dim + rank * per: c * dim + (rank + 1) * per] for c in range(3)])
  return ((y - yr).abs().max().item(), (x.grad - xr.grad).abs().max().item(), torch.equal(qkv.weight.data, want_rows))


def test_tensor_parallel_mlp_matches_dense_forward_and_backward():
  for err_y, err_g, rows_ok in run_ranks(_tp_matches_dense, 2):
    assert err_y < 1e-4 and err_g < 1e-4 and rows_ok


def _tp_wan(rank, world):
  """A Wan model sharded over the tensor group against the unsharded model with the same weights: forward output and
  the gradients of replicated and sharded parameters."""
  import torch
  import torch.distributed as dist

  from maxdiffusion_b200.models.wan.transformer_wan import WanConfig, WanModel
  from maxdiffusion_b200.parallel.tensor import apply_tensor_parallel_wan

  cfg = WanConfig(num_attention_heads=4, attention_head_dim=32, ffn_dim=96, num_layers=2, text_dim=48, freq_dim=32)
  torch.manual_seed(0)
  full = WanModel(cfg)
  torch.manual_seed(0)
  tp = WanModel(cfg)
  assert apply_tensor_parallel_wan(tp, dist.group.WORLD) == world
  torch.manual_seed(1)
  lat, text, t = torch.randn(1, 16, 2, 8, 8), torch.randn(1, 6, 48), torch.tensor([321.0])
  want = full(lat, t, text)
  got = tp(lat, t, text)
  err = (got - want).abs().max().item()
  want.square().mean().backward()
  got.square().mean().backward()
  n, r = world, rank
  g_full = dict(full.named_parameters())
  g_tp = dict(tp.named_parameters())
  dim, ffn = cfg.dim, cfg.ffn_dim
  checks = []
  # replicated parameter, row-parallel weight (columns), column-parallel fused qkv (rows of every chunk), sharded norm
  checks.append((g_tp["blocks.0.scale_shift_table"].grad - g_full["blocks.0.scale_shift_table"].grad).abs().max().item())
  checks.append((g_tp["blocks.1.ffn_out.weight"].grad - g_full["blocks.1.ffn_out.weight"].grad[:, r * ffn // n:(r + 1) * ffn // n]).abs().max().item())
  per = dim // n
  rows = torch.cat([g_full["blocks.0.attn1.to_qkv.weight"].grad[c * dim + r * per:c * dim + (r + 1) * per] for c in range(3)])
  checks.append((g_tp["blocks.0.attn1.to_qkv.weight"].grad - rows).abs().max().item())
  checks.append((g_tp["blocks.0.attn1.norm_q"].grad - g_full["blocks.0.attn1.norm_q"].grad[r * per:(r + 1) * per]).abs().max().item())
  checks.append((g_tp["patch_embedding.weight"].grad - g_full["patch_embedding.weight"].grad).abs().max().item())
  return err, checks


def test_wan_blocks_sharded_over_the_tensor_axis_match_the_unsharded_model():
  for err, checks in run_ranks(_tp_wan, 2):
    assert err < 2e-5, err
    assert max(checks) < 2e-5, checks
