"""Peer-memory kernels on 2 GPUs (NCCL ranks as child processes): fused reduce-scatter + AdamW, the flag-gated K/V
exchange feeding one flash-attention launch, and a training step that must agree with the NCCL path."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs",
                   "base_wan_14b.yml")


def _spawn(fn, world, *args):
  import socket

  import torch.multiprocessing as mp

  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
  ctx = mp.get_context("spawn")
  q = ctx.Queue()
  procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, q)) for r in range(world)]
  for p in procs:
    p.start()
  out = {}
  try:
    for _ in range(world):
      rank, status, payload = q.get(timeout=600)
      if status != "ok":
        raise RuntimeError(f"rank {rank} failed:\n{payload}")
      out[rank] = payload
  finally:
    for p in procs:
      p.join(timeout=30)
      if p.is_alive():
        p.kill()
  return [out[r] for r in range(world)]


def _entry(rank, world, port, fn, args, q):
  import traceback

  import torch.distributed as dist

  os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world),
                     "LOCAL_RANK": str(rank), "NCCL_NVLS_ENABLE": "0"})
  try:
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    out = fn(rank, world, *args)
    torch.cuda.synchronize()
    dist.barrier()  # peers may still be pulling from this rank's symmetric buffers: leave together
    from maxdiffusion_b200.ops import _lib

    _lib.raise_on_device_status()
    q.put((rank, "ok", out))
  except Exception:
    q.put((rank, "error", traceback.format_exc()))
  finally:
    if dist.is_initialized():
      dist.destroy_process_group()


def _rs_adamw(rank, world):
  import torch.distributed as dist

  from maxdiffusion_b200.ops import ref
  from maxdiffusion_b200.parallel import symm

  peer = symm.PeerGroup(dist.group.WORLD)
  n_full = 8 * 1024 * 64 * world
  shard = n_full // world
  torch.manual_seed(100 + rank)
  sym, ptrs, _ = peer.alloc(n_full, torch.bfloat16)
  grads = torch.randn(n_full, device="cuda", dtype=torch.bfloat16)
  sym.copy_(grads)
  torch.manual_seed(7)
  p = torch.randn(shard, device="cuda", dtype=torch.bfloat16)
  m = torch.zeros(shard, device="cuda", dtype=torch.float32)
  v = torch.zeros(shard, device="cuda", dtype=torch.float32)
  p2, m2, v2 = p.clone(), m.clone(), v.clone()
  stats = torch.zeros(2, device="cuda")
  scratch = torch.empty(128, device="cuda")
  hp = dict(lr=1e-2, b1=0.9, b2=0.999, eps=1e-8, wd=0.01)
  peer.signal(symm.FLAG_GRAD_READY, 1)
  peer.wait(symm.FLAG_GRAD_READY, 1)
  symm.rs_adamw([b + rank * shard * 2 for b in ptrs], shard, p, m, v, stats, scratch, step=1, stochastic=False, ctas=64, **hp)
  peer.signal(symm.FLAG_GRAD_ACK, 1)
  peer.wait(symm.FLAG_GRAD_ACK, 1)
  # reference: NCCL reduce-scatter in fp32, then the plain AdamW
  full32 = grads.float()
  red = torch.empty(shard, device="cuda")
  dist.reduce_scatter_tensor(red, full32)
  ref.adamw_step(p2, red, m2, v2, step=1, **hp)
  torch.cuda.synchronize()
  err_p = (p.float() - p2.float()).abs().max().item()
  err_m = (m - m2).abs().max().item()
  want_sq = (red * red).sum().item()
  return err_p, err_m, stats[0].item(), want_sq, stats[1].item(), red.abs().max().item()


def test_rs_adamw_matches_nccl_reduce_scatter_then_adamw():
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  for err_p, err_m, sq, want_sq, mx, want_mx in _spawn(_rs_adamw, 2):
    assert err_p <= 2e-2 and err_m < 1e-3
    assert abs(sq - want_sq) / want_sq < 1e-3 and abs(mx - want_mx) < 1e-2


def _kv_exchange(rank, world):
  import torch.distributed as dist

  from maxdiffusion_b200.ops import kernels as K, ref
  from maxdiffusion_b200.parallel import collectives as C, symm

  peer = symm.PeerGroup(dist.group.WORLD)
  B, S, H = 1, 520, 4
  ex = symm.PeerKVExchange(peer, B * S * H * 128)
  errs = []
  for it in range(3):  # three epochs exercise both slots and the ack protocol
    torch.manual_seed(1000 * it + rank)
    q = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
    k = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
    v = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
    if it == 1:
      kg, vg = ex.gather(k, v)                     # stand-alone pull (the recomputation path)
      out, _ = K.flash_fwd(q, list(kg), list(vg))
    else:
      kg, vg, flags, epoch, plan, keep = ex.plan(k, v)   # copy CTAs fused into the attention launch
      out, _ = K.flash_fwd(q, list(kg), list(vg), seg_flags=flags, flag_target=epoch, plan=plan)
    k_all = C.all_gather_stack(k, dist.group.WORLD)
    v_all = C.all_gather_stack(v, dist.group.WORLD)
    want = ref.attention(q, list(k_all), list(v_all))
    errs.append((out.float() - want.float()).abs().max().item())
    order = ex.order()
    assert all(torch.equal(kg[j], k_all[order[j]]) for j in range(world))
  # head-group slabs with a ragged last group (5 heads in groups of 2, 2, 1), two batch rows, on a NEW exchange of the
  # same peer group: its epochs continue where the first exchange stopped, so no wait is satisfied by a stale flag
  B, S, H = 2, 392, 5
  grouped = symm.PeerKVExchange(peer, B * S * H * 128, head_groups=3)
  for it in range(3):
    torch.manual_seed(77 * it + rank)
    q = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
    k = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
    v = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
    kg, vg, flags, epoch, plan, keep = grouped.plan(k, v)
    out, _ = K.flash_fwd(q, list(kg), list(vg), seg_flags=flags, flag_target=epoch, plan=plan)
    k_all = C.all_gather_stack(k, dist.group.WORLD)
    v_all = C.all_gather_stack(v, dist.group.WORLD)
    order = grouped.order()
    want = ref.attention(q, [k_all[r] for r in order], [v_all[r] for r in order])
    errs.append((out.float() - want.float()).abs().max().item())
    assert all(torch.equal(kg[j], k_all[order[j]]) and torch.equal(vg[j], v_all[order[j]]) for j in range(world))
  assert grouped.epoch == 6 and peer.epochs[symm.FLAG_KV_READY] == 6
  # full-occupancy case: more tiles than SMs, 42 MB per shard -- the copy CTAs must make progress while every
  # other SM holds a compute CTA; compared bit for bit with the same kernel on NCCL-gathered K/V
  B, S, H = 1, 4096, 40
  big = symm.PeerKVExchange(peer, B * S * H * 128)
  torch.manual_seed(rank)
  q = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
  k = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
  v = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
  kg, vg, flags, epoch, plan, keep = big.plan(k, v)
  out, _ = K.flash_fwd(q, list(kg), list(vg), seg_flags=flags, flag_target=epoch, plan=plan)
  k_all = C.all_gather_stack(k, dist.group.WORLD)
  v_all = C.all_gather_stack(v, dist.group.WORLD)
  order = big.order()
  want, _ = K.flash_fwd(q, [k_all[r] for r in order], [v_all[r] for r in order])
  errs.append((out.float() - want.float()).abs().max().item() * 1e3)
  return errs


def test_flag_gated_kv_exchange_feeds_flash_attention():
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  for errs in _spawn(_kv_exchange, 2):
    assert max(errs) < 3e-2


def _kv_exchange_dma(rank, world):
  import torch.distributed as dist

  from maxdiffusion_b200.ops import kernels as K
  from maxdiffusion_b200.parallel import collectives as C, symm

  peer = symm.PeerGroup(dist.group.WORLD)
  errs = []
  # small shards over four epochs (both slots, the acknowledgement from the side stream), then a full-occupancy case:
  # more tiles than SMs and 42 MB per shard, where nothing but copy engines and stream memory operations may move the data
  for (B, S, H, reps) in ((2, 392, 5, 4), (1, 4096, 40, 2)):
    ex = symm.PeerKVExchange(peer, B * S * H * 128, transport="dma")
    for it in range(reps):
      torch.manual_seed(31 * it + rank)
      q = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
      k = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
      v = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
      kg, vg, flags, epoch, plan, keep = ex.plan(k, v)
      assert plan is None and flags.numel() == world
      out, _ = K.flash_fwd(q, list(kg), list(vg), seg_flags=flags, flag_target=epoch)
      k_all = C.all_gather_stack(k, dist.group.WORLD)
      v_all = C.all_gather_stack(v, dist.group.WORLD)
      order = ex.order()
      want, _ = K.flash_fwd(q, [k_all[r] for r in order], [v_all[r] for r in order])
      errs.append((out.float() - want.float()).abs().max().item())
      assert all(torch.equal(kg[j], k_all[order[j]]) and torch.equal(vg[j], v_all[order[j]]) for j in range(world))
      assert flags.tolist() == [epoch] * world
  return errs


def test_copy_engine_kv_transport_feeds_flash_attention_bit_for_bit():
  """`ring_kv_transport=dma`: remote K/V arrive by copy-engine copies on a side stream, each segment's ready flag by a
  stream memory operation behind them; the attention launch has no copy CTAs and must equal the same kernel on
  NCCL-gathered K/V exactly."""
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  for errs in _spawn(_kv_exchange_dma, 2):
    assert max(errs) == 0.0


def test_training_step_with_copy_engine_kv_transport_matches():
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  a = _spawn(_train, 2, True, "tokamax_ring", True, "dma")[0]
  b = _spawn(_train, 2, True, "tokamax_ring", True, "sm")[0]
  assert a == pytest.approx(b, rel=1e-3, abs=1e-3)


def _train(rank, world, peer, attention="tokamax_ring", save_kv=True, kv_transport="sm"):
  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.parallel.mesh import create_device_mesh
  from maxdiffusion_b200.trainers.wan_trainer import WanTrainer

  config = pyconfig.initialize(
      ["t", CFG, "run_name=t", "height=128", "width=128", "num_frames=9", "dataset_type=synthetic", "wan_preset=tiny",
       'wan_config_overrides={"num_layers": 2, "ffn_dim": 1024}', "remat_policy=SAVE_ATTENTION",
       "warmup_steps_fraction=0.0", "log_config=false", "write_metrics=false", f"attention={attention}", "ulysses_shards=2",
       f"per_device_batch_size={1.0 / world}", f"peer_memory_transport={'true' if peer else 'false'}",
       "stochastic_rounding=false", f"ring_save_remote_kv={'true' if save_kv else 'false'}",
       f"ring_kv_transport={kv_transport}"], unittest=True)
  tr = WanTrainer(config, mesh=create_device_mesh(config))
  data = tr.load_dataset()
  return [float(tr.train_step(next(data))["learning/loss"]) for _ in range(3)]


def test_training_step_peer_transport_matches_nccl():
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  a = _spawn(_train, 2, True)[0]
  b = _spawn(_train, 2, False)[0]
  assert a == pytest.approx(b, rel=3e-2, abs=3e-2)


def test_training_step_that_refetches_remote_kv_in_the_backward_matches():
  """`ring_save_remote_kv=false`: only the own K/V shard is kept per layer and the others are pulled again for the
  backward; the losses of the following steps (which see the updated weights) must not move."""
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  a = _spawn(_train, 2, True, "tokamax_ring", False)[0]
  b = _spawn(_train, 2, True, "tokamax_ring", True)[0]
  assert a == pytest.approx(b, rel=1e-3, abs=1e-3)


def test_training_step_peer_transport_matches_nccl_on_4_ranks():
  """On more than 2 ranks the peer-memory exchange presents the K/V segments in backwards ring order while the NCCL
  path presents them in rank order: the joint dK/dV launch has to return every partial to the right owner in both."""
  if torch.cuda.device_count() < 4:
    pytest.skip("needs 4 GPUs")
  a = _spawn(_train, 4, True)[0]
  b = _spawn(_train, 4, False)[0]
  assert a == pytest.approx(b, rel=3e-2, abs=3e-2)


def test_two_dimensional_usp_on_4_ranks_peer_transport_matches_nccl():
  """Ulysses 2 x ring 2 with both axes larger than one: the peer-memory all-to-all inside the Ulysses pairs feeds the
  flag-gated ring launch across them; losses must agree with the NCCL transport of the same mesh."""
  if torch.cuda.device_count() < 4:
    pytest.skip("needs 4 GPUs")
  a = _spawn(_train, 4, True, "ulysses_ring")[0]
  b = _spawn(_train, 4, False, "ulysses_ring")[0]
  assert a == pytest.approx(b, rel=3e-2, abs=3e-2)


def _fused_ulysses(rank, world, strategy, ulysses):
  """`projected_self_attention` without autograd (exchanges folded into the norm / RoPE stores and the attention
  epilogue) against the same call with autograd enabled (norm + RoPE locally, pull all-to-all kernels)."""
  from maxdiffusion_b200.parallel.context import ContextParallel
  from maxdiffusion_b200.parallel.mesh import create_device_mesh

  mesh = create_device_mesh(shape={"data": 1, "fsdp": 1, "context": world, "tensor": 1}, ulysses_shards=ulysses)
  pctx = ContextParallel(mesh, strategy, peer_memory=True)
  B, S, H, D = 1, 200, 8, 128
  errs = []
  for it in range(4):  # more calls than buffer slots
    full_len = world * S - (5 if it % 2 else 0)
    pctx.full_len, pctx.local_len = (full_len, S) if it % 2 else (None, None)
    torch.manual_seed(50 * it + rank)
    q, k, v = (torch.randn(B, S, H * D, device="cuda").to(torch.bfloat16) for _ in range(3))
    wq, wk = (torch.rand(H * D, device="cuda") + 0.5).to(torch.bfloat16), (torch.rand(H * D, device="cuda") + 0.5).to(torch.bfloat16)
    ang = torch.rand(S, D // 2, device="cuda") * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    with torch.enable_grad():
      want = pctx.projected_self_attention(q, k, v, wq, wk, cos, sin, H, 1e-6)
    with torch.no_grad():
      got = pctx.projected_self_attention(q, k, v, wq, wk, cos, sin, H, 1e-6).clone()
    errs.append((got.float() - want.float()).abs().max().item())
  assert pctx._fused, "the fused exchange was not used"
  return errs


def test_ulysses_exchanges_folded_into_producer_and_consumer_kernels():
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  for errs in _spawn(_fused_ulysses, 2, "ulysses", 2):
    assert max(errs) < 2e-2, errs


def test_two_dimensional_usp_with_folded_ulysses_exchanges_on_4_ranks():
  if torch.cuda.device_count() < 4:
    pytest.skip("needs 4 GPUs")
  for errs in _spawn(_fused_ulysses, 4, "usp", 2):
    assert max(errs) < 2e-2, errs


def _small_allreduce(rank, world):
  import torch.distributed as dist

  from maxdiffusion_b200.parallel import symm

  peer = symm.PeerGroup(dist.group.WORLD)
  ar = symm.SmallAllReduce(peer, capacity=1024)
  outs = []
  for it in range(6):  # more calls than buffer halves: exercises the epoch alternation
    torch.manual_seed(1000 * it + rank)
    x = torch.randn(1 + 170 * it, device="cuda")
    got_sum, got_max = ar(x, "sum"), ar(x, "max")
    want_sum, want_max = x.clone(), x.clone()
    dist.all_reduce(want_sum)
    dist.all_reduce(want_max, op=dist.ReduceOp.MAX)
    outs.append(((got_sum - want_sum).abs().max().item(), (got_max - want_max).abs().max().item(),
                 got_sum.sum().item()))
  return outs


def test_small_allreduce_matches_nccl_and_is_identical_across_ranks():
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  res = _spawn(_small_allreduce, 2)
  for per_rank in res:
    for err_sum, err_max, _ in per_rank:
      assert err_sum < 1e-5 and err_max == 0.0
  for a, b in zip(res[0], res[1]):
    assert a[2] == b[2]  # bitwise identical sums on both ranks


def _peer_reduce_scatter(rank, world):
  import torch.distributed as dist

  from maxdiffusion_b200.parallel import symm

  peer = symm.PeerGroup(dist.group.WORLD)
  rs = symm.PeerReduceScatter(peer, 2 * 3 * 40 * 128)
  errs = []
  for it in range(5):  # more epochs than buffer slots
    shape = (2, 3, 8 * (it + 1), 128)
    torch.manual_seed(100 * it + rank)
    parts = [torch.randn(shape, device="cuda").to(torch.bfloat16) for _ in range(world)]
    views = rs.slices(shape)
    for v, p in zip(views, parts):
      v.copy_(p)
    got = rs.reduce()
    want = torch.empty(shape, device="cuda")
    dist.reduce_scatter_tensor(want, torch.stack([p.float() for p in parts]))
    errs.append(((got.float() - want).abs().max() / want.abs().max()).item())
  torch.cuda.synchronize()
  dist.barrier()  # a rank must not free its symmetric buffer while a peer's last pull is still reading it
  return errs


@pytest.mark.gpu
def test_peer_reduce_scatter_matches_fp32_sum():
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  res = _spawn(_peer_reduce_scatter, 2)
  for errs in res:
    assert max(errs) < 1e-2, errs  # one bf16 rounding of an fp32 sum


def _peer_all_to_all(rank, world):
  import torch.distributed as dist

  from maxdiffusion_b200.parallel import collectives as C
  from maxdiffusion_b200.parallel import symm

  peer = symm.PeerGroup(dist.group.WORLD)
  ex = symm.PeerAllToAll(peer, 2 * 160 * 4 * world * 128)
  same = []
  for it in range(5):  # more epochs than slots
    torch.manual_seed(10 * it + rank)
    B, S, H, D = 1 + it % 2, 32 * (it + 1) - 3, 4 * world, 128
    x = torch.randn((B, S, H, D), device="cuda").to(torch.bfloat16)
    a = ex.heads_to_seq(x)
    want = C.all_to_all_heads_to_seq(x, dist.group.WORLD)
    back = ex.seq_to_heads(a)
    same.append((torch.equal(a, want), torch.equal(back, x)))
  return same


def test_peer_all_to_all_equals_nccl_and_round_trips():
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  for res in _spawn(_peer_all_to_all, 2):
    assert all(a and b for a, b in res), res


def _spatial_vae(rank, world, peer_memory):
  import torch.distributed as dist

  from maxdiffusion_b200.models.wan.autoencoder_kl_wan import AutoencoderKLWan, WanVAEConfig
  from maxdiffusion_b200.parallel.spatial import HaloExchange

  torch.manual_seed(0)
  vae = AutoencoderKLWan(WanVAEConfig(base_dim=32)).eval().cuda()
  for p in vae.parameters():
    torch.nn.init.normal_(p, std=0.05)
  z = torch.randn(1, 16, 4, 6, 8 * world, device="cuda").to(torch.bfloat16)
  dist.broadcast(z, 0)
  cl = vae.channels_last_decoder()
  halo = HaloExchange(dist.group.WORLD, peer_memory=peer_memory)
  assert (halo.peer is not None) == peer_memory
  with torch.no_grad():
    whole = cl.decode(z, chunk=2)
    split = cl.decode(z, chunk=2, spatial=halo)
    again = cl.decode(z, chunk=1, spatial=halo)  # buffers and epochs carry over between decodes
  return (float((whole.float() - split.float()).abs().max()), float((whole.float() - again.float()).abs().max()),
          float(whole.float().abs().max()), tuple(split.shape), halo.exchanges)


@pytest.mark.parametrize("world,peer_memory", [(2, True), (2, False), (4, True)])
def test_vae_decode_split_over_the_width_with_halo_exchange(world, peer_memory):
  """Width-sharded Wan VAE decode on the convolution kernels: edge columns over peer memory (flags + pull) or NCCL
  point-to-point, against the one-GPU decode of the same latents."""
  if torch.cuda.device_count() < world:
    pytest.skip(f"needs {world} GPUs")
  for err, err2, scale, shape, exchanges in _spawn(_spatial_vae, world, peer_memory):
    assert shape == (1, 3, 13, 48, 64 * world)
    assert err <= 2e-2 * (1 + scale) and err2 <= 2e-2 * (1 + scale), (err, err2, scale)
    assert exchanges > 40


def _small_allreduce_peer_absent(rank, world):
  import torch.distributed as dist

  from maxdiffusion_b200.ops import _lib
  from maxdiffusion_b200.parallel import symm

  peer = symm.PeerGroup(dist.group.WORLD)
  ar = symm.SmallAllReduce(peer, capacity=64)
  x = torch.full((8,), float(rank + 1), device="cuda")
  before = ar(x).tolist()
  torch.cuda.synchronize()
  dist.barrier()
  raised = None
  if rank == 0:
    # the peer sits this call out: with a 50 ms budget the kernel gives up by itself and the host hears why
    old, symm.WAIT_BUDGET_S = symm.WAIT_BUDGET_S, 0.05
    try:
      ar(x)
      torch.cuda.synchronize()
      _lib.raise_on_device_status()
    except _lib.KernelError as e:
      raised = str(e)
    finally:
      symm.WAIT_BUDGET_S = old
  else:
    peer.next_epoch(symm.FLAG_SMALL_AR)  # keeps this rank's epoch count in step with the rank that tried
  dist.barrier()
  after = ar(x).tolist()  # the group goes on working
  return before, raised, after


def test_small_allreduce_whose_peer_never_joins_times_out_and_the_group_recovers():
  """Host-made failure on 2 GPUs: one rank does not make the call (it is between steps, nothing of its own in flight);
  the other rank's wait runs out after 50 ms, the status word names the site, and the next call of both ranks is right."""
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  res = _spawn(_small_allreduce_peer_absent, 2)
  for rank, (before, raised, after) in enumerate(res):
    assert before == [3.0] * 8 and after == [3.0] * 8
    assert (raised is not None and "timed out" in raised) if rank == 0 else raised is None
