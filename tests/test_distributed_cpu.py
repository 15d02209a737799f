"""Multi-rank logic on CPU (gloo, world_size 2): FSDP sharding + optimizer-in-backward and context parallelism
must reproduce the single-process training step; collectives must round-trip."""
import os

import pytest
import torch

from tests.dist_utils import run_ranks

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs",
                   "base_wan_14b.yml")
TINY = '{"num_attention_heads": 4, "attention_head_dim": 32, "ffn_dim": 96, "num_layers": 2, "text_dim": 48, "freq_dim": 32}'


def _make_trainer(attention, world, keep=0, extra=()):
  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.parallel.mesh import create_device_mesh
  from maxdiffusion_b200.trainers.wan_trainer import WanTrainer

  config = pyconfig.initialize(
      ["t", CFG, "run_name=t", "height=64", "width=48", "num_frames=9", "dataset_type=synthetic", "wan_preset=tiny",
       f"wan_config_overrides={TINY}", "remat_policy=FULL", "warmup_steps_fraction=0.0", "log_config=false",
       "write_metrics=false", "learning_rate=1e-3", f"attention={attention}", f"per_device_batch_size={1.0 / world}",
       "synthetic_override_text_dim=48", "max_sequence_length=16", "ulysses_shards=2", f"remat_keep_blocks={keep}", *extra],
      unittest=True)
  return WanTrainer(config, mesh=create_device_mesh(config), device="cpu")


def _train(rank, world, attention, steps, keep=0, extra=()):
  torch.manual_seed(0)
  tr = _make_trainer(attention, world, keep, extra)
  data = tr.load_dataset()
  losses = []
  for _ in range(steps):
    m = tr.train_step(next(data))
    losses.append(float(m["learning/loss"]))
  names = [[n for n, _ in b.named_parameters()] for b in tr.model.blocks]
  block_ids = {id(p) for b in tr.model.blocks for p in b.parameters()}
  root_names = [n for n, p in tr.model.named_parameters() if id(p) not in block_ids]
  sd = tr.engine.gather_state_dict(names, root_names)
  digest = {k: v.double().sum().item() for k, v in list(sd.items())[:6]}
  return losses, digest, float(m["learning/max_grad_norm"])


def test_single_process_reference_runs():
  losses, digest, gn = _train(0, 1, "flash", 2)
  assert all(l == l for l in losses) and gn > 0


@pytest.mark.parametrize("attention", ["tokamax_ring", "ulysses", "ulysses_ring"])
def test_two_rank_training_matches_single_process(attention):
  ref_losses, ref_digest, ref_gn = _train(0, 1, "flash", 2)
  out = run_ranks(_train, 2, attention, 2)
  for losses, digest, gn in out:
    assert losses == pytest.approx(ref_losses, rel=2e-4, abs=1e-5)
    assert gn == pytest.approx(ref_gn, rel=2e-3)
    for k, v in ref_digest.items():
      assert digest[k] == pytest.approx(v, rel=1e-4, abs=1e-4), k


def test_two_rank_training_with_kept_blocks_matches_single_process():
  """A block that keeps its activations still gets its weights gathered again before its backward (FSDP, 2 ranks)."""
  ref_losses, ref_digest, ref_gn = _train(0, 1, "flash", 2)
  for losses, digest, gn in run_ranks(_train, 2, "tokamax_ring", 2, 1):
    assert losses == pytest.approx(ref_losses, rel=2e-4, abs=1e-5)
    for k, v in ref_digest.items():
      assert digest[k] == pytest.approx(v, rel=1e-4, abs=1e-4), k


def _train_batch_axes(rank, world, axes, steps):
  """Global batch of 2 samples with fixed noise / timesteps; `axes` = (data, fsdp) sizes. Every batch replica trains
  on its own sample; with one process the same two samples form one batch."""
  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.parallel.mesh import create_device_mesh
  from maxdiffusion_b200.trainers.wan_trainer import WanTrainer

  data, fsdp = axes
  config = pyconfig.initialize(
      ["t", CFG, "run_name=t", "height=64", "width=48", "num_frames=9", "dataset_type=synthetic", "wan_preset=tiny",
       f"wan_config_overrides={TINY}", "remat_policy=FULL", "warmup_steps_fraction=0.0", "log_config=false",
       "write_metrics=false", "learning_rate=1e-3", "attention=flash", f"per_device_batch_size={2 // (data * fsdp)}",
       "synthetic_override_text_dim=48", "max_sequence_length=16", f"ici_data_parallelism={data}",
       f"ici_fsdp_parallelism={fsdp}", "ici_context_parallelism=1"], unittest=True)
  torch.manual_seed(0)
  tr = WanTrainer(config, mesh=create_device_mesh(config), device="cpu")
  g = torch.Generator().manual_seed(11)
  losses = []
  for _ in range(steps):
    full = {"latents": torch.randn(2, 16, 3, 8, 6, generator=g), "encoder_hidden_states": torch.randn(2, 16, 48, generator=g),
            "noise": torch.randn(2, 16, 3, 8, 6, generator=g), "timesteps": torch.tensor([200.0, 700.0])}
    if data * fsdp == 2:
      i = tr.batch_index()
      full = {k: v[i:i + 1] for k, v in full.items()}
    m = tr.train_step(full)
    losses.append(float(m["learning/loss"]))
  names = [[n for n, _ in b.named_parameters()] for b in tr.model.blocks]
  block_ids = {id(p) for b in tr.model.blocks for p in b.parameters()}
  root_names = [n for n, p in tr.model.named_parameters() if id(p) not in block_ids]
  sd = tr.engine.gather_state_dict(names, root_names)
  digest = {k: v.double().sum().item() for k, v in list(sd.items())[:6]}
  return losses, digest, float(m["learning/max_grad_norm"])


@pytest.mark.parametrize("axes", [(2, 1), (1, 2)])
def test_ranks_with_different_samples_match_one_process_with_the_whole_batch(axes):
  """data = 2 (replicated weights, gradient all-reduce) and fsdp = 2 (sharded weights, reduce-scatter): the applied
  update, the logged loss and the gradient norm are those of the mean over the global batch, and the replicas end
  up with identical weights."""
  ref_losses, ref_digest, ref_gn = _train_batch_axes(0, 1, (1, 1), 2)
  out = run_ranks(_train_batch_axes, 2, axes, 2)
  for losses, digest, gn in out:
    assert losses == pytest.approx(ref_losses, rel=2e-4, abs=1e-5)
    assert gn == pytest.approx(ref_gn, rel=2e-3)
    for k, v in ref_digest.items():
      assert digest[k] == pytest.approx(v, rel=1e-4, abs=1e-4), k
  assert out[0][1] == pytest.approx(out[1][1], rel=1e-9)


def _collectives(rank, world):
  import torch.distributed as dist

  from maxdiffusion_b200.parallel import collectives as C

  g = dist.group.WORLD
  x = torch.arange(2 * 6 * 4 * 3, dtype=torch.float32).reshape(2, 6, 4, 3) + 1000 * rank
  y = C.all_to_all_heads_to_seq(x, g)         # [2, 12, 2, 3]
  assert y.shape == (2, 12, 2, 3)
  # sequence block r of y comes from rank r, heads [rank*2, rank*2+2)
  for r in range(world):
    want = (torch.arange(2 * 6 * 4 * 3, dtype=torch.float32).reshape(2, 6, 4, 3) + 1000 * r)[:, :, rank * 2:(rank + 1) * 2]
    assert torch.equal(y[:, r * 6:(r + 1) * 6], want)
  z = C.all_to_all_seq_to_heads(y, g)
  assert torch.equal(z, x)
  st = C.all_gather_stack(x, g)
  assert st.shape[0] == world and torch.equal(st[rank], x)
  rs = C.reduce_scatter_stack(st.clone(), g)
  assert torch.allclose(rs, x * world)
  return True


def test_collective_round_trips():
  assert all(run_ranks(_collectives, 2))


def test_pull_all_to_all_strides_match_the_collective_semantics():
  """Index arithmetic of the peer-memory Ulysses exchange, emulated on the CPU: for every rank, pulling rows with the
  strides of `PeerAllToAll.pull_spec` from every rank's published tensor must give what all_to_all gives."""
  import numpy as np
  import torch

  from maxdiffusion_b200.parallel.symm import PeerAllToAll

  def emulate(kind, xs, rank):
    n, es = len(xs), 2
    sp = PeerAllToAll.pull_spec(kind, tuple(xs[0].shape), n, rank, es)
    out = np.zeros(int(np.prod(sp["out_shape"])) * es, dtype=np.uint8)
    for r in range(n):
      src = xs[r].view(torch.int16).numpy().view(np.uint8).reshape(-1)
      for b in range(sp["n_b"]):
        for s in range(sp["n_s"]):
          so = sp["src_off"] + b * sp["src_sb"] + s * sp["src_ss"]
          do = r * sp["dst_sr"] + b * sp["dst_sb"] + s * sp["dst_ss"]
          out[do:do + sp["row"]] = src[so:so + sp["row"]]
    return torch.from_numpy(out.view(np.int16)).view(torch.bfloat16).reshape(sp["out_shape"])

  n, B, S, hn, D = 3, 2, 5, 2, 8
  H = hn * n
  torch.manual_seed(0)
  xs = [torch.randn(B, S, H, D).to(torch.bfloat16) for _ in range(n)]
  head_sharded = []
  for me in range(n):
    got = emulate("heads_to_seq", xs, me)
    want = torch.cat([x[:, :, me * hn:(me + 1) * hn] for x in xs], dim=1)  # all rows, my heads
    assert torch.equal(got, want)
    head_sharded.append(got)
  for me in range(n):
    back = emulate("seq_to_heads", head_sharded, me)
    assert torch.equal(back, xs[me])


def test_four_rank_two_dimensional_usp_matches_single_process():
  """Ulysses (2, adjacent ranks) x ring (2, strided ranks) with BOTH axes larger than one: heads are exchanged inside
  the Ulysses pairs and the K/V segments travel between them (4 heads over 2 Ulysses ranks, 4 sequence shards)."""
  ref_losses, ref_digest, ref_gn = _train(0, 1, "flash", 2)
  out = run_ranks(_train, 4, "ulysses_ring", 2, timeout=600.0)
  for losses, digest, gn in out:
    assert losses == pytest.approx(ref_losses, rel=2e-4, abs=1e-5)
    assert gn == pytest.approx(ref_gn, rel=2e-3)
    for k, v in ref_digest.items():
      assert digest[k] == pytest.approx(v, rel=1e-4, abs=1e-4), k


def _cfg_pipeline(rank, world, data_axis):
  """Wan sampling with classifier-free guidance: as a batch of two on every rank (data axis 1) or split over the two
  ranks of the data axis, cond on one and uncond on the other, combined after an all-gather per step."""
  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.parallel.mesh import create_device_mesh
  from maxdiffusion_b200.pipelines.wan.wan_pipeline import WanPipeline2_1

  config = pyconfig.initialize(
      ["t", CFG, "run_name=t", "random_init=True", "height=32", "width=32", "num_frames=5", "wan_preset=tiny",
       f"wan_config_overrides={TINY}", "num_inference_steps=3", "log_config=false", "guidance_scale=4.0",
       f"ici_data_parallelism={data_axis}", "ici_fsdp_parallelism=1", f"ici_context_parallelism={world // data_axis}",
       "attention=flash" if world // data_axis == 1 else "attention=tokamax_ring"], unittest=True)
  torch.manual_seed(0)
  pipe = WanPipeline2_1.from_config(config, load_vae=False, mesh=create_device_mesh(config), device="cpu")
  g = torch.Generator().manual_seed(3)
  pe, ne = torch.randn(1, 8, 48, generator=g), torch.randn(1, 8, 48, generator=g)
  lat = pipe(prompt_embeds=pe, negative_prompt_embeds=ne, output_type="latent", generator=torch.Generator().manual_seed(5))
  return lat


def test_cfg_as_data_parallelism_matches_the_batched_form():
  want = _cfg_pipeline(0, 1, 1)
  got = run_ranks(_cfg_pipeline, 2, 2)
  for lat in got:
    assert torch.allclose(lat, want, atol=2e-5, rtol=1e-4)


def _train_tp(rank, world):
  """tensor = 2 (heads and FFN units split), through the trainer: losses and the gradient norm must be those of the
  single-process run (sharded parameters: the norm is the root of the summed squares of the shards)."""
  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.parallel.mesh import create_device_mesh
  from maxdiffusion_b200.trainers.wan_trainer import WanTrainer

  config = pyconfig.initialize(
      ["t", CFG, "run_name=t", "height=64", "width=48", "num_frames=9", "dataset_type=synthetic", "wan_preset=tiny",
       f"wan_config_overrides={TINY}", "remat_policy=FULL", "warmup_steps_fraction=0.0", "log_config=false",
       "write_metrics=false", "learning_rate=1e-3", "attention=flash", f"per_device_batch_size={1.0 / world}",
       "synthetic_override_text_dim=48", "max_sequence_length=16", "ici_data_parallelism=1", "ici_fsdp_parallelism=1",
       "ici_context_parallelism=1", f"ici_tensor_parallelism={world}"], unittest=True)
  torch.manual_seed(0)
  tr = WanTrainer(config, mesh=create_device_mesh(config), device="cpu")
  data = tr.load_dataset()
  return [float(tr.train_step(next(data))["learning/loss"]) for _ in range(2)]


def test_tensor_parallel_training_matches_single_process():
  ref = _train_tp(0, 1)
  for losses in run_ranks(_train_tp, 2):
    assert losses == pytest.approx(ref, rel=2e-4, abs=1e-5)


def _tp_checkpoint(rank, world, tmp, phase):
  """phase "save": two steps on `world` tensor ranks, checkpoint, two more steps (the uninterrupted run).
  phase "resume": a trainer on `world` tensor ranks whose weights were moved away restores and takes the same two steps."""
  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.checkpointing.wan_checkpointer import WanCheckpointer
  from maxdiffusion_b200.parallel.mesh import create_device_mesh
  from maxdiffusion_b200.trainers.wan_trainer import WanTrainer

  config = pyconfig.initialize(
      ["t", CFG, "run_name=tpck", f"output_dir={tmp}", "height=64", "width=48", "num_frames=9", "dataset_type=synthetic",
       "wan_preset=tiny", f"wan_config_overrides={TINY}", "remat_policy=FULL", "warmup_steps_fraction=0.0", "log_config=false",
       "write_metrics=false", "learning_rate=1e-3", "attention=flash", f"per_device_batch_size={1.0 / world}",
       "synthetic_override_text_dim=48", "max_sequence_length=16", "ici_data_parallelism=1", "ici_fsdp_parallelism=1",
       "ici_context_parallelism=1", f"ici_tensor_parallelism={world}", "save_optimizer=true",
       "enable_async_checkpointing=false"], unittest=True)
  torch.manual_seed(0)
  tr = WanTrainer(config, mesh=create_device_mesh(config), device="cpu")
  data = tr.load_dataset()
  batches = [next(data) for _ in range(4)]
  ck = WanCheckpointer(config)
  if phase == "save":
    for b in batches[:2]:
      tr.train_step(b)
    ck.save(2, tr)
    ck.manager.wait_until_finished()
  else:
    with torch.no_grad():  # everything must come from the checkpoint
      for flat in list(tr.engine.shards) + [tr.engine.root_flat]:
        flat.add_(0.25)
    assert ck.maybe_restore(tr) == 2
    tr.step = 2
  tr.gen = torch.Generator().manual_seed(1)
  return [float(tr.train_step(b)["learning/loss"]) for b in batches[2:]]


def test_tensor_parallel_checkpoint_resumes_on_the_same_and_on_another_tensor_axis(tmp_path):
  """A tensor-parallel run writes full parameters (gathered over the tensor axis) and every tensor rank's moments;
  restoring on 2 tensor ranks, on 1, and restoring a single-process checkpoint on 2 continues the uninterrupted run."""
  import json

  tmp = str(tmp_path / "tp2")
  ref = run_ranks(_tp_checkpoint, 2, tmp, "save")[0]
  meta = json.load(open(os.path.join(tmp, "tpck", "checkpoints", "2", "wan_state", "_METADATA")))["tree_metadata"]
  assert meta["blocks/attn1/query/kernel"]["shape"] == [2, 128, 128] and meta["blocks/ffn/proj_out/kernel"]["shape"] == [2, 96, 128]
  assert run_ranks(_tp_checkpoint, 2, tmp, "resume")[0] == pytest.approx(ref, rel=1e-5, abs=1e-7)
  assert _tp_checkpoint(0, 1, tmp, "resume") == pytest.approx(ref, rel=2e-4, abs=1e-5)
  tmp1 = str(tmp_path / "tp1")
  ref1 = _tp_checkpoint(0, 1, tmp1, "save")
  assert run_ranks(_tp_checkpoint, 2, tmp1, "resume")[0] == pytest.approx(ref1, rel=2e-4, abs=1e-5)


def _spatial_decode(rank, world, chunk):
  import torch.distributed as dist

  from maxdiffusion_b200.models.wan.autoencoder_kl_wan import AutoencoderKLWan, WanVAEConfig
  from maxdiffusion_b200.models.wan.vae_channels_last import ChannelsLastDecoder
  from maxdiffusion_b200.parallel.spatial import HaloExchange

  torch.manual_seed(0)
  vae = AutoencoderKLWan(WanVAEConfig(base_dim=8)).eval()
  for p in vae.parameters():
    torch.nn.init.normal_(p, std=0.2)
  z = torch.randn(1, 16, 3, 4, 6)
  cl = ChannelsLastDecoder(vae)
  halo = HaloExchange(dist.group.WORLD, peer_memory=False)
  with torch.no_grad():
    whole = cl.decode(z, chunk=chunk)
    split = cl.decode(z, chunk=chunk, spatial=halo)
  return float((whole - split).abs().max()), float(whole.abs().max()), tuple(split.shape), halo.exchanges


@pytest.mark.parametrize("world,chunk", [(2, 1), (3, 2)])
def test_vae_decode_split_over_the_width_matches_the_whole_frame(world, chunk):
  """Every rank decodes a vertical strip with its neighbours' edge columns in the halos (chunked decode with 2-frame
  histories, time and space up-sampling, the gathered mid-block attention): all ranks return the unsharded video."""
  for err, scale, shape, exchanges in run_ranks(_spatial_decode, world, chunk):
    assert shape == (1, 3, 9, 32, 48)
    assert err < 1e-4 * (1 + scale)
    assert exchanges > 20  # the strips really exchanged their edges


def test_ulysses_head_chunk_ranges():
  from maxdiffusion_b200.parallel.context import ulysses_head_chunks

  assert ulysses_head_chunks(40, 8, 1) == [(0, 40)]
  assert ulysses_head_chunks(40, 8, 2) == [(0, 16), (16, 40)]          # 5 groups of 8 heads: 2 + 3
  assert ulysses_head_chunks(40, 4, 5) == [(0, 8), (8, 16), (16, 24), (24, 32), (32, 40)]
  assert ulysses_head_chunks(8, 4, 16) == [(0, 4), (4, 8)]             # never more chunks than groups
  with pytest.raises(ValueError):
    ulysses_head_chunks(10, 4, 2)


def test_chunked_ulysses_training_matches_single_process():
  """`ulysses_attention_chunks=2`: every head-group chunk is exchanged and attended on its own (forward and backward);
  the step must equal the unchunked single-process one."""
  ref_losses, ref_digest, ref_gn = _train(0, 1, "flash", 2)
  for losses, digest, gn in run_ranks(_train, 2, "ulysses", 2, 0, ("ulysses_attention_chunks=2",)):
    assert losses == pytest.approx(ref_losses, rel=2e-4, abs=1e-5)
    assert gn == pytest.approx(ref_gn, rel=2e-3)
    for k, v in ref_digest.items():
      assert digest[k] == pytest.approx(v, rel=1e-4, abs=1e-4), k


def _cfg_fold(rank, world):
  from maxdiffusion_b200.ops import functional as OF
  from maxdiffusion_b200.parallel.context import ContextParallel
  from maxdiffusion_b200.parallel.mesh import create_device_mesh

  mesh = create_device_mesh(shape={"data": 1, "fsdp": 1, "context": world, "tensor": 1})
  ctx = ContextParallel(mesh, "ulysses")
  g = torch.Generator().manual_seed(0)
  B, S, H, D = 2, 8 * world, 3, 16  # 3 heads do not split over 2 ranks; 2 x 3 do
  q, k, v = (torch.randn((B, S, H, D), generator=g) for _ in range(3))
  want = OF.attention(q, k, v)
  local = lambda t: ctx.shard_sequence(t, dim=1)
  got = ctx.self_attention(local(q), local(k), local(v))
  return float((got - local(want)).abs().max())


def test_cfg_batch_folds_into_heads_when_the_heads_alone_do_not_split():
  for err in run_ranks(_cfg_fold, 2):
    assert err < 1e-5


def _single_replica_restore(rank, world, folder):
  """Rank 0 reads the state file; rank 1 is forbidden to open it and still ends up with the same tensors."""
  import safetensors.torch as st

  from maxdiffusion_b200.checkpointing.checkpointing_utils import WAN_CHECKPOINT, create_checkpoint_manager

  mgr = create_checkpoint_manager(folder, WAN_CHECKPOINT, enable_async=False, rank=rank, single_replica=True)
  if rank != 0:
    def forbidden(*a, **k):
      raise AssertionError("this rank must not read the checkpoint file")
    st.load_file = forbidden
  state = mgr.restore_state(mgr.latest_step(), "wan_state")
  return {k: (v.dtype, v.tolist()) for k, v in state.items()}


def test_single_replica_restore_reads_on_one_rank_and_broadcasts(tmp_path):
  from maxdiffusion_b200.checkpointing.checkpointing_utils import WAN_CHECKPOINT, create_checkpoint_manager

  mgr = create_checkpoint_manager(str(tmp_path), WAN_CHECKPOINT, enable_async=False)
  want = {"a/kernel": torch.arange(6, dtype=torch.float32).reshape(2, 3), "b/scale": torch.tensor([1.5, -2.0]).to(torch.bfloat16),
          "c/steps": torch.tensor([7], dtype=torch.int64)}
  mgr.save(4, {"wan_config": {"dim": 8}, "wan_state": want})
  mgr.wait_until_finished()
  got = run_ranks(_single_replica_restore, 2, str(tmp_path))
  expect = {k: (v.dtype, v.tolist()) for k, v in want.items()}
  assert got[0] == expect and got[1] == expect
  # one process, or the switch off: a plain read
  assert {k: v.tolist() for k, v in mgr.restore_state(4, "wan_state").items()} == {k: v.tolist() for k, v in want.items()}
