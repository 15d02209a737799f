"""Remat policy names, embedding / normalisation layers and the attention-kernel facade."""
import pytest
import torch

from maxdiffusion_b200 import kernels
from maxdiffusion_b200.models.embeddings import (CombinedTimestepGuidanceTextProjEmbeddings, FluxPosEmbed,
                                                 get_1d_rotary_pos_embed)
from maxdiffusion_b200.models.gradient_checkpoint import GradientCheckpointType, resolve_remat
from maxdiffusion_b200.models.normalization import AdaLayerNormContinuous, AdaLayerNormZero, AdaLayerNormZeroSingle
from maxdiffusion_b200.ops import functional as OF


def test_remat_policy_names():
  assert resolve_remat("NONE") == "NONE" and resolve_remat("full") == "FULL"
  assert resolve_remat("MATMUL_WITHOUT_BATCH") == resolve_remat("FLUX_OPTIMIZED") == "SAVE_ATTENTION"
  assert resolve_remat("OFFLOAD_MATMUL_WITHOUT_BATCH") == "SAVE_ATTENTION_OFFLOAD"
  assert resolve_remat("CUSTOM", ["self_attn"], []) == "SAVE_ATTENTION"
  assert resolve_remat("CUSTOM", [], ["hidden_states"]) == "FULL_OFFLOAD"
  with pytest.raises(ValueError):
    GradientCheckpointType.from_str("bogus")


def test_checkpoint_block_gradients_match_plain_autograd():
  torch.manual_seed(0)
  lin = torch.nn.Linear(8, 8)
  x = torch.randn(2, 3, 8, requires_grad=True)
  fn = lambda t: torch.tanh(lin(t)) * 2
  y = OF.checkpoint_block(fn, x, offload_input=True)  # on CPU the offload is a no-op; the path must still work
  y.sum().backward()
  gx, gw = x.grad.clone(), lin.weight.grad.clone()
  x.grad, lin.weight.grad = None, None
  fn(x).sum().backward()
  assert torch.allclose(gx, x.grad) and torch.allclose(gw, lin.weight.grad)


def test_keep_block_runs_hooks_in_order_and_matches_plain_autograd():
  torch.manual_seed(0)
  lin = torch.nn.Linear(8, 8)
  x = torch.randn(2, 3, 8, requires_grad=True)
  fn = lambda t: torch.tanh(lin(t)) * 2
  order = []

  def done():
    order.append(("done", lin.weight.grad is not None))  # parameter gradients are complete when the hook fires

  y = OF.keep_block(fn, x * 1.0, pre_backward=lambda: order.append(("pre", lin.weight.grad is None)), on_backward_done=done)
  assert y.requires_grad
  y.sum().backward()
  assert order == [("pre", True), ("done", True)]
  gx, gw = x.grad.clone(), lin.weight.grad.clone()
  x.grad, lin.weight.grad = None, None
  fn(x).sum().backward()
  assert torch.allclose(gx, x.grad) and torch.allclose(gw, lin.weight.grad)


def test_wan_training_step_is_the_same_with_kept_blocks(tmp_path):
  """`remat_keep_blocks` changes memory, not numbers: same loss and same updated weights after two steps."""
  import os

  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.parallel.mesh import create_device_mesh
  from maxdiffusion_b200.trainers.wan_trainer import WanTrainer

  cfg_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs", "base_wan_14b.yml")

  def run(keep):
    config = pyconfig.initialize(["t", cfg_path, "run_name=t", "height=64", "width=64", "num_frames=5", "dataset_type=synthetic",
                                  "wan_preset=tiny", "remat_policy=SAVE_ATTENTION", f"remat_keep_blocks={keep}", "warmup_steps_fraction=0.0",
                                  "log_config=false", "write_metrics=false", "stochastic_rounding=false"], unittest=True)
    tr = WanTrainer(config, mesh=create_device_mesh(config), device="cpu")
    data = tr.load_dataset()
    losses = [float(tr.train_step(next(data))["learning/loss"]) for _ in range(2)]
    return losses, [p.detach().clone() for p in tr.model.parameters()]

  l0, p0 = run(0)
  l1, p1 = run(1)
  l2, p2 = run(99)  # more than there are blocks: every block keeps its activations
  assert l0 == l1 == l2
  for a, b, c in zip(p0, p1, p2):
    assert torch.equal(a, b) and torch.equal(a, c)


def test_adaptive_norms_match_explicit_formula():
  torch.manual_seed(0)
  x, emb = torch.randn(2, 5, 16), torch.randn(2, 16)
  n = AdaLayerNormZero(16)
  out, gate_msa, shift_mlp, scale_mlp, gate_mlp = n(x, emb)
  mod = torch.nn.functional.linear(torch.nn.functional.silu(emb), n.linear.weight, n.linear.bias).chunk(6, dim=-1)
  want = torch.nn.functional.layer_norm(x, (16,), eps=1e-6) * (1 + mod[1][:, None]) + mod[0][:, None]
  assert torch.allclose(out, want, atol=1e-5) and torch.allclose(gate_msa, mod[2], atol=1e-6)
  s = AdaLayerNormZeroSingle(16)
  o2, g2 = s(x, emb)
  assert o2.shape == x.shape and g2.shape == (2, 16)
  c = AdaLayerNormContinuous(16, scale_shift_order="shift_scale")
  m2 = torch.nn.functional.linear(torch.nn.functional.silu(emb), c.linear.weight, c.linear.bias).chunk(2, dim=-1)
  want = torch.nn.functional.layer_norm(x, (16,), eps=1e-6) * (1 + m2[1][:, None]) + m2[0][:, None]
  assert torch.allclose(c(x, emb), want, atol=1e-5)


def test_embeddings_and_kernel_facade():
  e = CombinedTimestepGuidanceTextProjEmbeddings(32, 16)
  assert e(torch.tensor([1.0, 2.0]), torch.tensor([3.0, 3.0]), torch.randn(2, 16)).shape == (2, 32)
  cos, sin = get_1d_rotary_pos_embed(8, 4)
  cplx = get_1d_rotary_pos_embed(8, 4, use_real=False)
  assert torch.allclose(cplx.real, cos) and torch.allclose(cplx.imag, sin)
  ids = torch.tensor([[0, 1, 2], [0, 3, 4]])
  c2, _ = FluxPosEmbed(10000.0, (4, 6, 6))(ids)
  assert c2.shape == (2, 8)
  assert set(kernels.KERNEL_REGISTRY) >= {"dot_product", "flash", "tokamax_ring", "ulysses_ring_custom_bidir", "cudnn_flash_te"}
  q = torch.randn(1, 6, 2, 16)
  ref = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), q.transpose(1, 2), q.transpose(1, 2)).transpose(1, 2)
  assert torch.allclose(kernels.get_attention_kernel("tokamax_flash")(q, q, q), ref, atol=1e-5)


def test_fixed_m_plan_gate_smoothing_and_reference():
  """Fixed-exponent softmax: the bound dominates every score, heads over the gate stay online, smoothed keys give
  the same softmax, and the fp32 restatement with the fixed exponents equals plain attention."""
  import math

  from maxdiffusion_b200.ops import fixed_m as FM

  torch.manual_seed(0)
  B, S, H, D = 2, 50, 4, 16
  q = torch.randn(B, S, H, D)
  k = torch.randn(B, 70, H, D) + 0.5
  v = torch.randn(B, 70, H, D)
  q[:, :, 3] *= 30
  ks = FM.smooth_keys(k)
  assert ks.mean(dim=1).abs().max() < 1e-5
  m_fixed, heads = FM.plan(q, ks)
  assert heads.tolist() == [1, 1, 1, 0] and m_fixed.shape == (B, H, S)
  c = FM.LOG2E / math.sqrt(D)
  s = torch.einsum("bqhd,bkhd->bhqk", q, ks) * c
  assert (s.amax(-1) - m_fixed <= FM.RECENTER).all()  # exp2 never sees more than the re-centring constant
  assert (s.amax(-1) - m_fixed)[:, :3].min() > -126  # the largest term of a row of an eligible head survives
  want = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
  assert torch.allclose(FM.reference_attention(q, ks, v, None, (m_fixed, heads)), want, atol=1e-4)
  # unsmoothed segments use the halved gate
  q2 = q.clone()
  q2[:, :, 2] *= 9
  _, heads_smoothed = FM.plan(q2, ks)
  _, heads_ring = FM.plan(q2, [k[:, :30], k[:, 30:]], smoothed=False)
  assert heads_ring.sum() <= heads_smoothed.sum()
  got = FM.reference_attention(q, [k[:, :30], k[:, 30:]], [v[:, :30], v[:, 30:]], None,
                               FM.plan(q, [k[:, :30], k[:, 30:]], smoothed=False))
  assert torch.allclose(got, want, atol=1e-4)


def test_fixed_m_kernel_names_select_the_fixed_exponent_context():
  from maxdiffusion_b200 import common_types
  from maxdiffusion_b200.kernels import get_attention_kernel
  from maxdiffusion_b200.parallel.context import ContextParallel
  from maxdiffusion_b200.parallel.mesh import create_device_mesh

  assert set(common_types.FIXED_M_KERNELS) == {"ulysses_custom_fixed_m", "ulysses_ring_custom_fixed_m"}
  mesh = create_device_mesh()
  ctx = ContextParallel(mesh, "ulysses", fixed_m=True)
  assert ctx.fixed_m
  q = torch.randn(1, 12, 2, 16)
  # on CPU the exact SDPA path runs; the fixed-exponent option must not change the result
  want = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), q.transpose(1, 2), q.transpose(1, 2)).transpose(1, 2)
  assert torch.allclose(ctx.self_attention(q, q, q), want, atol=1e-5)
  fn = get_attention_kernel("ulysses_custom_fixed_m", mesh)
  assert torch.allclose(fn(q, q, q), want, atol=1e-5)


def test_ring_order_to_owner_mapping_of_the_joint_dkv_launch():
  """Segment i of the gathered K/V belongs to owner order[i]; the joint launch expresses that as (rot + i*step) % n."""
  from maxdiffusion_b200.parallel.context import _stackable

  kg = torch.zeros(8, 1, 4, 2, 8)
  for rank in range(8):
    backwards = [(rank - h) % 8 for h in range(8)]  # peer-memory exchange: own shard, then the ring predecessors
    rot, step = _stackable(kg, kg, backwards)
    assert [(rot + i * step) % 8 for i in range(8)] == backwards and step == 7
  assert _stackable(kg, kg, list(range(8))) == (0, 1)  # all-gather order
  assert _stackable(kg, kg, [0, 2, 1, 3, 4, 5, 6, 7]) is None  # not a rotation: per-segment launches
  assert _stackable(kg.transpose(0, 1), kg.transpose(0, 1), [0]) is None  # not stacked with one batch stride
  assert _stackable(kg[:2], kg[:2], [1, 0]) == (1, 1)
