"""Parity of the Wan transformer against an independent plain-PyTorch restatement of the published architecture, with
the weights travelling through the PRODUCTION key map (`loaders.wan_loader.diffusers_to_ours`).

The restatement below is written against the diffusers checkpoint format only (module names `attn1.to_q`,
`ffn.net.0.proj`, `norm2`, `scale_shift_table`, ...): unfused q / k / v, a Conv3d patch embedding, complex-number
rotary embedding, `nn.LayerNorm` in fp32. Nothing in it is shared with `models/wan/transformer_wan.py`. The reference
repository checks its own model the same way (src/maxdiffusion/tests/wan/wan_common_module_parity_test.py:330-420,
tolerance 2e-5 in fp32, "weight mapping covers all params" :332).
"""
import math

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from maxdiffusion_b200.loaders import wan_loader
from maxdiffusion_b200.loaders.lora_loader import lora_delta, merge_lora_into_wan, parse_lora_dict
from maxdiffusion_b200.models.wan.transformer_wan import WanConfig, WanModel

HEADS, HEAD_DIM, FFN, LAYERS, TEXT_DIM, FREQ = 3, 32, 160, 2, 48, 64
DIM = HEADS * HEAD_DIM


# ---------------------------------------------------------------------------------------------------------------
# independent restatement (diffusers naming)
# ---------------------------------------------------------------------------------------------------------------
class _RMSAcrossHeads(nn.Module):

  def __init__(self, dim, eps):
    super().__init__()
    self.weight = nn.Parameter(torch.ones(dim))
    self.eps = eps

  def forward(self, x):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight


def _rope_freqs(head_dim, f, h, w, theta=10000.0):
  """Complex rotary factors [f*h*w, head_dim/2]: the head's channel pairs are split between time, height and width."""
  h_dim = w_dim = 2 * (head_dim // 6)
  t_dim = head_dim - h_dim - w_dim

  def axis(dim, n):
    inv = 1.0 / theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim)
    return torch.polar(torch.ones(n, dim // 2, dtype=torch.float64), torch.outer(torch.arange(n, dtype=torch.float64), inv))

  ft, fh, fw = axis(t_dim, f), axis(h_dim, h), axis(w_dim, w)
  grid = torch.cat([ft[:, None, None, :].expand(f, h, w, -1), fh[None, :, None, :].expand(f, h, w, -1),
                    fw[None, None, :, :].expand(f, h, w, -1)], dim=-1)
  return grid.reshape(f * h * w, head_dim // 2)


def _apply_rope(x, freqs):  # x [B, S, H, D]
  xc = torch.view_as_complex(x.double().reshape(*x.shape[:-1], -1, 2))
  return torch.view_as_real(xc * freqs[None, :, None, :]).flatten(-2).to(x.dtype)


class _Attn(nn.Module):

  def __init__(self, dim, heads, eps):
    super().__init__()
    self.heads = heads
    self.to_q, self.to_k, self.to_v = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
    self.norm_q, self.norm_k = _RMSAcrossHeads(dim, eps), _RMSAcrossHeads(dim, eps)
    self.to_out = nn.ModuleList([nn.Linear(dim, dim)])

  def forward(self, x, context=None, freqs=None):
    ctx = x if context is None else context
    q, k, v = self.norm_q(self.to_q(x)), self.norm_k(self.to_k(ctx)), self.to_v(ctx)
    q, k, v = (t.unflatten(-1, (self.heads, -1)) for t in (q, k, v))
    if freqs is not None:
      q, k = _apply_rope(q, freqs), _apply_rope(k, freqs)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
    return self.to_out[0](o.flatten(2))


class _GELUProj(nn.Module):

  def __init__(self, a, b):
    super().__init__()
    self.proj = nn.Linear(a, b)

  def forward(self, x):
    return F.gelu(self.proj(x), approximate="tanh")


class _Block(nn.Module):

  def __init__(self, dim, heads, ffn, eps):
    super().__init__()
    self.norm1 = nn.LayerNorm(dim, eps, elementwise_affine=False)
    self.attn1 = _Attn(dim, heads, eps)
    self.norm2 = nn.LayerNorm(dim, eps, elementwise_affine=True)
    self.attn2 = _Attn(dim, heads, eps)
    self.norm3 = nn.LayerNorm(dim, eps, elementwise_affine=False)
    self.ffn = nn.Module()
    self.ffn.net = nn.ModuleList([_GELUProj(dim, ffn), nn.Identity(), nn.Linear(ffn, dim)])
    self.scale_shift_table = nn.Parameter(torch.randn(1, 6, dim) / dim ** 0.5)

  def forward(self, x, context, temb6, freqs):
    shift_msa, scale_msa, gate_msa, c_shift, c_scale, c_gate = (self.scale_shift_table + temb6).chunk(6, dim=1)
    x = x + self.attn1(self.norm1(x) * (1 + scale_msa) + shift_msa, freqs=freqs) * gate_msa
    x = x + self.attn2(self.norm2(x), context=context)
    h = self.norm3(x) * (1 + c_scale) + c_shift
    return x + self.ffn.net[2](self.ffn.net[0](h)) * c_gate


class _TimeText(nn.Module):

  def __init__(self, dim, freq, text_dim):
    super().__init__()
    self.freq = freq
    self.time_embedder = nn.Module()
    self.time_embedder.linear_1, self.time_embedder.linear_2 = nn.Linear(freq, dim), nn.Linear(dim, dim)
    self.time_proj = nn.Linear(dim, 6 * dim)
    self.text_embedder = nn.Module()
    self.text_embedder.linear_1, self.text_embedder.linear_2 = nn.Linear(text_dim, dim), nn.Linear(dim, dim)

  def forward(self, t, text):
    half = self.freq // 2
    ang = t.float()[:, None] * torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32) / half)[None]
    emb = torch.cat([ang.cos(), ang.sin()], dim=-1)  # flip_sin_to_cos
    temb = self.time_embedder.linear_2(F.silu(self.time_embedder.linear_1(emb)))
    return temb, self.time_proj(F.silu(temb)), self.text_embedder.linear_2(F.gelu(self.text_embedder.linear_1(text), approximate="tanh"))


class _RefWan(nn.Module):

  def __init__(self):
    super().__init__()
    self.patch_embedding = nn.Conv3d(16, DIM, (1, 2, 2), stride=(1, 2, 2))
    self.condition_embedder = _TimeText(DIM, FREQ, TEXT_DIM)
    self.blocks = nn.ModuleList([_Block(DIM, HEADS, FFN, 1e-6) for _ in range(LAYERS)])
    self.norm_out = nn.LayerNorm(DIM, 1e-6, elementwise_affine=False)
    self.proj_out = nn.Linear(DIM, 16 * 4)
    self.scale_shift_table = nn.Parameter(torch.randn(1, 2, DIM) / DIM ** 0.5)

  def forward(self, latents, t, text):
    B, C, Fr, H, W = latents.shape
    x = self.patch_embedding(latents)
    f, h, w = x.shape[2:]
    x = x.flatten(2).transpose(1, 2)
    freqs = _rope_freqs(HEAD_DIM, f, h, w)
    temb, tproj, ctx = self.condition_embedder(t, text)
    temb6 = tproj.unflatten(1, (6, -1))
    for blk in self.blocks:
      x = blk(x, ctx, temb6, freqs)
    shift, scale = (self.scale_shift_table + temb.unsqueeze(1)).chunk(2, dim=1)
    x = self.proj_out(self.norm_out(x) * (1 + scale) + shift)
    x = x.reshape(B, f, h, w, 1, 2, 2, 16).permute(0, 7, 1, 4, 2, 5, 3, 6)
    return x.reshape(B, 16, f, h * 2, w * 2)


def _models():
  torch.manual_seed(0)
  ref = _RefWan().eval()
  for n, p in ref.named_parameters():
    if n.endswith("norm_q.weight") or n.endswith("norm_k.weight") or "norm2" in n:
      torch.nn.init.normal_(p, mean=1.0 if n.endswith("weight") else 0.0, std=0.2)
  cfg = WanConfig(num_attention_heads=HEADS, attention_head_dim=HEAD_DIM, ffn_dim=FFN, num_layers=LAYERS,
                  text_dim=TEXT_DIM, freq_dim=FREQ)
  ours = WanModel(cfg).eval()
  return ref, ours, cfg


def test_key_map_covers_every_parameter_exactly_once_and_round_trips():
  ref, ours, cfg = _models()
  sd = {k: v.detach() for k, v in ref.state_dict().items()}
  mapped = wan_loader.diffusers_to_ours(sd)
  want = ours.state_dict()
  assert set(mapped) == set(want), (sorted(set(mapped) ^ set(want)))
  for k, v in mapped.items():
    assert tuple(v.shape) == tuple(want[k].shape), (k, v.shape, want[k].shape)
  # every source element lands in exactly one destination element
  assert sum(v.numel() for v in mapped.values()) == sum(v.numel() for v in sd.values())
  back = wan_loader.ours_to_diffusers(mapped, cfg.in_channels, tuple(cfg.patch_size))
  assert set(back) == set(sd)
  for k in sd:
    assert torch.equal(back[k], sd[k]), k
  # and the reference's flax tree (the checkpoint layout) round-trips through the same tables
  tree = wan_loader.diffusers_to_flax_tree(sd)
  again = wan_loader.flax_tree_to_diffusers(tree)
  assert set(again) == set(sd)
  for k in sd:
    assert torch.allclose(torch.as_tensor(again[k]).float(), sd[k].float()), k


def test_forward_matches_the_independent_restatement():
  ref, ours, cfg = _models()
  ours.load_state_dict(wan_loader.diffusers_to_ours({k: v.detach() for k, v in ref.state_dict().items()}), strict=True)
  torch.manual_seed(1)
  latents = torch.randn(2, 16, 3, 8, 12)
  text = torch.randn(2, 10, TEXT_DIM)
  t = torch.tensor([37.0, 911.0])
  with torch.no_grad():
    want = ref(latents, t, text)
    got = ours(latents, t, text)
  assert got.shape == want.shape
  assert (got - want).abs().max() < 2e-5 * (1 + want.abs().max())


def test_training_gradients_match_the_independent_restatement():
  ref, ours, cfg = _models()
  ours.load_state_dict(wan_loader.diffusers_to_ours({k: v.detach() for k, v in ref.state_dict().items()}), strict=True)
  ours.train()
  ref.train()
  torch.manual_seed(2)
  latents = torch.randn(1, 16, 2, 8, 8)
  text = torch.randn(1, 6, TEXT_DIM)
  t = torch.tensor([500.0])
  ref(latents, t, text).square().mean().backward()
  ours(latents, t, text).square().mean().backward()
  g_ref = wan_loader.diffusers_to_ours({k: p.grad for k, p in ref.named_parameters()})
  for k, p in ours.named_parameters():
    assert torch.allclose(p.grad, g_ref[k], atol=1e-6, rtol=2e-4), k


def test_lora_merge_equals_w_plus_scaled_up_down():
  """W' = W + scale * (alpha / rank) * up @ down on the right rows of the fused matrices, for PEFT and Kohya key
  styles, plus `.diff` / `.diff_b` deltas (reference: src/maxdiffusion/models/lora_nnx.py:150-245)."""
  _, ours, cfg = _models()
  before = {k: v.clone() for k, v in ours.state_dict().items()}
  torch.manual_seed(3)
  r = 4
  lora = {
      "transformer.blocks.0.attn1.to_k.lora_A.weight": torch.randn(r, DIM), "transformer.blocks.0.attn1.to_k.lora_B.weight": torch.randn(DIM, r),
      "diffusion_model.blocks.1.attn2.to_v.lora_down.weight": torch.randn(r, DIM), "diffusion_model.blocks.1.attn2.to_v.lora_up.weight": torch.randn(DIM, r),
      "diffusion_model.blocks.1.attn2.to_v.alpha": torch.tensor(2.0),
      "blocks.1.ffn.net.2.lora_A.weight": torch.randn(r, FFN), "blocks.1.ffn.net.2.lora_B.weight": torch.randn(DIM, r),
      "blocks.0.attn1.to_out.0.diff": torch.randn(DIM, DIM), "blocks.0.attn1.to_out.0.diff_b": torch.randn(DIM),
  }
  parsed = parse_lora_dict(lora)
  assert set(parsed) == {"blocks.0.attn1.to_k", "blocks.1.attn2.to_v", "blocks.1.ffn.net.2", "blocks.0.attn1.to_out.0"}
  assert torch.allclose(lora_delta(parsed["blocks.1.attn2.to_v"], 0.5),
                        0.5 * (2.0 / r) * lora["diffusion_model.blocks.1.attn2.to_v.lora_up.weight"] @ lora["diffusion_model.blocks.1.attn2.to_v.lora_down.weight"])
  n = merge_lora_into_wan(ours, lora, scale=0.5)
  assert n == 4  # three low-rank pairs and one module with `.diff` / `.diff_b` only
  after = ours.state_dict()
  k_rows = slice(DIM, 2 * DIM)  # to_k inside to_qkv
  d = 0.5 * lora["transformer.blocks.0.attn1.to_k.lora_B.weight"] @ lora["transformer.blocks.0.attn1.to_k.lora_A.weight"]
  assert torch.allclose(after["blocks.0.attn1.to_qkv.weight"][k_rows], before["blocks.0.attn1.to_qkv.weight"][k_rows] + d, atol=1e-5)
  assert torch.equal(after["blocks.0.attn1.to_qkv.weight"][:DIM], before["blocks.0.attn1.to_qkv.weight"][:DIM])
  v_rows = slice(DIM, 2 * DIM)  # to_v inside to_kv
  d = 0.5 * (2.0 / r) * lora["diffusion_model.blocks.1.attn2.to_v.lora_up.weight"] @ lora["diffusion_model.blocks.1.attn2.to_v.lora_down.weight"]
  assert torch.allclose(after["blocks.1.attn2.to_kv.weight"][v_rows], before["blocks.1.attn2.to_kv.weight"][v_rows] + d, atol=1e-5)
  d = 0.5 * lora["blocks.1.ffn.net.2.lora_B.weight"] @ lora["blocks.1.ffn.net.2.lora_A.weight"]
  assert torch.allclose(after["blocks.1.ffn_out.weight"], before["blocks.1.ffn_out.weight"] + d, atol=1e-5)
  assert torch.allclose(after["blocks.0.attn1.to_out.weight"], before["blocks.0.attn1.to_out.weight"] + 0.5 * lora["blocks.0.attn1.to_out.0.diff"], atol=1e-6)
  assert torch.allclose(after["blocks.0.attn1.to_out.bias"], before["blocks.0.attn1.to_out.bias"] + 0.5 * lora["blocks.0.attn1.to_out.0.diff_b"], atol=1e-6)
  untouched = [k for k in before if k not in ("blocks.0.attn1.to_qkv.weight", "blocks.1.attn2.to_kv.weight", "blocks.1.ffn_out.weight",
                                              "blocks.0.attn1.to_out.weight", "blocks.0.attn1.to_out.bias")]
  assert all(torch.equal(before[k], after[k]) for k in untouched)


def test_lora_in_the_original_wan_naming_reaches_embedders_norms_and_modulation_tables(tmp_path):
  """Distilled-step LoRA files of the original repository carry, beside the projections, deltas for the embedders,
  the head, q/k norm weights (`.diff`), the block norm (`norm3.diff` / `.diff_b`) and the modulation tables
  (`blocks.N.diff_m`, `head.diff_m`); reference: src/maxdiffusion/loaders/lora_conversion_utils.py:613-705. Wan 2.2
  entries name one file per expert (wan_lora_nnx_loader.py:64-111)."""
  import types

  from safetensors.torch import save_file

  from maxdiffusion_b200.loaders.lora_loader import merge_wan_loras

  _, ours, cfg = _models()
  before = {k: v.clone() for k, v in ours.state_dict().items()}
  torch.manual_seed(5)
  r, s = 2, 0.5
  pair = lambda name: (torch.randn(r, before[name].shape[1]) * 0.1, torch.randn(before[name].shape[0], r) * 0.1)
  lin = {"text_embedding.0": "condition_embedder.text_in", "text_embedding.2": "condition_embedder.text_out",
         "time_embedding.0": "condition_embedder.time_in", "time_embedding.2": "condition_embedder.time_out",
         "time_projection.1": "condition_embedder.time_proj", "head.head": "proj_out", "patch_embedding": "patch_embedding",
         "blocks.0.self_attn.o": "blocks.0.attn1.to_out", "blocks.1.ffn.0": "blocks.1.ffn_in"}
  lora, want = {}, {}
  for theirs, mine in lin.items():
    down, up = pair(mine + ".weight")
    lora[f"diffusion_model.{theirs}.lora_down.weight"], lora[f"diffusion_model.{theirs}.lora_up.weight"] = down, up
    want[mine + ".weight"] = before[mine + ".weight"] + s * up @ down
  vec = {"blocks.0.self_attn.norm_q": "blocks.0.attn1.norm_q", "blocks.1.cross_attn.norm_k": "blocks.1.attn2.norm_k"}
  for theirs, mine in vec.items():
    lora[f"diffusion_model.{theirs}.diff"] = torch.randn_like(before[mine])
    want[mine] = before[mine] + s * lora[f"diffusion_model.{theirs}.diff"]
  lora["diffusion_model.blocks.1.norm3.diff"], lora["diffusion_model.blocks.1.norm3.diff_b"] = torch.randn(DIM), torch.randn(DIM)
  want["blocks.1.norm2_weight"] = before["blocks.1.norm2_weight"] + s * lora["diffusion_model.blocks.1.norm3.diff"]
  want["blocks.1.norm2_bias"] = before["blocks.1.norm2_bias"] + s * lora["diffusion_model.blocks.1.norm3.diff_b"]
  lora["diffusion_model.blocks.0.diff_m"], lora["diffusion_model.head.diff_m"] = torch.randn(1, 6, DIM), torch.randn(1, 2, DIM)
  want["blocks.0.scale_shift_table"] = before["blocks.0.scale_shift_table"] + s * lora["diffusion_model.blocks.0.diff_m"]
  want["scale_shift_table"] = before["scale_shift_table"] + s * lora["diffusion_model.head.diff_m"]
  lora["diffusion_model.text_embedding.0.diff_b"] = torch.randn(DIM)
  want["condition_embedder.text_in.bias"] = before["condition_embedder.text_in.bias"] + s * lora["diffusion_model.text_embedding.0.diff_b"]
  assert merge_lora_into_wan(ours, lora, scale=s) == len(lin) + len(vec) + 3
  after = ours.state_dict()
  for k in before:
    assert torch.allclose(after[k], want.get(k, before[k]), atol=1e-6), k

  # Wan 2.2: one file per expert; an entry with `weight_name` only goes into both
  hi, lo = {k: v.clone() for k, v in lora.items() if "text_embedding" in k}, {k: v.clone() for k, v in lora.items() if "head" in k}
  save_file(hi, str(tmp_path / "high.safetensors"))
  save_file(lo, str(tmp_path / "low.safetensors"))
  _, a, _ = _models()
  _, b, _ = _models()
  pipe = types.SimpleNamespace(transformer=a, transformer_2=b)
  config = types.SimpleNamespace(lora_config={"lora_model_name_or_path": [str(tmp_path), str(tmp_path)], "scale": [s, s],
                                              "high_noise_weight_name": ["high.safetensors", None],
                                              "low_noise_weight_name": ["low.safetensors", None],
                                              "weight_name": [None, "low.safetensors"]})
  merge_wan_loras(pipe, config)
  sa, sb = a.state_dict(), b.state_dict()
  assert torch.allclose(sa["condition_embedder.text_in.weight"], want["condition_embedder.text_in.weight"], atol=1e-6)
  assert torch.equal(sb["condition_embedder.text_in.weight"], before["condition_embedder.text_in.weight"])
  # the head deltas: once into the high-noise expert (second entry), twice into the low-noise one (first + second entry)
  d = want["proj_out.weight"] - before["proj_out.weight"]
  assert torch.allclose(sa["proj_out.weight"], before["proj_out.weight"] + d, atol=1e-6)
  assert torch.allclose(sb["proj_out.weight"], before["proj_out.weight"] + 2 * d, atol=1e-6)
