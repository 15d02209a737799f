"""Flux transformer against an independent plain-PyTorch restatement of the published architecture, through the
production key map: a random diffusers-style state dict (separate to_q / to_k / to_v, `ff.net.0.proj`, `norm1.linear`,
...) is (a) run by the restatement below, written from the architecture description with diffusers' parameter names, and
(b) converted by `loaders.flux_loader.diffusers_to_ours` and run by `FluxTransformer2DModel` (fused qkv, fused
qkv + mlp in the single blocks, repository kernels' CPU paths). Outputs must agree: this pins the key map, the order of
the modulation chunks, the per-head RMS norms, the interleaved RoPE and the joint (text | image) attention.
reference: src/maxdiffusion/models/flux/transformers/transformer_flux_flax.py:41-560, models/embeddings_flax.py:437."""
import math

import torch
import torch.nn.functional as F

from maxdiffusion_b200.loaders import flux_loader
from maxdiffusion_b200.models.flux.transformer_flux import FLUX_PRESETS, FluxConfig, FluxTransformer2DModel, prepare_latent_image_ids
from tests.test_loader_keymaps_cpu import _diffusers_keys


def _lin(sd, name, x):
  return F.linear(x, sd[name + ".weight"], sd.get(name + ".bias"))


def _sinusoid(t, dim=256):
  half = dim // 2
  freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32) / half)
  ang = t.float()[:, None] * freqs[None]
  return torch.cat([ang.cos(), ang.sin()], dim=-1)  # flip_sin_to_cos


def _mlp_embed(sd, name, x):
  return _lin(sd, name + ".linear_2", F.silu(_lin(sd, name + ".linear_1", x)))


def _ln(x):
  return F.layer_norm(x, (x.shape[-1],), eps=1e-6)


def _rms(x, w):
  return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w


def _rope(ids, axes, theta=10000.0):
  cos, sin = [], []
  for i, d in enumerate(axes):
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    ang = ids[:, i].double()[:, None] * inv[None]
    cos.append(ang.cos().repeat_interleave(2, dim=-1))
    sin.append(ang.sin().repeat_interleave(2, dim=-1))
  return torch.cat(cos, -1).float(), torch.cat(sin, -1).float()


def _apply_rope(x, cos, sin):  # x [B, H, S, D]; pairs (2i, 2i+1) rotate together
  xr = torch.stack([-x[..., 1::2], x[..., 0::2]], dim=-1).flatten(-2)
  return x * cos + xr * sin


def _attention(q, k, v, heads, cos, sin, nq, nk):
  B, S, C = q.shape
  sh = lambda t: t.view(B, S, heads, C // heads).transpose(1, 2)
  q, k, v = sh(q), sh(k), sh(v)
  q, k = _rms(q, nq), _rms(k, nk)
  return q, k, v


def restatement(sd, cfg, x, txt, pooled, t, img_ids, txt_ids, guidance):
  H = cfg.num_attention_heads
  img = _lin(sd, "x_embedder", x)
  ctx = _lin(sd, "context_embedder", txt)
  temb = _mlp_embed(sd, "time_text_embed.timestep_embedder", _sinusoid(t * 1000.0))
  if cfg.guidance_embeds:
    temb = temb + _mlp_embed(sd, "time_text_embed.guidance_embedder", _sinusoid(guidance * 1000.0))
  temb = temb + _mlp_embed(sd, "time_text_embed.text_embedder", pooled)
  cos, sin = _rope(torch.cat([txt_ids, img_ids]), cfg.axes_dims_rope, cfg.theta)
  St = ctx.shape[1]
  for i in range(cfg.num_layers):
    p = f"transformer_blocks.{i}."
    m = _lin(sd, p + "norm1.linear", F.silu(temb)).chunk(6, dim=-1)      # shift, scale, gate (attention); shift, scale, gate (mlp)
    mc = _lin(sd, p + "norm1_context.linear", F.silu(temb)).chunk(6, dim=-1)
    xi = _ln(img) * (1 + m[1][:, None]) + m[0][:, None]
    xc = _ln(ctx) * (1 + mc[1][:, None]) + mc[0][:, None]
    qi, ki, vi = _attention(_lin(sd, p + "attn.to_q", xi), _lin(sd, p + "attn.to_k", xi), _lin(sd, p + "attn.to_v", xi), H, cos, sin,
                            sd[p + "attn.norm_q.weight"], sd[p + "attn.norm_k.weight"])
    qc, kc, vc = _attention(_lin(sd, p + "attn.add_q_proj", xc), _lin(sd, p + "attn.add_k_proj", xc), _lin(sd, p + "attn.add_v_proj", xc), H,
                            cos, sin, sd[p + "attn.norm_added_q.weight"], sd[p + "attn.norm_added_k.weight"])
    q, k, v = torch.cat([qc, qi], dim=2), torch.cat([kc, ki], dim=2), torch.cat([vc, vi], dim=2)
    o = F.scaled_dot_product_attention(_apply_rope(q, cos, sin), _apply_rope(k, cos, sin), v)
    o = o.transpose(1, 2).reshape(img.shape[0], -1, img.shape[-1])
    img = img + m[2][:, None] * _lin(sd, p + "attn.to_out.0", o[:, St:])
    ctx = ctx + mc[2][:, None] * _lin(sd, p + "attn.to_add_out", o[:, :St])
    h = _ln(img) * (1 + m[4][:, None]) + m[3][:, None]
    img = img + m[5][:, None] * _lin(sd, p + "ff.net.2", F.gelu(_lin(sd, p + "ff.net.0.proj", h), approximate="tanh"))
    h = _ln(ctx) * (1 + mc[4][:, None]) + mc[3][:, None]
    ctx = ctx + mc[5][:, None] * _lin(sd, p + "ff_context.net.2", F.gelu(_lin(sd, p + "ff_context.net.0.proj", h), approximate="tanh"))
  z = torch.cat([ctx, img], dim=1)
  for i in range(cfg.num_single_layers):
    p = f"single_transformer_blocks.{i}."
    shift, scale, gate = _lin(sd, p + "norm.linear", F.silu(temb)).chunk(3, dim=-1)
    h = _ln(z) * (1 + scale[:, None]) + shift[:, None]
    q, k, v = _attention(_lin(sd, p + "attn.to_q", h), _lin(sd, p + "attn.to_k", h), _lin(sd, p + "attn.to_v", h), H, cos, sin,
                         sd[p + "attn.norm_q.weight"], sd[p + "attn.norm_k.weight"])
    o = F.scaled_dot_product_attention(_apply_rope(q, cos, sin), _apply_rope(k, cos, sin), v).transpose(1, 2).reshape(z.shape)
    mlp = F.gelu(_lin(sd, p + "proj_mlp", h), approximate="tanh")
    z = z + gate[:, None] * _lin(sd, p + "proj_out", torch.cat([o, mlp], dim=-1))
  img = z[:, St:]
  scale, shift = _lin(sd, "norm_out.linear", F.silu(temb)).chunk(2, dim=-1)  # AdaLayerNormContinuous: (scale, shift)
  return _lin(sd, "proj_out", _ln(img) * (1 + scale[:, None]) + shift[:, None])


def test_flux_transformer_equals_the_restatement_through_the_diffusers_key_map():
  torch.manual_seed(0)
  cfg = FluxConfig(**FLUX_PRESETS["tiny"])
  g = torch.Generator().manual_seed(3)
  sd = {}
  for k, shape in _diffusers_keys(cfg).items():
    if k.endswith("norm_q.weight") or k.endswith("norm_k.weight") or "norm_added" in k:
      sd[k] = 1.0 + 0.2 * torch.randn(shape, generator=g)
    elif k.endswith(".bias"):
      sd[k] = 0.1 * torch.randn(shape, generator=g)
    else:
      sd[k] = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[-1]))
  model = FluxTransformer2DModel(cfg).eval()
  model.load_state_dict(flux_loader.diffusers_to_ours(sd), strict=True)
  B, T = 2, 6
  x = torch.randn(B, 16, cfg.in_channels, generator=g)
  txt = torch.randn(B, T, cfg.joint_attention_dim, generator=g)
  pooled = torch.randn(B, cfg.pooled_projection_dim, generator=g)
  t = torch.tensor([0.3, 0.9])
  guidance = torch.tensor([3.5, 1.0])
  img_ids = prepare_latent_image_ids(4, 4, "cpu")
  txt_ids = torch.zeros(T, 3)
  with torch.no_grad():
    want = restatement(sd, cfg, x, txt, pooled, t, img_ids, txt_ids, guidance)
    got = model(x, txt, pooled, t, img_ids, txt_ids, guidance)
  assert got.shape == want.shape == (B, 16, cfg.in_channels)
  assert (got - want).abs().max() < 2e-4 * (1 + want.abs().max()), (got - want).abs().max()
