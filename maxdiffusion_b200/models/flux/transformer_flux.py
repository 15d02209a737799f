"""Flux MMDiT (dev / schnell): 19 double-stream + 38 single-stream blocks, dim 3072, 24 heads of 128.

Reference: `FluxTransformer2DModel` and its blocks
(src/maxdiffusion/models/flux/transformers/transformer_flux_flax.py:68-720): double block = AdaLN-Zero (6-way)
on both streams, fused QKV, per-head RMSNorm on q,k, RoPE, joint attention over [txt ; img], output projection,
gate, LN+modulate, GELU(tanh) MLP, gate (:214-363); single block = AdaLN-Zero-Single (3-way), `lin_qkv` ||
`lin_mlp`, attention, `linear2` on concat[attn, gelu(mlp)], gate + residual (:68-211); bf16 clip at +-65504.

Kernel mapping: both projections of a single block are ONE GEMM (3072 -> 9216 + 12288); per-head RMSNorm + RoPE is
one fused row-wise kernel writing the [B,S,H,D] attention layout; attention is the tcgen05 flash kernel;
gate + residual run in the GEMM epilogue when no gradient is needed. Parameter names follow the diffusers
FluxTransformer2DModel with q/k/v fused (`loaders/flux_loader.py` converts both the diffusers and the BFL
single-file layouts).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as OF
from ..layers import Linear, project_gated_residual, sinusoidal_embedding


@dataclass
class FluxConfig:
  in_channels: int = 64
  num_layers: int = 19
  num_single_layers: int = 38
  attention_head_dim: int = 128
  num_attention_heads: int = 24
  joint_attention_dim: int = 4096
  pooled_projection_dim: int = 768
  guidance_embeds: bool = True
  axes_dims_rope: Sequence[int] = (16, 56, 56)
  mlp_ratio: float = 4.0
  theta: float = 10000.0

  @property
  def dim(self) -> int:
    return self.num_attention_heads * self.attention_head_dim

  @classmethod
  def from_dict(cls, d):
    return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

  def to_dict(self):
    return {k: (list(v) if isinstance(v, tuple) else v) for k, v in self.__dict__.items()}


FLUX_PRESETS = {
    "flux-dev": dict(guidance_embeds=True),
    "flux-schnell": dict(guidance_embeds=False),
    "tiny": dict(num_layers=2, num_single_layers=2, num_attention_heads=2, joint_attention_dim=64, pooled_projection_dim=32),
}


def flux_rope_tables(ids: torch.Tensor, axes_dims: Sequence[int], theta: float = 10000.0):
  """ids: [S, len(axes)] positions -> (cos, sin) fp32 [S, sum(axes)/2] for interleaved-pair rotation
  (reference: `FluxPosEmbed`, src/maxdiffusion/models/embeddings_flax.py:437)."""
  parts = []
  for i, d in enumerate(axes_dims):
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d))
    parts.append(torch.outer(ids[:, i].double(), inv))
  ang = torch.cat(parts, dim=-1)
  return ang.cos().float().contiguous(), ang.sin().float().contiguous()


def prepare_latent_image_ids(height: int, width: int, device=None) -> torch.Tensor:
  """[h*w, 3] ids of the 2x2-packed latent grid (h = H/16, w = W/16 of the image)."""
  ids = torch.zeros(height, width, 3, device=device)
  ids[..., 1] = torch.arange(height, device=device)[:, None]
  ids[..., 2] = torch.arange(width, device=device)[None, :]
  return ids.reshape(height * width, 3)


def pack_latents(latents: torch.Tensor) -> torch.Tensor:
  """[B,C,H,W] -> [B,(H/2)(W/2),4C] (reference: generate_flux.py:161-172)."""
  b, c, h, w = latents.shape
  x = latents.view(b, c, h // 2, 2, w // 2, 2).permute(0, 2, 4, 1, 3, 5)
  return x.reshape(b, (h // 2) * (w // 2), c * 4)


def unpack_latents(tokens: torch.Tensor, height: int, width: int) -> torch.Tensor:
  """Inverse of `pack_latents`; height/width are those of the latent grid."""
  b, _, ch = tokens.shape
  x = tokens.view(b, height // 2, width // 2, ch // 4, 2, 2).permute(0, 3, 1, 4, 2, 5)
  return x.reshape(b, ch // 4, height, width)


class _MLPEmbedder(nn.Module):

  def __init__(self, cin, dim):
    super().__init__()
    self.linear_1, self.linear_2 = Linear(cin, dim), Linear(dim, dim)

  def forward(self, x):
    return self.linear_2(F.silu(self.linear_1(x)))


def _modulation(linear: Linear, temb: torch.Tensor, n: int):
  """SiLU -> Linear -> n chunks with an fp32 result (M = batch). The modulation matrices are a quarter of Flux's
  parameters (18432 x 3072 per stream and double block), so on the GPU they are read once, as the bf16 they are stored
  in, by the GEMM kernel with fp32 accumulation and fp32 output; converting them to fp32 for every call moved five
  times their size and cost 5 % of a denoising step."""
  w = linear.weight
  if temb.is_cuda and w.dtype == torch.bfloat16 and not OF.library_mode() and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0:
    from ...ops import kernels as K

    x = F.silu(temb.float()).to(torch.bfloat16).contiguous()
    if torch.is_grad_enabled() and (w.requires_grad or temb.requires_grad):
      return OF.linear(x, w, linear.bias).float().chunk(n, dim=-1)  # differentiable: bf16 result of the same product
    bias = None if linear.bias is None else linear.bias.to(torch.bfloat16)
    out = K.gemm(x, w, bias=bias, out_dtype=torch.float32)
    return out.chunk(n, dim=-1)
  out = F.linear(F.silu(temb).float(), w.float(), linear.bias.float())
  return out.chunk(n, dim=-1)


def _clip(x):
  return x.clamp(-65504.0, 65504.0) if x.dtype == torch.float16 else x


class FluxDoubleBlock(nn.Module):

  def __init__(self, cfg: FluxConfig):
    super().__init__()
    dim, hidden = cfg.dim, int(cfg.dim * cfg.mlp_ratio)
    self.heads = cfg.num_attention_heads
    self.norm1 = Linear(dim, 6 * dim)          # AdaLN-Zero modulation of the image stream
    self.norm1_context = Linear(dim, 6 * dim)  # ... of the text stream
    self.to_qkv, self.add_qkv_proj = Linear(dim, 3 * dim), Linear(dim, 3 * dim)
    self.norm_q, self.norm_k = nn.Parameter(torch.ones(128)), nn.Parameter(torch.ones(128))
    self.norm_added_q, self.norm_added_k = nn.Parameter(torch.ones(128)), nn.Parameter(torch.ones(128))
    self.to_out, self.to_add_out = Linear(dim, dim), Linear(dim, dim)
    self.ff_in, self.ff_out = Linear(dim, hidden), Linear(hidden, dim)
    self.ff_context_in, self.ff_context_out = Linear(dim, hidden), Linear(hidden, dim)

  def forward(self, img, txt, temb, rope_img, rope_txt, pctx=None):
    from ..wan.transformer_wan import split_fused

    B, Si, C = img.shape
    St = txt.shape[1]
    H = self.heads
    sh_i, sc_i, g_i, sh2_i, sc2_i, g2_i = _modulation(self.norm1, temb, 6)
    sh_t, sc_t, g_t, sh2_t, sc2_t, g2_t = _modulation(self.norm1_context, temb, 6)
    qi, ki, vi = split_fused(self.to_qkv(OF.layer_norm_mod(img, scale=sc_i, shift=sh_i)), 3)
    qt, kt, vt = split_fused(self.add_qkv_proj(OF.layer_norm_mod(txt, scale=sc_t, shift=sh_t)), 3)
    qi = OF.rms_norm_rope(qi, self.norm_q, *rope_img, heads=H, per_head=True)
    ki = OF.rms_norm_rope(ki, self.norm_k, *rope_img, heads=H, per_head=True)
    qt = OF.rms_norm_rope(qt, self.norm_added_q, *rope_txt, heads=H, per_head=True)
    kt = OF.rms_norm_rope(kt, self.norm_added_k, *rope_txt, heads=H, per_head=True)
    q = torch.cat([qt, qi], dim=1)
    k = torch.cat([kt, ki], dim=1)
    v = torch.cat([vt.unflatten(-1, (H, C // H)), vi.unflatten(-1, (H, C // H))], dim=1)
    o = OF.attention(q, k, v).reshape(B, St + Si, C)
    ot, oi = o[:, :St], o[:, St:]
    # projections are called as modules so that wrappers (run-time LoRA adapters, quantised layers) take effect; a
    # plain `Linear` still gets the gate and the residual add in its GEMM epilogue
    img = project_gated_residual(self.to_out, oi, img, g_i)
    txt = project_gated_residual(self.to_add_out, ot, txt, g_t)
    h = self.ff_in(OF.layer_norm_mod(img, scale=sc2_i, shift=sh2_i), "gelu_tanh")
    img = project_gated_residual(self.ff_out, h, img, g2_i)
    h = self.ff_context_in(OF.layer_norm_mod(txt, scale=sc2_t, shift=sh2_t), "gelu_tanh")
    txt = project_gated_residual(self.ff_context_out, h, txt, g2_t)
    return _clip(img), _clip(txt)


class FluxSingleBlock(nn.Module):

  def __init__(self, cfg: FluxConfig):
    super().__init__()
    dim, hidden = cfg.dim, int(cfg.dim * cfg.mlp_ratio)
    self.heads, self.dim, self.hidden = cfg.num_attention_heads, dim, hidden
    self.norm = Linear(dim, 3 * dim)
    self.qkv_mlp = Linear(dim, 3 * dim + hidden)   # lin_qkv || lin_mlp as one GEMM
    self.norm_q, self.norm_k = nn.Parameter(torch.ones(128)), nn.Parameter(torch.ones(128))
    self.proj_out = Linear(dim + hidden, dim)

  def forward(self, x, temb, rope, pctx=None):
    B, S, C = x.shape
    H = self.heads
    shift, scale, gate = _modulation(self.norm, temb, 3)
    h = OF.layer_norm_mod(x, scale=scale, shift=shift)
    w = self.qkv_mlp.weight if type(self.qkv_mlp) is Linear else None
    if (w is not None and not torch.is_grad_enabled() and h.is_cuda and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        and not OF.library_mode() and C % 8 == 0 and self.hidden % 8 == 0):
      # Inference: the fused projection as two products over row slices of its matrix, so that the MLP half gets its
      # GELU in the GEMM epilogue and lands directly in the (attention | mlp) buffer the output projection reads --
      # no separate GELU pass and no concatenation copy (together 3 % of a denoising step).
      from ...ops import kernels as K

      b = self.qkv_mlp.bias
      h2 = h.reshape(B * S, C)
      f = K.gemm(h2, w[:3 * C], bias=None if b is None else b[:3 * C].contiguous()).view(B, S, 3 * C)
      cat = torch.empty((B, S, C + self.hidden), device=h.device, dtype=h.dtype)
      K.gemm(h2, w[3 * C:], bias=None if b is None else b[3 * C:].contiguous(), epi="gelu_tanh", out=cat.view(B * S, -1)[:, C:])
      q = OF.rms_norm_rope(f[..., :C], self.norm_q, *rope, heads=H, per_head=True)
      k = OF.rms_norm_rope(f[..., C:2 * C], self.norm_k, *rope, heads=H, per_head=True)
      cat[..., :C] = OF.attention(q, k, f[..., 2 * C:].unflatten(-1, (H, C // H))).reshape(B, S, C)
      return _clip(project_gated_residual(self.proj_out, cat, x, gate))
    f = self.qkv_mlp(h)
    q, k, v, mlp = f[..., :C], f[..., C:2 * C], f[..., 2 * C:3 * C], f[..., 3 * C:]
    q = OF.rms_norm_rope(q, self.norm_q, *rope, heads=H, per_head=True)
    k = OF.rms_norm_rope(k, self.norm_k, *rope, heads=H, per_head=True)
    o = OF.attention(q, k, v.unflatten(-1, (H, C // H))).reshape(B, S, C)
    cat = torch.cat([o, F.gelu(mlp, approximate="tanh")], dim=-1)
    return _clip(project_gated_residual(self.proj_out, cat, x, gate))


class FluxTransformer2DModel(nn.Module):

  def __init__(self, cfg: FluxConfig, remat_policy: str = "NONE"):
    super().__init__()
    self.cfg, self.remat_policy = cfg, remat_policy
    dim = cfg.dim
    self.x_embedder = Linear(cfg.in_channels, dim)
    self.context_embedder = Linear(cfg.joint_attention_dim, dim)
    self.time_embedder = _MLPEmbedder(256, dim)
    self.guidance_embedder = _MLPEmbedder(256, dim) if cfg.guidance_embeds else None
    self.text_embedder = _MLPEmbedder(cfg.pooled_projection_dim, dim)
    self.transformer_blocks = nn.ModuleList([FluxDoubleBlock(cfg) for _ in range(cfg.num_layers)])
    self.single_transformer_blocks = nn.ModuleList([FluxSingleBlock(cfg) for _ in range(cfg.num_single_layers)])
    self.norm_out = Linear(dim, 2 * dim)
    self.proj_out = Linear(dim, cfg.in_channels)
    self.block_hook = None

  @property
  def blocks(self):
    return list(self.transformer_blocks) + list(self.single_transformer_blocks)

  def forward(self, hidden_states, encoder_hidden_states, pooled_projections, timestep, img_ids, txt_ids,
              guidance=None, pctx=None):
    """hidden_states: packed latents [B,S_img,64]; encoder_hidden_states: T5 [B,S_txt,4096]; pooled: CLIP [B,768];
    timestep, guidance: [B] in [0,1] / raw scale (multiplied by 1000 for the sinusoid like the reference)."""
    cfg = self.cfg
    dtype = self.x_embedder.weight.dtype
    img = self.x_embedder(hidden_states.to(dtype))
    txt = self.context_embedder(encoder_hidden_states.to(dtype))
    temb = self.time_embedder(sinusoidal_embedding(timestep * 1000.0, 256).to(dtype))
    if self.guidance_embedder is not None:
      g = guidance if guidance is not None else torch.full_like(timestep, 3.5)
      temb = temb + self.guidance_embedder(sinusoidal_embedding(g * 1000.0, 256).to(dtype))
    temb = temb + self.text_embedder(pooled_projections.to(dtype))
    img_ids = img_ids[0] if img_ids.dim() == 3 else img_ids
    txt_ids = txt_ids[0] if txt_ids.dim() == 3 else txt_ids
    rope_img = flux_rope_tables(img_ids, cfg.axes_dims_rope, cfg.theta)
    rope_txt = flux_rope_tables(txt_ids, cfg.axes_dims_rope, cfg.theta)
    rope_all = (torch.cat([rope_txt[0], rope_img[0]]), torch.cat([rope_txt[1], rope_img[1]]))
    policy = self.remat_policy.upper() if torch.is_grad_enabled() else "NONE"
    idx = 0
    for blk in self.transformer_blocks:
      if self.block_hook is not None:
        self.block_hook(idx, "forward")
      if policy == "NONE":
        img, txt = blk(img, txt, temb, rope_img, rope_txt)
      else:
        done = (lambda i=idx: self.block_hook(i, "backward_done")) if self.block_hook is not None else None
        def run(a, b, t, blk=blk, i=idx):
          if self.block_hook is not None and torch.is_grad_enabled():
            self.block_hook(i, "recompute")
          return blk(a, b, t, rope_img, rope_txt)
        img, txt = OF.checkpoint_block(run, img, txt, temb, save_attention=(not policy.startswith("FULL")), on_backward_done=done,
                                offload_input=policy.endswith("_OFFLOAD"))
      idx += 1
    x = torch.cat([txt, img], dim=1)
    for blk in self.single_transformer_blocks:
      if self.block_hook is not None:
        self.block_hook(idx, "forward")
      if policy == "NONE":
        x = blk(x, temb, rope_all)
      else:
        done = (lambda i=idx: self.block_hook(i, "backward_done")) if self.block_hook is not None else None
        def run1(a, t, blk=blk, i=idx):
          if self.block_hook is not None and torch.is_grad_enabled():
            self.block_hook(i, "recompute")
          return blk(a, t, rope_all)
        x = OF.checkpoint_block(run1, x, temb, save_attention=(not policy.startswith("FULL")), on_backward_done=done,
                                offload_input=policy.endswith("_OFFLOAD"))
      idx += 1
    img = x[:, txt.shape[1]:]
    scale, shift = _modulation(self.norm_out, temb, 2)  # AdaLayerNormContinuous emits (scale, shift)
    img = OF.layer_norm_mod(img.contiguous(), scale=scale, shift=shift)
    return self.proj_out(img)
