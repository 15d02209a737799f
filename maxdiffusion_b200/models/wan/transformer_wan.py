"""Wan 2.1 / 2.2 diffusion transformer (T2V, I2V) on the sm_100a op set.

Architecture parity with the reference's `WanModel`
(src/maxdiffusion/models/wan/transformers/transformer_wan.py:539-956): Conv3d (1,2,2) patch embedding,
time / text (/ image) condition embedder (:98-217), N blocks of [AdaLN-modulated fp32 LayerNorm ->
self-attention with RMSNorm-across-heads on q,k and 3-D RoPE -> gated residual -> affine LayerNorm ->
cross-attention -> residual -> modulated LayerNorm -> GELU(tanh) FFN -> gated residual] (:333-536),
modulated output norm, projection and un-patchify; MagCache hooks (`skip_blocks`, `cached_residual`,
`return_residual`, :918-927) and a cross-attention K/V cache (:704-757).

What is different by design: q/k/v projections are one fused GEMM, the gate+residual runs in the output
projection's epilogue when no gradient is needed, the sequence dimension is explicitly sharded across the
context-parallel ranks (`pctx`) and each block is an explicit rematerialisation unit whose parameters live in
one flat buffer (see `parallel.fsdp`).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.nn as nn

from ...ops import functional as OF
from ..layers import Linear, project_gated_residual, sinusoidal_embedding


@dataclass
class WanConfig:
  patch_size: Sequence[int] = (1, 2, 2)
  num_attention_heads: int = 40
  attention_head_dim: int = 128
  in_channels: int = 16
  out_channels: int = 16
  text_dim: int = 4096
  freq_dim: int = 256
  ffn_dim: int = 13824
  num_layers: int = 40
  cross_attn_norm: bool = True
  qk_norm: str = "rms_norm_across_heads"
  eps: float = 1e-6
  image_dim: Optional[int] = None
  added_kv_proj_dim: Optional[int] = None
  rope_max_seq_len: int = 1024
  pos_embed_seq_len: Optional[int] = None

  @property
  def dim(self) -> int:
    return self.num_attention_heads * self.attention_head_dim

  @classmethod
  def from_dict(cls, d: dict) -> "WanConfig":
    keys = cls.__dataclass_fields__.keys()
    return cls(**{k: v for k, v in d.items() if k in keys})

  def to_dict(self) -> dict:
    return {k: (list(v) if isinstance(v, tuple) else v) for k, v in self.__dict__.items()}


WAN_PRESETS = {
    "wan2.1-t2v-14b": dict(num_attention_heads=40, ffn_dim=13824, num_layers=40),
    "wan2.1-t2v-1.3b": dict(num_attention_heads=12, ffn_dim=8960, num_layers=30),
    "wan2.1-i2v-14b": dict(num_attention_heads=40, ffn_dim=13824, num_layers=40, in_channels=36, image_dim=1280,
                           added_kv_proj_dim=5120),
    "wan2.2-t2v-a14b": dict(num_attention_heads=40, ffn_dim=13824, num_layers=40),
    "wan2.2-i2v-a14b": dict(num_attention_heads=40, ffn_dim=13824, num_layers=40, in_channels=36),
    "tiny": dict(num_attention_heads=12, ffn_dim=8960, num_layers=2),
}


def wan_rope_tables(head_dim: int, grid: tuple[int, int, int], theta: float = 10000.0, max_seq_len: int = 1024,
                    device=None):
  """cos/sin tables [F*H*W, head_dim/2] (fp32) of the 3-D rotary embedding.

  head_dim is split t/h/w = (d - 4*(d//6)) / 2*(d//6) / 2*(d//6) channels, i.e. 22/21/21 rotation pairs for
  d = 128 (reference: transformer_wan.py:43-95).
  """
  f, h, w = grid
  h_dim = w_dim = 2 * (head_dim // 6)
  t_dim = head_dim - h_dim - w_dim
  parts = []
  for dim, n, axis in ((t_dim, f, 0), (h_dim, h, 1), (w_dim, w, 2)):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64, device=device)[: dim // 2] / dim))
    ang = torch.outer(torch.arange(n, dtype=torch.float64, device=device), inv)  # [n, dim/2]
    shape = [1, 1, 1, dim // 2]
    shape[axis] = n
    parts.append(ang.view(shape).expand(f, h, w, dim // 2))
  ang = torch.cat(parts, dim=-1).reshape(f * h * w, head_dim // 2)
  return ang.cos().float().contiguous(), ang.sin().float().contiguous()


class _SplitFused(torch.autograd.Function):
  """Views of a fused projection output; the backward writes the pieces' gradients with one concatenation."""

  @staticmethod
  def forward(ctx, fused, n):
    c = fused.shape[-1] // n
    return tuple(fused[..., i * c:(i + 1) * c] for i in range(n))

  @staticmethod
  def backward(ctx, *grads):
    return torch.cat([g.reshape(*g.shape[:2], -1) for g in grads], dim=-1), None


def split_fused(fused: torch.Tensor, n: int):
  if fused.requires_grad:
    return _SplitFused.apply(fused, n)
  c = fused.shape[-1] // n
  return tuple(fused[..., i * c:(i + 1) * c] for i in range(n))


def _norm_rope(mod, x, weight, cos=None, sin=None):
  """RMSNorm across all heads (+ RoPE) of a projection; under tensor parallelism (`mod.tp_group`, set by
  `parallel.tensor.apply_tensor_parallel_wan`) the projection holds this rank's heads only and the statistic is summed
  over the tensor group."""
  tp = getattr(mod, "tp_group", None)
  if tp is not None:
    from ...parallel.tensor import tp_rms_norm_rope

    return tp_rms_norm_rope(x, weight, cos, sin, mod.heads, mod.eps, tp, mod.tp_full_dim)
  return OF.rms_norm_rope(x, weight, cos, sin, heads=mod.heads, eps=mod.eps)


class WanSelfAttention(nn.Module):

  def __init__(self, dim: int, heads: int, eps: float):
    super().__init__()
    self.heads, self.eps = heads, eps
    self.to_qkv = Linear(dim, 3 * dim)
    self.norm_q = nn.Parameter(torch.ones(dim))
    self.norm_k = nn.Parameter(torch.ones(dim))
    self.to_out = Linear(dim, dim)

  def forward(self, x, rope, pctx, residual, gate):
    B, S, C = x.shape
    q, k, v = split_fused(self.to_qkv(x), 3)
    cos, sin = rope
    if pctx is not None and getattr(self, "tp_group", None) is None:
      # the strategy object sees the raw projections: under Ulysses the exchanges ride on the norm / RoPE stores and
      # on the attention epilogue instead of running as kernels of their own
      o = pctx.projected_self_attention(q, k, v, self.norm_q, self.norm_k, cos, sin, self.heads, self.eps)
      return project_gated_residual(self.to_out, o, residual, gate)
    q = _norm_rope(self, q, self.norm_q, cos, sin)
    k = _norm_rope(self, k, self.norm_k, cos, sin)
    v = v.unflatten(-1, (self.heads, v.shape[-1] // self.heads))
    o = pctx.self_attention(q, k, v) if pctx is not None else OF.attention(q, k, v)
    return project_gated_residual(self.to_out, o.reshape(B, S, -1), residual, gate)


class WanCrossAttention(nn.Module):

  def __init__(self, dim: int, heads: int, eps: float, added_kv_proj_dim: Optional[int] = None):
    super().__init__()
    self.heads, self.eps = heads, eps
    self.to_q = Linear(dim, dim)
    self.to_kv = Linear(dim, 2 * dim)
    self.norm_q = nn.Parameter(torch.ones(dim))
    self.norm_k = nn.Parameter(torch.ones(dim))
    self.to_out = Linear(dim, dim)
    self.has_image = added_kv_proj_dim is not None
    if self.has_image:
      self.add_kv_proj = Linear(added_kv_proj_dim, 2 * dim)
      self.norm_added_k = nn.Parameter(torch.ones(dim))

  def compute_kv(self, context, context_image=None):
    """K/V of the conditioning tokens; constant over the denoising loop, so pipelines cache it per prompt."""
    if context_image is not None and not self.has_image:
      # no separate image K/V projection (Wan-Animate): the image tokens join the text tokens
      context = torch.cat([context_image, context], dim=1)
    B, T, C = context.shape[0], context.shape[1], self.to_q.weight.shape[0]
    k, v = split_fused(self.to_kv(context), 2)
    k = _norm_rope(self, k, self.norm_k)
    out = {"text": (k, v.unflatten(-1, (self.heads, C // self.heads)))}
    if self.has_image and context_image is not None:
      ki, vi = split_fused(self.add_kv_proj(context_image), 2)
      ki = _norm_rope(self, ki, self.norm_added_k)
      out["image"] = (ki, vi.unflatten(-1, (self.heads, C // self.heads)))
    return out

  def forward(self, x, context, context_image, residual, cached_kv=None):
    B, S, C = x.shape
    q = _norm_rope(self, self.to_q(x), self.norm_q)
    kv = cached_kv if cached_kv is not None else self.compute_kv(context, context_image)
    o = OF.attention(q, *kv["text"])
    if "image" in kv:
      o = o + OF.attention(q, *kv["image"])
    return project_gated_residual(self.to_out, o.reshape(B, S, -1), residual, None)


class WanBlock(nn.Module):

  def __init__(self, cfg: WanConfig):
    super().__init__()
    dim = cfg.dim
    self.eps = cfg.eps
    self.scale_shift_table = nn.Parameter(torch.randn(1, 6, dim) / math.sqrt(dim))
    self.attn1 = WanSelfAttention(dim, cfg.num_attention_heads, cfg.eps)
    self.attn2 = WanCrossAttention(dim, cfg.num_attention_heads, cfg.eps, cfg.added_kv_proj_dim)
    self.norm2_weight = nn.Parameter(torch.ones(dim))
    self.norm2_bias = nn.Parameter(torch.zeros(dim))
    self.ffn_in = Linear(dim, cfg.ffn_dim)
    self.ffn_out = Linear(cfg.ffn_dim, dim)

  def forward(self, x, context, temb6, rope, pctx=None, context_image=None, cached_kv=None):
    """x: [B,S,dim]; context: [B,T,dim] (already embedded); temb6: fp32 [B,6,dim]; rope: (cos, sin) [S,64]."""
    mod = self.scale_shift_table.float() + temb6.float()  # [B,6,dim]
    shift_msa, scale_msa, gate_msa, c_shift, c_scale, c_gate = mod.unbind(1)
    h = OF.layer_norm_mod(x, scale=scale_msa, shift=shift_msa, eps=self.eps)
    x = self.attn1(h, rope, pctx, residual=x, gate=gate_msa)
    h = OF.layer_norm_mod(x, gamma=self.norm2_weight, beta=self.norm2_bias, eps=self.eps)
    x = self.attn2(h, context, context_image, residual=x, cached_kv=cached_kv)
    h = OF.layer_norm_mod(x, scale=c_scale, shift=c_shift, eps=self.eps)
    h = self.ffn_in(h, activation="gelu_tanh")
    return project_gated_residual(self.ffn_out, h, x, c_gate)


class WanImageEmbedding(nn.Module):
  """CLIP image tokens -> model width (I2V); reference: embeddings_flax.py:253."""

  def __init__(self, in_features: int, out_features: int, pos_embed_seq_len: Optional[int] = None):
    super().__init__()
    self.norm1 = nn.LayerNorm(in_features)
    self.ff_in = Linear(in_features, in_features)
    self.ff_out = Linear(in_features, out_features)
    self.norm2 = nn.LayerNorm(out_features)
    self.pos_embed = nn.Parameter(torch.zeros(1, pos_embed_seq_len, in_features)) if pos_embed_seq_len else None

  def forward(self, x):
    if self.pos_embed is not None:
      b, s, c = x.shape
      x = (x.reshape(-1, 2 * s, c) + self.pos_embed.to(x.dtype)).reshape(b, s, c) if self.pos_embed.shape[1] == 2 * s \
          else x + self.pos_embed.to(x.dtype)
    ln = lambda m, t: torch.nn.functional.layer_norm(t.float(), m.normalized_shape, m.weight.float(), m.bias.float(), m.eps)
    h = ln(self.norm1, x).to(x.dtype)
    h = torch.nn.functional.gelu(self.ff_in(h))
    h = self.ff_out(h)
    return ln(self.norm2, h).to(x.dtype)


class WanConditionEmbedder(nn.Module):

  def __init__(self, cfg: WanConfig):
    super().__init__()
    dim = cfg.dim
    self.freq_dim = cfg.freq_dim
    self.time_in = Linear(cfg.freq_dim, dim)
    self.time_out = Linear(dim, dim)
    self.time_proj = Linear(dim, 6 * dim)
    self.text_in = Linear(cfg.text_dim, dim)
    self.text_out = Linear(dim, dim)
    self.image_embedder = WanImageEmbedding(cfg.image_dim, dim, cfg.pos_embed_seq_len) if cfg.image_dim else None

  def time(self, timestep, dtype):
    """timestep: [B] (or [B,S] per token) -> (temb [.., dim], timestep_proj fp32 [.., 6*dim])."""
    emb = sinusoidal_embedding(timestep.reshape(-1), self.freq_dim).to(dtype)
    temb = self.time_out(torch.nn.functional.silu(self.time_in(emb)))
    proj = torch.nn.functional.linear(torch.nn.functional.silu(temb).float(), self.time_proj.weight.float(),
                                      self.time_proj.bias.float())
    return temb.reshape(*timestep.shape, -1), proj.reshape(*timestep.shape, -1)

  def text(self, context):
    return self.text_out(OF.linear(context, self.text_in.weight, self.text_in.bias, activation="gelu_tanh"))


class WanModel(nn.Module):

  def __init__(self, cfg: WanConfig, remat_policy: str = "NONE"):
    super().__init__()
    self.cfg = cfg
    self.remat_policy = remat_policy
    dim = cfg.dim
    pt, ph, pw = cfg.patch_size
    self.patch_embedding = Linear(cfg.in_channels * pt * ph * pw, dim)
    self.condition_embedder = WanConditionEmbedder(cfg)
    self.blocks = nn.ModuleList([WanBlock(cfg) for _ in range(cfg.num_layers)])
    self.scale_shift_table = nn.Parameter(torch.randn(1, 2, dim) / math.sqrt(dim))
    self.proj_out = Linear(dim, cfg.out_channels * pt * ph * pw)
    self.block_hook = None  # optional callable(block_index, phase) used by the FSDP engine

  # ---- layout helpers -----------------------------------------------------------------------
  def patchify(self, latents, channel_last: bool = False):
    """[B,C,F,H,W] -> tokens [B, F'*H'*W', C*pt*ph*pw].

    Patch vectors are channel-major (the Conv3d weight order) for the model input, and channel-last
    (pt, ph, pw, C — the order `proj_out` emits and `unpatchify` consumes) for training targets.
    """
    B, C, F, H, W = latents.shape
    pt, ph, pw = self.cfg.patch_size
    x = latents.reshape(B, C, F // pt, pt, H // ph, ph, W // pw, pw)
    order = (0, 2, 4, 6, 3, 5, 7, 1) if channel_last else (0, 2, 4, 6, 1, 3, 5, 7)
    x = x.permute(*order).reshape(B, (F // pt) * (H // ph) * (W // pw), C * pt * ph * pw)
    return x, (F // pt, H // ph, W // pw)

  def unpatchify(self, tokens, grid):
    B = tokens.shape[0]
    f, h, w = grid
    pt, ph, pw = self.cfg.patch_size
    x = tokens.reshape(B, f, h, w, pt, ph, pw, -1)
    x = x.permute(0, 7, 1, 4, 2, 5, 3, 6)
    return x.reshape(B, -1, f * pt, h * ph, w * pw)

  def compute_kv_cache(self, encoder_hidden_states, encoder_hidden_states_image=None):
    """Per-layer cross-attention K/V for a prompt (reference: transformer_wan.py:704-757)."""
    dtype = self.patch_embedding.weight.dtype
    context = self.condition_embedder.text(encoder_hidden_states.to(dtype))
    image = None
    if encoder_hidden_states_image is not None and self.condition_embedder.image_embedder is not None:
      image = self.condition_embedder.image_embedder(encoder_hidden_states_image.to(dtype))
    return [blk.attn2.compute_kv(context, image) for blk in self.blocks]

  # ---- forward ------------------------------------------------------------------------------
  def forward(self, hidden_states, timestep, encoder_hidden_states, encoder_hidden_states_image=None, pctx=None,
              skip_blocks: bool = False, cached_residual=None, return_residual: bool = False, kv_cache=None,
              rope=None, return_tokens: bool = False, hints: Optional[dict] = None, block_post=None, token_bias=None):
    """hidden_states: latents [B,C,F,H,W]; timestep: [B]; encoder_hidden_states: [B,T,text_dim]. Returns [B,C,F,H,W].

    With a context-parallel `pctx` every rank passes the full latents and receives the output of its own
    token shard scattered back into a full-size tensor only on request (`pctx.gather_output`).
    """
    cfg = self.cfg
    dtype = self.patch_embedding.weight.dtype
    tokens, grid = self.patchify(hidden_states.to(dtype))
    if rope is None:
      rope = wan_rope_tables(cfg.attention_head_dim, grid, max_seq_len=cfg.rope_max_seq_len, device=tokens.device)
    if pctx is not None:
      tokens = pctx.shard_sequence(tokens)
      rope = (pctx.shard_sequence(rope[0], dim=0), pctx.shard_sequence(rope[1], dim=0))
    x = self.patch_embedding(tokens)
    if token_bias is not None:  # pose embedding of Wan-Animate, added to the embedded patches
      x = x + (pctx.shard_sequence(token_bias) if pctx is not None else token_bias).to(x.dtype)

    temb, tproj = self.condition_embedder.time(timestep, dtype)
    temb6 = tproj.reshape(tproj.shape[0], 6, -1)
    context = context_image = None
    if kv_cache is None:
      context = self.condition_embedder.text(encoder_hidden_states.to(dtype))
      if encoder_hidden_states_image is not None and self.condition_embedder.image_embedder is not None:
        context_image = self.condition_embedder.image_embedder(encoder_hidden_states_image.to(dtype))

    x_in = x
    if skip_blocks:
      if cached_residual is None:
        raise ValueError("cached_residual must be provided when skip_blocks is True")
      x = x + cached_residual
    else:
      if callable(hints):
        # control branches (VACE) need the embedded tokens and conditioning: they are computed here, once
        hints = hints(x, context, temb6, rope, pctx)
      x = self.run_blocks(x, context, temb6, rope, pctx, context_image, kv_cache, hints, block_post)
    residual = (x - x_in) if return_residual else None

    shift, scale = (self.scale_shift_table.float() + temb.float().unsqueeze(1)).unbind(1)
    x = OF.layer_norm_mod(x, scale=scale, shift=shift, eps=cfg.eps)
    x = self.proj_out(x)
    if return_tokens:
      # training: the loss is taken on this rank's token shard, in patch space
      return x
    if pctx is not None:
      x = pctx.unshard_sequence(x)
    out = self.unpatchify(x, grid)
    return (out, residual) if return_residual else out

  def run_blocks(self, x, context, temb6, rope, pctx, context_image, kv_cache, hints=None, block_post=None):
    """`hints` {block index: tensor} are added to the stream after that block (VACE); `block_post(i, x)` may
    transform the stream after block i (Wan-Animate face adapter)."""
    policy = self.remat_policy.upper() if torch.is_grad_enabled() else "NONE"
    # the last `remat_keep_blocks` blocks keep their activations instead of recomputing them (memory permitting)
    first_kept = len(self.blocks) - int(getattr(self, "remat_keep_blocks", 0) or 0)
    for i, blk in enumerate(self.blocks):
      if self.block_hook is not None:
        self.block_hook(i, "forward")
      layer_kv = kv_cache[i] if kv_cache is not None else None
      if policy == "NONE":
        x = blk(x, context, temb6, rope, pctx, context_image, layer_kv)
      elif i >= first_kept:
        def run_keep(x_, context_, temb6_, blk=blk, layer_kv=layer_kv):
          return blk(x_, context_, temb6_, rope, pctx, context_image, layer_kv)

        pre = done = None
        if self.block_hook is not None:
          pre = (lambda idx=i: self.block_hook(idx, "recompute"))
          done = (lambda idx=i: self.block_hook(idx, "backward_done"))
        x = OF.keep_block(run_keep, x, context, temb6, pre_backward=pre, on_backward_done=done)
      else:
        def run(x_, context_, temb6_, blk=blk, layer_kv=layer_kv, idx=i):
          if self.block_hook is not None and torch.is_grad_enabled():
            self.block_hook(idx, "recompute")
          return blk(x_, context_, temb6_, rope, pctx, context_image, layer_kv)

        done = None
        if self.block_hook is not None:
          done = (lambda idx=i: self.block_hook(idx, "backward_done"))
        x = OF.checkpoint_block(run, x, context, temb6, save_attention=(not policy.startswith("FULL")), on_backward_done=done,
                                offload_input=policy.endswith("_OFFLOAD"))
      if hints is not None and i in hints:
        x = x + hints[i].to(x.dtype)
      if block_post is not None:
        x = block_post(i, x)
    return x
