"""Differentiable ops of the framework.

Dispatch rule: CUDA bf16 tensors run the hand-written sm_100a kernels (`ops.kernels`) inside
`torch.autograd.Function`s whose backward passes are kernels as well; every other tensor (CPU, fp32)
runs the PyTorch reference (`ops.ref`) under ordinary autograd. There is no silent fallback for CUDA
bf16 inputs: if the kernel library cannot be loaded the call raises.

Selective rematerialisation: inside `remat.record()` the self-attention forward stores (O, LSE) and inside
`remat.replay()` it reuses them instead of running the forward kernel again, which is the
"save attention, recompute the rest" policy (the reference spells such policies as lists of checkpoint
names, src/maxdiffusion/models/gradient_checkpoint.py:30-103).
"""
from __future__ import annotations

import contextlib
import math
import threading
from typing import Sequence

import torch
import torch.nn.functional as F

from . import conv as OC
from . import kernels as K
from . import ref


_LIBRARY_MODE = False


def set_library_mode(on: bool) -> None:
  """Yardstick switch: when on, no op of this module (and no optimizer step of `parallel.fsdp`) runs a kernel of this
  repository; CUDA tensors take the PyTorch path instead (`F.linear` = cuBLAS, `scaled_dot_product_attention`, eager
  norms and elementwise ops, `torch._foreach` AdamW). Used by `bench.py --impl library` only."""
  global _LIBRARY_MODE
  _LIBRARY_MODE = bool(on)


def library_mode() -> bool:
  return _LIBRARY_MODE


def _fast(t: torch.Tensor) -> bool:
  return t.is_cuda and t.dtype == torch.bfloat16 and not _LIBRARY_MODE


# ---------------------------------------------------------------------------------------------
# remat bookkeeping for attention outputs
# ---------------------------------------------------------------------------------------------
class _RematState(threading.local):

  def __init__(self):
    self.mode = None  # None | "record" | "replay"
    self.store = None
    self.cursor = 0


_remat = _RematState()


class remat:
  """Context managers used by `checkpoint_block`."""

  @staticmethod
  @contextlib.contextmanager
  def record(store: list):
    prev = (_remat.mode, _remat.store, _remat.cursor)
    _remat.mode, _remat.store, _remat.cursor = "record", store, 0
    try:
      yield
    finally:
      _remat.mode, _remat.store, _remat.cursor = prev

  @staticmethod
  @contextlib.contextmanager
  def replay(store: list):
    prev = (_remat.mode, _remat.store, _remat.cursor)
    _remat.mode, _remat.store, _remat.cursor = "replay", store, 0
    try:
      yield
    finally:
      _remat.mode, _remat.store, _remat.cursor = prev


# ---------------------------------------------------------------------------------------------
# linear (+ bias, + GELU-tanh / SiLU), the GEMM family
# ---------------------------------------------------------------------------------------------
class _LinearFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, w, b, act, residual=None):
    x2 = x.reshape(-1, x.shape[-1])
    need_grad = any(ctx.needs_input_grad[:3])
    ctx.act = act
    ctx.x_shape = x.shape
    ctx.has_bias = b is not None
    if residual is not None:
      # y = residual + x W^T + b: the add rides in the GEMM epilogue; its gradient is dy itself
      r2 = residual.reshape(-1, w.shape[0])
      y = K.gemm(x2, w, bias=b, epi="add_res", residual=r2 if r2.is_contiguous() else r2.contiguous())
      ctx.save_for_backward(x2, w, None)
    elif act in ("gelu_tanh",) and need_grad:
      u = K.gemm(x2, w, bias=b)
      y = K.gelu_fwd(u)
      ctx.save_for_backward(x2, w, u)
    else:
      y = K.gemm(x2, w, bias=b, epi=act or "none")
      if act == "silu" and need_grad:
        raise NotImplementedError("silu epilogue has no fused backward; apply silu as a separate op when training")
      ctx.save_for_backward(x2, w, None)
    return y.view(*x.shape[:-1], w.shape[0])

  @staticmethod
  def backward(ctx, dy):
    x2, w, u = ctx.saved_tensors
    dy2 = dy.reshape(-1, dy.shape[-1])
    if not dy2.is_contiguous():
      dy2 = dy2.contiguous()
    if u is not None:
      dy2 = K.gelu_bwd(dy2, u)
    dx = dw = db = None
    if ctx.needs_input_grad[0]:
      dx = K.gemm(dy2, w, b_mn=True).view(ctx.x_shape)       # dX = dY · W
    if ctx.needs_input_grad[1]:
      dw = K.gemm(dy2, x2, a_mn=True, b_mn=True)              # dW = dYᵀ · X
    if ctx.has_bias and ctx.needs_input_grad[2]:
      db = K.colsum(dy2).to(torch.bfloat16)
    return dx, dw, db, None, (dy if ctx.needs_input_grad[4] else None)


def linear(x, weight, bias=None, activation: str | None = None, residual=None):
  """y = act(x @ weightᵀ + bias) (+ residual, without activation); weight is [out, in] (PyTorch / diffusers
  orientation). The residual add runs in the GEMM epilogue."""
  if _fast(x) and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0:
    if weight.dtype != torch.bfloat16:
      weight = weight.to(torch.bfloat16)
    if bias is not None and bias.dtype != torch.bfloat16:
      bias = bias.to(torch.bfloat16)
    if residual is not None and (activation is not None or residual.dtype != torch.bfloat16):
      return residual + _LinearFn.apply(x, weight, bias, activation)
    return _LinearFn.apply(x, weight, bias, activation, residual)
  y = F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
  if activation == "gelu_tanh":
    y = F.gelu(y, approximate="tanh")
  elif activation == "silu":
    y = F.silu(y)
  return y if residual is None else residual + y


def linear_gated_residual(x, weight, bias, residual, gate):
  """residual + gate[:,None,:] * (x @ weightᵀ + bias), the output projection of an AdaLN-gated branch.

  Without autograd the gate and the residual add run in the GEMM epilogue; with autograd the product is
  materialised because the gate's gradient needs it.
  """
  if _fast(x) and not torch.is_grad_enabled():
    B, S, _ = x.shape
    out = K.gemm(x.reshape(B * S, -1), weight, bias=bias, epi="gated_res" if gate is not None else "add_res",
                 residual=residual.reshape(B * S, -1), gate=gate, rows_per_batch=S)
    return out.view(B, S, -1)
  return gated_residual(residual, linear(x, weight, bias), gate)


# ---------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------
# attention outputs are kept across the rematerialisation of a block only when recomputing them is expensive
_REMAT_MIN_KV = 2048


class _AttentionFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, q, scale, n_seg, fixed_m, *kv):
    ks, vs = list(kv[:n_seg]), list(kv[n_seg:])
    saved = None
    keep = _remat.mode is not None and sum(k.shape[1] for k in ks) >= _REMAT_MIN_KV
    if keep and _remat.mode == "replay":
      saved = _remat.store[_remat.cursor]
      _remat.cursor += 1
    if saved is not None:
      out, lse = saved
    else:
      out, lse = K.flash_fwd(q, ks, vs, scale, fixed_m=fixed_m)
      if keep and _remat.mode == "record":
        _remat.store.append((out, lse))
    ctx.scale, ctx.n_seg = scale, n_seg
    ctx.save_for_backward(q, out, lse, *ks, *vs)
    return out

  @staticmethod
  def backward(ctx, d_o):
    q, out, lse, *kv = ctx.saved_tensors
    n = ctx.n_seg
    ks, vs = kv[:n], kv[n:]
    if d_o.stride(-1) != 1:
      d_o = d_o.contiguous()
    delta = K.flash_delta(out, d_o)
    dq = K.flash_bwd_dq(q, d_o, ks, vs, lse, delta, ctx.scale)
    dks, dvs = [], []
    for k, v in zip(ks, vs):
      dk, dv = K.flash_bwd_dkv(q, d_o, k, v, lse, delta, ctx.scale)
      dks.append(dk)
      dvs.append(dv)
    return (dq, None, None, None, *dks, *dvs)


_KEPT: dict = {}


def _kept_indices(keep: torch.Tensor):
  """Per batch row, the indices of the kept keys (one host synchronisation per mask tensor, then cached on the
  tensor object and its version counter: the same mask serves every layer and step of a sampling loop)."""
  import weakref

  hit = _KEPT.get(id(keep))
  if hit is not None and hit[0]() is keep and hit[1] == keep._version:
    return hit[2]
  if len(_KEPT) >= 32:
    _KEPT.clear()
  idx = [keep[b].nonzero(as_tuple=True)[0] for b in range(keep.shape[0])]
  _KEPT[id(keep)] = (weakref.ref(keep), keep._version, idx)
  return idx


def attention(q, k, v, scale: float | None = None, fixed_m=None, keep_mask=None):
  """Softmax attention. q: [B,Sq,H,D]; k, v: [B,Skv,H,D] or equal-length lists of KV segments.

  `fixed_m` (from `ops.fixed_m.plan`) runs the marked heads of the flash kernel with a fixed softmax exponent; the
  result and the saved log-sum-exp are those of the plain softmax, so the backward is unchanged. Paths that do
  not run the flash kernel ignore it.

  `keep_mask` (bool [B,Skv], True = attend) drops keys per batch row. On the flash path the kept keys of a row are
  compacted and the kernel runs on the shorter sequence (dropped keys cost nothing); a row without kept keys
  yields zeros. Elsewhere the mask goes to SDPA."""
  ks = list(k) if isinstance(k, (list, tuple)) else [k]
  vs = list(v) if isinstance(v, (list, tuple)) else [v]
  D = q.shape[-1]
  scale = scale if scale is not None else 1.0 / math.sqrt(D)
  if _fast(q) and D not in K.FLASH_HEAD_DIMS and D < max(K.FLASH_HEAD_DIMS) and D % 8 == 0:
    # other head sizes (Stable Diffusion 1.x / 2.x: 40, 80) ride the next built size: zero channels add nothing to
    # q.k and produce zero output channels, which are cut off again; the scale stays that of the true size
    Dp = min(d for d in K.FLASH_HEAD_DIMS if d > D)
    pad = lambda t: F.pad(t, (0, Dp - D))
    out = attention(pad(q), [pad(t) for t in ks], [pad(t) for t in vs], scale, None, keep_mask)
    return out[..., :D]
  fast = _fast(q) and D in K.FLASH_HEAD_DIMS
  if keep_mask is not None:
    assert keep_mask.dtype == torch.bool and keep_mask.dim() == 2 and len(ks) == 1
    kc, vc = ks[0], vs[0]
    if not fast:
      out = F.scaled_dot_product_attention(q.transpose(1, 2), kc.transpose(1, 2), vc.transpose(1, 2),
                                           attn_mask=keep_mask[:, None, None, :], scale=scale)
      return out.transpose(1, 2)
    rows = []
    for b, idx in enumerate(_kept_indices(keep_mask)):
      if idx.numel() == 0:
        rows.append(torch.zeros_like(q[b:b + 1]))
      elif idx.numel() == kc.shape[1]:
        rows.append(_AttentionFn.apply(q[b:b + 1], scale, 1, None, kc[b:b + 1], vc[b:b + 1]))
      else:
        rows.append(_AttentionFn.apply(q[b:b + 1], scale, 1, None, kc[b:b + 1].index_select(1, idx),
                                       vc[b:b + 1].index_select(1, idx)))
    return rows[0] if len(rows) == 1 else torch.cat(rows, dim=0)
  if fast:
    return _AttentionFn.apply(q, scale, len(ks), fixed_m, *ks, *vs)
  kc = torch.cat(ks, dim=1) if len(ks) > 1 else ks[0]
  vc = torch.cat(vs, dim=1) if len(vs) > 1 else vs[0]
  out = F.scaled_dot_product_attention(q.transpose(1, 2), kc.transpose(1, 2), vc.transpose(1, 2), scale=scale)
  return out.transpose(1, 2)


# ---------------------------------------------------------------------------------------------
# norms
# ---------------------------------------------------------------------------------------------
class _LayerNormModFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, gamma, beta, scale, shift, eps):
    need = any(ctx.needs_input_grad[:5])
    if need:
      y, mean, rstd = K.ln_fwd(x, gamma, beta, scale, shift, eps, save_stats=True)
      ctx.save_for_backward(x, mean, rstd, gamma, scale)
    else:
      y = K.ln_fwd(x, gamma, beta, scale, shift, eps)
    return y

  @staticmethod
  def backward(ctx, dy):
    x, mean, rstd, gamma, scale = ctx.saved_tensors
    if not dy.is_contiguous():
      dy = dy.contiguous()
    need_sums = any(ctx.needs_input_grad[1:5])
    dx, sums = K.ln_bwd(dy, x, mean, rstd, gamma, scale, need_sums=need_sums)
    dgamma = dbeta = dscale = dshift = None
    if sums is not None:
      if gamma is not None:
        # with affine the first sum is d/dgamma only when there is no modulation on top
        dgamma = sums[:, 0].sum(0).to(gamma.dtype) if ctx.needs_input_grad[1] else None
        dbeta = sums[:, 1].sum(0).to(gamma.dtype) if ctx.needs_input_grad[2] else None
      if scale is not None:
        dscale = sums[:, 0] if ctx.needs_input_grad[3] else None
        dshift = sums[:, 1] if ctx.needs_input_grad[4] else None
    return dx, dgamma, dbeta, dscale, dshift, None


def layer_norm_mod(x, gamma=None, beta=None, scale=None, shift=None, eps: float = 1e-6):
  """fp32 LayerNorm with optional affine (gamma, beta) xor AdaLN modulation (scale, shift: fp32 [B, C])."""
  if _fast(x) and x.dim() == 3 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192 and not (gamma is not None and scale is not None):
    x = x if x.is_contiguous() else x.contiguous()
    if scale is not None:
      scale = scale.float() if scale.dtype != torch.float32 else scale
      shift = shift.float() if shift.dtype != torch.float32 else shift
      if scale.stride(-1) != 1 or shift.stride(-1) != 1 or scale.stride(0) != shift.stride(0):
        scale, shift = scale.contiguous(), shift.contiguous()
    return _LayerNormModFn.apply(x, gamma, beta, scale, shift, eps)
  return ref.layer_norm_mod(x, gamma, beta, scale, shift, eps)


class _GegluFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, u):
    ctx.save_for_backward(u)
    return K.geglu_fwd(u)

  @staticmethod
  def backward(ctx, dy):
    (u,) = ctx.saved_tensors
    return K.geglu_bwd(dy if dy.is_contiguous() else dy.contiguous(), u)


def geglu(u: torch.Tensor) -> torch.Tensor:
  """u [..., 2 * inner] = (h | gate) -> h * gelu(gate), exact GELU; one kernel forward, one backward."""
  if _fast(u) and u.shape[-1] % 16 == 0:
    return _GegluFn.apply(u if u.is_contiguous() else u.contiguous())
  h, gate = u.chunk(2, dim=-1)
  return h * torch.nn.functional.gelu(gate)


class _RmsRopeFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, w, cos, sin, heads, per_head, eps):
    need = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
    ctx.per_head = per_head
    ctx.has_rope = cos is not None
    if need:
      y, rstd = K.rms_rope_fwd(x, w, cos, sin, heads, per_head, eps, save_stats=True)
      ctx.save_for_backward(x, rstd, w, cos, sin)
    else:
      y = K.rms_rope_fwd(x, w, cos, sin, heads, per_head, eps)
    return y

  @staticmethod
  def backward(ctx, dy):
    x, rstd, w, cos, sin = ctx.saved_tensors
    dx, dw = K.rms_rope_bwd(dy, x, rstd, w, cos, sin, per_head=ctx.per_head, need_dw=ctx.needs_input_grad[1])
    if dw is not None:
      dw = dw.to(w.dtype)
    return dx, dw, None, None, None, None, None


def rms_norm_rope(x, weight=None, cos=None, sin=None, heads: int = 1, per_head: bool = False, eps: float = 1e-6):
  """RMSNorm (across all channels or per 128-wide head) then RoPE on interleaved pairs. [B,S,C] -> [B,S,H,D]."""
  B, S, C = x.shape
  if _fast(x) and C % 128 == 0 and C // heads == 128 and C <= 8192 and x.stride(-1) == 1 and x.stride(0) == S * x.stride(1):
    if cos is not None:
      cos = cos.float().contiguous() if (cos.dtype != torch.float32 or not cos.is_contiguous()) else cos
      sin = sin.float().contiguous() if (sin.dtype != torch.float32 or not sin.is_contiguous()) else sin
    return _RmsRopeFn.apply(x, weight, cos, sin, heads, per_head, eps)
  return ref.rms_norm_rope(x, weight, cos, sin, heads, per_head, eps)


# ---------------------------------------------------------------------------------------------
# elementwise
# ---------------------------------------------------------------------------------------------
class _GatedResFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, res, y, gate):
    ctx.save_for_backward(y if ctx.needs_input_grad[2] else None, gate)
    return K.gated_res_fwd(res, y, gate)

  @staticmethod
  def backward(ctx, dout):
    y, gate = ctx.saved_tensors
    if not dout.is_contiguous():
      dout = dout.contiguous()
    if gate is None:
      return dout, dout, None
    if y is not None:
      dy, dgate = K.gated_res_bwd(dout, y, gate)
    else:
      dy, dgate = (dout.float() * gate.unsqueeze(1)).to(dout.dtype), None
    return dout, dy, dgate


def gated_residual(res, y, gate=None):
  """res + gate[:, None, :] * y with one rounding; gate is fp32 [B, C] (None means 1)."""
  if _fast(res) and res.dim() == 3 and res.shape[-1] % 8 == 0 and res.shape[-1] <= 8192:
    res = res if res.is_contiguous() else res.contiguous()
    y = y if y.is_contiguous() else y.contiguous()
    if gate is not None and (gate.dtype != torch.float32 or gate.stride(-1) != 1):
      gate = gate.float().contiguous()
    return _GatedResFn.apply(res, y, gate)
  return ref.gated_residual(res, y, gate)


# ---------------------------------------------------------------------------------------------
# block-level rematerialisation
# ---------------------------------------------------------------------------------------------
class _CheckpointFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, fn, save_attention, on_backward_done, n_tensors, *args):
    ctx.fn = fn
    ctx.on_backward_done = on_backward_done
    offload = save_attention == "offload" or (isinstance(save_attention, tuple) and save_attention[1])
    save_attention = save_attention[0] if isinstance(save_attention, tuple) else (save_attention is True)
    ctx.store = [] if save_attention else None
    tensors = args[:n_tensors]
    ctx.rest = args[n_tensors:]
    ctx.offloaded = None
    if offload and tensors and tensors[0].is_cuda:
      # the block input (the residual stream) waits for the backward pass in pinned host memory
      x = tensors[0]
      host = torch.empty(x.shape, dtype=x.dtype, device="cpu", pin_memory=True)
      host.copy_(x, non_blocking=True)
      ctx.offloaded = (host, x.device, x.requires_grad)
      ctx.offload_event = torch.cuda.Event()
      ctx.offload_event.record()
      tensors = (None,) + tuple(tensors[1:])
    ctx.save_for_backward(*tensors)
    with torch.no_grad():
      if ctx.store is not None:
        with remat.record(ctx.store):
          out = fn(*args)
      else:
        out = fn(*args)
    return out

  @staticmethod
  def backward(ctx, *douts):
    saved = list(ctx.saved_tensors)
    if ctx.offloaded is not None:
      host, device, req = ctx.offloaded
      ctx.offload_event.synchronize()
      saved[0] = host.to(device, non_blocking=True).requires_grad_(req)
      ctx.offloaded = None
    tensors = [t.detach().requires_grad_(t.requires_grad) if t is not None else None for t in saved]
    # only tensors that took part in autograd need gradients; floating point inputs are assumed to
    inputs = []
    for t, orig in zip(tensors, saved):
      if t is not None and orig.is_floating_point():
        t.requires_grad_(True)
      inputs.append(t)
    with torch.enable_grad():
      if ctx.store is not None:
        with remat.replay(ctx.store):
          out = ctx.fn(*inputs, *ctx.rest)
      else:
        out = ctx.fn(*inputs, *ctx.rest)
    outs = out if isinstance(out, tuple) else (out,)
    torch.autograd.backward([o for o in outs if o.requires_grad], [g for o, g in zip(outs, douts) if o.requires_grad])
    ctx.store = None
    grads = [t.grad if (t is not None and t.is_floating_point()) else None for t in inputs]
    if ctx.on_backward_done is not None:
      ctx.on_backward_done()
    return (None, None, None, None, *grads, *([None] * len(ctx.rest)))


class _KeepGraphFn(torch.autograd.Function):
  """A block whose activations are kept (no recomputation) but whose backward still runs as one unit, so that the
  same hooks as for a rematerialised block fire: `pre_backward()` before it (the FSDP engine gathers the block's
  weights again) and `on_backward_done()` once its parameter gradients are complete."""

  @staticmethod
  def forward(ctx, fn, pre_backward, on_backward_done, n_tensors, *args):
    tensors, rest = args[:n_tensors], args[n_tensors:]
    inputs = [t.detach().requires_grad_(True) if (t is not None and t.is_floating_point()) else t for t in tensors]
    with torch.enable_grad():
      out = fn(*inputs, *rest)
    ctx.inputs, ctx.out = inputs, out
    ctx.pre_backward, ctx.on_backward_done, ctx.n_rest = pre_backward, on_backward_done, len(rest)
    if isinstance(out, tuple):
      return tuple(o.detach() for o in out)
    return out.detach()

  @staticmethod
  def backward(ctx, *douts):
    if ctx.pre_backward is not None:
      ctx.pre_backward()
    outs = ctx.out if isinstance(ctx.out, tuple) else (ctx.out,)
    torch.autograd.backward([o for o in outs if o.requires_grad], [g for o, g in zip(outs, douts) if o.requires_grad])
    grads = [t.grad if (t is not None and t.is_floating_point()) else None for t in ctx.inputs]
    ctx.out, ctx.inputs = None, None
    if ctx.on_backward_done is not None:
      ctx.on_backward_done()
    return (None, None, None, None, *grads, *([None] * ctx.n_rest))


def keep_block(fn, *tensor_args, extra_args: Sequence = (), pre_backward=None, on_backward_done=None):
  """Runs `fn(*tensor_args, *extra_args)` keeping its activations; see `_KeepGraphFn`."""
  return _KeepGraphFn.apply(fn, pre_backward, on_backward_done, len(tensor_args), *tensor_args, *extra_args)


def checkpoint_block(fn, *tensor_args, extra_args: Sequence = (), save_attention: bool = False,
                     on_backward_done=None, offload_input: bool = False):
  """Runs `fn(*tensor_args, *extra_args)` storing only its tensor inputs; the backward pass recomputes it.

  Parameters used inside `fn` receive their gradients during the recomputation. With `save_attention`
  the flash-attention outputs of the first pass are kept and not recomputed. `on_backward_done()` is called
  once the parameter gradients of the block are complete (the FSDP engine reduces and applies them there).
  With `offload_input` the first tensor argument is parked in pinned host memory between the two passes.
  """
  mode = (bool(save_attention), True) if offload_input else bool(save_attention)
  return _CheckpointFn.apply(fn, mode, on_backward_done, len(tensor_args), *tensor_args, *extra_args)


# ---------------------------------------------------------------------------------------------
# GroupNorm (+SiLU) and the elementwise step family
# ---------------------------------------------------------------------------------------------
class _GroupNormFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, gamma, beta, groups, eps, act):
    y, stats = K.groupnorm_fwd(x, groups, gamma, beta, eps, act)
    ctx.save_for_backward(x, gamma, beta, stats)
    ctx.groups, ctx.act = groups, act
    return y

  @staticmethod
  def backward(ctx, dy):
    x, gamma, beta, stats = ctx.saved_tensors
    dx, dgamma, dbeta = K.groupnorm_bwd(dy, x, stats, ctx.groups, gamma, beta, ctx.act)
    return (dx, dgamma.to(gamma.dtype) if gamma is not None else None,
            dbeta.to(beta.dtype) if beta is not None else None, None, None, None)


class _GroupNormCLFn(torch.autograd.Function):
  """GroupNorm (+ SiLU) of an NCHW tensor held in channels-last memory, on the channels-last kernels."""

  @staticmethod
  def forward(ctx, x, gamma, beta, groups, eps, act):
    N, C, H, W = x.shape
    x3 = x.permute(0, 2, 3, 1).reshape(N, H * W, C)  # a view: the memory is [N, H, W, C]
    y3, a, b, mean, rstd = OC.group_norm_cl_fwd(x3, groups, gamma, beta, eps, act)
    ctx.save_for_backward(x3, gamma, a, b, mean, rstd)
    ctx.groups, ctx.act, ctx.shape = groups, act, (N, C, H, W)
    ctx.has_beta = beta is not None
    return y3.view(N, H, W, C).permute(0, 3, 1, 2)

  @staticmethod
  def backward(ctx, dy):
    x3, gamma, a, b, mean, rstd = ctx.saved_tensors
    N, C, H, W = ctx.shape
    dy3 = dy.contiguous(memory_format=torch.channels_last).permute(0, 2, 3, 1).reshape(N, H * W, C)
    dx3, dgamma, dbeta = OC.group_norm_cl_bwd(dy3, x3, ctx.groups, gamma, a, b, mean, rstd, ctx.act)
    return (dx3.view(N, H, W, C).permute(0, 3, 1, 2), dgamma.to(gamma.dtype) if gamma is not None else None,
            dbeta.to(gamma.dtype) if (ctx.has_beta and gamma is not None) else None, None, None, None)


def _is_channels_last(x: torch.Tensor) -> bool:
  return x.dim() == 4 and x.shape[1] > 1 and x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous()


def group_norm(x, groups: int, gamma=None, beta=None, eps: float = 1e-6, act: bool = False):
  """GroupNorm over a channels-first tensor [N, C, *spatial] with optional fused SiLU. A 4-D bf16 tensor in
  channels-last memory (what `conv2d` produces) stays in that layout."""
  if _fast(x) and _is_channels_last(x) and x.shape[1] % 8 == 0 and x.shape[1] <= 2048:
    return _GroupNormCLFn.apply(x, gamma, beta, groups, eps, act)
  if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and not _LIBRARY_MODE:
    x = x if x.is_contiguous() else x.contiguous()
    return _GroupNormFn.apply(x, gamma, beta, groups, eps, act)
  return ref.group_norm(x, groups, gamma, beta, eps, act)


# ---------------------------------------------------------------------------------------------
# conv2d (NCHW interface, channels-last memory, implicit-GEMM kernels)
# ---------------------------------------------------------------------------------------------
_PACKED: dict = {}


def _packed(weight: torch.Tensor, bias, kind: str, make):
  """Packed form of a convolution weight, re-packed when the parameter changes (optimizer step, load)."""
  key = (id(weight), kind)
  ver = (weight.data_ptr(), weight._version, None if bias is None else bias._version)
  hit = _PACKED.get(key)
  if hit is None or hit[0] != ver or hit[2]() is not weight:
    import weakref

    if len(_PACKED) > 4096:
      _PACKED.clear()
    hit = (ver, make(), weakref.ref(weight))
    _PACKED[key] = hit
  return hit[1]


class _Conv2dFn(torch.autograd.Function):
  """3x3 convolution, stride 1 or 2, optionally preceded by a nearest-2x up-sampling (fused), on channels-last memory.
  Forward and input gradient run on the implicit-GEMM kernel; the weight gradient on `ops.conv.conv2d_wgrad`."""

  @staticmethod
  def forward(ctx, x, weight, bias, stride, pad, upsample):
    N, C, H, W = x.shape
    xc = x.contiguous(memory_format=torch.channels_last).permute(0, 2, 3, 1)  # [N, H, W, C], dense
    if upsample:
      pk = _packed(weight, bias, "up", lambda: OC.pack_upsample_conv2d(weight.detach(), None if bias is None else bias.detach()))
      y = OC.upsample2x_conv2d(OC.pad_channels(xc, pk.c_in), pk)
    else:
      pk = _packed(weight, bias, f"s{stride}p{pad}", lambda: OC.pack_conv2d(weight.detach(), None if bias is None else bias.detach(),
                                                                           stride=stride, pad_top_left=pad))
      y = OC.conv2d(OC.pad_channels(xc, pk.c_in), pk)
    ctx.save_for_backward(xc, weight)
    ctx.cfg = (stride, pad, upsample, bias is not None)
    return y.permute(0, 3, 1, 2)

  @staticmethod
  def backward(ctx, dy):
    xc, weight = ctx.saved_tensors
    stride, pad, upsample, has_bias = ctx.cfg
    dyc = dy.contiguous(memory_format=torch.channels_last).permute(0, 2, 3, 1)  # [N, Ho, Wo, Co]
    co, ci = weight.shape[:2]
    dx = dw = db = None
    if ctx.needs_input_grad[0]:
      if upsample:
        pk = _packed(weight, None, "dgrad_s1p1", lambda: OC.pack_conv2d_dgrad(weight.detach(), 1, 1))
        du = OC.conv2d_dgrad(OC.pad_channels(dyc, pk.c_in), pk)[..., :ci]  # gradient of the up-sampled image
        n, h2, w2, _ = du.shape
        dxc = du.reshape(n, h2 // 2, 2, w2 // 2, 2, ci).float().sum(dim=(2, 4)).to(du.dtype)
      else:
        pk = _packed(weight, None, f"dgrad_s{stride}p{pad}", lambda: OC.pack_conv2d_dgrad(weight.detach(), stride, pad))
        dxc = OC.conv2d_dgrad(OC.pad_channels(dyc, pk.c_in), pk)[..., :ci]
      dx = dxc.permute(0, 3, 1, 2)
    if ctx.needs_input_grad[1]:
      xin = xc
      if upsample:
        n, h, w, c = xc.shape
        xin = xc.reshape(n, h, 1, w, 1, c).expand(n, h, 2, w, 2, c).reshape(n, 2 * h, 2 * w, c)
      dw = OC.conv2d_wgrad(xin, dyc, weight.shape[2], stride, pad).to(weight.dtype)
    if has_bias and ctx.needs_input_grad[2]:
      db = K.colsum(dyc.reshape(-1, co)).to(weight.dtype) if co % 8 == 0 else dyc.float().sum(dim=(0, 1, 2)).to(weight.dtype)
    return dx, dw, db, None, None, None


def conv2d(x, weight, bias=None, stride: int = 1, padding=1, upsample: bool = False):
  """2-D convolution of an NCHW tensor. `padding` is an int (all sides) or "far" (zero rows / columns after the image
  only: the VAE's stride-2 down-sampling). With `upsample` the input is nearest-2x up-sampled first (fused).

  CUDA bf16 3x3 convolutions run on the implicit-GEMM kernels and return channels-last memory; 1x1 convolutions are
  GEMMs over the pixel rows; everything else is `torch.nn.functional.conv2d`."""
  k = weight.shape[-1]
  pad_tl = 0 if padding == "far" else int(padding)
  co, ci = weight.shape[:2]
  if _fast(x) and k == 1 and stride == 1 and pad_tl == 0 and not upsample and ci % 8 == 0 and co % 8 == 0:
    n, c, h, w = x.shape
    rows = x.contiguous(memory_format=torch.channels_last).permute(0, 2, 3, 1).reshape(n, h * w, c)
    y = linear(rows, weight.reshape(co, ci), bias)
    return y.view(n, h, w, co).permute(0, 3, 1, 2)
  even = x.shape[2] % 2 == 0 and x.shape[3] % 2 == 0
  if (_fast(x) and k == 3 and stride in (1, 2) and (stride == 1 or even) and
      ((stride == 1 and pad_tl == 1) or (stride == 2 and pad_tl in (0, 1)))):
    if weight.dtype != torch.bfloat16:
      weight = weight.to(torch.bfloat16)
    return _Conv2dFn.apply(x, weight, bias, stride, pad_tl, upsample)
  if upsample:
    x = F.interpolate(x, scale_factor=2.0, mode="nearest")
  if padding == "far":
    x = F.pad(x, (0, 1, 0, 1))
  return F.conv2d(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype), stride=stride, padding=pad_tl)


def lincomb(xs, coefs, out_dtype=None):
  """sum_i coefs[(b,) i] * xs[i]; no gradient (sampling-loop updates)."""
  x0 = xs[0]
  per = x0.numel() // (len(coefs) if isinstance(coefs[0], (list, tuple)) else 1)
  if x0.is_cuda and per % 8 == 0 and all(x.dtype in (torch.bfloat16, torch.float32) for x in xs) and not _LIBRARY_MODE:
    return K.lincomb(list(xs), coefs, out_dtype=out_dtype)
  return ref.lincomb(xs, coefs, out_dtype)


class _MseFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, pred, target, weights):
    loss, dpred = K.mse_fwd_bwd(pred, target, weights, need_grad=True)
    ctx.save_for_backward(dpred)
    return loss

  @staticmethod
  def backward(ctx, dloss):
    (dpred,) = ctx.saved_tensors
    return dpred * dloss.to(dpred.dtype), None, None


def weighted_mse(pred, target, weights=None):
  """mean over all elements of w_b * (pred - target)^2; the gradient with respect to pred comes from the same pass."""
  B = pred.shape[0]
  if (pred.is_cuda and pred.dtype in (torch.bfloat16, torch.float32) and target.dtype in (torch.bfloat16, torch.float32)
      and B <= 16 and (pred.numel() // B) % 8 == 0 and not _LIBRARY_MODE):
    w = None if weights is None else [float(v) for v in (weights.tolist() if torch.is_tensor(weights) else weights)]
    return _MseFn.apply(pred, target.detach(), w)
  return ref.weighted_mse(pred, target, weights)
