"""Pure-PyTorch reference implementation of every op in `maxdiffusion_b200.ops`.

These are the oracles the CUDA kernels are tested against (run in fp32), and they are what the ops
dispatch to for CPU tensors, so that the whole framework — models, schedulers, trainers — runs and is
testable on a machine without a GPU.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def gemm(a, b, *, a_mn=False, b_mn=False, bias=None, epi="none", residual=None, gate=None, rows_per_batch=0,
         out_dtype=None, alpha=1.0):
  """D = epi(alpha * A @ B^T + bias); A is [M,K] ([K,M] when a_mn), B is [N,K] ([K,N] when b_mn)."""
  af = a.float().t() if a_mn else a.float()
  bf = b.float() if b_mn else b.float().t()
  y = alpha * (af @ bf)
  if bias is not None:
    y = y + bias.float()
  if epi == "gelu_tanh":
    y = F.gelu(y, approximate="tanh")
  elif epi == "silu":
    y = F.silu(y)
  elif epi == "gated_res":
    m = y.shape[0]
    g = gate.float()
    if rows_per_batch > 0:
      g = g.repeat_interleave(rows_per_batch, dim=0)[:m]
    else:
      g = g[:1].expand(m, -1)
    y = residual.float() + g[:, : y.shape[1]] * y
  elif epi == "add_res":
    y = residual.float() + y
  elif epi != "none":
    raise ValueError(epi)
  return y.to(out_dtype or a.dtype)


def attention(q, k_list, v_list, scale=None, return_lse=False):
  """Softmax attention over the concatenation of KV segments. q: [B,Sq,H,D]; k,v: lists of [B,Skv,H,D]."""
  if isinstance(k_list, torch.Tensor):
    k_list, v_list = [k_list], [v_list]
  k = torch.cat(list(k_list), dim=1)
  v = torch.cat(list(v_list), dim=1)
  d = q.shape[-1]
  scale = scale if scale is not None else 1.0 / math.sqrt(d)
  qf, kf, vf = q.float(), k.float(), v.float()
  s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
  lse = torch.logsumexp(s, dim=-1)  # natural log, [B,H,Sq]
  p = torch.exp(s - lse.unsqueeze(-1))
  o = torch.einsum("bhqk,bkhd->bqhd", p, vf).to(q.dtype)
  if return_lse:
    return o, lse * (1.0 / math.log(2.0))  # log2 domain, like the kernel
  return o


def attention_bwd(q, k, v, o, do, lse2, scale=None):
  """Gradients of `attention` for a single KV segment. lse2 is the log2-domain LSE [B,H,Sq]."""
  d = q.shape[-1]
  scale = scale if scale is not None else 1.0 / math.sqrt(d)
  qf, kf, vf, dof, of = q.float(), k.float(), v.float(), do.float(), o.float()
  s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
  p = torch.exp(s - (lse2 * math.log(2.0)).unsqueeze(-1))
  dv = torch.einsum("bhqk,bqhd->bkhd", p, dof)
  dp = torch.einsum("bqhd,bkhd->bhqk", dof, vf)
  delta = (dof * of).sum(-1).permute(0, 2, 1)  # [B,H,Sq]
  ds = p * (dp - delta.unsqueeze(-1)) * scale
  dq = torch.einsum("bhqk,bkhd->bqhd", ds, kf)
  dk = torch.einsum("bhqk,bqhd->bkhd", ds, qf)
  return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def _expand_mod(t, rows_per_batch, rows):
  # t: [num_batches, C] -> [rows, C]
  return t.float().repeat_interleave(rows_per_batch, dim=0)[:rows]


def layer_norm_mod(x, gamma=None, beta=None, scale=None, shift=None, eps=1e-6, return_stats=False):
  """y = ((x-mean)*rstd*gamma+beta)*(1+scale)+shift with fp32 statistics. x: [B,S,C]; scale/shift: [B,C]."""
  xf = x.float()
  mean = xf.mean(-1, keepdim=True)
  var = ((xf - mean) ** 2).mean(-1, keepdim=True)
  rstd = torch.rsqrt(var + eps)
  y = (xf - mean) * rstd
  if gamma is not None:
    y = y * gamma.float()
  if beta is not None:
    y = y + beta.float()
  if scale is not None:
    y = y * (1.0 + scale.float().unsqueeze(1)) + shift.float().unsqueeze(1)
  y = y.to(x.dtype)
  if return_stats:
    return y, mean.squeeze(-1), rstd.squeeze(-1)
  return y


def rope_rotate(y, cos, sin):
  """Rotary embedding on interleaved pairs. y: [B,S,H,D]; cos/sin: [S,D/2] fp32."""
  yf = y.float()
  y0, y1 = yf[..., 0::2], yf[..., 1::2]
  c = cos[None, :, None, :].float()
  s = sin[None, :, None, :].float()
  out = torch.stack([y0 * c - y1 * s, y0 * s + y1 * c], dim=-1)
  return out.reshape(y.shape)


def rms_norm_rope(x, w=None, cos=None, sin=None, heads=1, per_head=False, eps=1e-6):
  """RMSNorm over all channels (per_head=False) or per 128-wide head, then RoPE. x: [B,S,C] -> [B,S,H,D]."""
  b, s, c = x.shape
  d = c // heads
  xf = x.float()
  if per_head:
    xh = xf.view(b, s, heads, d)
    y = xh * torch.rsqrt((xh * xh).mean(-1, keepdim=True) + eps)
    if w is not None:
      y = y * w.float()
  else:
    y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
    if w is not None:
      y = y * w.float()
    y = y.view(b, s, heads, d)
  if cos is not None:
    y = rope_rotate(y, cos, sin)
  return y.to(x.dtype)


def gated_residual(res, y, gate=None):
  """res + gate[:,None,:] * y in fp32, rounded once. res,y: [B,S,C]; gate: [B,C] fp32 or None."""
  if gate is None:
    return (res.float() + y.float()).to(res.dtype)
  return (res.float() + gate.float().unsqueeze(1) * y.float()).to(res.dtype)


def gelu_tanh(u):
  return F.gelu(u.float(), approximate="tanh").to(u.dtype)


def adamw_step(p, g, m, v, *, lr, b1, b2, eps, wd, step, grad_scale=1.0, clip_value=0.0):
  """In-place AdamW with decoupled weight decay (optax.adamw semantics), fp32 math."""
  gf = g.float() * grad_scale
  if clip_value > 0:
    gf = gf.clamp(-clip_value, clip_value)
  mf = b1 * m.float() + (1 - b1) * gf
  vf = b2 * v.float() + (1 - b2) * gf * gf
  m.copy_(mf.to(m.dtype))
  v.copy_(vf.to(v.dtype))
  mhat = mf / (1 - b1**step)
  vhat = vf / (1 - b2**step)
  pf = p.float()
  pf = pf - lr * (mhat / (vhat.sqrt() + eps) + wd * pf)
  p.copy_(pf.to(p.dtype))


def sumsq_maxabs(x):
  xf = x.float()
  return torch.stack([(xf * xf).sum(), xf.abs().max()])


def group_norm(x, groups, gamma=None, beta=None, eps=1e-6, act=False):
  y = torch.nn.functional.group_norm(x.float(), groups, None if gamma is None else gamma.float(),
                                     None if beta is None else beta.float(), eps)
  if act:
    y = torch.nn.functional.silu(y)
  return y.to(x.dtype)


def lincomb(xs, coefs, out_dtype=None):
  x0 = xs[0]
  rows = list(coefs) if isinstance(coefs[0], (list, tuple)) else [list(coefs)]
  c = torch.tensor(rows, dtype=torch.float32, device=x0.device)  # [B or 1, n_in]
  shape = [c.shape[0]] + [1] * (x0.dim() - 1)
  acc = torch.zeros(x0.shape, dtype=torch.float32, device=x0.device)
  for i, x in enumerate(xs):
    acc = acc + c[:, i].reshape(shape) * x.float()
  return acc.to(out_dtype or x0.dtype)


def weighted_mse(pred, target, weights=None):
  e = (pred.float() - target.float()) ** 2
  if weights is not None:
    w = torch.as_tensor(weights, dtype=torch.float32, device=pred.device)
    e = e * w.reshape([-1] + [1] * (pred.dim() - 1))
  return e.mean()


def to_uint8(x):
  return ((x.float() * 0.5 + 0.5).clamp(0, 1) * 255.0).round().to(torch.uint8)


def channel_affine(x, mean, scale, channel_dim, denorm=False, out_dtype=None):
  shape = [1] * x.dim()
  shape[channel_dim] = -1
  m = mean.float().to(x.device).reshape(shape)
  s = scale.float().to(x.device).reshape(shape)
  y = x.float() * s + m if denorm else (x.float() - m) * s
  return y.to(out_dtype or x.dtype)


def blend_ramp(a, b, dim):
  n = a.shape[dim]
  shape = [1] * a.dim()
  shape[dim] = n
  w = (torch.arange(n, device=a.device, dtype=torch.float32) / n).reshape(shape)
  return (a.float() * (1 - w) + b.float() * w).to(a.dtype)
