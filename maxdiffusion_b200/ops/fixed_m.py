"""Fixed-exponent softmax for the flash-attention forward ("fixed-m").

Online softmax tracks a running row maximum and rescales the output accumulator when it moves. For heads whose
logits are provably small that work can be dropped: by Cauchy-Schwarz every score of query i obeys
q_i.k_j <= |q_i| * max_j |k_j|, so

    m_i = ceil(|q_i| * max_j|k_j| * scale * log2(e)) - 88

is an upper bound (minus a re-centring constant) that can be subtracted from every exponent of the row instead of
the running maximum: exp2 never sees more than 88, and as long as the bound stays below a gate the largest term of
a row stays above the fp32 flush-to-zero floor. The result is the same softmax (the shift cancels in p / sum p).

A head is eligible when max_i|q_i| * max_j|k_j| * scale * log2(e) <= 213. That gate assumes the keys were
smoothed (k - mean over the sequence, which leaves softmax unchanged and guarantees a row maximum >= 0); without
smoothing (ring attention, where no rank holds all keys) the gate halves to 106.5. Heads over the gate keep the
online softmax inside the same kernel launch. Norm maxima carry a 1 % margin and are max-reduced over the
process group that shares the keys.

Reference: src/maxdiffusion/kernels/custom_splash_attention.py:50-66,120-128,173-190,243-251 (kernel side) and
src/maxdiffusion/models/attention_flax.py:892-912,1357-1385 (k-smoothing and the per-head statistics).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist

RECENTER = 88.0
SAFE_BOUND = 213.0
RING_SAFE_BOUND = SAFE_BOUND / 2.0
NORM_MARGIN = 1.01
LOG2E = 1.4426950408889634


def smooth_keys(k: torch.Tensor) -> torch.Tensor:
  """k - mean over the sequence axis (per batch, head and channel). k: [B, S, H, D]. Softmax over the keys is
  unchanged because every score of a row moves by the same q_i . mean(k)."""
  return k - k.mean(dim=1, keepdim=True, dtype=torch.float32).to(k.dtype)


def head_statistics(q: torch.Tensor, ks: Sequence[torch.Tensor], group=None):
  """(row norms of q as fp32 [B, H, Sq], max row norm of q per head [H], max row norm of the keys per head [H]);
  the two maxima include the margin and are max-reduced over `group`."""
  with torch.no_grad():
    # fp32 accumulation inside the reduction: no fp32 copy of q or k is materialised
    qn = torch.linalg.vector_norm(q, dim=-1, dtype=torch.float32).permute(0, 2, 1).contiguous()  # [B, H, Sq]
    qmax = qn.amax(dim=(0, 2))
    kmax = torch.stack([torch.linalg.vector_norm(k, dim=-1, dtype=torch.float32).amax(dim=(0, 1))
                        for k in ks]).amax(dim=0)
    both = torch.stack([qmax, kmax]) * NORM_MARGIN
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
      dist.all_reduce(both, op=dist.ReduceOp.MAX, group=group)
  return qn, both[0], both[1]


def plan(q: torch.Tensor, ks, scale: Optional[float] = None, *, smoothed: bool = True,
         group=None) -> Tuple[torch.Tensor, torch.Tensor]:
  """(m_fixed fp32 [B, H, Sq] in the log2 domain, fixed_heads int32 [H]) for `kernels.flash_fwd(fixed_m=...)`.

  `ks` is one key tensor or the list of key segments this rank attends to; `group` is the process group whose
  ranks hold the other segments of the same keys (ring), or None. `smoothed` says whether `smooth_keys` was
  applied over the FULL key sequence; it selects the gate."""
  ks = list(ks) if isinstance(ks, (list, tuple)) else [ks]
  D = q.shape[-1]
  c = (scale if scale is not None else 1.0 / math.sqrt(D)) * LOG2E
  qn, qmax, kmax = head_statistics(q, ks, group)
  with torch.no_grad():
    m_fixed = torch.ceil(qn * (kmax * c)[None, :, None]) - RECENTER
    gate = SAFE_BOUND if smoothed else RING_SAFE_BOUND
    fixed_heads = (qmax * kmax * c <= gate).to(torch.int32)
  return m_fixed.contiguous(), fixed_heads.contiguous()


def reference_attention(q, ks, vs, scale: Optional[float] = None, fixed_m=None) -> torch.Tensor:
  """fp32 restatement of what the kernel computes, for tests: p = exp2(s*c - m) with m = m_fixed on the marked
  heads and the row maximum elsewhere; out = (p @ v) / sum p. q: [B,Sq,H,D]; ks / vs: tensors or segment lists."""
  ks = list(ks) if isinstance(ks, (list, tuple)) else [ks]
  vs = list(vs) if isinstance(vs, (list, tuple)) else [vs]
  k = torch.cat(ks, dim=1).float()
  v = torch.cat(vs, dim=1).float()
  D = q.shape[-1]
  c = (scale if scale is not None else 1.0 / math.sqrt(D)) * LOG2E
  s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k) * c
  m = s.amax(dim=-1)
  if fixed_m is not None:
    m_fixed, fixed_heads = fixed_m
    m = torch.where(fixed_heads.bool()[None, :, None], m_fixed.to(m.device), m)
  p = torch.exp2(s - m[..., None])
  out = torch.einsum("bhqk,bkhd->bqhd", p, v) / p.sum(-1).permute(0, 2, 1)[..., None]
  return out.to(q.dtype)
