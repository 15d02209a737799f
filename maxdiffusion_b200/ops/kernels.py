"""Thin, typed Python wrappers over the C entry points of `_kernels.so` (no autograd here).

Every function takes CUDA tensors, checks layout assumptions, launches on the current stream and
returns freshly allocated outputs. `maxdiffusion_b200.ops.functional` builds the differentiable ops
on top of these.
"""
from __future__ import annotations

import ctypes
import math
from typing import Sequence

import torch

from . import _lib

_EPI = {"none": 0, "gelu_tanh": 1, "gated_res": 2, "silu": 3, "add_res": 4}
_TARGET_CTAS = 148 * 4


def _ctas_per_batch(num_batches: int, rows_per_batch: int) -> int:
  return max(1, min(rows_per_batch, _TARGET_CTAS // max(1, num_batches)))


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
  return t if t.stride(-1) == 1 else t.contiguous()


_SM_COUNT = 148


def split_k_for(M: int, N: int, K: int, sms: int = _SM_COUNT) -> int:
  """How many ranges to cut the contraction into (1 = no split). A product whose output has fewer 128 x 256 tiles
  than the GPU has SMs leaves SMs idle for the whole contraction (weight gradients: K is the token count); splitting
  K makes more work items at the price of fp32 partials that a fold kernel sums. The model: waves of work items
  times k-blocks per item (about 0.4 us per k-block), plus the write and read of every partial at HBM speed."""
  tiles = -(-M // 128) * -(-N // 256)
  num_kb = -(-K // 64)
  if tiles * 2 > sms or num_kb < 16:
    return 1
  fold_us = M * N * 8 / 5e6  # one partial written and read, in microseconds at 5 TB/s
  best, best_cost = 1, -(-tiles // sms) * num_kb * 0.41
  for s in range(2, 33):
    per = -(-num_kb // s)
    if per < 4:
      break
    s_eff = -(-num_kb // per)
    cost = -(-tiles * s_eff // sms) * per * 0.41 + s_eff * fold_us + 2.0
    if cost < best_cost * 0.9:
      best, best_cost = s_eff, cost
  return best


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, bias=None, epi: str = "none",
         residual=None, gate=None, rows_per_batch: int = 0, out=None, out_dtype=torch.bfloat16, alpha: float = 1.0,
         split_k: int = 0):
  """D[M,N] = epi(alpha * A·Bᵀ + bias) on the tcgen05 GEMM. A: [M,K] (or [K,M] if a_mn); B: [N,K] (or [K,N]).
  `split_k`: 0 = chosen by `split_k_for` for plain products (no bias / epilogue), 1 = never, n = that many ranges."""
  assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
  a, b = _rowmajor(a), _rowmajor(b)
  K, M = (a.shape if a_mn else a.shape[::-1])
  Kb, N = (b.shape if b_mn else b.shape[::-1])
  assert K == Kb, f"contraction mismatch {a.shape} {b.shape} a_mn={a_mn} b_mn={b_mn}"
  if out is None:
    out = torch.empty((M, N), device=a.device, dtype=out_dtype)
  assert out.stride(-1) == 1 and out.shape == (M, N)
  if residual is not None:
    residual = _rowmajor(residual)
    assert residual.dtype == torch.bfloat16
  if gate is not None:
    assert gate.dtype == torch.float32 and gate.stride(-1) == 1
  if bias is not None:
    assert bias.dtype == torch.bfloat16 and bias.is_contiguous()
  plain = bias is None and epi == "none" and residual is None and gate is None
  splits = (split_k_for(M, N, K) if split_k == 0 else split_k) if plain else 1
  if splits > 1:
    partial = torch.empty((splits, -(-M // 128) * 128, N), device=a.device, dtype=torch.float32)  # splits a whole tile apart
    rc = _lib.lib().mdb_gemm_bf16_splitk(_lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0),
                                         out.stride(0), int(a_mn), int(b_mn), int(out.dtype == torch.float32), float(alpha),
                                         _lib.ptr(partial), splits, _lib.stream())
    _lib.check(rc, "mdb_gemm_bf16_splitk")
    return out
  rc = _lib.lib().mdb_gemm_bf16(
      _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(residual), _lib.ptr(gate), M, N, K,
      a.stride(0), b.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
      gate.stride(0) if gate is not None and gate.dim() == 2 else 0, rows_per_batch, int(a_mn), int(b_mn), _EPI[epi],
      int(out.dtype == torch.float32), float(alpha), _lib.stream())
  _lib.check(rc, "mdb_gemm_bf16")
  return out


def gemm_epilogue_mode(direct: bool = False) -> None:
  """True pins the direct-store epilogue (16-byte stores from one thread per row); False restores the default
  (128-byte slabs staged in shared memory and written by TMA stores). For benchmarks and tests."""
  _lib.check(_lib.lib().mdb_gemm_epilogue_mode(int(direct)), "mdb_gemm_epilogue_mode")


def gemm_force_tile_n(bn: int = 0) -> None:
  """Tile width of the bf16 GEMM: 0 is the default (256), 128 / 256 pin it (tile search, benchmarks, tests)."""
  _lib.check(_lib.lib().mdb_gemm_force_tile_n(int(bn)), "mdb_gemm_force_tile_n")


FLASH_HEAD_DIMS = (64, 128)


def _flash_entry(name: str, D: int):
  """The C entry point of an attention kernel for head_dim D (128: `name`, 64: `name_d64`)."""
  if D not in FLASH_HEAD_DIMS:
    raise ValueError(f"the flash-attention kernels are built for head_dim {FLASH_HEAD_DIMS}, got {D}")
  return getattr(_lib.lib(), name if D == 128 else name + "_d64")


# ---------------------------------------------------------------------------------------------
# launch shapes chosen by the tile search (`utils/tile_size_grid_search.py`): {(q_len, head_dim, heads, segments):
# (kv_stages, copy_ctas)}; `flash_fwd` applies the entry of its shape before it launches
# ---------------------------------------------------------------------------------------------
_FLASH_TUNED: dict = {}
_FLASH_CURRENT = (0, 0)


def flash_tune(kv_stages: int = 0, copy_ctas: int = 0) -> None:
  """Pins the launch shape of the attention forward: K / V pipeline stages (2..5, 0 = default 4) and the number of
  copy CTAs of a context-parallel launch (0 = automatic)."""
  global _FLASH_CURRENT
  _lib.check(_lib.lib().mdb_flash_fwd_tune(int(kv_stages), int(copy_ctas)), "mdb_flash_fwd_tune")
  _FLASH_CURRENT = (int(kv_stages), int(copy_ctas))


def flash_last_variant() -> tuple:
  a, b = ctypes.c_int(0), ctypes.c_int(0)
  _lib.lib().mdb_flash_fwd_last_variant(ctypes.byref(a), ctypes.byref(b))
  return a.value, b.value


def flash_tuned_key(q_len: int, head_dim: int, heads: int, segments: int) -> str:
  return f"flash:{q_len}:{head_dim}:{heads}:{segments}"


def load_flash_tuning(path: str) -> int:
  """Reads the tile-search cache (`tile_search_cache.json`) and registers its attention entries. Returns how many."""
  import json
  import os

  if not path or not os.path.exists(path):
    return 0
  with open(path) as f:
    data = json.load(f)
  n = 0
  for key, c in data.items():
    if key.startswith("flash:"):
      _FLASH_TUNED[key] = (int(c.get("stages", 0)), int(c.get("copy_ctas", 0)))
      n += 1
  return n


def flash_fwd(q: torch.Tensor, k_list: Sequence[torch.Tensor], v_list: Sequence[torch.Tensor], scale: float | None = None,
              return_lse: bool = True, seg_flags: torch.Tensor | None = None, flag_target: int = 0, plan=None,
              fixed_m=None):
  """Flash attention forward over KV segments. q: [B,Sq,H,D]; k/v: lists of [B,Skv_i,H,D] sharing strides; D is 64 or 128.

  `seg_flags` gates segment i on flags[i] >= flag_target; `plan` (an `_lib.CopyPlan`) adds copy CTAs that stage
  the remote segments from peer memory inside the same launch. `fixed_m` = (m_fixed fp32 [B,H,Sq] in the log2
  domain, fixed_heads int32 [H]) switches the marked heads to the fixed-exponent softmax (`ops.fixed_m`)."""
  if isinstance(k_list, torch.Tensor):
    k_list, v_list = [k_list], [v_list]
  B, Sq, H, D = q.shape
  assert D in FLASH_HEAD_DIMS and q.dtype == torch.bfloat16 and q.stride(-1) == 1
  if _FLASH_TUNED:
    want = _FLASH_TUNED.get(flash_tuned_key(Sq, D, H, len(k_list)), (0, 0))  # shapes without an entry: the default
    if want != _FLASH_CURRENT:
      flash_tune(*want)
  k0, v0 = k_list[0], v_list[0]
  for k, v in zip(k_list, v_list):
    assert k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    assert k.stride() == k0.stride() and v.stride() == v0.stride() and k.stride(-1) == 1 and v.stride(-1) == 1
  n = len(k_list)
  out = torch.empty((B, Sq, H, D), device=q.device, dtype=torch.bfloat16)
  lse = torch.empty((B, H, Sq), device=q.device, dtype=torch.float32) if return_lse else None
  kp = (ctypes.c_void_p * n)(*[k.data_ptr() for k in k_list])
  vp = (ctypes.c_void_p * n)(*[v.data_ptr() for v in v_list])
  lens = (ctypes.c_int * n)(*[k.shape[1] for k in k_list])
  scale = scale if scale is not None else 1.0 / math.sqrt(D)
  args = (_lib.ptr(q), kp, vp, _lib.ptr(out), _lib.ptr(lse), B, H, Sq, n, lens,
          q.stride(0), q.stride(1), q.stride(2), k0.stride(0), k0.stride(1), k0.stride(2),
          v0.stride(0), v0.stride(1), v0.stride(2), out.stride(0), out.stride(1), out.stride(2),
          float(scale), _lib.ptr(seg_flags), int(flag_target), ctypes.byref(plan) if plan is not None else None,
          _lib.stream())
  if fixed_m is None:
    rc = _flash_entry("mdb_flash_fwd", D)(*args)
  else:
    m_fixed, fixed_heads = fixed_m
    assert m_fixed.dtype == torch.float32 and m_fixed.shape == (B, H, Sq) and m_fixed.is_contiguous()
    assert fixed_heads.dtype == torch.int32 and fixed_heads.shape == (H,) and fixed_heads.is_contiguous()
    rc = _flash_entry("mdb_flash_fwd_fixed_m", D)(*args, _lib.ptr(m_fixed), _lib.ptr(fixed_heads))
  _lib.check(rc, "mdb_flash_fwd")
  return (out, lse) if return_lse else out


def flash_fwd_scatter(q, k_list, v_list, peer_out_ptrs, rows_per_rank: int, heads_total: int, head_off: int,
                      scale: float | None = None, seg_flags=None, flag_target: int = 0, plan=None) -> None:
  """Attention forward (head_dim 128) whose epilogue stores the output rows straight into the ranks that own them:
  query row r of this launch is row r % rows_per_rank of rank r // rows_per_rank, whose tensor at `peer_out_ptrs[rank]`
  is [B, rows_per_rank, heads_total, 128]; this launch's head h becomes head head_off + h there. The reverse
  head <-> sequence exchange of Ulysses attention then needs no kernel of its own. Nothing is returned."""
  if isinstance(k_list, torch.Tensor):
    k_list, v_list = [k_list], [v_list]
  B, Sq, H, D = q.shape
  assert D == 128 and q.dtype == torch.bfloat16 and q.stride(-1) == 1
  k0, v0 = k_list[0], v_list[0]
  for k, v in zip(k_list, v_list):
    assert k.stride() == k0.stride() and v.stride() == v0.stride() and k.stride(-1) == 1 and v.stride(-1) == 1
  n = len(k_list)
  kp = (ctypes.c_void_p * n)(*[k.data_ptr() for k in k_list])
  vp = (ctypes.c_void_p * n)(*[v.data_ptr() for v in v_list])
  lens = (ctypes.c_int * n)(*[k.shape[1] for k in k_list])
  sc = _lib.OutScatter()
  sc.n, sc.rows_per_rank, sc.head_off = len(peer_out_ptrs), int(rows_per_rank), int(head_off)
  for i, p in enumerate(peer_out_ptrs):
    sc.ptrs[i] = int(p)
  scale = scale if scale is not None else 1.0 / math.sqrt(D)
  rc = _lib.lib().mdb_flash_fwd_scatter(
      _lib.ptr(q), kp, vp, B, H, Sq, n, lens, q.stride(0), q.stride(1), q.stride(2), k0.stride(0), k0.stride(1), k0.stride(2),
      v0.stride(0), v0.stride(1), v0.stride(2), rows_per_rank * heads_total * D, heads_total * D, D, float(scale),
      _lib.ptr(seg_flags), int(flag_target), ctypes.byref(plan) if plan is not None else None, ctypes.byref(sc), _lib.stream())
  _lib.check(rc, "mdb_flash_fwd_scatter")


def rms_rope_scatter(x, peer_ptrs, me: int, w=None, cos=None, sin=None, mode: str = "row", eps: float = 1e-6) -> None:
  """RMSNorm (+ RoPE) of x [B, S, C] whose stores ARE the Ulysses exchange: head h of row (b, s) lands in rank
  h // (H / n)'s buffer [B, n S, H / n, 128] at position me * S + s. `mode`: "row" (RMS over all C channels), "head"
  (per 128-channel head) or "copy" (no normalisation: the value projection)."""
  B, S, C = x.shape
  assert x.dtype == torch.bfloat16 and x.stride(-1) == 1 and x.stride(0) == S * x.stride(1)
  group = {"row": C, "head": 128, "copy": 0}[mode]
  if cos is not None:
    assert cos.dtype == torch.float32 and cos.shape == (S, 64) and cos.is_contiguous() and sin.is_contiguous()
  arr = (ctypes.c_ulonglong * len(peer_ptrs))(*[int(p) for p in peer_ptrs])
  rc = _lib.lib().mdb_rms_rope_fwd_scatter(_lib.ptr(x), x.stride(1), _lib.ptr(w), int(mode == "head"), _lib.ptr(cos), _lib.ptr(sin),
                                           B, S, C, group, float(eps), arr, len(peer_ptrs), int(me), _ctas_per_batch(B, S),
                                           _lib.stream())
  _lib.check(rc, "mdb_rms_rope_fwd_scatter")


def _strides3(t):
  return (ctypes.c_longlong * 3)(t.stride(0), t.stride(1), t.stride(2))


def flash_delta(o, d_o):
  """delta[b,h,s] = sum_d dO*O (fp32), the row term of the softmax backward."""
  B, S, H, D = o.shape
  assert D in FLASH_HEAD_DIMS and o.stride(-1) == 1 and d_o.stride(-1) == 1
  delta = torch.empty((B, H, S), device=o.device, dtype=torch.float32)
  rc = _flash_entry("mdb_flash_delta", D)(_lib.ptr(o), _lib.ptr(d_o), _lib.ptr(delta), B, S, H, o.stride(0), o.stride(1),
                                  o.stride(2), d_o.stride(0), d_o.stride(1), d_o.stride(2), _lib.stream())
  _lib.check(rc, "mdb_flash_delta")
  return delta


def flash_bwd_dkv(q, d_o, k, v, lse, delta, scale=None, out_dtype=torch.bfloat16, dk=None, dv=None):
  """dK, dV of one KV segment [B,Skv,H,D] from the local queries q/dO [B,Sq,H,D]. `dk` / `dv` may be given
  (e.g. views of a symmetric buffer); they must be [B,Skv,H,D] with unit head_dim stride."""
  B, Sq, H, D = q.shape
  Skv = k.shape[1]
  assert D in FLASH_HEAD_DIMS and all(t.stride(-1) == 1 for t in (q, d_o, k, v))
  if dk is None:
    dk = torch.empty((B, Skv, H, D), device=q.device, dtype=out_dtype)
  if dv is None:
    dv = torch.empty((B, Skv, H, D), device=q.device, dtype=out_dtype)
  assert dk.shape == (B, Skv, H, D) and dv.shape == (B, Skv, H, D) and dk.dtype == out_dtype and dv.dtype == out_dtype
  scale = scale if scale is not None else 1.0 / math.sqrt(D)
  rc = _flash_entry("mdb_flash_bwd_dkv", D)(_lib.ptr(q), _lib.ptr(d_o), _lib.ptr(k), _lib.ptr(v), _lib.ptr(lse),
                                    _lib.ptr(delta), _lib.ptr(dk), _lib.ptr(dv), B, H, Sq, Skv, _strides3(q),
                                    _strides3(d_o), _strides3(k), _strides3(v), _strides3(dk), _strides3(dv),
                                    float(scale), int(out_dtype == torch.float32), _lib.stream())
  _lib.check(rc, "mdb_flash_bwd_dkv")
  return dk, dv


def flash_bwd_dkv_stacked(q, d_o, kg, vg, lens, lse, delta, scale=None, dk=None, dv=None, out_rot: int = 0,
                          out_step: int = 1, out_dtype=torch.bfloat16):
  """dK, dV of ALL stacked KV segments kg / vg [n, B, Skv, H, D] from the local queries in ONE launch (the segments
  ride the batch axis of the grid; a launch per 4k-token segment costs about half as much again).

  `lens[i]` are the valid rows of segment i. The result of segment i is written to dk[(out_rot + i * out_step) % n]
  (ring order -> owner order, whichever way the ring turns); dk / dv are [n, B, Skv, H, D] with any stride along the first axis (slices of a symmetric
  buffer) and are allocated when not given. Rows beyond lens[i] are left untouched."""
  n, B, Skv, H, D = kg.shape
  Sq = q.shape[1]
  assert D in FLASH_HEAD_DIMS and q.stride(-1) == 1 and d_o.stride(-1) == 1 and 1 <= n <= 8 and len(lens) == n
  for t in (kg, vg):
    assert t.stride(-1) == 1 and t.stride(0) == B * t.stride(1), "segments must be stacked with one batch stride"
  if dk is None:
    dk = torch.empty((n, B, Skv, H, D), device=q.device, dtype=out_dtype)
  if dv is None:
    dv = torch.empty((n, B, Skv, H, D), device=q.device, dtype=out_dtype)
  assert dk.shape == kg.shape and dv.shape == kg.shape and dk.dtype == out_dtype and dv.dtype == out_dtype
  assert dk.stride(0) == dv.stride(0) and dk.stride(-1) == 1 and dv.stride(-1) == 1
  scale = scale if scale is not None else 1.0 / math.sqrt(D)
  seg_lens = (ctypes.c_int * n)(*[int(x) for x in lens])
  rc = _flash_entry("mdb_flash_bwd_dkv_stacked", D)(
      _lib.ptr(q), _lib.ptr(d_o), _lib.ptr(kg), _lib.ptr(vg), _lib.ptr(lse), _lib.ptr(delta), _lib.ptr(dk), _lib.ptr(dv),
      B, H, Sq, Skv, _strides3(q), _strides3(d_o), _strides3(kg[0]), _strides3(vg[0]), _strides3(dk[0]), _strides3(dv[0]),
      float(scale), int(out_dtype == torch.float32), _lib.stream(), n, seg_lens, int(out_rot), int(out_step) % n,
      dk.stride(0))
  _lib.check(rc, "mdb_flash_bwd_dkv_stacked")
  return dk, dv


def flash_bwd_dq(q, d_o, k_list, v_list, lse, delta, scale=None, out_dtype=torch.bfloat16):
  """dQ of the local queries over every KV segment."""
  if isinstance(k_list, torch.Tensor):
    k_list, v_list = [k_list], [v_list]
  B, Sq, H, D = q.shape
  k0, v0 = k_list[0], v_list[0]
  for k, v in zip(k_list, v_list):
    assert k.stride() == k0.stride() and v.stride() == v0.stride() and k.stride(-1) == 1 and v.stride(-1) == 1
  n = len(k_list)
  dq = torch.empty((B, Sq, H, D), device=q.device, dtype=out_dtype)
  kp = (ctypes.c_void_p * n)(*[k.data_ptr() for k in k_list])
  vp = (ctypes.c_void_p * n)(*[v.data_ptr() for v in v_list])
  lens = (ctypes.c_int * n)(*[k.shape[1] for k in k_list])
  scale = scale if scale is not None else 1.0 / math.sqrt(D)
  rc = _flash_entry("mdb_flash_bwd_dq", D)(_lib.ptr(q), _lib.ptr(d_o), kp, vp, _lib.ptr(lse), _lib.ptr(delta), _lib.ptr(dq), B,
                                   H, Sq, n, lens, _strides3(q), _strides3(d_o), _strides3(k0), _strides3(v0),
                                   _strides3(dq), float(scale), int(out_dtype == torch.float32), _lib.stream())
  _lib.check(rc, "mdb_flash_bwd_dq")
  return dq


def ln_fwd(x, gamma=None, beta=None, scale=None, shift=None, eps=1e-6, save_stats=False):
  """x: [B,S,C] bf16 contiguous; scale/shift: fp32 [B,C] (row stride arbitrary)."""
  assert x.dtype == torch.bfloat16 and x.is_contiguous()
  B, S, C = x.shape
  y = torch.empty_like(x)
  mean = torch.empty((B, S), device=x.device, dtype=torch.float32) if save_stats else None
  rstd = torch.empty((B, S), device=x.device, dtype=torch.float32) if save_stats else None
  if scale is not None:
    assert scale.dtype == torch.float32 and shift.dtype == torch.float32
    assert scale.stride(-1) == 1 and shift.stride(-1) == 1 and scale.stride(0) == shift.stride(0)
  rc = _lib.lib().mdb_ln_fwd(_lib.ptr(x), _lib.ptr(y), _lib.ptr(gamma), _lib.ptr(beta), _lib.ptr(scale),
                             _lib.ptr(shift), scale.stride(0) if scale is not None else 0, B, S, C, float(eps),
                             _lib.ptr(mean), _lib.ptr(rstd), _ctas_per_batch(B, S), _lib.stream())
  _lib.check(rc, "mdb_ln_fwd")
  return (y, mean, rstd) if save_stats else y


def ln_bwd(dy, x, mean, rstd, gamma=None, scale=None, need_sums=True):
  """Returns dx and fp32 sums [B,2,C]: (sum dy*xhat, sum dy) per batch."""
  assert dy.is_contiguous() and x.is_contiguous()
  B, S, C = x.shape
  dx = torch.empty_like(x)
  cpb = _ctas_per_batch(B, S)
  sums = scratch = None
  if need_sums:
    sums = torch.empty((B, 2, C), device=x.device, dtype=torch.float32)
    scratch = torch.empty((B * cpb * 2 * C,), device=x.device, dtype=torch.float32)
  rc = _lib.lib().mdb_ln_bwd(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(gamma),
                             _lib.ptr(scale), scale.stride(0) if scale is not None else 0, B, S, C, _lib.ptr(dx),
                             _lib.ptr(sums), _lib.ptr(scratch), cpb, _lib.stream())
  _lib.check(rc, "mdb_ln_bwd")
  return dx, sums


def rms_rope_fwd(x, w=None, cos=None, sin=None, heads=1, per_head=False, eps=1e-6, save_stats=False):
  """x: [B,S,C] bf16 (row stride arbitrary, e.g. a slice of a fused QKV output) -> [B,S,H,D] contiguous."""
  B, S, C = x.shape
  assert x.dtype == torch.bfloat16 and x.stride(-1) == 1 and x.stride(0) == S * x.stride(1)
  y = torch.empty((B, S, C), device=x.device, dtype=torch.bfloat16)
  group = 128 if per_head else C
  rstd = None
  if save_stats:
    rstd = torch.empty((B, S, heads) if per_head else (B, S), device=x.device, dtype=torch.float32)
  if cos is not None:
    assert cos.dtype == torch.float32 and cos.shape == (S, 64) and cos.is_contiguous() and sin.is_contiguous()
  rc = _lib.lib().mdb_rms_rope_fwd(_lib.ptr(x), x.stride(1), _lib.ptr(y), C, _lib.ptr(w), int(per_head),
                                   _lib.ptr(cos), _lib.ptr(sin), B, S, C, group, float(eps), _lib.ptr(rstd),
                                   _ctas_per_batch(B, S), _lib.stream())
  _lib.check(rc, "mdb_rms_rope_fwd")
  y = y.view(B, S, heads, C // heads)
  return (y, rstd) if save_stats else y


def rms_rope_bwd(dy, x, rstd, w=None, cos=None, sin=None, per_head=False, need_dw=True):
  """dy: [B,S,H,D] (any strides with unit inner stride over [H*D]); returns dx [B,S,C] and dw fp32 [C]."""
  B, S, C = x.shape
  dy2 = dy.reshape(B, S, C) if dy.is_contiguous() else dy.contiguous().view(B, S, C)
  dx = torch.empty((B, S, C), device=x.device, dtype=torch.bfloat16)
  cpb = _ctas_per_batch(B, S)
  group = 128 if per_head else C
  dw = scratch = None
  if need_dw and w is not None:
    dw = torch.empty((C,), device=x.device, dtype=torch.float32)
    scratch = torch.empty((B * cpb * C,), device=x.device, dtype=torch.float32)
  rc = _lib.lib().mdb_rms_rope_bwd(_lib.ptr(dy2), C, _lib.ptr(x), x.stride(1), _lib.ptr(rstd), _lib.ptr(w),
                                   int(per_head), _lib.ptr(cos), _lib.ptr(sin), B, S, C, group, _lib.ptr(dx), C,
                                   _lib.ptr(dw), _lib.ptr(scratch), cpb, _lib.stream())
  _lib.check(rc, "mdb_rms_rope_bwd")
  if dw is not None and per_head:
    dw = dw.view(C // 128, 128).sum(0)
  return dx, dw


def gated_res_fwd(res, y, gate=None):
  assert res.is_contiguous() and y.is_contiguous() and res.dtype == torch.bfloat16
  B, S, C = res.shape
  out = torch.empty_like(res)
  rc = _lib.lib().mdb_gated_res_fwd(_lib.ptr(res), _lib.ptr(y), _lib.ptr(gate), gate.stride(0) if gate is not None else 0,
                                    B, S, C, _lib.ptr(out), _ctas_per_batch(B, S), _lib.stream())
  _lib.check(rc, "mdb_gated_res_fwd")
  return out


def gated_res_bwd(dout, y, gate):
  assert dout.is_contiguous() and y.is_contiguous()
  B, S, C = y.shape
  dy = torch.empty_like(y)
  cpb = _ctas_per_batch(B, S)
  dgate = torch.empty((B, C), device=y.device, dtype=torch.float32)
  scratch = torch.empty((B * cpb * C,), device=y.device, dtype=torch.float32)
  rc = _lib.lib().mdb_gated_res_bwd(_lib.ptr(dout), _lib.ptr(y), _lib.ptr(gate), gate.stride(0), B, S, C, _lib.ptr(dy),
                                    _lib.ptr(dgate), _lib.ptr(scratch), cpb, _lib.stream())
  _lib.check(rc, "mdb_gated_res_bwd")
  return dy, dgate


def colsum(x2d):
  """fp32 column sums of a bf16 [rows, C] matrix (bias gradient)."""
  assert x2d.dim() == 2 and x2d.stride(-1) == 1 and x2d.dtype == torch.bfloat16
  rows, C = x2d.shape
  ctas = max(1, min(rows, _TARGET_CTAS))
  out = torch.empty((C,), device=x2d.device, dtype=torch.float32)
  scratch = torch.empty((ctas * C,), device=x2d.device, dtype=torch.float32)
  rc = _lib.lib().mdb_colsum(_lib.ptr(x2d), x2d.stride(0), rows, C, _lib.ptr(out), _lib.ptr(scratch), ctas,
                             _lib.stream())
  _lib.check(rc, "mdb_colsum")
  return out


def gelu_fwd(u):
  assert u.is_contiguous() and u.dtype == torch.bfloat16
  y = torch.empty_like(u)
  _lib.check(_lib.lib().mdb_gelu_fwd(_lib.ptr(u), _lib.ptr(y), u.numel(), _lib.stream()), "mdb_gelu_fwd")
  return y


def gelu_bwd(dy, u):
  assert u.is_contiguous() and dy.is_contiguous()
  du = torch.empty_like(u)
  _lib.check(_lib.lib().mdb_gelu_bwd(_lib.ptr(dy), _lib.ptr(u), _lib.ptr(du), u.numel(), _lib.stream()),
             "mdb_gelu_bwd")
  return du


def geglu_fwd(u):
  """u [..., 2 * inner] bf16 (h | gate) -> h * gelu(gate) [..., inner] (exact GELU)."""
  assert u.is_contiguous() and u.dtype == torch.bfloat16 and u.shape[-1] % 16 == 0
  inner = u.shape[-1] // 2
  y = torch.empty((*u.shape[:-1], inner), dtype=u.dtype, device=u.device)
  _lib.check(_lib.lib().mdb_geglu_fwd(_lib.ptr(u), _lib.ptr(y), u.numel() // (2 * inner), inner, _lib.stream()), "mdb_geglu_fwd")
  return y


def geglu_bwd(dy, u):
  assert u.is_contiguous() and dy.is_contiguous() and dy.dtype == u.dtype == torch.bfloat16
  inner = u.shape[-1] // 2
  du = torch.empty_like(u)
  _lib.check(_lib.lib().mdb_geglu_bwd(_lib.ptr(dy), _lib.ptr(u), _lib.ptr(du), u.numel() // (2 * inner), inner, _lib.stream()),
             "mdb_geglu_bwd")
  return du


def adamw(p, g, m, v, *, lr, b1, b2, eps, wd, step, grad_scale=1.0, clip_value=0.0, seed=0, stochastic=True):
  """Fused in-place AdamW on flat buffers. p: bf16; g: bf16|fp32; m, v: bf16|fp32 (same dtype)."""
  assert p.dtype == torch.bfloat16 and p.is_contiguous() and g.is_contiguous() and m.is_contiguous()
  assert m.dtype == v.dtype and g.numel() == p.numel() == m.numel() == v.numel()
  rc = _lib.lib().mdb_adamw(_lib.ptr(p), _lib.ptr(g), _lib.ptr(m), _lib.ptr(v), p.numel(), float(lr), float(b1),
                            float(b2), float(eps), float(wd), float(1 - b1**step), float(1 - b2**step),
                            float(grad_scale), float(clip_value), int(seed) & (2**64 - 1), int(stochastic),
                            int(g.dtype == torch.float32), int(m.dtype == torch.float32), _lib.stream())
  _lib.check(rc, "mdb_adamw")


def sumsq_maxabs(x, out=None, accumulate=False):
  """out (fp32 [2]) = {sum x², max |x|}; with accumulate the result is folded into `out`."""
  assert x.is_contiguous()
  if out is None:
    out = torch.zeros((2,), device=x.device, dtype=torch.float32)
  scratch = torch.empty((2048,), device=x.device, dtype=torch.float32)
  rc = _lib.lib().mdb_sumsq_maxabs(_lib.ptr(x), x.numel(), int(x.dtype == torch.float32), _lib.ptr(out),
                                   _lib.ptr(scratch), int(accumulate), _lib.stream())
  _lib.check(rc, "mdb_sumsq_maxabs")
  return out


# ---------------------------------------------------------------------------------------------
# elementwise step family and GroupNorm
# ---------------------------------------------------------------------------------------------
def _declare_extra(L):
  c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
  L.mdb_lincomb.argtypes = [c_void_p, c_int, c_int, ctypes.POINTER(c_void_p), ctypes.POINTER(c_int),
                            ctypes.POINTER(c_float), c_int, c_ll, c_void_p, c_int, c_void_p]
  L.mdb_lincomb.restype = c_int
  L.mdb_mse_fwd_bwd.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, ctypes.POINTER(c_float), c_int, c_ll,
                                c_float, c_void_p, c_int, c_void_p]
  L.mdb_mse_fwd_bwd.restype = c_int
  L.mdb_channel_affine.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_ll, c_int, c_ll,
                                   c_void_p]
  L.mdb_channel_affine.restype = c_int
  L.mdb_to_uint8.argtypes = [c_void_p, c_int, c_void_p, c_ll, c_void_p]
  L.mdb_to_uint8.restype = c_int
  L.mdb_blend_ramp.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_ll, ctypes.POINTER(c_ll), c_int, c_ll, c_void_p]
  L.mdb_blend_ramp.restype = c_int
  L.mdb_groupnorm_fwd.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_ll,
                                  c_int, c_float, c_int, c_void_p, c_void_p, c_void_p]
  L.mdb_groupnorm_fwd.restype = c_int
  L.mdb_groupnorm_bwd.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                  c_int, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p]
  L.mdb_groupnorm_bwd.restype = c_int


_lib.register(_declare_extra)

_PARTIAL_BLOCKS = 148 * 4


def _is_f32(t):
  assert t.dtype in (torch.float32, torch.bfloat16), t.dtype
  return int(t.dtype == torch.float32)


def lincomb(xs: Sequence[torch.Tensor], coefs, out_dtype=None, out=None, want_sumsq: bool = False):
  """out = sum_i coefs[b][i] * xs[i]. `coefs` is [n_in] (shared) or [B][n_in] (per sample along dim 0).

  All inputs share one shape (bf16 or fp32 each). Returns out, or (out, sum(out^2) as a 0-d fp32 tensor)."""
  x0 = xs[0]
  n_in = len(xs)
  assert 1 <= n_in <= 6
  xs = [x if x.is_contiguous() else x.contiguous() for x in xs]
  for x in xs:
    assert x.shape == x0.shape
  rows = list(coefs) if isinstance(coefs[0], (list, tuple)) else [list(coefs)]
  B = len(rows)
  assert B <= 16 and (B == 1 or B == x0.shape[0])
  n = x0.numel()
  per_batch = n // B
  assert per_batch % 8 == 0, "element count per sample must be a multiple of 8"
  if out is None:
    out = torch.empty(x0.shape, device=x0.device, dtype=out_dtype or x0.dtype)
  assert out.is_contiguous()
  ptrs = (ctypes.c_void_p * n_in)(*[x.data_ptr() for x in xs])
  f32s = (ctypes.c_int * n_in)(*[_is_f32(x) for x in xs])
  flat = [float(c) for r in rows for c in r]
  cf = (ctypes.c_float * len(flat))(*flat)
  partial = torch.empty((_PARTIAL_BLOCKS,), device=x0.device, dtype=torch.float32) if want_sumsq else None
  rc = _lib.lib().mdb_lincomb(_lib.ptr(out), _is_f32(out), n_in, ptrs, f32s, cf, B, per_batch, _lib.ptr(partial),
                              _PARTIAL_BLOCKS, _lib.stream())
  _lib.check(rc, "mdb_lincomb")
  return (out, partial.sum()) if want_sumsq else out


def mse_fwd_bwd(pred, target, weights=None, need_grad: bool = True, grad_dtype=None):
  """loss = sum_b w_b * sum (pred-target)^2 / numel and d(loss)/d(pred) in one pass. Returns (loss, dpred)."""
  pred = pred if pred.is_contiguous() else pred.contiguous()
  target = target if target.is_contiguous() else target.contiguous()
  assert pred.shape == target.shape
  B = pred.shape[0] if weights is not None else 1
  w = [float(x) for x in weights] if weights is not None else [1.0]
  assert len(w) == B and B <= 16
  n = pred.numel()
  per_batch = n // B
  assert per_batch % 8 == 0
  dpred = torch.empty(pred.shape, device=pred.device, dtype=grad_dtype or pred.dtype) if need_grad else None
  partial = torch.empty((_PARTIAL_BLOCKS,), device=pred.device, dtype=torch.float32)
  wf = (ctypes.c_float * B)(*w)
  rc = _lib.lib().mdb_mse_fwd_bwd(_lib.ptr(pred), _is_f32(pred), _lib.ptr(target), _is_f32(target), _lib.ptr(dpred),
                                  _is_f32(dpred) if need_grad else 0, wf, B, per_batch, 2.0 / n, _lib.ptr(partial),
                                  _PARTIAL_BLOCKS, _lib.stream())
  _lib.check(rc, "mdb_mse_fwd_bwd")
  return partial.sum() / n, dpred


def channel_affine(x, mean, scale, channel_dim: int, denorm: bool = False, out_dtype=None):
  """(x - mean[c]) * scale[c], or x * scale[c] + mean[c] with `denorm`; c indexes `channel_dim`."""
  x = x if x.is_contiguous() else x.contiguous()
  C = x.shape[channel_dim]
  inner = 1
  for d in x.shape[channel_dim + 1:]:
    inner *= d
  out = torch.empty(x.shape, device=x.device, dtype=out_dtype or x.dtype)
  mean = mean.to(device=x.device, dtype=torch.float32).contiguous()
  scale = scale.to(device=x.device, dtype=torch.float32).contiguous()
  assert mean.numel() == C and scale.numel() == C
  rc = _lib.lib().mdb_channel_affine(_lib.ptr(x), _is_f32(x), _lib.ptr(out), _is_f32(out), _lib.ptr(mean),
                                     _lib.ptr(scale), C, inner, int(denorm), x.numel(), _lib.stream())
  _lib.check(rc, "mdb_channel_affine")
  return out


def to_uint8(x):
  """clamp(x/2 + 0.5, 0, 1) * 255, rounded to uint8."""
  x = x if x.is_contiguous() else x.contiguous()
  n = x.numel()
  assert n % 8 == 0
  out = torch.empty(x.shape, device=x.device, dtype=torch.uint8)
  _lib.check(_lib.lib().mdb_to_uint8(_lib.ptr(x), _is_f32(x), _lib.ptr(out), n, _lib.stream()), "mdb_to_uint8")
  return out


def blend_ramp(a, b, dim: int):
  """a * (1 - i/extent) + b * (i/extent) along `dim` (i the index along it); a and b are views of equal shape whose
  dims after `dim` are contiguous and whose dims before `dim` collapse to one stride."""
  assert a.shape == b.shape and a.dtype == b.dtype
  extent = a.shape[dim]
  inner = 1
  for d in a.shape[dim + 1:]:
    inner *= d
  outer = a.numel() // (extent * inner)

  def strides(t):
    tt = t.reshape(outer, extent, inner) if t.is_contiguous() else None
    if tt is None:
      tt = t.contiguous().reshape(outer, extent, inner)
    return tt, tt.stride(0), tt.stride(1)

  a3, ao, ae = strides(a)
  b3, bo, be = strides(b)
  out = torch.empty((outer, extent, inner), device=a.device, dtype=a.dtype)
  st = (ctypes.c_longlong * 6)(ao, bo, out.stride(0), ae, be, out.stride(1))
  rc = _lib.lib().mdb_blend_ramp(_lib.ptr(a3), _lib.ptr(b3), _lib.ptr(out), _is_f32(a), outer, st, extent, inner,
                                 _lib.stream())
  _lib.check(rc, "mdb_blend_ramp")
  return out.reshape(a.shape)


def _gn_splits(N, C, hw):
  rows = N * C
  s = max(1, min((_TARGET_CTAS + rows - 1) // rows, hw // 2048))
  return int(min(s, 64))


def groupnorm_fwd(x, groups, gamma=None, beta=None, eps=1e-6, act: bool = False, save_stats: bool = True):
  """GroupNorm over [N, C, *spatial] (contiguous), optional fused SiLU. Returns (y, mean_rstd [N, G, 2] or None)."""
  assert x.is_contiguous()
  N, C = x.shape[:2]
  hw = x.numel() // (N * C)
  S = _gn_splits(N, C, hw)
  y = torch.empty_like(x)
  partial = torch.empty((N * C * S, 2), device=x.device, dtype=torch.float32)
  stats = torch.empty((N, groups, 2), device=x.device, dtype=torch.float32) if save_stats else None
  g32 = gamma.float().contiguous() if gamma is not None else None
  b32 = beta.float().contiguous() if beta is not None else None
  rc = _lib.lib().mdb_groupnorm_fwd(_lib.ptr(x), _is_f32(x), _lib.ptr(y), _is_f32(y), _lib.ptr(g32), _lib.ptr(b32), N, C,
                                    groups, hw, S, float(eps), int(act), _lib.ptr(partial), _lib.ptr(stats),
                                    _lib.stream())
  _lib.check(rc, "mdb_groupnorm_fwd")
  return y, stats


def groupnorm_bwd(dy, x, stats, groups, gamma=None, beta=None, act: bool = False):
  """Returns (dx, dgamma fp32 [C], dbeta fp32 [C])."""
  assert x.is_contiguous()
  dy = dy if dy.is_contiguous() else dy.contiguous()
  N, C = x.shape[:2]
  hw = x.numel() // (N * C)
  S = _gn_splits(N, C, hw)
  dx = torch.empty_like(x)
  partial = torch.empty((N, C, S, 2), device=x.device, dtype=torch.float32)
  g32 = gamma.float().contiguous() if gamma is not None else None
  b32 = beta.float().contiguous() if beta is not None else None
  rc = _lib.lib().mdb_groupnorm_bwd(_lib.ptr(dy), _is_f32(dy), _lib.ptr(x), _is_f32(x), _lib.ptr(dx), _is_f32(dx),
                                    _lib.ptr(g32), _lib.ptr(b32), N, C, groups, hw, S, int(act), _lib.ptr(stats),
                                    _lib.ptr(partial), _lib.stream())
  _lib.check(rc, "mdb_groupnorm_bwd")
  sums = partial.sum(dim=(0, 2))
  return dx, sums[:, 1], sums[:, 0]


# ---------------------------------------------------------------------------------------------
# fp8 GEMM with per-tensor absmax scales
# ---------------------------------------------------------------------------------------------
def _declare_fp8(L):
  c_void_p, c_int, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
  L.mdb_gemm_fp8.argtypes = [c_void_p] * 6 + [c_int] * 3 + [c_ll] * 3 + [c_int, c_int, c_void_p]
  L.mdb_gemm_fp8.restype = c_int
  L.mdb_quantize_fp8.argtypes = [c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_int, c_void_p]
  L.mdb_quantize_fp8.restype = c_int
  L.mdb_gemm_int8.argtypes = [c_void_p] * 6 + [c_int] * 3 + [c_ll] * 3 + [c_void_p]
  L.mdb_gemm_int8.restype = c_int
  L.mdb_quantize_int8.argtypes = [c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p]
  L.mdb_quantize_int8.restype = c_int


_lib.register(_declare_fp8)


def quantize_fp8(x: torch.Tensor, e5m2: bool = False):
  """Per-tensor absmax quantisation of a bf16 tensor. Returns (q uint8 same shape, scale fp32 [1] on device) with
  x ~= q * scale; no host synchronisation."""
  assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 8 == 0
  stats = sumsq_maxabs(x)
  q = torch.empty(x.shape, device=x.device, dtype=torch.uint8)
  scale = torch.empty((1,), device=x.device, dtype=torch.float32)
  rc = _lib.lib().mdb_quantize_fp8(_lib.ptr(x), _lib.ptr(q), x.numel(), _lib.ptr(stats), _lib.ptr(scale), int(e5m2),
                                   _lib.stream())
  _lib.check(rc, "mdb_quantize_fp8")
  return q, scale


def gemm_fp8(aq, a_scale, bq, b_scale, bias=None, a_e5m2: bool = False, b_e5m2: bool = False):
  """bf16 D[M,N] = (a_scale * b_scale) * Aq[M,K] · Bq[N,K]ᵀ + bias on the fp8 tensor-core path (K % 16 == 0)."""
  assert aq.dtype == torch.uint8 and bq.dtype == torch.uint8 and aq.dim() == 2 and bq.dim() == 2
  assert aq.stride(-1) == 1 and bq.stride(-1) == 1 and aq.shape[1] == bq.shape[1]
  M, K = aq.shape
  N = bq.shape[0]
  out = torch.empty((M, N), device=aq.device, dtype=torch.bfloat16)
  rc = _lib.lib().mdb_gemm_fp8(_lib.ptr(aq), _lib.ptr(bq), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(a_scale),
                               _lib.ptr(b_scale), M, N, K, aq.stride(0), bq.stride(0), out.stride(0), int(a_e5m2),
                               int(b_e5m2), _lib.stream())
  _lib.check(rc, "mdb_gemm_fp8")
  return out


def quantize_int8(x: torch.Tensor):
  """Symmetric per-tensor int8 quantisation of a bf16 tensor: (q int8 same shape, scale fp32 [1] on device) with
  x ~= q * scale and q in [-127, 127]; no host synchronisation."""
  assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 8 == 0
  stats = sumsq_maxabs(x)
  q = torch.empty(x.shape, device=x.device, dtype=torch.int8)
  scale = torch.empty((1,), device=x.device, dtype=torch.float32)
  rc = _lib.lib().mdb_quantize_int8(_lib.ptr(x), _lib.ptr(q), x.numel(), _lib.ptr(stats), _lib.ptr(scale), _lib.stream())
  _lib.check(rc, "mdb_quantize_int8")
  return q, scale


def gemm_int8(aq, a_scale, bq, b_scale, bias=None):
  """bf16 D[M,N] = (a_scale * b_scale) * Aq[M,K] · Bq[N,K]ᵀ + bias with int8 operands and exact int32 accumulation
  (tcgen05 kind::i8; K % 16 == 0)."""
  assert aq.dtype == torch.int8 and bq.dtype == torch.int8 and aq.dim() == 2 and bq.dim() == 2
  assert aq.stride(-1) == 1 and bq.stride(-1) == 1 and aq.shape[1] == bq.shape[1]
  M, K = aq.shape
  N = bq.shape[0]
  out = torch.empty((M, N), device=aq.device, dtype=torch.bfloat16)
  rc = _lib.lib().mdb_gemm_int8(_lib.ptr(aq), _lib.ptr(bq), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(a_scale),
                                _lib.ptr(b_scale), M, N, K, aq.stride(0), bq.stride(0), out.stride(0), _lib.stream())
  _lib.check(rc, "mdb_gemm_int8")
  return out


# ---------------------------------------------------------------------------------------------
# anti-aliased snake activation (vocoder)
# ---------------------------------------------------------------------------------------------
def _declare_snake(L):
  c_void_p, c_int, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
  fp = ctypes.POINTER(ctypes.c_float)
  L.mdb_snake_aa.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, fp, fp, c_ll, c_int, c_int, c_int, c_void_p]
  L.mdb_snake_aa.restype = c_int


_lib.register(_declare_snake)


def snake_aa(x, alpha, inv_beta, f_up, f_dn, leaky_slope: float | None = None):
  """Anti-aliased activation over [B, C, L]: 2x up-sample, snake(alpha, 1/beta) (or leaky ReLU), 2x down-sample.
  alpha / inv_beta: fp32 [C] on the device; f_up / f_dn: 12 filter taps each (host sequences)."""
  assert x.dim() == 3 and x.is_contiguous() and x.dtype in (torch.float32, torch.bfloat16)
  B, C, L = x.shape
  out = torch.empty_like(x)
  up = (ctypes.c_float * 12)(*[float(v) for v in f_up])
  dn = (ctypes.c_float * 12)(*[float(v) for v in f_dn])
  mode = 0 if leaky_slope is None else 1
  if mode == 1:
    alpha = torch.full((1,), float(leaky_slope), device=x.device, dtype=torch.float32)
    inv_beta = alpha
  rows, step = B * C, 65535
  xf, of = x.view(rows, L), out.view(rows, L)
  for r0 in range(0, rows, step):
    n = min(step, rows - r0)
    if r0 % C != 0 and mode == 0:
      raise ValueError("row chunks must start on a channel boundary")
    rc = _lib.lib().mdb_snake_aa(_lib.ptr(xf[r0:r0 + n]), _lib.ptr(of[r0:r0 + n]), _is_f32(x), _lib.ptr(alpha), _lib.ptr(inv_beta),
                                 up, dn, n, C, L, mode, _lib.stream())
    _lib.check(rc, "mdb_snake_aa")
  return out
