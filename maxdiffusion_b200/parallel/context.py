"""Context (sequence) parallelism for self-attention: gather/ring, Ulysses, and 2-D Ulysses x ring.

Strategy names follow the reference's attention-kernel registry
(src/maxdiffusion/models/attention_flax.py:1589-1867; dispatch in `common_types.ATTENTION_KERNELS`):

  gather / ring : every rank keeps its query shard; the K/V shards of all ranks are presented to ONE flash
                  kernel launch as KV segments, so the running (O, m, l) never leaves the SM between hops (the
                  reference merges per-hop partial results through HBM, ring_attention_kernel.py:1099-1131).
                  Backward: dQ over all segments in one launch, dK/dV per segment, then a reduce-scatter returns
                  the partial sums to the owners (reference: ring_attention_kernel.py:181-289).
  ulysses       : all-to-all heads <-> sequence, local full-sequence attention on H/U heads, all-to-all back
                  (reference: attention_flax.py:817-1061).
  usp           : Ulysses inside `ulysses` groups, gather/ring across `ring` groups (reference: :1064-1254).

Cross-attention never communicates: K/V are the 512 text tokens, replicated (reference: :2405-2437).
This module is the NCCL baseline; `parallel.symm` provides the peer-memory transport used on NVLink.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import fixed_m as FM
from ..ops import functional as OF
from ..ops import kernels as K
from . import collectives as C


class _GatherSeq(torch.autograd.Function):
  """all-gather along a new leading axis; backward returns each owner the sum of the partial gradients."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return C.all_gather_stack(x, group)

  @staticmethod
  def backward(ctx, g):
    return C.reduce_scatter_stack(g.contiguous(), ctx.group), None


def _a2a(x, group, exch, to_seq: bool):
  """One Ulysses exchange: over peer memory when an exchange object is given and the tensor qualifies, else NCCL."""
  if exch is not None and exch.supports(x, exch.n) and x.numel() <= exch.numel:
    x = x.contiguous()
    return exch.heads_to_seq(x) if to_seq else exch.seq_to_heads(x)
  return C.all_to_all_heads_to_seq(x, group) if to_seq else C.all_to_all_seq_to_heads(x, group)


class _HeadsToSeq(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, group, exch=None):
    ctx.group, ctx.exch = group, exch
    return _a2a(x, group, exch, True)

  @staticmethod
  def backward(ctx, g):
    return _a2a(g.contiguous(), ctx.group, ctx.exch, False), None, None


class _SeqToHeads(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, group, exch=None):
    ctx.group, ctx.exch = group, exch
    return _a2a(x, group, exch, False)

  @staticmethod
  def backward(ctx, g):
    return _a2a(g.contiguous(), ctx.group, ctx.exch, True), None, None


def _stackable(kg, vg, order):
  """(rot, step) when the gathered K/V [n, B, S, H, D] can ride one dK/dV launch, else None: stacked with a single
  batch stride, and segment i belongs to owner (rot + i * step) % n (the ring order, whichever way it turns)."""
  n, B = kg.shape[0], kg.shape[1]
  if not all(t.stride(-1) == 1 and t.stride(0) == B * t.stride(1) for t in (kg, vg)):
    return None
  rot = order[0]
  step = (order[1] - order[0]) % n if n > 1 else 0
  if any(order[i] != (rot + i * step) % n for i in range(n)):
    return None
  return rot, step


def ulysses_head_chunks(heads: int, shards: int, chunks: int) -> list:
  """Half-open head ranges for the chunked Ulysses exchange: every range is a whole number of `shards`-sized head
  groups (each chunk is exchanged on its own, so it must split evenly over the shards); the groups are dealt out
  floor(groups / chunks) per chunk and the last chunk takes the rest. One range when `chunks` <= 1.
  (reference: `_ulysses_head_chunk_ranges`, src/maxdiffusion/models/attention_flax.py:483-520)"""
  if chunks <= 1:
    return [(0, heads)]
  if heads % shards:
    raise ValueError(f"Ulysses needs heads ({heads}) divisible by the shard count ({shards})")
  groups = heads // shards
  chunks = min(chunks, groups)
  per = max(1, groups // chunks)
  bounds = [min(i * per, groups) for i in range(chunks)] + [groups]
  return [(a * shards, b * shards) for a, b in zip(bounds, bounds[1:]) if b > a]


class _SegmentAttentionFn(torch.autograd.Function):
  """Kernel path of gather/ring attention: local q against the stacked K/V shards [n, B, S_loc, H, D]."""

  @staticmethod
  def forward(ctx, q, k, v, scale, group, valid_lens, exchange, reducer=None, fixed_m=None, save_kv=True):
    state = OF._remat
    saved = None
    if state.mode == "replay":
      saved = state.store[state.cursor]
      state.cursor += 1
    flags, epoch, plan, keep = None, 0, None, None
    if exchange is not None:
      # peer-memory transport: segments in ring order (own shard first)
      order = exchange.order()
      if saved is None:
        kg, vg, flags, epoch, plan, keep = exchange.plan(k.contiguous(), v.contiguous())
      else:
        kg, vg = exchange.gather(k.contiguous(), v.contiguous())
    else:
      kg = C.all_gather_stack(k, group)
      vg = C.all_gather_stack(v, group)
      order = list(range(kg.shape[0]))
    n = kg.shape[0]
    lens = tuple(valid_lens[r] for r in order)
    ks = [kg[i][:, :lens[i]] for i in range(n)]
    vs = [vg[i][:, :lens[i]] for i in range(n)]
    if saved is not None:
      out, lse = saved
    else:
      # with a plan the copy CTAs of this launch stage the remote segments while the math starts on the own one
      out, lse = K.flash_fwd(q, ks, vs, scale, seg_flags=flags, flag_target=epoch, plan=plan, fixed_m=fixed_m)
      if state.mode == "record":
        state.store.append((out, lse))
    ctx.scale, ctx.group, ctx.valid_lens, ctx.order, ctx.reducer = scale, group, lens, order, reducer
    ctx.save_kv, ctx.exchange = save_kv, exchange
    if save_kv:
      ctx.save_for_backward(q, out, lse, kg, vg)
    else:
      # only this rank's shard waits for the backward pass: the K/V memory of a layer then shrinks with the context
      # axis; the other shards are fetched again when the backward needs them
      ctx.save_for_backward(q, out, lse, k, v)
    return out

  @staticmethod
  def backward(ctx, d_o):
    q, out, lse, kg, vg = ctx.saved_tensors
    if not ctx.save_kv:
      if ctx.exchange is not None:
        kg, vg = ctx.exchange.gather(kg.contiguous(), vg.contiguous())
      else:
        kg, vg = C.all_gather_stack(kg, ctx.group), C.all_gather_stack(vg, ctx.group)
    n = kg.shape[0]
    lens = ctx.valid_lens
    if d_o.stride(-1) != 1:
      d_o = d_o.contiguous()
    ks = [kg[i][:, :lens[i]] for i in range(n)]
    vs = [vg[i][:, :lens[i]] for i in range(n)]
    delta = K.flash_delta(out, d_o)
    rs = ctx.reducer
    if rs is not None:
      # peer-memory return of the partials: the dK/dV kernels write the partial for owner r straight into slice r of
      # a symmetric buffer ([dK | dV] per owner), and every owner pulls and sums its slice with one kernel. That
      # kernel is bound by NVLink, so it runs on a side stream underneath the dQ kernel.
      shape = (2,) + tuple(kg.shape[1:])
      parts = rs.slices(shape)
      for i in range(n):
        if lens[i] < kg.shape[2]:  # pad rows of a ragged shard: no kernel writes them, the owner sums them
          parts[ctx.order[i]][:, :, lens[i]:].zero_()
      ring = _stackable(kg, vg, ctx.order)
      if ring is not None:
        both_parts = rs.stacked()  # [owner, 2, B, S, H, D]
        K.flash_bwd_dkv_stacked(q, d_o, kg, vg, lens, lse, delta, ctx.scale, dk=both_parts[:, 0], dv=both_parts[:, 1],
                                out_rot=ring[0], out_step=ring[1])
      else:
        for i in range(n):
          part = parts[ctx.order[i]]
          K.flash_bwd_dkv(q, d_o, ks[i], vs[i], lse, delta, ctx.scale, dk=part[0][:, :lens[i]], dv=part[1][:, :lens[i]])
      main = torch.cuda.current_stream()
      produced = torch.cuda.Event()
      produced.record(main)
      with torch.cuda.stream(rs.stream):
        rs.stream.wait_event(produced)
        both = rs.reduce()
        reduced = torch.cuda.Event()
        reduced.record(rs.stream)
      dq = K.flash_bwd_dq(q, d_o, ks, vs, lse, delta, ctx.scale)
      main.wait_event(reduced)
      both.record_stream(main)
      return dq, both[0], both[1], None, None, None, None, None, None, None
    dq = K.flash_bwd_dq(q, d_o, ks, vs, lse, delta, ctx.scale)
    dkg, dvg = torch.empty_like(kg), torch.empty_like(vg)
    for i in range(n):
      if lens[i] < kg.shape[2]:  # pad rows of a ragged shard: no kernel writes them, the reduce-scatter sums them
        dkg[ctx.order[i]][:, lens[i]:].zero_()
        dvg[ctx.order[i]][:, lens[i]:].zero_()
    ring = _stackable(kg, vg, ctx.order)
    if ring is not None:
      # partial gradients are stored by OWNER rank so that the reduce-scatter returns each owner its sum
      K.flash_bwd_dkv_stacked(q, d_o, kg, vg, lens, lse, delta, ctx.scale, dk=dkg, dv=dvg, out_rot=ring[0],
                              out_step=ring[1])
    else:
      for i in range(n):
        dk, dv = K.flash_bwd_dkv(q, d_o, ks[i], vs[i], lse, delta, ctx.scale)
        dkg[ctx.order[i]][:, :lens[i]].copy_(dk)
        dvg[ctx.order[i]][:, :lens[i]].copy_(dv)
    dk = C.reduce_scatter_stack(dkg, ctx.group)
    dv = C.reduce_scatter_stack(dvg, ctx.group)
    return dq, dk, dv, None, None, None, None, None, None, None


class ContextParallel:
  """Sequence sharding + the self-attention strategy of one rank.

  `mesh` is a `parallel.mesh.DeviceMesh`; `strategy` one of local / gather / ring / ulysses / usp.
  """

  def __init__(self, mesh, strategy: str = "ring", peer_memory: bool = False, fixed_m: bool = False,
               save_remote_kv: bool = True, ulysses_chunks: int = 1, kv_transport: str = "sm"):
    self.mesh = mesh
    # ring K/V over peer memory: "sm" stages the remote shards with copy CTAs of the attention launch itself, "dma" with
    # copy-engine copies and stream memory operations on a side stream (every CTA of the launch then computes)
    self.kv_transport = kv_transport
    self.strategy = strategy
    self.peer_memory = peer_memory
    # Ulysses: exchange and attend in this many head-group chunks (`ulysses_attention_chunks`), so that the exchange
    # of one chunk can run beside the attention of another; forwards outside autograd over peer memory fold the
    # exchanges into the producer / consumer kernels instead and ignore it
    self.ulysses_chunks = max(1, int(ulysses_chunks))
    # ring / gather attention: keep every rank's K/V of a layer for its backward (fastest), or keep the own shard only
    # and fetch the others again in the backward (K/V memory per layer then falls with the context axis)
    self.save_remote_kv = save_remote_kv
    # fixed-exponent softmax (`ops.fixed_m`): keys are smoothed where a rank sees the whole key sequence (local,
    # Ulysses); ring segments stay unsmoothed and take the halved gate, with the key norms max-reduced over the ring
    self.fixed_m = fixed_m
    self._exchanges: dict = {}
    self._peers: dict = {}
    self._reducers: dict = {}
    self._a2as: dict = {}
    self._fused: dict = {}
    self.group = mesh.group("context")
    self.size = mesh.size("context")
    self.rank = mesh.index_in("context") if self.size > 1 else 0
    self.ulysses_group = mesh.group("ulysses")
    self.ring_group = mesh.group("ring")
    self.ulysses_size = len(mesh.ranks("ulysses"))
    self.ring_size = len(mesh.ranks("ring"))
    self.ring_rank = mesh.index_in("ring") if self.ring_size > 1 else 0
    self.full_len: Optional[int] = None
    self.local_len: Optional[int] = None

  def _exchange_for(self, group, k):
    """The peer-memory K/V transport of `group` (created on first use), or None for the NCCL path."""
    if not self.peer_memory or group is None:
      return None
    key = id(group)
    ex = self._exchanges.get(key)
    if ex is None or ex.numel < k.numel():
      from . import symm

      if not symm.peer_memory_available(group):
        self._exchanges[key] = None
        return None
      if key not in self._peers:
        self._peers[key] = symm.PeerGroup(group)
      old = ex
      # a larger tensor arrived: the new exchange continues the group's epochs with new buffers; the old buffers go
      # only after the constructor's device synchronisation + barrier, when no peer can still be reading them
      ex = symm.PeerKVExchange(self._peers[key], k.numel(), k.dtype, transport=self.kv_transport)
      if old is not None:
        old.release()
      self._exchanges[key] = ex
    return ex

  def _a2a_for(self, group, x):
    """The peer-memory all-to-all of `group` (created on first use), or None for the NCCL path."""
    if not self.peer_memory or group is None or not x.is_cuda:
      return None
    key = id(group)
    ex = self._a2as.get(key, False)
    if ex is False or (ex is not None and ex.numel < x.numel()):
      from . import symm

      if not symm.peer_memory_available(group):
        self._a2as[key] = None
        return None
      if key not in self._peers:
        self._peers[key] = symm.PeerGroup(group)
      old = ex
      ex = symm.PeerAllToAll(self._peers[key], x.numel(), x.dtype)
      if old:
        old.release()
      self._a2as[key] = ex
    return ex

  def _reducer_for(self, group, k):
    """The peer-memory reduce-scatter that returns dK / dV partials to their owners (created on first use)."""
    key = id(group)
    rs = self._reducers.get(key)
    need = 2 * k.numel()
    if rs is None or rs.numel < need:
      from . import symm

      old = rs
      rs = symm.PeerReduceScatter(self._peers[key], need, k.dtype)
      if old is not None:
        old.release()
      self._reducers[key] = rs
    return rs

  # ---- sequence layout ---------------------------------------------------------------------
  def shard_sequence(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
    """Local shard of a full-length tensor; the length is padded (zeros) to a multiple of the axis size."""
    if self.size == 1:
      return x
    S = x.shape[dim]
    # a multiple of 8 rows per rank keeps every per-row fp32 statistic of the attention kernels (log-sum-exp, delta)
    # on 16-byte boundaries, which their bulk copies need; 32760 tokens on 8 ranks become 8 x 4096 with 8 pad rows
    per = ((S + self.size - 1) // self.size + 7) // 8 * 8
    self.full_len, self.local_len = S, per
    if per * self.size != S:
      pad = [0, 0] * (x.dim() - dim - 1) + [0, per * self.size - S]
      x = torch.nn.functional.pad(x, pad)
    return x.narrow(dim, self.rank * per, per).contiguous()

  def valid_lengths(self, ranks: int, per: int, group_stride: int = 1) -> list[int]:
    """Unpadded length of every shard along an axis of `ranks` shards of `per` tokens."""
    if self.full_len is None:
      return [per] * ranks
    out = []
    for r in range(ranks):
      start = r * per
      out.append(max(0, min(per, self.full_len - start)))
    return out

  def unshard_sequence(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
    """Inverse of `shard_sequence` (no gradient flows through it; training takes its loss on the shard)."""
    if self.size == 1:
      return x
    with torch.no_grad():
      full = C.all_gather_cat(x.transpose(0, dim).contiguous(), self.group, dim=0).transpose(0, dim)
    return full.narrow(dim, 0, self.full_len) if self.full_len is not None else full

  # ---- attention ---------------------------------------------------------------------------
  def _uses_flash(self, q) -> bool:
    return q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in K.FLASH_HEAD_DIMS and not OF.library_mode()

  def _full_attention(self, q, k, v, scale=None):
    """Attention of a rank that holds the whole key sequence of its heads."""
    if self.fixed_m and self._uses_flash(q):
      k = FM.smooth_keys(k)
      return OF.attention(q, k, v, scale, fixed_m=FM.plan(q, k, scale, smoothed=True))
    return OF.attention(q, k, v, scale)

  def _segment_attention(self, q, k, v, group, n, valid_lens, scale=None):
    if n == 1:
      if valid_lens[0] < k.shape[1]:  # padded tail rows of the sequence are no keys
        k, v = k[:, :valid_lens[0]], v[:, :valid_lens[0]]
      return self._full_attention(q, k, v, scale)
    D = q.shape[-1]
    scale = scale if scale is not None else D ** -0.5
    if self._uses_flash(q):
      ex = self._exchange_for(group, k)
      rs = self._reducer_for(group, k) if (ex is not None and torch.is_grad_enabled() and k.requires_grad) else None
      fixed = None
      if self.fixed_m:
        # padded tail rows of the own shard are zeros and do not raise the norm maximum
        fixed = FM.plan(q, k, scale, smoothed=False, group=group)
      return _SegmentAttentionFn.apply(q, k, v, scale, group, tuple(valid_lens), ex, rs, fixed, self.save_remote_kv)
    kg = _GatherSeq.apply(k, group)
    vg = _GatherSeq.apply(v, group)
    ks = [kg[i][:, :valid_lens[i]] for i in range(n)]
    vs = [vg[i][:, :valid_lens[i]] for i in range(n)]
    return OF.attention(q, ks, vs, scale)

  # ---- attention from the raw projections (lets the exchanges ride on the producer / consumer kernels) ---------
  def _fused_ulysses_for(self, group, numel_qkv, numel_out, dtype):
    key = id(group)
    ex = self._fused.get(key)
    if ex is None or ex.qkv_numel < numel_qkv or ex.out_numel < numel_out:
      from . import symm

      if not symm.peer_memory_available(group):
        return None
      if key not in self._peers:
        self._peers[key] = symm.PeerGroup(group)
      old = ex
      ex = symm.PeerFusedUlysses(self._peers[key], numel_qkv, numel_out, dtype)
      if old is not None:
        old.release()
      self._fused[key] = ex
    return ex

  def projected_self_attention(self, q, k, v, norm_q, norm_k, cos, sin, heads: int, eps: float, scale=None):
    """Self-attention from the raw q / k / v projections [B, S_loc, C] of this rank's rows: RMSNorm across heads +
    RoPE on q and k, attention under this object's strategy, output [B, S_loc, C].

    Under Ulysses (and the Ulysses half of the 2-D split), without autograd and over peer memory, neither exchange is
    a kernel of its own: the norm / RoPE kernel stores every head into the rank that owns it and the attention epilogue
    stores every output row into the rank that owns it (`symm.PeerFusedUlysses`; the reference runs two XLA
    all-to-alls around the kernel, src/maxdiffusion/models/attention_flax.py:875-877, 980-986). Everything else takes
    the generic path: norm + RoPE locally, then `self_attention`."""
    B, S, C = q.shape
    D = C // heads
    group = self.ulysses_group if self.strategy == "usp" else self.group
    U = self.ulysses_size if self.strategy == "usp" else self.size
    # a recorded forward of a rematerialised block also runs without autograd, but its replay expects the attention
    # output and statistics in the store: only a forward outside any recording takes the folded path
    fused = (self.strategy in ("ulysses", "usp") and self.peer_memory and U > 1 and group is not None and not torch.is_grad_enabled()
             and OF._remat.mode is None and not self.fixed_m and q.is_cuda and q.dtype == torch.bfloat16 and D == 128 and heads % U == 0 and U <= 8
             and not OF.library_mode() and all(t.stride(-1) == 1 and t.stride(0) == S * t.stride(1) for t in (q, k, v)))
    ex = self._fused_ulysses_for(group, B * U * S * (heads // U) * D, B * S * C, q.dtype) if fused else None
    if ex is None:
      qn = OF.rms_norm_rope(q, norm_q, cos, sin, heads=heads, eps=eps)
      kn = OF.rms_norm_rope(k, norm_k, cos, sin, heads=heads, eps=eps)
      return self.self_attention(qn, kn, v.unflatten(-1, (heads, D)), scale).reshape(B, S, C)
    cosf = cos.float().contiguous() if cos is not None else None
    sinf = sin.float().contiguous() if sin is not None else None
    qh, kh, vh = ex.scatter_qkv(q, k, v, norm_q, norm_k, cosf, sinf, eps)
    if self.strategy == "ulysses":
      if self.full_len is not None and self.full_len < S * U:
        kh, vh = kh[:, :self.full_len], vh[:, :self.full_len]
      return ex.attention(qh, kh, vh, heads, scale).reshape(B, S, C)
    # 2-D: the K / V of the other ring ranks are pulled by the copy CTAs of the same launch
    R, seg = self.ring_size, S * U
    lens = [seg] * R
    if self.full_len is not None:
      lens = [max(0, min(seg, self.full_len - r * seg)) for r in range(R)]
    if R == 1:
      return ex.attention(qh, kh[:, :lens[0]], vh[:, :lens[0]], heads, scale).reshape(B, S, C)
    rex = self._exchange_for(self.ring_group, kh)
    order = rex.order()
    kg, vg, flags, epoch, plan, keep = rex.plan(kh.contiguous(), vh.contiguous())
    ks = [kg[i][:, :lens[order[i]]] for i in range(R)]
    vs = [vg[i][:, :lens[order[i]]] for i in range(R)]
    return ex.attention(qh, ks, vs, heads, scale, seg_flags=flags, flag_target=epoch, plan=plan).reshape(B, S, C)

  def self_attention(self, q, k, v, scale=None):
    """q, k, v: [B, S_loc, H, D] (sequence-sharded). Returns the attention output with the same layout."""
    if self.size == 1 or self.strategy == "local":
      return self._full_attention(q, k, v, scale)
    per = q.shape[1]
    if self.strategy in ("gather", "ring"):
      return self._segment_attention(q, k, v, self.group, self.size, self.valid_lengths(self.size, per), scale)
    if self.strategy in ("ulysses", "usp") and q.shape[0] > 1:
      # CFG fold: every (batch, head) pair is an attention problem of its own, so a batch that makes the head count
      # divisible by the Ulysses shards is folded into the head axis around the exchange (40 heads over 8 shards
      # work with the CFG batch of 2; reference: src/maxdiffusion/models/attention_flax.py:995-1020)
      U = self.size if self.strategy == "ulysses" else self.ulysses_size
      B, S, H, D = q.shape
      if H % U != 0 and (B * H) % U == 0:
        fold = lambda t: t.permute(1, 0, 2, 3).reshape(1, t.shape[1], B * H, D)
        o = self.self_attention(fold(q), fold(k), fold(v), scale)
        return o.reshape(S, B, H, D).permute(1, 0, 2, 3)
    if self.strategy in ("ulysses", "usp") and self.ulysses_chunks > 1:
      U = self.size if self.strategy == "ulysses" else self.ulysses_size
      ranges = ulysses_head_chunks(q.shape[2], U, self.ulysses_chunks)
      if len(ranges) > 1:
        chunks, self.ulysses_chunks = self.ulysses_chunks, 1
        try:  # every chunk is a Ulysses attention of its own over fewer heads; the outputs concatenate along heads
          outs = [self.self_attention(q[:, :, a:b], k[:, :, a:b], v[:, :, a:b], scale) for a, b in ranges]
        finally:
          self.ulysses_chunks = chunks
        return torch.cat(outs, dim=2)
    if self.strategy == "ulysses":
      H = q.shape[2]
      if H % self.size != 0:
        raise ValueError(f"Ulysses needs heads ({H}) divisible by the context axis ({self.size})")
      ex = self._a2a_for(self.group, q)
      qh, kh, vh = (_HeadsToSeq.apply(t, self.group, ex) for t in (q, k, v))
      if self.full_len is not None and self.full_len < per * self.size:
        kh, vh = kh[:, :self.full_len], vh[:, :self.full_len]
      o = self._full_attention(qh, kh, vh, scale)
      return _SeqToHeads.apply(o, self.group, ex)
    if self.strategy == "usp":
      H = q.shape[2]
      U, R = self.ulysses_size, self.ring_size
      if H % U != 0:
        raise ValueError(f"ulysses_shards ({U}) must divide the number of heads ({H})")
      ex = self._a2a_for(self.ulysses_group, q)
      qh, kh, vh = (_HeadsToSeq.apply(t, self.ulysses_group, ex) for t in (q, k, v))
      # after the exchange a rank holds U consecutive shards of the sequence: the ring segment r covers the
      # global tokens [r*U*per, (r+1)*U*per)
      seg = per * U
      lens = [seg] * R
      if self.full_len is not None:
        lens = [max(0, min(seg, self.full_len - r * seg)) for r in range(R)]
      o = self._segment_attention(qh, kh, vh, self.ring_group, R, lens, scale)
      return _SeqToHeads.apply(o, self.ulysses_group, ex)
    raise ValueError(f"unknown context strategy {self.strategy}")
