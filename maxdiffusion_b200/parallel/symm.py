"""Symmetric peer memory over NVLink: buffers every rank of a group can load from / store to directly.

Allocation and the exchange of the memory handles are plumbing and go through
`torch.distributed._symmetric_memory`; everything that moves data or synchronises — epoch flags with
release/acquire semantics at system scope, bounded waits, pull copies, the fused reduce-scatter + AdamW — is this
repository's own kernels (`csrc/comm.cu`). Flags are monotonically increasing epoch numbers, so buffers are reused
without reset barriers; every device-side wait gives up after a time budget and records the failure in the device
status word, which the host raises as an exception at the next check.

The reference has no counterpart: its collectives are inserted by XLA and run through NCCL on GPUs
(src/maxdiffusion/max_utils.py:925-955, gpu_multi_process_run.sh:18-77).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import _lib

# flag kinds (rows of the signal pad); each row has one slot per source rank
FLAG_GRAD_READY = 0
FLAG_GRAD_ACK = 1
FLAG_KV_READY = 2
FLAG_KV_ACK = 3
FLAG_SHARD_READY = 4
FLAG_USER = 5
FLAG_SMALL_AR = 6
FLAG_RS_READY = 7
FLAG_RS_ACK = 8
FLAG_A2A_READY = 9
FLAG_A2A_ACK = 10
FLAG_O_READY = 11   # fused Ulysses: attention output rows stored into their owners
FLAG_O_ACK = 12
FLAG_QKV_READY = 13  # fused Ulysses: q / k / v heads stored into their owners
FLAG_QKV_ACK = 14
FLAG_TP_READY = 15   # tensor-parallel partial products (parallel.tensor.PeerAllReduce)
FLAG_TP_ACK = 16
FLAG_HALO_READY = 17  # width-sharded VAE: edge columns published for the neighbours (parallel.spatial.HaloExchange)
FLAG_HALO_ACK = 18
NUM_FLAG_KINDS = 20
WAIT_BUDGET_S = 10.0  # waits on other ranks: long enough for host-side skew (first-step allocation, logging)


def _declare(L):
  c_void_p, c_int, c_ll, c_float, c_uint = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_uint
  ullp = ctypes.POINTER(ctypes.c_ulonglong)
  L.mdb_signal_peers.argtypes = [ullp, c_int, c_int, c_uint, c_void_p]
  L.mdb_signal_peers.restype = c_int
  L.mdb_wait_flags.argtypes = [c_void_p, c_int, c_int, c_uint, ctypes.c_double, c_void_p]
  L.mdb_wait_flags.restype = c_int
  L.mdb_set_flag.argtypes = [c_void_p, c_uint, c_void_p]
  L.mdb_set_flag.restype = c_int
  L.mdb_peer_copy.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_void_p]
  L.mdb_peer_copy.restype = c_int
  L.mdb_memcpy_async.argtypes = [c_void_p, c_void_p, c_ll, c_void_p]
  L.mdb_memcpy_async.restype = c_int
  L.mdb_rs_adamw.argtypes = ([ullp, c_int, c_ll] + [c_void_p] * 6 + [c_int] + [c_float] * 9 +
                             [ctypes.c_ulonglong, c_int, c_int, c_int, c_void_p])
  L.mdb_rs_adamw.restype = c_int
  L.mdb_small_allreduce.argtypes = [c_void_p, c_void_p, c_int, c_int, ullp, ullp, c_int, c_int, c_int, c_int, c_uint,
                                    ctypes.c_double, c_void_p]
  L.mdb_small_allreduce.restype = c_int
  L.mdb_pull_reduce.argtypes = [ullp, c_int, c_void_p, c_ll, c_int, c_void_p]
  L.mdb_pull_reduce.restype = c_int
  L.mdb_pull_gather.argtypes = [ullp, c_int, c_void_p, c_ll, c_int, c_void_p]
  L.mdb_pull_gather.restype = c_int
  L.mdb_pull_a2a.argtypes = [ullp, c_int, c_void_p, c_int, c_int, c_int] + [c_ll] * 5 + [c_int, c_void_p]
  L.mdb_pull_a2a.restype = c_int


_lib.register(_declare)


def peer_memory_available(group) -> bool:
  """Peer kernels need CUDA, a multi-rank NCCL group on one node, and the symmetric-memory allocator."""
  if group is None or not torch.cuda.is_available() or dist.get_backend(group) != "nccl":
    return False
  try:
    import importlib

    importlib.import_module("torch.distributed._symmetric_memory")
  except Exception:
    return False
  return True


class PeerGroup:
  """A group of ranks with a shared signal pad and symmetric buffers."""

  def __init__(self, group):
    import torch.distributed._symmetric_memory as symm_mem

    self._symm = symm_mem
    self.group = group
    self.world = dist.get_world_size(group)
    self.rank = dist.get_rank(group)
    self.device = torch.device("cuda", torch.cuda.current_device())
    self.flags = symm_mem.empty(NUM_FLAG_KINDS * self.world, dtype=torch.int32, device=self.device)
    self.flags.zero_()
    self._flags_hdl = symm_mem.rendezvous(self.flags, group)
    self.flag_ptrs = [int(p) for p in self._flags_hdl.buffer_ptrs]
    self._buffers = []
    # One epoch counter per flag kind, owned by the group and not by the exchange objects: the pad keeps the largest
    # epoch ever signalled, so an object created later (a larger tensor arrived) has to continue from there. An
    # object that started again at zero would find every one of its waits satisfied by the stale values.
    self.epochs = [0] * NUM_FLAG_KINDS
    torch.cuda.synchronize()
    dist.barrier(group=group)

  def next_epoch(self, kind: int) -> int:
    """Advances and returns the epoch of a flag kind (every rank of the group calls it in the same order)."""
    self.epochs[kind] += 1
    return self.epochs[kind]

  def release(self, tensors) -> None:
    """Forgets symmetric buffers handed out by `alloc` (their memory returns to the allocator once unused)."""
    ids = {id(t) for t in tensors}
    self._buffers = [(t, h) for (t, h) in self._buffers if id(t) not in ids]

  # ---- buffers ----------------------------------------------------------------------------
  def alloc(self, numel: int, dtype: torch.dtype):
    """Symmetric buffer of `numel` elements; returns (local tensor, [address of the buffer on every rank])."""
    t = self._symm.empty(numel, dtype=dtype, device=self.device)
    hdl = self._symm.rendezvous(t, self.group)
    self._buffers.append((t, hdl))
    return t, [int(p) for p in hdl.buffer_ptrs], hdl

  # ---- flags ------------------------------------------------------------------------------
  def signal(self, kind: int, value: int, stream=None, peers: Optional[Sequence[int]] = None) -> None:
    """Stores `value` into slot (kind, my rank) of every peer's pad (all ranks by default, self included)."""
    ranks = list(range(self.world)) if peers is None else list(peers)
    arr = (ctypes.c_ulonglong * len(ranks))(*[self.flag_ptrs[r] for r in ranks])
    rc = _lib.lib().mdb_signal_peers(arr, len(ranks), kind * self.world + self.rank, int(value) & 0xffffffff,
                                     stream if stream is not None else _lib.stream())
    _lib.check(rc, "mdb_signal_peers")

  def wait(self, kind: int, value: int, sources: Optional[Sequence[int]] = None, stream=None) -> None:
    """Waits (bounded) until the slots (kind, src) of MY pad reached `value`, for every src (all by default)."""
    if value <= 0:
      return
    base = self.flags.data_ptr() + 4 * kind * self.world
    if sources is None:
      rc = _lib.lib().mdb_wait_flags(ctypes.c_void_p(base), self.world, 1, int(value), WAIT_BUDGET_S,
                                     stream if stream is not None else _lib.stream())
      _lib.check(rc, "mdb_wait_flags")
    else:
      for s in sources:
        rc = _lib.lib().mdb_wait_flags(ctypes.c_void_p(base + 4 * s), 1, 1, int(value), WAIT_BUDGET_S,
                                       stream if stream is not None else _lib.stream())
        _lib.check(rc, "mdb_wait_flags")


class SmallAllReduce:
  """One-launch all-reduce (sum or max) of up to `capacity` fp32 values over peer memory.

  Every rank reduces all ranks' vectors in rank order, so the result is bitwise identical everywhere. Calls must be
  made by every rank of the group in the same order (each call advances the epoch by one)."""

  def __init__(self, peers: "PeerGroup", capacity: int = 4096):
    self.peers = peers
    self.capacity = capacity
    self.buf, self.buf_ptrs, self._hdl = peers.alloc(2 * capacity, torch.float32)
    self.buf.zero_()
    n = peers.world
    self._bufs = (ctypes.c_ulonglong * n)(*self.buf_ptrs)
    self._flags = (ctypes.c_ulonglong * n)(*peers.flag_ptrs)
    torch.cuda.synchronize()
    dist.barrier(group=peers.group)

  def __call__(self, x: torch.Tensor, op: str = "sum", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    assert x.dtype == torch.float32 and x.is_contiguous() and 0 < x.numel() <= self.capacity
    out = torch.empty_like(x) if out is None else out
    self.epoch = self.peers.next_epoch(FLAG_SMALL_AR)
    rc = _lib.lib().mdb_small_allreduce(_lib.ptr(x), _lib.ptr(out), x.numel(), {"sum": 0, "max": 1}[op], self._bufs,
                                        self._flags, self.peers.world, self.peers.rank,
                                        FLAG_SMALL_AR * self.peers.world, self.capacity, self.epoch, WAIT_BUDGET_S,
                                        _lib.stream())
    _lib.check(rc, "mdb_small_allreduce")
    return out


def set_flag(flag_tensor: torch.Tensor, index: int, value: int, stream=None) -> None:
  rc = _lib.lib().mdb_set_flag(ctypes.c_void_p(flag_tensor.data_ptr() + 4 * index), int(value),
                               stream if stream is not None else _lib.stream())
  _lib.check(rc, "mdb_set_flag")


def peer_copy(src_ptr: int, dst: torch.Tensor, nbytes: int, ctas: int = 16, stream=None) -> None:
  rc = _lib.lib().mdb_peer_copy(ctypes.c_void_p(src_ptr), ctypes.c_void_p(dst.data_ptr()), nbytes, ctas,
                                stream if stream is not None else _lib.stream())
  _lib.check(rc, "mdb_peer_copy")


def memcpy_async(dst_ptr: int, src_ptr: int, nbytes: int, stream=None) -> None:
  """Copy-engine copy (local or peer source); occupies no SM, so it can run beside a kernel that fills the GPU."""
  rc = _lib.lib().mdb_memcpy_async(ctypes.c_void_p(dst_ptr), ctypes.c_void_p(src_ptr), nbytes,
                                   stream if stream is not None else _lib.stream())
  _lib.check(rc, "mdb_memcpy_async")


def stream_write_value32(addr: int, value: int, stream=None) -> None:
  """Stream memory operation: the stream stores `value` at device address `addr` once its earlier work is done; no
  kernel is launched, so the store lands even while a persistent kernel holds every SM."""
  rc = _lib.lib().mdb_stream_write_value32(ctypes.c_void_p(addr), int(value) & 0xffffffff,
                                           stream if stream is not None else _lib.stream())
  _lib.check(rc, "mdb_stream_write_value32")


class PeerKVExchange:
  """Ring-schedule K/V exchange for context-parallel attention over peer memory.

  Every rank publishes its K/V shard in a symmetric buffer and raises an epoch flag on all peers. The attention
  kernel is then launched with a copy plan: its last CTAs wait for the owners' flags, pull the other shards
  straight from their owners over NVLink (no store-and-forward chain: through NVSwitch every peer is one hop away)
  into a local staging tensor and raise each staged segment's ready flag, while the compute CTAs of the same
  launch start on the rank's own shard and wait — bounded — on a segment's flag before its first TMA load. The
  transfer of hop h+1 thus overlaps the math of hop h, the running (O, m, l) never leave the SM, and nothing
  but this one kernel is involved; afterwards the copy CTAs acknowledge to the owners so the buffers can be
  reused two epochs later without a barrier.
  """

  def __init__(self, peer: "PeerGroup", max_numel_per_tensor: int, dtype=torch.bfloat16, copy_ctas: int = 12,
               head_groups: int = 0, transport: str = "sm"):
    if transport not in ("sm", "dma"):
      raise ValueError(f"ring K/V transport must be 'sm' (copy CTAs of the attention launch) or 'dma' (copy engines), got {transport!r}")
    self.transport = transport
    self.peer = peer
    self.n, self.rank = peer.world, peer.rank
    self.numel = max_numel_per_tensor
    self.copy_ctas = copy_ctas
    self.head_groups = head_groups  # 0: the launcher picks one head group per round of work items; 1: whole segments
    self._dma_stream = None
    self.slots, self.slot_ptrs = [], []
    for _ in range(2):
      t, ptrs, _h = peer.alloc(2 * max_numel_per_tensor, dtype)
      self.slots.append(t)
      self.slot_ptrs.append(ptrs)
    self.epoch = peer.epochs[FLAG_KV_READY]
    self.elem = torch.tensor([], dtype=dtype).element_size()
    torch.cuda.synchronize()
    dist.barrier(group=peer.group)

  def release(self) -> None:
    self.peer.release(self.slots)

  def order(self):
    """Ranks in the order the segments are consumed: own shard, then the ring predecessors."""
    return [(self.rank - h) % self.n for h in range(self.n)]

  def publish(self, k: torch.Tensor, v: torch.Tensor):
    """Copies this rank's shard into the symmetric slot of a new epoch and raises KV_READY on every peer."""
    numel = k.numel()
    assert numel == v.numel() and numel <= self.numel and k.dtype == self.slots[0].dtype
    self.epoch = self.peer.next_epoch(FLAG_KV_READY)
    e = self.epoch
    slot = e % 2
    sym = self.slots[slot]
    self.peer.wait(FLAG_KV_ACK, e - 2)              # the previous content of this slot has been pulled by all
    sym[:numel].view(k.shape).copy_(k)
    sym[self.numel:self.numel + numel].view(v.shape).copy_(v)
    self.peer.signal(FLAG_KV_READY, e)
    kg = torch.empty((self.n,) + tuple(k.shape), dtype=k.dtype, device=k.device)
    vg = torch.empty((self.n,) + tuple(v.shape), dtype=v.dtype, device=v.device)
    kg[0].copy_(k)
    vg[0].copy_(v)
    return kg, vg, e, slot, numel * self.elem

  def plan(self, k: torch.Tensor, v: torch.Tensor):
    """Returns (kg, vg, flags, epoch, plan) for a fused launch: staging tensors [n, *k.shape] in consumption order,
    the int32 ready flags (one row of `COPY_FLAG_STRIDE` head-group flags per segment; row 0, the own shard, is already
    raised) and the copy plan for `kernels.flash_fwd`. With the copy-engine transport the plan is None and there is one
    flag per segment (`stage_dma`)."""
    if self.transport == "dma":
      kg, vg, flags, e = self.stage_dma(k, v)
      return kg, vg, flags, e, None, flags
    kg, vg, e, slot, nbytes = self.publish(k, v)
    fs = _lib.COPY_FLAG_STRIDE
    state = torch.zeros(self.n * fs + _lib.COPY_NUM_COUNTERS + 7, dtype=torch.int32, device=k.device)  # [flags | counters]
    flags = state[:self.n * fs]
    flags[:fs].fill_(e)
    plan = _lib.CopyPlan()
    plan.n_remote = self.n - 1
    plan.n_copy_ctas = self.copy_ctas
    plan.n_groups = self.head_groups
    pad = self.peer.flags.data_ptr()
    for i, src in enumerate(self.order()[1:]):
      base = self.slot_ptrs[slot][src]
      plan.src[i][0], plan.src[i][1] = base, base + self.numel * self.elem
      plan.dst[i][0], plan.dst[i][1] = kg[i + 1].data_ptr(), vg[i + 1].data_ptr()
      plan.ready[i] = pad + 4 * (FLAG_KV_READY * self.n + src)
    plan.nbytes = nbytes
    plan.epoch = e
    plan.counters = state.data_ptr() + 4 * self.n * fs
    plan.seg_flags = flags.data_ptr()
    plan.n_ack = self.n
    for r in range(self.n):
      plan.ack[r] = self.peer.flag_ptrs[r] + 4 * (FLAG_KV_ACK * self.n + self.rank)
    return kg, vg, flags, e, plan, state

  def stage_dma(self, k: torch.Tensor, v: torch.Tensor):
    """Copy-engine transport. Returns (kg, vg, flags, epoch): staging tensors in consumption order and one int32 ready
    flag per segment (flag 0, the own shard, already raised) for `kernels.flash_fwd(..., seg_flags=, flag_target=)`.

    Once every owner has published, a side stream pulls the remote shards in ring order with copy-engine copies and,
    after each segment's pair of copies, stores the epoch into that segment's flag with a stream memory operation.
    Neither the copies nor the flag stores need an SM, so every CTA of the attention launch computes, and the only
    thing its bounded flag waits depend on is the DMA engines. The acknowledgement to the owners follows the last
    copy on the side stream."""
    kg, vg, e, slot, nbytes = self.publish(k, v)
    flags = torch.zeros(self.n, dtype=torch.int32, device=k.device)
    flags[:1].fill_(e)
    self.peer.wait(FLAG_KV_READY, e)
    main = torch.cuda.current_stream()
    if self._dma_stream is None:
      self._dma_stream = torch.cuda.Stream(device=k.device)
    side = self._dma_stream
    side.wait_stream(main)
    sp = ctypes.c_void_p(side.cuda_stream)
    for i, src in enumerate(self.order()[1:]):
      base = self.slot_ptrs[slot][src]
      memcpy_async(kg[i + 1].data_ptr(), base, nbytes, stream=sp)
      memcpy_async(vg[i + 1].data_ptr(), base + self.numel * self.elem, nbytes, stream=sp)
      stream_write_value32(flags.data_ptr() + 4 * (i + 1), e, stream=sp)
    self.peer.signal(FLAG_KV_ACK, e, stream=sp)
    for t in (kg, vg, flags):
      t.record_stream(side)
    return kg, vg, flags, e

  def gather(self, k: torch.Tensor, v: torch.Tensor):
    """Stand-alone variant (no attention kernel to fuse with): waits for every owner, pulls, acknowledges."""
    kg, vg, e, slot, nbytes = self.publish(k, v)
    self.peer.wait(FLAG_KV_READY, e)
    for i, src in enumerate(self.order()[1:]):
      base = self.slot_ptrs[slot][src]
      peer_copy(base, kg[i + 1], nbytes, ctas=32)
      peer_copy(base + self.numel * self.elem, vg[i + 1], nbytes, ctas=32)
    self.peer.signal(FLAG_KV_ACK, e)
    return kg, vg


def pull_gather(src_ptrs: Sequence[int], dst: torch.Tensor, nbytes_per_rank: int, ctas: int = 16, stream=None) -> None:
  """dst = concatenation over ranks of the `nbytes_per_rank` bytes at src_ptrs[r] (peer addresses), one kernel."""
  arr = (ctypes.c_ulonglong * len(src_ptrs))(*src_ptrs)
  rc = _lib.lib().mdb_pull_gather(arr, len(src_ptrs), _lib.ptr(dst), int(nbytes_per_rank), ctas,
                                  stream if stream is not None else _lib.stream())
  _lib.check(rc, "mdb_pull_gather")


class PeerAllToAll:
  """The Ulysses exchanges over peer memory: [B, S, H, D] sequence-sharded <-> [B, n S, H / n, D] head-sharded.

  A rank publishes its tensor in a symmetric slot and raises an epoch flag; every rank then pulls, with ONE kernel,
  the rows it keeps from every peer straight into their final place (`pull_a2a` in csrc/comm.cu), so the layout change
  rides on the transfer: no permute + contiguous pass before or after, every byte crosses NVLink once. An
  acknowledge flag lets the two slots be reused without a barrier.
  """

  def __init__(self, peer: "PeerGroup", max_numel: int, dtype=torch.bfloat16):
    self.peer, self.n, self.rank = peer, peer.world, peer.rank
    self.numel = -(-max_numel // 8) * 8
    self.dtype = dtype
    self.elem = torch.tensor([], dtype=dtype).element_size()
    self.slots, self.slot_ptrs = [], []
    for _ in range(2):
      t, ptrs, _h = peer.alloc(self.numel, dtype)
      self.slots.append(t)
      self.slot_ptrs.append(ptrs)
    self.epoch = peer.epochs[FLAG_A2A_READY]
    torch.cuda.synchronize()
    dist.barrier(group=peer.group)

  def release(self) -> None:
    self.peer.release(self.slots)

  @staticmethod
  def supports(x: torch.Tensor, n: int) -> bool:
    return x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and (x.shape[-1] * x.element_size()) % 16 == 0

  def _publish(self, x: torch.Tensor):
    assert x.numel() <= self.numel and x.dtype == self.dtype
    self.epoch = self.peer.next_epoch(FLAG_A2A_READY)
    e, slot = self.epoch, self.epoch % 2
    self.peer.wait(FLAG_A2A_ACK, e - 2)  # every peer has pulled the previous content of this slot
    self.slots[slot][:x.numel()].view(x.shape).copy_(x)
    self.peer.signal(FLAG_A2A_READY, e)
    self.peer.wait(FLAG_A2A_READY, e)
    return e, slot

  def _pull(self, slot, src_off_bytes, out, n_b, n_s, row_bytes, src_sb, src_ss, dst_sr, dst_sb, dst_ss, e):
    arr = (ctypes.c_ulonglong * self.n)(*[self.slot_ptrs[slot][r] + src_off_bytes for r in range(self.n)])
    rc = _lib.lib().mdb_pull_a2a(arr, self.n, _lib.ptr(out), n_b, n_s, row_bytes, src_sb, src_ss, dst_sr, dst_sb, dst_ss,
                                 24, _lib.stream())
    _lib.check(rc, "mdb_pull_a2a")
    self.peer.signal(FLAG_A2A_ACK, e)
    return out

  @staticmethod
  def pull_spec(kind: str, shape, n: int, rank: int, es: int) -> dict:
    """The byte strides of one exchange as the pull kernel takes them (`pull_a2a_kernel`), for a rank of an
    n-rank group; `kind` is 'heads_to_seq' ([B,S,H,D] -> [B,nS,H/n,D]) or 'seq_to_heads' (the inverse)."""
    if kind == "heads_to_seq":
      B, S, H, D = shape
      hn = H // n
      row = hn * D * es
      return dict(out_shape=(B, n * S, hn, D), src_off=rank * row, n_b=B, n_s=S, row=row, src_sb=S * H * D * es,
                  src_ss=H * D * es, dst_sr=S * row, dst_sb=n * S * row, dst_ss=row)
    B, Sf, hn, D = shape
    S, H = Sf // n, hn * n
    row = hn * D * es
    return dict(out_shape=(B, S, H, D), src_off=rank * S * row, n_b=B, n_s=S, row=row, src_sb=Sf * row, src_ss=row,
                dst_sr=row, dst_sb=S * H * D * es, dst_ss=H * D * es)

  def _exchange(self, kind: str, x: torch.Tensor) -> torch.Tensor:
    sp = self.pull_spec(kind, tuple(x.shape), self.n, self.rank, self.elem)
    e, slot = self._publish(x)
    out = torch.empty(sp["out_shape"], dtype=x.dtype, device=x.device)
    return self._pull(slot, sp["src_off"], out, sp["n_b"], sp["n_s"], sp["row"], sp["src_sb"], sp["src_ss"], sp["dst_sr"],
                      sp["dst_sb"], sp["dst_ss"], e)

  def heads_to_seq(self, x: torch.Tensor) -> torch.Tensor:
    """[B, S, H, D] (every rank: its S rows, all heads) -> [B, n S, H / n, D] (all rows, this rank's heads)."""
    return self._exchange("heads_to_seq", x)

  def seq_to_heads(self, x: torch.Tensor) -> torch.Tensor:
    """[B, n S, H / n, D] (all rows, this rank's heads) -> [B, S, H, D] (this rank's rows, all heads)."""
    return self._exchange("seq_to_heads", x)


class PeerFusedUlysses:
  """Both Ulysses exchanges WITHOUT an exchange kernel (inference; nothing is kept for a backward pass).

  Forward exchange: the RMSNorm + RoPE kernel of q and k, and a layout-only pass of the same kernel for v, store every
  head straight into the receive buffer of the rank that owns it (`kernels.rms_rope_scatter`), already in the
  [B, n S, H / n, D] layout attention wants. Reverse exchange: the attention epilogue stores every output row straight
  into the [B, S, H, D] buffer of the rank that owns the row (`kernels.flash_fwd_scatter`). What remains of the
  collectives are the epoch flags: READY after a rank's stores (peers wait for all of them before they read), ACK after
  a rank has consumed a receive slot (peers wait for it before they overwrite the slot two epochs later).
  """

  def __init__(self, peer: "PeerGroup", qkv_numel: int, out_numel: int, dtype=torch.bfloat16):
    self.peer, self.n, self.rank = peer, peer.world, peer.rank
    self.qkv_numel, self.out_numel = -(-qkv_numel // 8) * 8, -(-out_numel // 8) * 8
    self.elem = torch.tensor([], dtype=dtype).element_size()
    self.recv, self.recv_ptrs, self.out, self.out_ptrs = [], [], [], []
    for _ in range(2):
      t, ptrs, _h = peer.alloc(3 * self.qkv_numel, dtype)
      self.recv.append(t)
      self.recv_ptrs.append(ptrs)
      t, ptrs, _h = peer.alloc(self.out_numel, dtype)
      self.out.append(t)
      self.out_ptrs.append(ptrs)
    self._qkv_epoch = self._out_epoch = None
    torch.cuda.synchronize()
    dist.barrier(group=peer.group)

  def release(self) -> None:
    self.peer.release(self.recv + self.out)

  def scatter_qkv(self, q, k, v, norm_q, norm_k, cos, sin, eps: float):
    """q, k, v: raw projections [B, S, C] of this rank's rows. Returns (qh, kh, vh) [B, n S, H / n, 128]: views of the
    receive slot, valid until `attention` has consumed them."""
    from ..ops import kernels as K

    B, S, C = q.shape
    hn = C // 128 // self.n
    numel = B * self.n * S * hn * 128
    assert numel <= self.qkv_numel
    e = self.peer.next_epoch(FLAG_QKV_READY)
    slot = e % 2
    self.peer.wait(FLAG_QKV_ACK, e - 2)  # every peer has consumed what it received in this slot two epochs ago
    for i, (t, w, rope) in enumerate(((q, norm_q, True), (k, norm_k, True), (v, None, False))):
      ptrs = [p + i * self.qkv_numel * self.elem for p in self.recv_ptrs[slot]]
      K.rms_rope_scatter(t, ptrs, self.rank, w, cos if rope else None, sin if rope else None,
                         mode="row" if rope else "copy", eps=eps)
    self.peer.signal(FLAG_QKV_READY, e)
    self.peer.wait(FLAG_QKV_READY, e)    # every peer's stores into MY slot are complete
    self._qkv_epoch = e
    views = [self.recv[slot][i * self.qkv_numel:i * self.qkv_numel + numel].view(B, self.n * S, hn, 128) for i in range(3)]
    return views

  def attention(self, qh, kh, vh, heads_total: int, scale=None, seg_flags=None, flag_target: int = 0, plan=None):
    """Attention on this rank's heads; the output rows go to their owners. Returns this rank's [B, S, H, 128] output
    (a view of the receive slot, valid until the call after next)."""
    from ..ops import kernels as K

    B, Sn, hn, D = qh.shape
    S = Sn // self.n
    if self._out_epoch is not None:
      self.peer.signal(FLAG_O_ACK, self._out_epoch)  # the consumer of the previous output has been enqueued by now
    e = self.peer.next_epoch(FLAG_O_READY)
    slot = e % 2
    self.peer.wait(FLAG_O_ACK, e - 2)
    K.flash_fwd_scatter(qh, kh, vh, self.out_ptrs[slot], S, heads_total, self.rank * hn, scale, seg_flags, flag_target, plan)
    self.peer.signal(FLAG_QKV_ACK, self._qkv_epoch)  # q, k, v of this epoch have been read
    self.peer.signal(FLAG_O_READY, e)
    self.peer.wait(FLAG_O_READY, e)
    self._out_epoch = e
    return self.out[slot][:B * S * heads_total * D].view(B, S, heads_total, D)


class PeerReduceScatter:
  """Reduce-scatter over peer memory for tensors that are produced slice by slice (the dK / dV partials of ring
  attention's backward, one slice per owner rank).

  Every rank's producers write their partial for owner r straight into slice r of a symmetric bf16 buffer
  (`slices()` hands out the views). `reduce()` then raises this rank's READY flag on every peer, waits (bounded) for
  all peers, and ONE kernel pulls this rank's slice from every rank over NVLink in 16-byte loads, sums the partials
  in rank order in fp32 and writes bf16: every byte crosses NVLink once, the sum is rounded once, and the result is
  bitwise reproducible. An ACK flag lets the two buffer slots be reused without a barrier.
  """

  def __init__(self, peer: "PeerGroup", max_slice_numel: int, dtype=torch.bfloat16):
    assert dtype == torch.bfloat16
    self.peer, self.n, self.rank = peer, peer.world, peer.rank
    self.numel = -(-max_slice_numel // 8) * 8
    self.slots, self.slot_ptrs = [], []
    for _ in range(2):
      t, ptrs, _h = peer.alloc(self.n * self.numel, dtype)
      self.slots.append(t)
      self.slot_ptrs.append(ptrs)
    self.epoch = peer.epochs[FLAG_RS_READY]
    self.stream = torch.cuda.Stream()  # callers may run `reduce` here, underneath compute on their own stream
    torch.cuda.synchronize()
    dist.barrier(group=peer.group)

  def release(self) -> None:
    self.peer.release(self.slots)

  def slices(self, shape):
    """Starts an epoch: views [n][*shape] of the slot to be filled (slice r = partial for owner r)."""
    numel = 1
    for d in shape:
      numel *= int(d)
    assert numel <= self.numel and numel % 8 == 0, (numel, self.numel)
    self.epoch = self.peer.next_epoch(FLAG_RS_READY)
    self.peer.wait(FLAG_RS_ACK, self.epoch - 2)  # every owner has pulled the previous content of this slot
    sym = self.slots[self.epoch % 2]
    self._shape, self._numel = tuple(shape), numel
    return [sym[r * self.numel:r * self.numel + numel].view(shape) for r in range(self.n)]

  def stacked(self) -> torch.Tensor:
    """The slices of the current epoch as one strided view [n, *shape] (owner r at index r)."""
    sym = self.slots[self.epoch % 2]
    strides, acc = [], 1
    for d in reversed(self._shape):
      strides.append(acc)
      acc *= int(d)
    return sym.as_strided((self.n,) + self._shape, (self.numel,) + tuple(reversed(strides)))

  def reduce(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    e, slot = self.epoch, self.epoch % 2
    self.peer.signal(FLAG_RS_READY, e)
    self.peer.wait(FLAG_RS_READY, e)
    if out is None:
      out = torch.empty(self._shape, dtype=torch.bfloat16, device=self.slots[0].device)
    off = self.rank * self.numel * 2
    arr = (ctypes.c_ulonglong * self.n)(*[self.slot_ptrs[slot][r] + off for r in range(self.n)])
    rc = _lib.lib().mdb_pull_reduce(arr, self.n, _lib.ptr(out), self._numel, 32, _lib.stream())
    _lib.check(rc, "mdb_pull_reduce")
    self.peer.signal(FLAG_RS_ACK, e)
    return out


def rs_adamw(grad_ptrs: Sequence[int], n: int, p, m, v, stats, scratch, *, lr, b1, b2, eps, wd, step, grad_scale=1.0,
             clip_value=0.0, seed=0, stochastic=True, apply=True, reduced_out=None, ctas=32, stream=None) -> None:
  """Fused reduce-scatter + statistics + AdamW on this rank's parameter slice (see csrc/comm.cu)."""
  arr = (ctypes.c_ulonglong * len(grad_ptrs))(*grad_ptrs)
  rc = _lib.lib().mdb_rs_adamw(arr, len(grad_ptrs), n, _lib.ptr(p), _lib.ptr(m), _lib.ptr(v), _lib.ptr(reduced_out),
                               _lib.ptr(stats), _lib.ptr(scratch), int(apply), float(lr), float(b1), float(b2),
                               float(eps), float(wd), float(1 - b1 ** step), float(1 - b2 ** step), float(grad_scale),
                               float(clip_value), int(seed) & (2 ** 64 - 1), int(stochastic),
                               int(m.dtype == torch.float32), ctas, stream if stream is not None else _lib.stream())
  _lib.check(rc, "mdb_rs_adamw")
