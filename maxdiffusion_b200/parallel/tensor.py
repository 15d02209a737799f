"""Tensor parallelism over the mesh's `tensor` axis: column-parallel and row-parallel linears (Megatron layout).

The reference shards `heads` / `mlp` kernels over the `tensor` mesh axis and lets XLA insert the all-reduce
(logical axis rules in src/maxdiffusion/configs/base_wan_14b.yml:204-222, src/maxdiffusion/common_types.py:72-110).
Here the two halves are explicit:

  * `ColumnParallelLinear`: weight rows (output features) split over the group; input replicated, output sharded;
    backward all-reduces the input gradient;
  * `RowParallelLinear`: weight columns (input features) split; input sharded, partial outputs summed over the
    group. With peer memory the sum is `parallel.symm`'s pull-reduce over symmetric buffers, else an NCCL all-reduce;
  * `shard_attention_heads` / `shard_mlp` split an existing block's fused projections in place.
  * `apply_tensor_parallel_wan` shards the blocks of a `WanModel` in place (heads and FFN units over the group) and
    is what the trainers and pipelines call when the mesh's `tensor` axis is larger than one.
GEMMs run on the tcgen05 kernel (`ops.functional.linear`); only the reduction crosses NVLink. With peer memory the
row-parallel GEMM writes its partial product straight into a symmetric buffer and every rank sums the partials of all
ranks in rank order with one pull kernel (`PeerAllReduce`: bitwise identical results on every rank, no NCCL call);
otherwise the reduction is an NCCL all-reduce.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as OF


class PeerAllReduce:
  """Sum of one bf16 tensor per rank over peer memory: producers write their partial into `buffer(shape)` (a view of a
  symmetric slot, e.g. as the `out=` of the row-parallel GEMM), `reduce()` raises the epoch flag, waits (bounded) for
  the peers and pulls every rank's partial in rank order, adding in fp32 and rounding once."""

  def __init__(self, group, max_numel: int):
    from . import symm

    self._symm = symm
    self.peer = symm.PeerGroup(group)
    self.n, self.rank = self.peer.world, self.peer.rank
    self.numel = -(-max_numel // 8) * 8
    self.slots, self.slot_ptrs = [], []
    for _ in range(2):
      t, ptrs, _h = self.peer.alloc(self.numel, torch.bfloat16)
      self.slots.append(t)
      self.slot_ptrs.append(ptrs)
    self.epoch = 0
    torch.cuda.synchronize()
    dist.barrier(group=group)

  def buffer(self, shape) -> torch.Tensor:
    numel = 1
    for d in shape:
      numel *= int(d)
    assert numel <= self.numel and numel % 8 == 0
    self.epoch = self.peer.next_epoch(self._symm.FLAG_TP_READY)
    self.peer.wait(self._symm.FLAG_TP_ACK, self.epoch - 2)  # every peer has read this slot's previous content
    self._shape, self._numel = tuple(shape), numel
    return self.slots[self.epoch % 2][:numel].view(shape)

  def reduce(self) -> torch.Tensor:
    import ctypes

    from ..ops import _lib

    symm, e = self._symm, self.epoch
    self.peer.signal(symm.FLAG_TP_READY, e)
    self.peer.wait(symm.FLAG_TP_READY, e)
    out = torch.empty(self._shape, dtype=torch.bfloat16, device=self.slots[0].device)
    arr = (ctypes.c_ulonglong * self.n)(*self.slot_ptrs[e % 2])
    rc = _lib.lib().mdb_pull_reduce(arr, self.n, _lib.ptr(out), self._numel, 32, _lib.stream())
    _lib.check(rc, "mdb_pull_reduce")
    self.peer.signal(symm.FLAG_TP_ACK, e)
    return out


_PEER_AR: dict = {}


def _peer_allreduce_for(group, numel: int):
  """The peer-memory all-reduce of a group (created on first use and grown when a larger tensor arrives), or None."""
  from . import symm

  if group is None or not symm.peer_memory_available(group):
    return None
  ar = _PEER_AR.get(id(group))
  if ar is None or ar.numel < numel:
    ar = PeerAllReduce(group, numel)
    _PEER_AR[id(group)] = ar
  return ar


def all_reduce_sum(x: torch.Tensor, group, peer_memory: bool = True) -> torch.Tensor:
  """Sum over the group; over peer memory for CUDA bf16 tensors when available, else NCCL / Gloo."""
  if group is None:
    return x
  if peer_memory and x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
    ar = _peer_allreduce_for(group, x.numel())
    if ar is not None:
      ar.buffer(x.shape).copy_(x)
      return ar.reduce()
  x = x.contiguous()
  dist.all_reduce(x, group=group)
  return x


class _CopyToGroup(torch.autograd.Function):
  """Identity forward, all-reduce backward (input of a column-parallel layer)."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return x

  @staticmethod
  def backward(ctx, g):
    return all_reduce_sum(g, ctx.group), None


class _ReduceFromGroup(torch.autograd.Function):
  """All-reduce forward, identity backward (output of a row-parallel layer)."""

  @staticmethod
  def forward(ctx, x, group):
    return all_reduce_sum(x, group)

  @staticmethod
  def backward(ctx, g):
    return g, None


def _size_rank(group):
  if group is None:
    return 1, 0
  return dist.get_world_size(group), dist.get_rank(group)


class ColumnParallelLinear(nn.Module):

  def __init__(self, in_features: int, out_features: int, bias: bool = True, group=None, chunks: int = 1):
    """`chunks` > 1 keeps fused projections (q|k|v) aligned: every chunk of the output is split separately."""
    super().__init__()
    self.group = group
    n, r = _size_rank(group)
    if out_features % (n * chunks) != 0:
      raise ValueError(f"out_features={out_features} is not divisible by tensor ranks x chunks = {n * chunks}")
    self.in_features, self.out_features, self.chunks, self.n, self.r = in_features, out_features, chunks, n, r
    self.weight = nn.Parameter(torch.empty(out_features // n, in_features))
    self.bias = nn.Parameter(torch.zeros(out_features // n)) if bias else None
    nn.init.normal_(self.weight, std=in_features ** -0.5)

  def shard_of(self, full: torch.Tensor) -> torch.Tensor:
    """This rank's rows of a full [out, ...] tensor."""
    per = self.out_features // self.chunks
    loc = per // self.n
    return torch.cat([full[c * per + self.r * loc: c * per + (self.r + 1) * loc] for c in range(self.chunks)], dim=0)

  def load_full(self, weight: torch.Tensor, bias=None) -> None:
    with torch.no_grad():
      self.weight.copy_(self.shard_of(weight))
      if self.bias is not None and bias is not None:
        self.bias.copy_(self.shard_of(bias))

  def forward(self, x, activation=None):
    return OF.linear(_CopyToGroup.apply(x, self.group), self.weight, self.bias, activation)


class RowParallelLinear(nn.Module):

  def __init__(self, in_features: int, out_features: int, bias: bool = True, group=None):
    super().__init__()
    self.group = group
    n, r = _size_rank(group)
    if in_features % n != 0:
      raise ValueError(f"in_features={in_features} is not divisible by the tensor ranks ({n})")
    self.in_features, self.out_features, self.n, self.r = in_features, out_features, n, r
    self.weight = nn.Parameter(torch.empty(out_features, in_features // n))
    self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
    nn.init.normal_(self.weight, std=in_features ** -0.5)

  def load_full(self, weight: torch.Tensor, bias=None) -> None:
    loc = self.in_features // self.n
    with torch.no_grad():
      self.weight.copy_(weight[:, self.r * loc:(self.r + 1) * loc])
      if self.bias is not None and bias is not None:
        self.bias.copy_(bias)

  def forward(self, x):
    if (self.group is not None and not torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.bfloat16
        and not OF.library_mode()):
      # inference: the GEMM writes its partial product straight into the symmetric slot the peers pull from
      from ..ops import kernels as K

      rows = x.reshape(-1, x.shape[-1])
      ar = _peer_allreduce_for(self.group, rows.shape[0] * self.out_features)
      if ar is not None and self.out_features % 8 == 0 and rows.shape[1] % 8 == 0:
        K.gemm(rows, self.weight.to(torch.bfloat16), out=ar.buffer((rows.shape[0], self.out_features)))
        y = ar.reduce().view(*x.shape[:-1], self.out_features)
        return y + self.bias.to(y.dtype) if self.bias is not None else y
    y = _ReduceFromGroup.apply(OF.linear(x, self.weight, None), self.group)
    return y + self.bias.to(y.dtype) if self.bias is not None else y


def parallel_mlp(dim: int, hidden: int, group=None):
  """(up, down) projections of a feed-forward block split over `group`: hidden units are sharded."""
  return ColumnParallelLinear(dim, hidden, group=group), RowParallelLinear(hidden, dim, group=group)


def parallel_attention_projections(dim: int, group=None):
  """(fused qkv, out) projections split by heads: every rank computes attention for heads/n heads."""
  return ColumnParallelLinear(dim, 3 * dim, group=group, chunks=3), RowParallelLinear(dim, dim, group=group)


# ---------------------------------------------------------------------------------------------------------------
# Wan blocks over the tensor axis
# ---------------------------------------------------------------------------------------------------------------
class _AllReduceSum(torch.autograd.Function):
  """Sum over the group in both directions (a statistic every rank needs and every rank contributes to)."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    y = x.clone()
    dist.all_reduce(y, group=group)
    return y

  @staticmethod
  def backward(ctx, g):
    g = g.contiguous().clone()
    dist.all_reduce(g, group=ctx.group)
    return g, None


def tp_rms_norm_rope(x, w, cos, sin, heads_local: int, eps: float, group, full_dim: int):
  """RMSNorm over ALL heads of the model (`full_dim` channels, of which this rank holds x.shape[-1]) followed by RoPE:
  the sum of squares of the local slice is summed over the tensor group (reference: the norm spans the `heads` axis
  that the `tensor` mesh axis shards, src/maxdiffusion/models/attention_flax.py:2468-2525)."""
  from ..ops import ref

  B, S, C = x.shape
  xf = x.float()
  ss = (xf * xf).sum(-1, keepdim=True)
  if group is not None:
    ss = _AllReduceSum.apply(ss, group)
  y = xf * torch.rsqrt(ss / full_dim + eps)
  if w is not None:
    y = y * w.float()
  y = y.view(B, S, heads_local, C // heads_local)
  if cos is not None:
    y = ref.rope_rotate(y, cos, sin)
  return y.to(x.dtype)


def _column(lin, group, chunks=1):
  new = ColumnParallelLinear(lin.in_features, lin.out_features, bias=lin.bias is not None, group=group, chunks=chunks)
  new = new.to(device=lin.weight.device, dtype=lin.weight.dtype)
  new.load_full(lin.weight.data, None if lin.bias is None else lin.bias.data)
  return new


def _row(lin, group):
  new = RowParallelLinear(lin.in_features, lin.out_features, bias=lin.bias is not None, group=group)
  new = new.to(device=lin.weight.device, dtype=lin.weight.dtype)
  new.load_full(lin.weight.data, None if lin.bias is None else lin.bias.data)
  return new


def apply_tensor_parallel_wan(model, group) -> int:
  """Shards every block of a `WanModel` over `group` in place: attention heads (q / k / v column-parallel, output
  projection row-parallel, the across-heads RMSNorm with a summed statistic) and FFN units (up column-, down
  row-parallel). Every rank must hold the same full weights when this is called. Returns the group size."""
  n, r = _size_rank(group)
  if n == 1:
    return 1
  for blk in model.blocks:
    for attn, fused, chunks in ((blk.attn1, "to_qkv", 3), (blk.attn2, "to_kv", 2)):
      heads = attn.heads
      if heads % n != 0:
        raise ValueError(f"{heads} attention heads cannot be split over {n} tensor ranks")
      dim = attn.to_out.in_features
      setattr(attn, fused, _column(getattr(attn, fused), group, chunks))
      if fused == "to_kv":
        attn.to_q = _column(attn.to_q, group)
        if getattr(attn, "has_image", False):
          attn.add_kv_proj = _column(attn.add_kv_proj, group, 2)
          attn.norm_added_k = torch.nn.Parameter(attn.norm_added_k.data[r * dim // n:(r + 1) * dim // n].clone())
      attn.to_out = _row(attn.to_out, group)
      for name in ("norm_q", "norm_k"):
        w = getattr(attn, name)
        setattr(attn, name, torch.nn.Parameter(w.data[r * dim // n:(r + 1) * dim // n].clone()))
      attn.heads = heads // n
      attn.tp_group, attn.tp_full_dim = group, dim
    blk.ffn_in = _column(blk.ffn_in, group)
    blk.ffn_out = _row(blk.ffn_out, group)
  model.tp_group = group
  return n


# ---- full <-> per-rank parameter layout (checkpoints of tensor-parallel runs) -----------------------------------------
def tensor_parallel_specs(block) -> dict:
  """name -> (kind, chunks) for every parameter of `block` that holds a slice of the full tensor: "col" = rows
  [out, ...] split (per chunk of a fused projection), "row" = columns split. Parameters that are not listed are
  replicated over the tensor ranks."""
  specs = {}
  for mod_name, mod in block.named_modules():
    prefix = f"{mod_name}." if mod_name else ""
    if isinstance(mod, ColumnParallelLinear):
      specs[prefix + "weight"] = ("col", mod.chunks)
      if mod.bias is not None:
        specs[prefix + "bias"] = ("col", mod.chunks)
    elif isinstance(mod, RowParallelLinear):
      specs[prefix + "weight"] = ("row", 1)
    if getattr(mod, "tp_group", None) is not None:
      for nm in ("norm_q", "norm_k", "norm_added_k"):
        if isinstance(getattr(mod, nm, None), nn.Parameter):
          specs[prefix + nm] = ("col", 1)
  return specs


def shard_of_full(full: torch.Tensor, spec, n: int, r: int) -> torch.Tensor:
  """Rank r's slice (of n) of a full parameter."""
  if spec is None or n == 1:
    return full
  kind, chunks = spec
  if kind == "row":
    loc = full.shape[1] // n
    return full[:, r * loc:(r + 1) * loc]
  per = full.shape[0] // chunks
  loc = per // n
  return torch.cat([full[c * per + r * loc:c * per + (r + 1) * loc] for c in range(chunks)], dim=0)


def full_from_shards(parts, spec) -> torch.Tensor:
  """Inverse of `shard_of_full` over the slices of all ranks, in rank order."""
  if spec is None or len(parts) == 1:
    return parts[0]
  kind, chunks = spec
  if kind == "row":
    return torch.cat(list(parts), dim=1)
  loc = parts[0].shape[0] // chunks
  return torch.cat([p[c * loc:(c + 1) * loc] for c in range(chunks) for p in parts], dim=0)


def gather_full(local: torch.Tensor, spec, group) -> torch.Tensor:
  """All ranks of `group` call this with their slice; every rank gets the full parameter."""
  n, _ = _size_rank(group)
  if spec is None or n == 1:
    return local
  parts = [torch.empty_like(local) for _ in range(n)]
  dist.all_gather(parts, local.contiguous(), group=group)
  return full_from_shards(parts, spec)
