"""Tensor parallelism over the mesh's `tensor` axis: column-parallel and row-parallel linears (Megatron layout).

The reference shards `heads` / `mlp` kernels over the `tensor` mesh axis and lets XLA insert the all-reduce
(logical axis rules in src/maxdiffusion/configs/base_wan_14b.yml:204-222, src/maxdiffusion/common_types.py:72-110).
Here the two halves are explicit:

  * `ColumnParallelLinear`: weight rows (output features) split over the group; input replicated, output sharded;
    backward all-reduces the input gradient;
  * `RowParallelLinear`: weight columns (input features) split; input sharded, partial outputs summed over the
    group. With peer memory the sum is `parallel.symm`'s pull-reduce over symmetric buffers, else an NCCL all-reduce;
  * `shard_attention_heads` / `shard_mlp` split an existing block's fused projections in place.
GEMMs run on the tcgen05 kernel (`ops.functional.linear`); only the reduction crosses NVLink.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as OF


class _CopyToGroup(torch.autograd.Function):
  """Identity forward, all-reduce backward (input of a column-parallel layer)."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return x

  @staticmethod
  def backward(ctx, g):
    if ctx.group is not None:
      g = g.contiguous()
      dist.all_reduce(g, group=ctx.group)
    return g, None


class _ReduceFromGroup(torch.autograd.Function):
  """All-reduce forward, identity backward (output of a row-parallel layer)."""

  @staticmethod
  def forward(ctx, x, group):
    if group is not None:
      x = x.contiguous()
      dist.all_reduce(x, group=group)
    return x

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
    y = _ReduceFromGroup.apply(OF.linear(x, self.weight, None), self.group)
    return y + self.bias.to(y.dtype) if self.bias is not None else y


def parallel_mlp(dim: int, hidden: int, group=None):
  """(up, down) projections of a feed-forward block split over `group`: hidden units are sharded."""
  return ColumnParallelLinear(dim, hidden, group=group), RowParallelLinear(hidden, dim, group=group)


def parallel_attention_projections(dim: int, group=None):
  """(fused qkv, out) projections split by heads: every rank computes attention for heads/n heads."""
  return ColumnParallelLinear(dim, 3 * dim, group=group, chunks=3), RowParallelLinear(dim, dim, group=group)
