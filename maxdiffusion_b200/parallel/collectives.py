"""Collective helpers that behave the same on NCCL (GPU) and Gloo (CPU tests).

These are the library-collective baseline of every communication site; the fused peer-memory kernels in
`parallel.symm` replace them on the hot paths and are A/B-timed against them.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _is_gloo(group) -> bool:
  return dist.get_backend(group) == "gloo"


def group_size(group) -> int:
  return dist.get_world_size(group) if group is not None else 1


def all_gather_cat(x: torch.Tensor, group, dim: int = 0) -> torch.Tensor:
  """Concatenation of every rank's `x` along `dim` (equal shapes)."""
  n = group_size(group)
  if n == 1:
    return x
  out = all_gather_stack(x, group)
  if dim == 0:
    return out.reshape((n * x.shape[0],) + tuple(x.shape[1:]))
  return torch.cat(list(out.unbind(0)), dim=dim)


def all_gather_stack(x: torch.Tensor, group) -> torch.Tensor:
  """[n, *x.shape] with the ranks' tensors stacked on a new leading axis."""
  n = group_size(group)
  x = x.contiguous()
  if n == 1:
    return x.unsqueeze(0)
  if x.dim() == 0:
    x = x.reshape(1)
  # the concatenated form of the output is the one every backend accepts
  out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
  dist.all_gather_into_tensor(out, x, group=group)
  return out.view((n,) + tuple(x.shape))


def reduce_scatter_stack(x: torch.Tensor, group) -> torch.Tensor:
  """x: [n, ...] where slice r is this rank's contribution to rank r; returns the sum of everyone's slice for me."""
  n = group_size(group)
  if n == 1:
    return x[0]
  x = x.contiguous()
  if _is_gloo(group):
    dist.all_reduce(x, group=group)
    return x[dist.get_rank(group)].clone()
  out = torch.empty(tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
  dist.reduce_scatter_tensor(out, x, group=group)
  return out


def reduce_scatter_flat(out: torch.Tensor, full: torch.Tensor, group) -> None:
  if _is_gloo(group):
    dist.all_reduce(full, group=group)
    r, n = dist.get_rank(group), dist.get_world_size(group)
    out.copy_(full.view(n, -1)[r])
  else:
    dist.reduce_scatter_tensor(out, full, group=group)


def all_to_all_heads_to_seq(x: torch.Tensor, group) -> torch.Tensor:
  """[B, S_loc, H, D] sequence-sharded -> [B, S_loc*n, H/n, D] head-sharded (the Ulysses exchange)."""
  n = group_size(group)
  if n == 1:
    return x
  B, S, H, D = x.shape
  send = x.reshape(B, S, n, H // n, D).permute(2, 0, 1, 3, 4).contiguous()  # [n, B, S, H/n, D]
  recv = torch.empty_like(send)
  dist.all_to_all_single(recv, send, group=group)
  return recv.permute(1, 0, 2, 3, 4).reshape(B, n * S, H // n, D)


def all_to_all_seq_to_heads(x: torch.Tensor, group) -> torch.Tensor:
  """Inverse of `all_to_all_heads_to_seq`: [B, S, H/n, D] -> [B, S/n, H, D]."""
  n = group_size(group)
  if n == 1:
    return x
  B, S, Hn, D = x.shape
  send = x.reshape(B, n, S // n, Hn, D).permute(1, 0, 2, 3, 4).contiguous()  # [n, B, S/n, H/n, D]
  recv = torch.empty_like(send)
  dist.all_to_all_single(recv, send, group=group)
  return recv.permute(1, 2, 0, 3, 4).reshape(B, S // n, n * Hn, D)
