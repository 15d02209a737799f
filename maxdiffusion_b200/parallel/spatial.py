"""Spatial parallelism of the VAE: every rank of a group decodes a vertical strip of the frame.

Channels-last activations [.., H, W, C] are split along W. A 3x3 (or 3x3x3) convolution of a strip needs one column
of each neighbouring strip; `HaloExchange.fill` puts them into the halo columns of a tensor that was produced with
room for them ([.., H, W_local + 2, C]), and the convolution kernels read the halo without producing output for it
(`ops.conv.conv3d_causal(halo=1)`). The columns beyond the first / last strip are zeros: the padding the unsharded
convolution reads there. Everything between two convolutions (norms, activations, 1x1 convolutions, the time
up-sampling) is per pixel and needs no exchange; the single-head attention of the mid block gathers the frame.

Reference: the `vae_spatial` mesh axis and the activation sharding of the Wan VAE
(src/maxdiffusion/pipelines/wan/wan_pipeline.py:560-640, src/maxdiffusion/models/wan/autoencoder_kl_wan.py:70-147, where
the halo traffic is whatever the XLA partitioner emits for a convolution over a sharded axis).

Transport. Over peer memory every rank copies its two edge columns into a symmetric buffer (two alternating slots),
signals its neighbours, waits for theirs and pulls their columns with one copy kernel per side; an ACK flag two
exchanges later frees the slot. Each wait is bounded and reports through the device status word. Without peer memory
(CPU ranks, or a group that spans hosts) the columns travel as point-to-point sends of the process group.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import collectives as C


class HaloExchange:

  def __init__(self, group, peer_memory: bool = True):
    self.group = group
    self.size = C.group_size(group)
    self.rank = dist.get_rank(group) if self.size > 1 else 0
    self.left = self.rank - 1 if self.rank > 0 else None
    self.right = self.rank + 1 if self.rank < self.size - 1 else None
    self.peer = None
    self._buf = None
    self._cap = 0
    self.exchanges = 0  # how many halo fills ran (tests, profiles)
    if peer_memory and self.size > 1 and torch.cuda.is_available():
      from . import symm

      if symm.peer_memory_available(group):
        self.peer = symm.PeerGroup(group)

  # ---- sharding --------------------------------------------------------------------------------
  def shard(self, x: torch.Tensor, dim: int = -2) -> torch.Tensor:
    """This rank's strip of a replicated tensor (the width must divide by the group size)."""
    W = x.shape[dim]
    if W % self.size:
      raise ValueError(f"width {W} does not divide over {self.size} ranks")
    per = W // self.size
    return x.narrow(dim, self.rank * per, per).contiguous()

  def gather(self, x: torch.Tensor, dim: int = -2) -> torch.Tensor:
    """The whole tensor from every rank's strip."""
    if self.size == 1:
      return x
    dim = dim % x.dim()
    stacked = C.all_gather_stack(x, self.group)  # [n, .., W_local, ..]
    return torch.cat(list(stacked.unbind(0)), dim=dim)

  # ---- halos -------------------------------------------------------------------------------------
  def extend(self, x: torch.Tensor) -> torch.Tensor:
    """[.., H, W, C] -> [.., H, W + 2, C] with the neighbours' edge columns (one extra copy of x; producers that can
    write into the interior of a wider tensor use `fill` on their own output instead)."""
    y = torch.empty((*x.shape[:-2], x.shape[-2] + 2, x.shape[-1]), dtype=x.dtype, device=x.device)
    y[..., 1:-1, :].copy_(x)
    return self.fill(y)

  def fill(self, y: torch.Tensor) -> torch.Tensor:
    """Fills the halo columns y[.., 0, :] and y[.., -1, :] in place from the neighbours' edge columns y[.., -2, :] and
    y[.., 1, :]; zeros at the outer sides of the frame. Every rank of the group calls it in the same order."""
    self.exchanges += 1
    if self.left is None:
      y[..., 0, :].zero_()
    if self.right is None:
      y[..., -1, :].zero_()
    if self.size == 1:
      return y
    if self.peer is not None and y.is_cuda:
      self._fill_peer(y)
    else:
      self._fill_p2p(y)
    return y

  def _fill_p2p(self, y):
    ops, recv = [], []
    for nbr, mine, theirs in ((self.left, 1, 0), (self.right, -2, -1)):
      if nbr is None:
        continue
      g = dist.get_global_rank(self.group, nbr) if self.group is not None else nbr
      buf = torch.empty_like(y[..., theirs, :]).contiguous()
      ops.append(dist.P2POp(dist.isend, y[..., mine, :].contiguous(), g, group=self.group))
      ops.append(dist.P2POp(dist.irecv, buf, g, group=self.group))
      recv.append((theirs, buf))
    for w in dist.batch_isend_irecv(ops):
      w.wait()
    for col, buf in recv:
      y[..., col, :].copy_(buf)

  def reserve(self, numel: int, dtype) -> None:
    """Sizes the symmetric edge buffers for edge columns of up to `numel` elements (every rank of the group, with
    the same numbers). A decode reserves once for its largest layer, so that no exchange has to grow them."""
    if self.peer is None or (self._buf is not None and self._cap >= numel and self._buf.dtype == dtype):
      return
    old = self._buf
    if old is not None:
      # neighbours may still be pulling from the old buffers: every rank drains its stream before any rank lets go
      torch.cuda.synchronize()
      dist.barrier(group=self.group)
    cap = (max(numel, 2 * self._cap) + 7) // 8 * 8
    # [slot][side][cap]: side 0 = my left edge column (read by the left neighbour), side 1 = my right edge column
    self._buf, self._ptrs, self._hdl = self.peer.alloc(4 * cap, dtype)
    self._cap = cap
    if old is not None:
      self.peer.release([old])
    torch.cuda.synchronize()
    dist.barrier(group=self.group)

  def _fill_peer(self, y):
    from . import symm

    peer = self.peer
    edge = y[..., 0, :]
    n, es = edge.numel(), y.element_size()
    self.reserve(n, y.dtype)
    buf = self._buf.view(2, 2, self._cap)
    nbrs = [r for r in (self.left, self.right) if r is not None]
    e = peer.next_epoch(symm.FLAG_HALO_READY)
    slot = e & 1
    # the slot's previous content (exchange e - 2) has been pulled by both neighbours (a fresh buffer has none, but
    # the acknowledgements of the exchanges before it were sent all the same)
    peer.wait(symm.FLAG_HALO_ACK, e - 2, sources=nbrs)
    buf[slot, 0, :n].view(edge.shape).copy_(y[..., 1, :])
    buf[slot, 1, :n].view(edge.shape).copy_(y[..., -2, :])
    peer.signal(symm.FLAG_HALO_READY, e, peers=nbrs)
    peer.wait(symm.FLAG_HALO_READY, e, sources=nbrs)
    for nbr, side, col in ((self.left, 1, 0), (self.right, 0, -1)):
      if nbr is None:
        continue
      tmp = torch.empty(edge.shape, dtype=y.dtype, device=y.device)
      symm.peer_copy(self._ptrs[nbr] + ((slot * 2 + side) * self._cap) * es, tmp, n * es, ctas=8)
      y[..., col, :].copy_(tmp)
    peer.signal(symm.FLAG_HALO_ACK, e, peers=nbrs)
