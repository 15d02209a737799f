"""Fully-sharded parameters with the optimizer step taken inside the backward pass.

The reference shards every Wan weight over the `('context', 'fsdp')` mesh axes and lets XLA insert the
all-gather before use, the reduce-scatter of the gradients and the optax update
(src/maxdiffusion/configs/base_wan_14b.yml:217, src/maxdiffusion/trainers/wan_trainer.py:116-189,
src/maxdiffusion/max_utils.py:683-696). Here the unit of sharding is a transformer block:

  * the parameters of a block live in ONE flat bf16 buffer; each rank owns 1/W of it (`shard`), together with the
    AdamW moments of that slice;
  * before a block runs (forward, or recomputation in backward) its flat buffer is all-gathered into one of two
    rotating full-size slots on a side stream, one block ahead of the compute stream;
  * when the backward of a block ends, its gradients are packed into a flat buffer, reduce-scattered (sum) to
    the owners, the gradient statistics (sum of squares, max-abs) are accumulated, and — unless global-norm
    clipping needs the whole gradient first — the fused AdamW kernel updates the owner's slice at once, so no
    full-model gradient is ever resident.

With one rank the same code runs without communication (the slot is the shard itself).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import kernels as K
from ..ops import ref

def _library_mode() -> bool:
  from ..ops import functional as OF

  return OF.library_mode()


_ALIGN = 64  # elements; keeps every parameter view 128-byte aligned (TMA needs 16)


@dataclass
class AdamWConfig:
  lr: float = 1e-5
  b1: float = 0.9
  b2: float = 0.999
  eps: float = 1e-8
  weight_decay: float = 0.0
  clip_value: float = 0.0        # > 0: clip each gradient element to [-v, v]  (opt_enable_grad_clipping)
  clip_global_norm: float = 0.0  # > 0: scale gradients so that their global L2 norm is at most this
  state_dtype: torch.dtype = torch.bfloat16
  stochastic_rounding: bool = True


def lr_schedule(step: int, base_lr: float, schedule_steps: int, warmup_fraction: float) -> float:
  """Linear warm-up from 0 over `warmup_fraction * schedule_steps`, then constant
  (reference: src/maxdiffusion/max_utils.py:658-680)."""
  warmup = int(schedule_steps * warmup_fraction)
  if warmup > 0 and step < warmup:
    return base_lr * step / warmup
  return base_lr


class FlatParamGroup:
  """Parameters of one module packed into a flat buffer of `dtype`; the parameters become views of it."""

  def __init__(self, params: Sequence[nn.Parameter], world: int, dtype: torch.dtype, device):
    self.params = list(params)
    self.shapes = [p.shape for p in self.params]
    self.offsets = []
    off = 0
    for p in self.params:
      self.offsets.append(off)
      off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
    unit = world * _ALIGN
    self.numel = max(unit, (off + unit - 1) // unit * unit)
    self.dtype, self.device, self.world = dtype, device, world
    self.shard_numel = self.numel // world
    # alignment gaps and the tail are not covered by any parameter; they are zeroed whenever gradients are packed
    self.gaps = []
    for p, o in zip(self.params, self.offsets):
      end = o + p.numel()
      nxt = (end + _ALIGN - 1) // _ALIGN * _ALIGN
      if nxt > end:
        self.gaps.append((end, nxt))
    if self.numel > off:
      self.gaps.append((off, self.numel))

  def pack_from_params(self) -> torch.Tensor:
    flat = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
    for p, off in zip(self.params, self.offsets):
      flat[off:off + p.numel()].copy_(p.detach().reshape(-1))
    return flat

  def views(self, flat: torch.Tensor) -> list[torch.Tensor]:
    return [flat[off:off + math.prod(s)].view(s) for off, s in zip(self.offsets, self.shapes)]

  def point_params_to(self, flat: torch.Tensor) -> None:
    for p, v in zip(self.params, self.views(flat)):
      p.data = v

  def pack_grads(self, flat_grad: torch.Tensor) -> None:
    """Copies every parameter's .grad into `flat_grad` (zeros for unused parameters) and frees the .grad."""
    views = self.views(flat_grad)
    dst, src = [], []
    for p, v in zip(self.params, views):
      if p.grad is None:
        v.zero_()
      else:
        dst.append(v)
        src.append(p.grad.to(flat_grad.dtype) if p.grad.dtype != flat_grad.dtype else p.grad)
    if dst:
      torch._foreach_copy_(dst, src)
    for a, b in self.gaps:
      flat_grad[a:b].zero_()
    for p in self.params:
      p.grad = None


class FSDPEngine:

  def __init__(self, blocks: Sequence[nn.Module], root_params: Sequence[nn.Parameter], opt: AdamWConfig, *,
               group=None, replica_group=None, device=None, param_dtype=torch.bfloat16, seed: int = 0,
               train: bool = True, peer_memory: bool = False):
    self.blocks = list(blocks)
    self.opt = opt
    self.group, self.replica_group = group, replica_group
    self.world = dist.get_world_size(group) if group is not None else 1
    self.rank = dist.get_rank(group) if group is not None else 0
    self.device = device if device is not None else next(self.blocks[0].parameters()).device
    self.on_cuda = torch.device(self.device).type == "cuda"
    self.param_dtype = param_dtype
    self.seed = seed
    self.step_count = 0
    self.lr = opt.lr
    self.train = train

    self.groups = [FlatParamGroup(list(b.parameters()), self.world, param_dtype, self.device) for b in self.blocks]
    self.root = FlatParamGroup(list(root_params), 1, param_dtype, self.device)
    self.max_numel = max(g.numel for g in self.groups)

    # owner shards (the persistent copy of the weights) and optimizer moments
    self.shards = []
    for g in self.groups:
      flat = g.pack_from_params()
      shard = flat[self.rank * g.shard_numel:(self.rank + 1) * g.shard_numel].clone() if self.world > 1 else flat
      self.shards.append(shard)
      for p in g.params:  # drop the original storage
        p.data = torch.empty(0, dtype=param_dtype, device=self.device)
    self.root_flat = self.root.pack_from_params()
    self.root.point_params_to(self.root_flat)
    if train:
      sd = opt.state_dtype
      self.m = [torch.zeros_like(s, dtype=sd) for s in self.shards]
      self.v = [torch.zeros_like(s, dtype=sd) for s in self.shards]
      self.root_m = torch.zeros_like(self.root_flat, dtype=sd)
      self.root_v = torch.zeros_like(self.root_flat, dtype=sd)
      self.grad_stats = torch.zeros(2, dtype=torch.float32, device=self.device)
      self.pending: list[tuple[int, torch.Tensor]] = []  # shard grads kept for global-norm clipping

    self.peer = None
    self._small_ar = None
    if self.world > 1:
      self.slots = [torch.empty(self.max_numel, dtype=param_dtype, device=self.device) for _ in range(2)]
      self.grad_slots = [torch.zeros(self.max_numel, dtype=param_dtype, device=self.device) for _ in range(2)] if train else []
      if peer_memory and train and self.on_cuda and param_dtype == torch.bfloat16:
        from . import symm

        if symm.peer_memory_available(group):
          self.peer = symm.PeerGroup(group)
          self._small_ar = symm.SmallAllReduce(self.peer)
          self.sym_grad, self.sym_grad_ptrs = [], []
          for _ in range(2):
            t, ptrs, _h = self.peer.alloc(self.max_numel, param_dtype)
            t.zero_()
            self.sym_grad.append(t)
            self.sym_grad_ptrs.append(ptrs)
          self.grad_slots = self.sym_grad
          self.rs_scratch = torch.empty(2 * 64, dtype=torch.float32, device=self.device)
          self.grad_epoch = 0
          # the owner shards move into one symmetric buffer so that peers can pull them: the parameter all-gather
          # of a block is then one kernel of this repository (`symm.pull_gather`) instead of an NCCL collective
          offs, total = [], 0
          for sh in self.shards:
            offs.append(total)
            total += -(-sh.numel() // 8) * 8
          sym, ptrs, _h = self.peer.alloc(total, param_dtype)
          for k, sh in enumerate(self.shards):
            view = sym[offs[k]:offs[k] + sh.numel()]
            view.copy_(sh)
            self.shards[k] = view
          self.sym_shards, self.shard_ptrs, self.shard_offs = sym, ptrs, offs
          self.shards_version = 0  # optimizer steps whose updates are complete in `sym_shards`
          torch.cuda.synchronize()
          dist.barrier(group=group)
      self.comm_stream = torch.cuda.Stream() if self.on_cuda else None
      self.gather_done = [None, None]
      self.slot_block = [-1, -1]
      self.grad_slot_free = [None, None]
      self.grad_use = 0
    else:
      for g, s in zip(self.groups, self.shards):
        g.point_params_to(s)
      self.flat_grad = torch.empty(self.max_numel, dtype=param_dtype, device=self.device) if train else None

  # ------------------------------------------------------------------ gathering
  def _issue_gather(self, i: int) -> None:
    slot = i % 2
    if self.slot_block[slot] == i:
      return
    g = self.groups[i]
    full = self.slots[slot][:g.numel]
    if self.on_cuda:
      ready = torch.cuda.Event()
      ready.record()  # everything enqueued so far (the previous user of this slot included)
      with torch.cuda.stream(self.comm_stream):
        self.comm_stream.wait_event(ready)
        if self.peer is not None:
          from . import symm

          # every owner has finished the optimizer step that this gather must see (the flag carries its step count)
          self.peer.wait(symm.FLAG_SHARD_READY, self.shards_version)
          esz = self.shards[i].element_size()
          symm.pull_gather([p + self.shard_offs[i] * esz for p in self.shard_ptrs], full, g.shard_numel * esz, ctas=12)
        else:
          dist.all_gather_into_tensor(full, self.shards[i], group=self.group)
        done = torch.cuda.Event()
        done.record()
      self.gather_done[slot] = done
    else:
      dist.all_gather_into_tensor(full, self.shards[i], group=self.group)
    self.slot_block[slot] = i

  def materialize(self, i: int, prefetch: Optional[int] = None) -> None:
    """Makes block i's parameters usable on the compute stream and starts fetching block `prefetch`."""
    if self.world == 1:
      return
    self._issue_gather(i)
    slot = i % 2
    if self.on_cuda and self.gather_done[slot] is not None:
      torch.cuda.current_stream().wait_event(self.gather_done[slot])
    self.groups[i].point_params_to(self.slots[slot][:self.groups[i].numel])
    if prefetch is not None and 0 <= prefetch < len(self.blocks):
      self._issue_gather(prefetch)

  def block_hook(self, i: int, phase: str) -> None:
    """Called by the model: phase is 'forward', 'recompute' (start of a block's backward) or 'backward_done'."""
    if phase == "forward":
      self.materialize(i, prefetch=i + 1)
    elif phase == "recompute":
      self.materialize(i, prefetch=i - 1)
    elif phase == "backward_done":
      self.reduce_and_step(i)

  # ------------------------------------------------------------------ optimizer
  def begin_step(self, lr: Optional[float] = None) -> None:
    self.step_count += 1
    if lr is not None:
      self.lr = lr
    self.grad_stats.zero_()
    self.pending.clear()

  def _adamw(self, p, g, m, v, grad_scale: float, salt: int) -> None:
    o = self.opt
    kw = dict(lr=self.lr, b1=o.b1, b2=o.b2, eps=o.eps, wd=o.weight_decay, step=self.step_count, grad_scale=grad_scale,
              clip_value=o.clip_value)
    if p.is_cuda and not _library_mode():
      K.adamw(p, g, m, v, seed=(self.seed * 1000003 + self.step_count) * 4099 + salt,
              stochastic=o.stochastic_rounding, **kw)
    else:
      ref.adamw_step(p, g, m, v, **kw)

  def _stats(self, g: torch.Tensor) -> None:
    if g.is_cuda and not _library_mode():
      K.sumsq_maxabs(g, out=self.grad_stats, accumulate=True)
    else:
      s = ref.sumsq_maxabs(g)
      self.grad_stats[0] += s[0]
      self.grad_stats[1] = torch.maximum(self.grad_stats[1], s[1])

  def reduce_and_step(self, i: int) -> None:
    """Gradient of block i: pack -> reduce-scatter -> statistics -> AdamW on the owned slice."""
    g = self.groups[i]
    deferred = self.opt.clip_global_norm > 0
    if self.world == 1:
      flat = self.flat_grad[:g.numel]
      g.pack_grads(flat)
      if self.replica_group is not None:
        dist.all_reduce(flat, group=self.replica_group)
      self._stats(flat)
      if deferred:
        self.pending.append((i, flat.clone()))
      else:
        self._adamw(self.shards[i], flat, self.m[i], self.v[i], 1.0, i)
      return
    if self.peer is not None:
      return self._reduce_and_step_peer(i)
    slot = self.grad_use % 2
    self.grad_use += 1
    full = self.grad_slots[slot][:g.numel]
    if self.on_cuda and self.grad_slot_free[slot] is not None:
      torch.cuda.current_stream().wait_event(self.grad_slot_free[slot])
    g.pack_grads(full)
    shard_grad = torch.empty(g.shard_numel, dtype=self.param_dtype, device=self.device)
    if self.on_cuda:
      ready = torch.cuda.Event()
      ready.record()
      with torch.cuda.stream(self.comm_stream):
        self.comm_stream.wait_event(ready)
        shard_grad.record_stream(self.comm_stream)
        dist.reduce_scatter_tensor(shard_grad, full, group=self.group)
        free = torch.cuda.Event()
        free.record()
        self.grad_slot_free[slot] = free
        if self.replica_group is not None:
          dist.all_reduce(shard_grad, group=self.replica_group)
        self._stats(shard_grad)
        if deferred:
          self.pending.append((i, shard_grad))
        else:
          self._adamw(self.shards[i], shard_grad, self.m[i], self.v[i], 1.0, i)
      # the updated shard invalidates any gathered copy of this block
      for s in range(2):
        if self.slot_block[s] == i:
          self.slot_block[s] = -1
    else:
      dist.reduce_scatter_tensor(shard_grad, full, group=self.group)
      if self.replica_group is not None:
        dist.all_reduce(shard_grad, group=self.replica_group)
      self._stats(shard_grad)
      if deferred:
        self.pending.append((i, shard_grad))
      else:
        self._adamw(self.shards[i], shard_grad, self.m[i], self.v[i], 1.0, i)
      for s in range(2):
        if self.slot_block[s] == i:
          self.slot_block[s] = -1

  def _reduce_and_step_peer(self, i: int) -> None:
    """Peer-memory path: gradients are packed into a symmetric buffer and every owner pulls, sums and applies its
    slice with one fused kernel (`symm.rs_adamw`); no NCCL collective is involved."""
    from . import symm

    g = self.groups[i]
    # With replicas (a `data` axis), the reduced slice still has to be summed over the replica group before the
    # statistics and the update may see it, so the kernel only reduces and the rest follows the all-reduce.
    replicated = self.replica_group is not None
    deferred = self.opt.clip_global_norm > 0
    fused_apply = not deferred and not replicated
    e = self.grad_epoch = self.peer.next_epoch(symm.FLAG_GRAD_READY)
    slot = e % 2
    self.peer.wait(symm.FLAG_GRAD_ACK, e - 2)           # everyone has consumed the previous content of this slot
    g.pack_grads(self.sym_grad[slot][:g.numel])
    self.peer.signal(symm.FLAG_GRAD_READY, e)
    ready = torch.cuda.Event()
    ready.record()
    o = self.opt
    with torch.cuda.stream(self.comm_stream):
      self.comm_stream.wait_event(ready)
      self.peer.wait(symm.FLAG_GRAD_READY, e)
      off_bytes = self.rank * g.shard_numel * 2
      ptrs = [base + off_bytes for base in self.sym_grad_ptrs[slot]]
      reduced = None
      if not fused_apply:
        reduced = torch.empty(g.shard_numel, dtype=self.param_dtype, device=self.device)
        reduced.record_stream(self.comm_stream)
      # the statistics of a slice that is not final yet (replicas pending) go to a throw-away accumulator
      stats = self.grad_stats if not replicated else torch.zeros_like(self.grad_stats)
      symm.rs_adamw(ptrs, g.shard_numel, self.shards[i], self.m[i], self.v[i], stats, self.rs_scratch,
                    lr=self.lr, b1=o.b1, b2=o.b2, eps=o.eps, wd=o.weight_decay, step=self.step_count,
                    clip_value=o.clip_value,
                    seed=(self.seed * 1000003 + self.step_count) * 4099 + i,
                    stochastic=o.stochastic_rounding, apply=fused_apply, reduced_out=reduced, ctas=64)
      self.peer.signal(symm.FLAG_GRAD_ACK, e)
      if replicated:
        dist.all_reduce(reduced, group=self.replica_group)
        self._stats(reduced)
      if deferred:
        self.pending.append((i, reduced))
      elif replicated:
        self._adamw(self.shards[i], reduced, self.m[i], self.v[i], 1.0, i)
    for s in range(2):
      if self.slot_block[s] == i:
        self.slot_block[s] = -1

  def finish_step(self, model_group=None) -> dict:
    """Root (replicated) parameters, deferred clipped updates, and the step's gradient metrics."""
    if self.world > 1 and self.on_cuda:
      torch.cuda.current_stream().wait_stream(self.comm_stream)
    root_grad = torch.empty_like(self.root_flat)
    self.root.pack_grads(root_grad)
    if model_group is not None:
      dist.all_reduce(root_grad, group=model_group)
    if self.replica_group is not None:
      dist.all_reduce(root_grad, group=self.replica_group)
    stats = self.grad_stats.clone()
    if self.group is not None and self.peer is not None:
      # one-launch peer-memory all-reduces (sum of squares, max-abs); identical bits on every rank
      stats = torch.cat([self._small_ar(stats[0:1].contiguous(), "sum"), self._small_ar(stats[1:2].contiguous(), "max")])
    elif self.group is not None:
      sq, mx = stats[0:1].clone(), stats[1:2].clone()
      dist.all_reduce(sq, group=self.group)
      dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.group)
      stats = torch.cat([sq, mx])
    root_stats = K.sumsq_maxabs(root_grad) if (root_grad.is_cuda and not _library_mode()) else ref.sumsq_maxabs(root_grad)
    total_sq = stats[0] + root_stats[0]
    max_abs = torch.maximum(stats[1], root_stats[1])
    grad_norm = total_sq.sqrt()
    scale = 1.0
    if self.opt.clip_global_norm > 0:
      scale = float(min(1.0, self.opt.clip_global_norm / (grad_norm.item() + 1e-6)))
      for i, sg in self.pending:
        self._adamw(self.shards[i], sg, self.m[i], self.v[i], scale, i)
      self.pending.clear()
    self._adamw(self.root_flat, root_grad, self.root_m, self.root_v, scale, 7919)
    if self.world > 1 and self.peer is not None:
      # every shard of this rank now holds the weights of step `step_count`: peers may gather them. (A peer cannot
      # still be reading the old values: it published its gradient of a block only after its last use of the block.)
      from . import symm

      self.shards_version = self.step_count
      self.peer.signal(symm.FLAG_SHARD_READY, self.shards_version)
    return {"grad_norm": grad_norm, "max_abs_grad": max_abs}

  # ------------------------------------------------------------------ state access
  def full_block_flat(self, i: int) -> torch.Tensor:
    if self.world == 1:
      return self.shards[i]
    full = torch.empty(self.groups[i].numel, dtype=self.param_dtype, device=self.device)
    dist.all_gather_into_tensor(full, self.shards[i], group=self.group)
    return full

  def gather_state_dict(self, names_per_block: Sequence[Sequence[str]], root_names: Sequence[str]) -> dict:
    """Full (unsharded) parameters by name; collective when sharded."""
    out = {}
    for i, (g, names) in enumerate(zip(self.groups, names_per_block)):
      full = self.full_block_flat(i)
      for n, v in zip(names, g.views(full)):
        out[n] = v.clone()
    for n, v in zip(root_names, self.root.views(self.root_flat)):
      out[n] = v.clone()
    return out

  def load_full_block(self, i: int, tensors: Sequence[torch.Tensor]) -> None:
    g = self.groups[i]
    flat = torch.zeros(g.numel, dtype=self.param_dtype, device=self.device)
    for t, off in zip(tensors, g.offsets):
      flat[off:off + t.numel()].copy_(t.reshape(-1))
    if self.world == 1:
      self.shards[i].copy_(flat)
    else:
      self.shards[i].copy_(flat[self.rank * g.shard_numel:(self.rank + 1) * g.shard_numel])
      self.slot_block = [-1, -1]
      if self.peer is not None:
        # peers pull this shard without a collective: it has to be complete before any of them gathers it
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

  def optimizer_state(self) -> dict:
    return {"step": self.step_count, "m": self.m, "v": self.v, "root_m": self.root_m, "root_v": self.root_v}

  def load_optimizer_state(self, state: dict) -> None:
    self.step_count = int(state["step"])
    for dst, src in zip(self.m, state["m"]):
      dst.copy_(src)
    for dst, src in zip(self.v, state["v"]):
      dst.copy_(src)
    self.root_m.copy_(state["root_m"])
    self.root_v.copy_(state["root_v"])


class FlatShardedOptimizer:
  """AdamW over ALL parameters of a model as one flat buffer, with gradient and optimizer-state sharding (ZeRO-2).

  For models without a uniform block structure (UNet, VAE, text encoders): parameters stay resident (replicated),
  gradients are packed, reduce-scattered over `group`, every rank updates its slice with the fused AdamW kernel and
  the updated slices are all-gathered back into the flat parameter buffer. With one rank it is a plain fused AdamW.
  """

  def __init__(self, params: Sequence[nn.Parameter], opt: AdamWConfig, group=None, seed: int = 0):
    params = [p for p in params if p.requires_grad]
    self.opt, self.group, self.seed = opt, group, seed
    self.world = dist.get_world_size(group) if group is not None else 1
    self.rank = dist.get_rank(group) if group is not None else 0
    device, dtype = params[0].device, params[0].dtype
    self.flat_group = FlatParamGroup(params, self.world, dtype, device)
    self.flat = self.flat_group.pack_from_params()
    self.flat_group.point_params_to(self.flat)
    n = self.flat_group.shard_numel
    self.m = torch.zeros(n, dtype=opt.state_dtype if dtype == torch.bfloat16 else torch.float32, device=device)
    self.v = torch.zeros_like(self.m)
    self.grad = torch.zeros(self.flat_group.numel, dtype=dtype, device=device)
    self.step_count = 0
    self.lr = opt.lr

  def step(self, lr: Optional[float] = None) -> dict:
    from . import collectives as C

    self.step_count += 1
    if lr is not None:
      self.lr = lr
    g = self.flat_group
    g.pack_grads(self.grad)
    n = g.shard_numel
    if self.world > 1:
      shard_grad = torch.empty(n, dtype=self.grad.dtype, device=self.grad.device)
      C.reduce_scatter_flat(shard_grad, self.grad, self.group)
      shard_grad.div_(self.world)
    else:
      shard_grad = self.grad
    stats = K.sumsq_maxabs(shard_grad) if shard_grad.is_cuda and shard_grad.dtype in (torch.bfloat16, torch.float32) else ref.sumsq_maxabs(shard_grad)
    if self.group is not None:
      sq, mx = stats[0:1].clone(), stats[1:2].clone()
      dist.all_reduce(sq, group=self.group)
      dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.group)
      stats = torch.cat([sq, mx])
    norm = stats[0].sqrt()
    scale = 1.0
    if self.opt.clip_global_norm > 0:
      scale = float(min(1.0, self.opt.clip_global_norm / (norm.item() + 1e-6)))
    p = self.flat[self.rank * n:(self.rank + 1) * n]
    o = self.opt
    kw = dict(lr=self.lr, b1=o.b1, b2=o.b2, eps=o.eps, wd=o.weight_decay, step=self.step_count, grad_scale=scale,
              clip_value=o.clip_value)
    if p.is_cuda and p.dtype == torch.bfloat16:
      K.adamw(p, shard_grad, self.m, self.v, seed=self.seed * 7919 + self.step_count, stochastic=o.stochastic_rounding, **kw)
    else:
      ref.adamw_step(p, shard_grad, self.m, self.v, **kw)
    if self.world > 1:
      dist.all_gather_into_tensor(self.flat, p.clone(), group=self.group)
    return {"grad_norm": norm, "max_abs_grad": stats[1]}
