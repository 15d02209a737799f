"""Attention-kernel entry points under the names the reference's users import
(src/maxdiffusion/models/attention_flax.py:1589-1867 `KERNEL_REGISTRY`; src/maxdiffusion/kernels/*).

Every name of the reference's registry resolves to one of five strategies implemented in `parallel.context`
(`common_types.ATTENTION_KERNELS`): the distinction between `flash`, `tokamax_flash` and `cudnn_flash_te`, or
between `ulysses` and `ulysses_custom`, is a choice of TPU kernel library in the reference and has no counterpart
here: all of them run the tcgen05 flash kernel, with K/V moved over NVLink peer memory.

  make_splash_mha(...)            -> callable(q, k, v): local flash attention
  make_ring_attention(...)        -> callable(q, k, v): ring / gather context parallelism over a group
  make_custom_ring_attention(...) -> same as make_ring_attention (the reference's own ring kernel)
  get_attention_kernel(name, mesh)-> callable for any registry name
"""
from __future__ import annotations

from typing import Callable, Optional

from ..common_types import ATTENTION_KERNELS, FIXED_M_KERNELS, USP_KERNELS, context_strategy
from ..ops import functional as OF

KERNEL_REGISTRY = dict(ATTENTION_KERNELS)


def make_splash_mha(scale: Optional[float] = None, **unused_block_sizes) -> Callable:
  """Local attention. Block sizes are accepted for call compatibility only: the kernel works on pairs of 128-row
  query tiles against 64-key blocks (its TMEM layout); what `utils.tile_size_grid_search` chooses per shape is the
  depth of the K / V pipeline and the number of copy CTAs (`ops.kernels.load_flash_tuning`)."""
  return lambda q, k, v: OF.attention(q, k, v, scale)


def make_ring_attention(mesh, peer_memory: bool = True, scale: Optional[float] = None, **unused) -> Callable:
  from ..parallel.context import ContextParallel

  ctx = ContextParallel(mesh, "ring", peer_memory=peer_memory)
  return lambda q, k, v: ctx.self_attention(q, k, v, scale)


make_custom_ring_attention = make_ring_attention


def get_attention_kernel(name: str, mesh=None, peer_memory: bool = True, scale: Optional[float] = None) -> Callable:
  strategy = context_strategy(name)
  fixed_m = name in FIXED_M_KERNELS
  if mesh is None or ((strategy == "local" or mesh.size("context") == 1) and not fixed_m):
    return make_splash_mha(scale)
  from ..parallel.context import ContextParallel

  ctx = ContextParallel(mesh, strategy, peer_memory=peer_memory, fixed_m=fixed_m)
  return lambda q, k, v: ctx.self_attention(q, k, v, scale)


__all__ = ["KERNEL_REGISTRY", "FIXED_M_KERNELS", "USP_KERNELS", "make_splash_mha", "make_ring_attention",
           "make_custom_ring_attention", "get_attention_kernel"]
