"""Names shared across the framework: mesh axes, attention kernels, model families.

The mesh axes and the attention-kernel names are the reference's public vocabulary
(src/maxdiffusion/common_types.py:36-110, src/maxdiffusion/models/attention_flax.py:1589-1867); what they
select here is an explicit per-rank strategy, not a set of GSPMD annotation rules.
"""
from __future__ import annotations

DATA = "data"
FSDP = "fsdp"
CONTEXT = "context"
TENSOR = "tensor"
MESH_AXES = (DATA, FSDP, CONTEXT, TENSOR)

# activation / parameter logical names accepted in `logical_axis_rules` (kept for config compatibility)
BATCH = "activation_batch"
LENGTH = "activation_length"
KV_LENGTH = "activation_kv_length"
HEAD = "activation_heads"
EMBED = "activation_embed"
D_KV = "activation_kv"

WAN2_1 = "wan2.1"
WAN2_2 = "wan2.2"
WAN_MODELS = (WAN2_1, WAN2_2)
TRAINABLE_WAN_MODELS = (WAN2_1,)

# attention kernel name -> context-parallel strategy of the self-attention layers
#   local   : every rank holds the whole sequence
#   gather  : q is sequence-sharded, K/V are all-gathered (the reference's SEQUENCE_PARALLEL rules)
#   ring    : K/V shards visit every rank, one flash kernel keeps (O, m, l) on chip across hops
#   ulysses : all-to-all heads<->sequence around a local full-sequence kernel
#   usp     : 2-D, Ulysses inside `ulysses_shards` ranks, ring across the rest
ATTENTION_KERNELS = {
    "dot_product": "local",
    "flash": "gather",
    "tokamax_flash": "gather",
    "cudnn_flash_te": "gather",
    "tokamax_ring": "ring",
    "tokamax_ring_custom": "ring",
    "ring": "ring",
    "ulysses": "ulysses",
    "ulysses_custom": "ulysses",
    "ulysses_custom_fixed_m": "ulysses",
    "ulysses_ring": "usp",
    "ulysses_ring_custom": "usp",
    "ulysses_ring_custom_fixed_m": "usp",
    "ulysses_ring_custom_bidir": "usp",
}
FIXED_M_KERNELS = ("ulysses_custom_fixed_m", "ulysses_ring_custom_fixed_m")
USP_KERNELS = tuple(k for k, v in ATTENTION_KERNELS.items() if v == "usp")


def context_strategy(attention: str) -> str:
  if attention not in ATTENTION_KERNELS:
    raise ValueError(f"unknown attention kernel '{attention}'; known: {sorted(ATTENTION_KERNELS)}")
  return ATTENTION_KERNELS[attention]
