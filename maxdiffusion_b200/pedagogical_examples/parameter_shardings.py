"""Shows how parameters are laid out for sharded training: every transformer block becomes one flat buffer cut into
equal per-rank shards (the unit of all-gather before use and of reduce-scatter + AdamW after backward), and the few
root parameters (embedders, head) form one more.

  python -m maxdiffusion_b200.pedagogical_examples.parameter_shardings wan2.1-t2v-14b 8

The reference's counterpart prints the logical-axis annotations of the SDXL UNet
(pedagogical_examples/unet_shardings.py); here the sharding is positional, so the table lists offsets instead.
"""
from __future__ import annotations

import sys

import torch

from .parameter_count import build


def run(name: str = "wan2.1-t2v-14b", world: int = 8, show_blocks: int = 1) -> dict:
  model = build(name)
  blocks = list(getattr(model, "blocks", []))
  ids = {id(p) for b in blocks for p in b.parameters()}
  root = [(n, p) for n, p in model.named_parameters() if id(p) not in ids]
  out = {"blocks": len(blocks), "world": world}
  for bi, b in enumerate(blocks[:show_blocks]):
    off = 0
    print(f"block {bi}:")
    for n, p in b.named_parameters():
      print(f"  {n:<40} {str(tuple(p.shape)):<18} flat[{off}:{off + p.numel()}]")
      off += p.numel()
    padded = -(-off // (world * 8)) * world * 8  # shards stay 16-byte aligned in bf16
    out["block_numel"], out["block_shard"] = off, padded // world
    print(f"  flat size {off} -> padded {padded}, {padded // world} elements ({padded // world * 2 / 2**20:.1f} MiB bf16) per rank")
  rn = sum(p.numel() for _, p in root)
  out["root_numel"] = rn
  print(f"root group: {len(root)} tensors, {rn} elements, {-(-rn // world)} per rank")
  per_rank = (out.get("block_shard", 0) * len(blocks) + -(-rn // world))
  print(f"per-rank resident: {per_rank * 2 / 2**30:.2f} GiB bf16 weights + {per_rank * 8 / 2**30:.2f} GiB fp32 AdamW moments")
  return out


if __name__ == "__main__":
  run(sys.argv[1] if len(sys.argv) > 1 else "wan2.1-t2v-14b", int(sys.argv[2]) if len(sys.argv) > 2 else 8)
