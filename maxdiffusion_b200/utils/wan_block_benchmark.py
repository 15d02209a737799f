"""Wan plug for the tile search: times one self-attention layer of the configured shape per candidate.

  python -m maxdiffusion_b200.utils.wan_block_benchmark <config.yml> key=value ...

Reference: `WanBlockBenchmark` and its CLI (src/maxdiffusion/utils/wan_block_benchmark.py:115-328). The kernels of
this build have fixed tile shapes (128-row q tiles in pairs, 128-key blocks, 2 K/V stages); the search therefore
currently ranks the feasible launch variants — the number of copy CTAs under context parallelism — and records the
result in the autotune cache (`aot_cache_dir`).
"""
from __future__ import annotations

import os
import sys

import torch

from .tile_size_grid_search import Candidate, grid_search, smart_grid, full_grid


class WanBlockBenchmark:

  def __init__(self, heads: int, q_len: int, kv_lens, device="cuda"):
    self.heads, self.q_len, self.kv_lens, self.device = heads, q_len, list(kv_lens), device
    self.tensors = None

  def setup(self, candidate: Candidate):
    from ..ops import kernels as K

    if (candidate.block_q, candidate.block_kv, candidate.stages) != (256, 128, 2):
      raise ValueError("tile shape is fixed in this build")
    g = torch.Generator(device=self.device).manual_seed(0)
    mk = lambda s: torch.randn((1, s, self.heads, 128), device=self.device, dtype=torch.bfloat16, generator=g)
    q, ks, vs = mk(self.q_len), [mk(s) for s in self.kv_lens], [mk(s) for s in self.kv_lens]
    self.tensors = (q, ks, vs)
    return lambda: K.flash_fwd(q, ks, vs, return_lse=False)

  def teardown(self):
    self.tensors = None


def tune_wan_block_sizes(config):
  from ..trainers.wan_trainer import resolve_wan_config

  cfg = resolve_wan_config(config)
  world = int(os.environ.get("WORLD_SIZE", "1"))
  seq = ((int(config.num_frames) - 1) // 4 + 1) * (int(config.height) // 16) * (int(config.width) // 16)
  per = -(-seq // world)
  bench = WanBlockBenchmark(cfg.num_attention_heads, per, [per] * world)
  grid = smart_grid if str(config.get("tile_search_mode", "smart")) == "smart" else full_grid
  cache = os.path.join(config.get("aot_cache_dir", "") or ".", "tile_search_cache.json")
  best = grid_search(bench, grid(per, seq, 1), iters=int(config.get("tile_search_iters", 10)),
                     out_dir=config.get("tile_search_out", ""), cache_path=cache,
                     cache_key=f"wan:{cfg.num_attention_heads}:{per}:{world}", sync=torch.cuda.synchronize)
  return best


def main(argv=None):
  from .. import pyconfig

  print(tune_wan_block_sizes(pyconfig.initialize(list(sys.argv if argv is None else argv))))


if __name__ == "__main__":
  main()
