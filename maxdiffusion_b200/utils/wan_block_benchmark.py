"""Wan plug for the tile search: times one self-attention layer of the configured shape per candidate.

  python -m maxdiffusion_b200.utils.wan_block_benchmark <config.yml> key=value ...
  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m maxdiffusion_b200.utils.wan_block_benchmark <config.yml> ...

Reference: `WanBlockBenchmark` and its CLI (src/maxdiffusion/utils/wan_block_benchmark.py:115-328). What the search
ranks here are the launch variants the attention forward is built in: the depth of the K / V pipeline (2 to 5
stages; the q tile pair of 2 x 128 rows and the 64-key block are fixed by the kernel's TMEM layout, other tile
shapes are rejected as infeasible) and, under context parallelism, the number of copy CTAs that pull the remote K / V
shards inside the launch. The winner is written to `tile_search_cache.json` under `aot_cache_dir`;
`ops.kernels.load_flash_tuning` registers it and `ops.kernels.flash_fwd` launches the cached variant for that shape.
"""
from __future__ import annotations

import os
import sys

import torch

from .tile_size_grid_search import Candidate, grid_search

KERNEL_BLOCK_Q, KERNEL_BLOCK_KV = 256, 64


def kernel_supports(c: Candidate) -> bool:
  return c.block_q == KERNEL_BLOCK_Q and c.block_kv == KERNEL_BLOCK_KV and 2 <= c.stages <= 5


def candidates(n_ranks: int = 1, full: bool = False):
  """The launch variants of the forward kernel, plus (full mode) neighbouring tile shapes that the search records as
  rejected so that the CSV shows what was considered."""
  out = []
  for stages in (2, 3, 4, 5):
    for cc in ((0,) if n_ranks == 1 else (8, 12, 16, 20, 24)):
      out.append(Candidate(KERNEL_BLOCK_Q, KERNEL_BLOCK_KV, stages, cc))
  if full:
    out += [Candidate(256, 128, 2, 0), Candidate(128, 64, 4, 0)]
  return out


class WanBlockBenchmark:

  def __init__(self, heads: int, q_len: int, kv_lens, device="cuda", exchange=None, head_dim: int = 128):
    self.heads, self.q_len, self.kv_lens, self.device = heads, q_len, list(kv_lens), device
    self.exchange, self.head_dim = exchange, head_dim
    self.tensors = None

  def setup(self, candidate: Candidate):
    from ..ops import kernels as K

    if not kernel_supports(candidate):
      raise ValueError(f"the attention kernel is not built with tiles {candidate.block_q} x {candidate.block_kv} / {candidate.stages} stages")
    K.flash_tune(candidate.stages, candidate.copy_ctas)
    g = torch.Generator(device=self.device).manual_seed(0)
    mk = lambda s: torch.randn((1, s, self.heads, self.head_dim), device=self.device, dtype=torch.bfloat16, generator=g)
    q = mk(self.q_len)
    if self.exchange is not None:
      # context parallelism: this rank's shard is published, the others are pulled by the launch's copy CTAs
      k, v = mk(self.kv_lens[0]), mk(self.kv_lens[0])
      self.tensors = (q, k, v)

      def run():
        kg, vg, flags, epoch, plan, keep = self.exchange.plan(k, v)
        K.flash_fwd(q, list(kg), list(vg), return_lse=False, seg_flags=flags, flag_target=epoch, plan=plan)

      return run
    ks, vs = [mk(s) for s in self.kv_lens], [mk(s) for s in self.kv_lens]
    self.tensors = (q, ks, vs)
    return lambda: K.flash_fwd(q, ks, vs, return_lse=False)

  def teardown(self):
    from ..ops import kernels as K

    self.tensors = None
    K.flash_tune(0, 0)


def tune_wan_block_sizes(config):
  import torch.distributed as dist

  from ..ops import kernels as K
  from ..parallel.mesh import init_distributed
  from ..trainers.wan_trainer import resolve_wan_config

  cfg = resolve_wan_config(config)
  rank, world, _ = init_distributed()
  seq = ((int(config.num_frames) - 1) // 4 + 1) * (int(config.height) // 16) * (int(config.width) // 16)
  per = (-(-seq // world) + 7) // 8 * 8
  exchange = None
  if world > 1:
    from ..parallel import symm

    peer = symm.PeerGroup(dist.group.WORLD)
    exchange = symm.PeerKVExchange(peer, per * cfg.num_attention_heads * cfg.attention_head_dim)
  bench = WanBlockBenchmark(cfg.num_attention_heads, per, [per] * world, exchange=exchange, head_dim=cfg.attention_head_dim)
  cache = os.path.join(config.get("aot_cache_dir", "") or ".", "tile_search_cache.json")
  key = K.flash_tuned_key(per, cfg.attention_head_dim, cfg.num_attention_heads, world)
  best = grid_search(bench, candidates(world, full=str(config.get("tile_search_mode", "smart")) != "smart"),
                     iters=int(config.get("tile_search_iters", 10)), out_dir=config.get("tile_search_out", "") if rank == 0 else "",
                     cache_path=cache if rank == 0 else "", cache_key=key, sync=torch.cuda.synchronize)
  if world > 1:
    torch.cuda.synchronize()
    dist.barrier()
  return best


def main(argv=None):
  from .. import pyconfig

  print(tune_wan_block_sizes(pyconfig.initialize(list(sys.argv if argv is None else argv))))


if __name__ == "__main__":
  main()
