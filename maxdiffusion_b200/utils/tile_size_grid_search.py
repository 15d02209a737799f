"""Attention tile autotuner: searches kernel launch parameters for a given (sequence, heads, mode, #GPUs).

Same structure as the reference's model-agnostic tuner (src/maxdiffusion/utils/tile_size_grid_search.py:86-533):
candidate generation, a `BlockBenchmark` plug interface (:277-310), `time_callable` that excludes warm-up (:249-274),
aggregation across ranks (max over ranks; a candidate that fails on any rank is rejected, :328-392), an orchestrator
`grid_search` with CSV output (:448-533) and an on-disk cache. The budget that bounds candidates is the SM's
TMEM (512 columns) and shared memory (227 KB) instead of the TPU's VMEM.
"""
from __future__ import annotations

import csv
import dataclasses
import json
import os
import time
from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional, Protocol, Sequence

SMEM_LIMIT_BYTES = 227 * 1024
TMEM_COLUMNS = 512


@dataclass(frozen=True)
class Candidate:
  block_q: int
  block_kv: int
  stages: int = 2
  copy_ctas: int = 0

  def as_dict(self) -> dict:
    return dataclasses.asdict(self)


def padding_of(length: int, block: int) -> int:
  """Rows of padding when `length` is covered by blocks of `block`."""
  return (-length) % block


def block_for_count(length: int, count: int, align: int = 128) -> int:
  """Smallest `align`-multiple block that covers `length` in `count` blocks."""
  per = -(-length // count)
  return -(-per // align) * align


def local_tiled_seq_len(seq_len: int, attention: str, context_shards: int = 1, ulysses_shards: int = -1,
                        row_multiple: int = 8) -> int:
  """Key / query rows ONE attention launch of a rank tiles over, for a sequence of `seq_len` tokens split the way
  production splits it (reference: src/maxdiffusion/utils/tile_size_grid_search.py `local_tiled_seq_len`).

  The context axis holds `context_shards` ranks; every rank keeps ceil(seq_len / shards) tokens rounded up to
  `row_multiple` (`ContextParallel.shard_sequence`: a shard has to start on a 16-byte boundary for the bulk copies).
  ring: a launch sees one shard per segment; Ulysses: the whole padded sequence of a head group; Ulysses x ring: the
  `ulysses_shards` shards of a Ulysses group joined; gather / local: the whole sequence."""
  from ..common_types import context_strategy

  strategy = context_strategy(attention)
  if context_shards <= 1 or strategy in ("local", "gather"):
    return seq_len
  per = -(-seq_len // context_shards)
  per = -(-per // row_multiple) * row_multiple
  if strategy == "ring":
    return per
  if strategy == "ulysses":
    return per * context_shards
  u = ulysses_shards if ulysses_shards and ulysses_shards > 0 else 1
  if context_shards % u != 0:
    raise ValueError(f"the context axis ({context_shards} ranks) must be divisible by ulysses_shards ({u})")
  return per * u


def smem_bytes(c: Candidate, head_dim: int = 128, elem: int = 2) -> int:
  return (c.block_q + 2 * c.stages * c.block_kv) * head_dim * elem + 2048


def tmem_columns(c: Candidate, head_dim: int = 128) -> int:
  q_tiles = c.block_q // 128
  return q_tiles * (c.block_kv + head_dim)  # S (fp32, block_kv columns) + O accumulator per 128-row q tile


def feasible(c: Candidate, head_dim: int = 128) -> bool:
  return (c.block_q % 128 == 0 and c.block_kv % 64 == 0 and smem_bytes(c, head_dim) <= SMEM_LIMIT_BYTES and
          tmem_columns(c, head_dim) <= TMEM_COLUMNS)


def bq_candidates(q_len: int, max_bq: int = 256) -> List[int]:
  out = [b for b in (128, 256, 384, 512) if b <= max_bq]
  return sorted(set(out), key=lambda b: (padding_of(q_len, b), -b))


def bkv_candidates(kv_len: int) -> List[int]:
  return sorted({64, 128, 256}, key=lambda b: (padding_of(kv_len, b), -b))


def smart_grid(q_len: int, kv_len: int, n_ranks: int = 1, head_dim: int = 128) -> List[Candidate]:
  """Candidate ladder capped by the on-chip budgets; with ranks > 1 the number of copy CTAs is searched too."""
  out = []
  for bq in bq_candidates(q_len):
    for bkv in bkv_candidates(kv_len):
      for stages in (2, 3):
        for cc in ((0,) if n_ranks == 1 else (8, 12, 16)):
          c = Candidate(bq, bkv, stages, cc)
          if feasible(c, head_dim):
            out.append(c)
  return out


def full_grid(q_len: int, kv_len: int, n_ranks: int = 1, head_dim: int = 128) -> List[Candidate]:
  out = []
  for bq in (128, 256, 384, 512):
    for bkv in (64, 128, 192, 256):
      for stages in (2, 3, 4):
        for cc in ((0,) if n_ranks == 1 else (4, 8, 12, 16, 24)):
          c = Candidate(bq, bkv, stages, cc)
          if feasible(c, head_dim):
            out.append(c)
  return out


class BlockBenchmark(Protocol):
  """Plug for one model: builds the workload for a candidate and runs it once."""

  def setup(self, candidate: Candidate) -> Callable[[], None]: ...

  def teardown(self) -> None: ...


def time_callable(fn: Callable[[], None], iters: int = 10, warmup: int = 2, sync: Optional[Callable[[], None]] = None,
                  timer: Callable[[], float] = time.perf_counter) -> float:
  """Mean seconds per call over `iters` calls after `warmup` untimed ones."""
  for _ in range(warmup):
    fn()
  if sync:
    sync()
  t0 = timer()
  for _ in range(iters):
    fn()
  if sync:
    sync()
  return (timer() - t0) / iters


def aggregate_across_ranks(per_rank_seconds: Sequence[Optional[float]]) -> Optional[float]:
  """Max over ranks; None (failure / out of memory on any rank) rejects the candidate."""
  if any(s is None for s in per_rank_seconds):
    return None
  return max(per_rank_seconds)


def _gather_ranks(value: Optional[float]) -> List[Optional[float]]:
  import torch.distributed as dist

  if not (dist.is_available() and dist.is_initialized()):
    return [value]
  out = [None] * dist.get_world_size()
  dist.all_gather_object(out, value)
  return out


def grid_search(bench: BlockBenchmark, candidates: Iterable[Candidate], iters: int = 10, out_dir: str = "",
                cache_path: str = "", cache_key: str = "", sync: Optional[Callable[[], None]] = None,
                gather: Callable[[Optional[float]], List[Optional[float]]] = _gather_ranks) -> Optional[Candidate]:
  """Times every candidate, writes `tile_search.csv`, returns the fastest one (and remembers it under `cache_key`)."""
  if cache_path and cache_key and os.path.exists(cache_path):
    with open(cache_path) as f:
      cached = json.load(f).get(cache_key)
    if cached:
      return Candidate(**cached)
  rows, best, best_t = [], None, float("inf")
  for c in candidates:
    local: Optional[float]
    try:
      fn = bench.setup(c)
      local = time_callable(fn, iters=iters, sync=sync)
    except Exception:  # launch failure or out of memory: the candidate is rejected on every rank
      local = None
    finally:
      bench.teardown()
    t = aggregate_across_ranks(gather(local))
    rows.append({**c.as_dict(), "seconds": t if t is not None else "failed"})
    if t is not None and t < best_t:
      best, best_t = c, t
  if out_dir:
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "tile_search.csv"), "w", newline="") as f:
      w = csv.DictWriter(f, fieldnames=list(rows[0].keys()) if rows else ["block_q"])
      w.writeheader()
      w.writerows(rows)
  if best is not None and cache_path and cache_key:
    data = {}
    if os.path.exists(cache_path):
      with open(cache_path) as f:
        data = json.load(f)
    data[cache_key] = best.as_dict()
    os.makedirs(os.path.dirname(os.path.abspath(cache_path)), exist_ok=True)
    with open(cache_path, "w") as f:
      json.dump(data, f, indent=1)
  return best
