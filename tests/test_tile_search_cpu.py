"""Tile-search logic on the host: candidate ladders, timing that excludes warm-up, rank aggregation, CSV, cache."""
import csv
import os

from maxdiffusion_b200.utils import tile_size_grid_search as T


def test_candidate_math():
  assert T.padding_of(4095, 128) == 1 and T.padding_of(4096, 128) == 0
  assert T.block_for_count(4095, 16) == 256
  assert T.feasible(T.Candidate(256, 128, 2)) and not T.feasible(T.Candidate(512, 256, 4))
  assert T.tmem_columns(T.Candidate(256, 128)) == 512
  grid = T.smart_grid(4095, 32760, n_ranks=8)
  assert grid and all(T.feasible(c) for c in grid) and {c.copy_ctas for c in grid} == {8, 12, 16}


def test_time_callable_excludes_warmup():
  ticks = iter(range(1000))
  calls = []
  t = T.time_callable(lambda: calls.append(1), iters=4, warmup=3, timer=lambda: next(ticks))
  assert len(calls) == 7 and t == 0.25


def test_rank_aggregation():
  assert T.aggregate_across_ranks([1.0, 3.0, 2.0]) == 3.0
  assert T.aggregate_across_ranks([1.0, None]) is None


class _MockBench:
  """Synthetic cost model: cost falls with block_kv, one candidate fails."""

  def setup(self, c):
    if c.block_kv == 256:
      raise MemoryError("synthetic out of memory")
    import time
    return lambda: time.sleep(0.001 * (3 - c.block_kv // 64))

  def teardown(self):
    pass


def test_grid_search_csv_and_cache(tmp_path):
  cands = [T.Candidate(256, 64), T.Candidate(256, 128), T.Candidate(128, 256)]
  cache = str(tmp_path / "cache.json")
  best = T.grid_search(_MockBench(), cands, iters=2, out_dir=str(tmp_path), cache_path=cache, cache_key="k", gather=lambda v: [v])
  assert best == T.Candidate(256, 128)
  rows = list(csv.DictReader(open(os.path.join(tmp_path, "tile_search.csv"))))
  assert len(rows) == 3 and rows[2]["seconds"] == "failed"
  assert T.grid_search(_MockBench(), [], cache_path=cache, cache_key="k") == best  # served from the cache


def test_wan_plug_offers_the_kernels_launch_variants_and_rejects_other_tiles():
  from maxdiffusion_b200.utils import wan_block_benchmark as W

  one = W.candidates(1)
  assert [c.stages for c in one] == [2, 3, 4, 5] and all(W.kernel_supports(c) and c.copy_ctas == 0 for c in one)
  eight = W.candidates(8)
  assert {c.copy_ctas for c in eight} == {8, 12, 16, 20, 24} and len(eight) == 20
  extra = [c for c in W.candidates(1, full=True) if not W.kernel_supports(c)]
  assert extra  # recorded as rejected in the CSV
  import pytest

  with pytest.raises(ValueError, match="not built"):
    W.WanBlockBenchmark(4, 256, [256], device="cpu").setup(extra[0])


def test_cached_choice_is_registered_for_the_attention_launcher(tmp_path):
  import json

  from maxdiffusion_b200.ops import kernels as K

  key = K.flash_tuned_key(4096, 128, 40, 8)
  path = tmp_path / "tile_search_cache.json"
  path.write_text(json.dumps({key: {"block_q": 256, "block_kv": 64, "stages": 3, "copy_ctas": 16}, "ltx2:32:100": {"stages": 2}}))
  K._FLASH_TUNED.clear()
  assert K.load_flash_tuning(str(path)) == 1
  assert K._FLASH_TUNED[key] == (3, 16)
  K._FLASH_TUNED.clear()


def test_local_tiled_sequence_length_follows_the_production_split():
  import pytest

  assert T.local_tiled_seq_len(6144, "tokamax_ring", context_shards=8) == 768
  assert T.local_tiled_seq_len(6144, "ulysses_ring", context_shards=8, ulysses_shards=2) == 1536
  assert T.local_tiled_seq_len(6144, "ulysses", context_shards=8) == 6144
  assert T.local_tiled_seq_len(6144, "flash", context_shards=8) == 6144
  # shards are padded to 8 rows (16-byte starts for the bulk copies): 32760 tokens on 8 ranks are 8 x 4096
  assert T.local_tiled_seq_len(32760, "tokamax_ring", context_shards=8) == 4096
  assert T.local_tiled_seq_len(10, "tokamax_ring", context_shards=4) == 8
  assert T.local_tiled_seq_len(10, "tokamax_ring", context_shards=4, row_multiple=1) == 3
  assert T.local_tiled_seq_len(10, "ulysses_ring", context_shards=4, ulysses_shards=2, row_multiple=1) == 6
  with pytest.raises(ValueError, match="must be divisible"):
    T.local_tiled_seq_len(6144, "ulysses_ring_custom", context_shards=8, ulysses_shards=3)
