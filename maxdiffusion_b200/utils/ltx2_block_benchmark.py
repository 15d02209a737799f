"""LTX-2 plug for the attention tile search: times ONE transformer block of the configured size on synthetic tokens.

reference: src/maxdiffusion/utils/ltx2_block_benchmark.py (`LTX2BlockBenchmark`, CLI). Candidates are the launch
variants of the attention forward (`utils.wan_block_benchmark.candidates`: K / V pipeline depth); the block is built once, every candidate only changes the attention
configuration, warm-up is excluded and the maximum over ranks is kept.
"""
from __future__ import annotations

import sys
from typing import Optional

import torch

from .. import max_logging, pyconfig
from ..models.ltx2.transformer_ltx2 import LTX2_PRESETS, LTX2Config, LTX2VideoTransformer3DModel
from .tile_size_grid_search import Candidate, full_grid, grid_search, smart_grid


class LTX2BlockBenchmark:

  def __init__(self, config, device=None):
    self.config = config
    self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    cfg = dict(LTX2_PRESETS[str(config.get("ltx2_preset", "ltx2-19b"))])
    cfg.update(config.get("ltx2_config_overrides", {}) or {})
    cfg["num_layers"] = 1
    self.cfg = LTX2Config(**cfg)
    dtype = config.weights_dtype if self.device.type == "cuda" else torch.float32
    self.model = LTX2VideoTransformer3DModel(self.cfg).to(self.device, dtype).eval()
    self.lf = (int(config.num_frames) - 1) // 8 + 1
    self.lh, self.lw = int(config.height) // 32, int(config.width) // 32
    self.audio_frames = round(int(config.num_frames) / float(config.fps) * self.cfg.audio_sampling_rate / self.cfg.audio_hop_length / 4)
    g = torch.Generator().manual_seed(0)
    S = self.lf * self.lh * self.lw
    self.x = torch.randn((1, S, self.cfg.in_channels), generator=g).to(self.device, dtype)
    self.a = torch.randn((1, self.audio_frames, self.cfg.audio_in_channels), generator=g).to(self.device, dtype)
    self.text = torch.randn((1, 128, self.cfg.caption_channels), generator=g).to(self.device, dtype)

  def sequence_length(self) -> int:
    return self.x.shape[1]

  def setup(self, candidate: Candidate):
    from ..ops import kernels as K
    from .wan_block_benchmark import kernel_supports

    if not kernel_supports(candidate):
      raise ValueError(f"the attention kernel is not built with tiles {candidate.block_q} x {candidate.block_kv} / {candidate.stages} stages")
    if self.device.type == "cuda":
      K.flash_tune(candidate.stages, candidate.copy_ctas)  # every attention launch of the block uses this variant
    t = torch.full((1,), 500.0, device=self.device)

    @torch.no_grad()
    def step():
      return self.model(self.x, self.a, self.text, self.text, t, num_frames=self.lf, height=self.lh, width=self.lw,
                        audio_num_frames=self.audio_frames, fps=float(self.config.fps))

    return step

  def teardown(self):
    if self.device.type == "cuda":
      from ..ops import kernels as K

      K.flash_tune(0, 0)


def run_tile_search(config, device=None):
  import os

  bench = LTX2BlockBenchmark(config, device)
  seq = bench.sequence_length()
  from .wan_block_benchmark import candidates

  grid = lambda q, kv, n: candidates(n, full=str(config.get("tile_search_mode", "smart")) != "smart")
  cache = os.path.join(config.get("aot_cache_dir", "") or ".", "tile_search_cache.json")
  sync = torch.cuda.synchronize if bench.device.type == "cuda" else None
  best = grid_search(bench, grid(seq, seq, 1), iters=int(config.get("tile_search_iters", 10)),
                     out_dir=config.get("tile_search_out", ""), cache_path=cache,
                     cache_key=f"ltx2:{bench.cfg.num_attention_heads}:{seq}", sync=sync)
  max_logging.log(f"tile search: best candidate {best}")
  return best


def main(argv=None):
  run_tile_search(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
