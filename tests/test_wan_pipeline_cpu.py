"""Wan pipeline, VAE chunking and cache policies on CPU (fp32, tiny random-init models)."""
import os

import numpy as np
import pytest
import torch

from maxdiffusion_b200 import pyconfig
from maxdiffusion_b200.models.wan.autoencoder_kl_wan import AutoencoderKLWan, WanVAEConfig
from maxdiffusion_b200.pipelines.wan import cache_policies as CP
from maxdiffusion_b200.pipelines.wan.wan_pipeline import WanPipeline2_1, WanPipeline2_2

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs")
TINY = '{"num_attention_heads": 2, "attention_head_dim": 32, "ffn_dim": 64, "num_layers": 2, "text_dim": 32, "freq_dim": 32}'
VAE = '{"base_dim": 8, "z_dim": 16}'


def _config(name="base_wan_14b.yml", *extra):
  return pyconfig.initialize(["t", os.path.join(CFG, name), "run_name=t", "height=32", "width=32", "num_frames=9",
                              "wan_preset=tiny", f"wan_config_overrides={TINY}", f"vae_config_overrides={VAE}",
                              "num_inference_steps=6", "log_config=false", *extra], unittest=True)


def test_vae_chunked_decode_and_encode_match_whole_clip():
  torch.manual_seed(0)
  vae = AutoencoderKLWan(WanVAEConfig(base_dim=8))
  z = torch.randn(1, 16, 3, 4, 4)
  full = vae.decode_full(z)
  assert full.shape == (1, 3, 9, 32, 32)
  assert torch.allclose(vae.decode(z, chunk=1), full, atol=1e-5)
  assert torch.allclose(vae.decode(z, chunk=2), full, atol=1e-5)
  x = torch.randn(1, 3, 9, 32, 32)
  assert torch.allclose(vae.encode(x, chunk=4).mean, vae.encode_full(x).mean, atol=1e-5)
  assert vae.encode(x).mean.shape == (1, 16, 3, 4, 4)


def test_pipeline_runs_and_caches_change_little():
  config = _config()
  pipe = WanPipeline2_1.from_config(config, device="cpu")
  emb = torch.randn(1, 8, 32)
  neg = torch.randn(1, 8, 32)
  g = lambda: torch.Generator().manual_seed(3)
  video = pipe(prompt_embeds=emb, negative_prompt_embeds=neg, generator=g())
  assert video.shape == (1, 9, 32, 32, 3) and video.dtype == torch.uint8
  base = pipe(prompt_embeds=emb, negative_prompt_embeds=neg, generator=g(), output_type="latent")
  kv = pipe(prompt_embeds=emb, negative_prompt_embeds=neg, generator=g(), output_type="latent", use_kv_cache=True)
  assert torch.allclose(base, kv, atol=1e-4)  # the K/V cache is exact
  for kw in (dict(use_cfg_cache=True), dict(use_magcache=True)):
    out = pipe(prompt_embeds=emb, negative_prompt_embeds=neg, generator=g(), output_type="latent", **kw)
    assert torch.isfinite(out).all()


def test_wan22_switches_experts_and_sen_cache_runs():
  config = _config("base_wan_27b.yml")
  pipe = WanPipeline2_2.from_config(config, device="cpu", load_vae=False)
  emb, neg = torch.randn(1, 8, 32), torch.randn(1, 8, 32)
  calls = {"high": 0, "low": 0}
  f1, f2 = pipe.transformer.forward, pipe.transformer_2.forward
  pipe.transformer.forward = lambda *a, **k: (calls.__setitem__("high", calls["high"] + 1), f1(*a, **k))[1]
  pipe.transformer_2.forward = lambda *a, **k: (calls.__setitem__("low", calls["low"] + 1), f2(*a, **k))[1]
  out = pipe(prompt_embeds=emb, negative_prompt_embeds=neg, output_type="latent", num_inference_steps=10)
  assert calls["high"] > 0 and calls["low"] > 0 and calls["high"] + calls["low"] == 10
  out = pipe(prompt_embeds=emb, negative_prompt_embeds=neg, output_type="latent", num_inference_steps=10, use_sen_cache=True)
  assert torch.isfinite(out).all()


def test_cache_schedules():
  sched = CP.cfg_cache_schedule(50, 720)
  assert not any(sched[:16]) and not any(sched[45:]) and sum(sched) > 15 and not sched[16]
  mag = CP.magcache_schedule(40, np.ones(80) * 0.999, thresh=0.12, K=2, retention_ratio=0.2)
  assert not any(mag[:8]) and sum(mag) > 10
  # never more than K consecutive skips
  run = 0
  for s in mag:
    run = run + 1 if s else 0
    assert run <= 2
  x = torch.randn(1, 4, 2, 16, 18)
  assert torch.allclose(CP.fft_compensate(x, x, x, 1.2, 1.0), x, atol=1e-5)  # zero bias -> identity


@pytest.mark.parametrize("shape", [(1, 4, 3, 90, 160), (2, 3, 2, 45, 80), (1, 2, 1, 31, 53), (1, 1, 1, 3, 5)])
def test_band_filter_as_two_gemms_matches_the_fft_form(shape):
  """The GEMM form of the CFG-cache compensation equals rfft2 -> band weights -> irfft2 (even, odd, tiny sizes)."""
  from maxdiffusion_b200.ops import dft

  torch.manual_seed(0)
  a, b, c = (torch.randn(shape) for _ in range(3))
  for w1, w2 in ((1.2, 1.0), (1.0, 1.2), (0.7, 0.7)):
    got = CP.fft_compensate(a, b, c, w1, w2)
    want = CP.fft_compensate_reference(a, b, c, w1, w2)
    assert torch.allclose(got, want, atol=2e-5), (got - want).abs().max()
  # the projector is idempotent and symmetric, and keeps the mean (frequency 0)
  p = dft.band_projector(shape[-2], max(1, shape[-2] // 4), False)
  assert torch.allclose(p @ p, p, atol=1e-5) and torch.allclose(p, p.T, atol=1e-6)
  assert torch.allclose(p.sum(1), torch.ones(shape[-2]), atol=1e-5)


def test_split_bf16_product_keeps_fp32_accuracy():
  """[x_hi|x_lo|x_hi]·[P_hi|P_hi|P_lo]ᵀ with bf16 operands and fp32 accumulation is within 1e-4 of the fp32 product."""
  from maxdiffusion_b200.ops import dft

  torch.manual_seed(1)
  x = torch.randn(64, 160)
  p = dft.band_projector(160, 20, True)
  x_hi, x_lo = dft._split_bf16(x)
  p_hi, p_lo = dft._split_bf16(p)
  a = torch.cat([x_hi, x_lo, x_hi], 1).float()
  b = torch.cat([p_hi, p_hi, p_lo], 1).float()
  assert (a @ b.T - x @ p).abs().max() < 1e-4
  assert (x_hi.float() @ p_hi.float().T - x @ p).abs().max() > 1e-3  # a single bf16 product is not enough


def test_wan22_vae_chunked_matches_whole_clip_and_patchify_round_trip():
  from maxdiffusion_b200.models.wan.autoencoder_kl_wan_2p2 import (AutoencoderKLWan2p2, WanAvgDown3D, WanDupUp3D,
                                                                    WanVAE2p2Config, patchify, unpatchify)

  torch.manual_seed(0)
  x = torch.randn(1, 3, 2, 8, 12)
  p = patchify(x, 2)
  assert p.shape == (1, 12, 2, 4, 6) and torch.equal(unpatchify(p, 2), x)
  # channel index = c*4 + w_in_patch*2 + h_in_patch
  assert torch.equal(p[0, 1 * 4 + 1 * 2 + 0, 0, 1, 2], x[0, 1, 0, 2, 5])
  down = WanAvgDown3D(4, 8, 2, 2)
  assert down(torch.randn(1, 4, 1, 4, 4)).shape == (1, 8, 1, 2, 2)  # a single frame is padded in front
  up = WanDupUp3D(8, 4, 2, 2)
  assert up(torch.randn(1, 8, 3, 2, 2), True).shape == (1, 4, 5, 4, 4)
  cfg = WanVAE2p2Config(base_dim=8, base_dec_dim=8, z_dim=6, latents_mean=[0.0] * 6, latents_std=[1.0] * 6)
  vae = AutoencoderKLWan2p2(cfg).eval()
  video = torch.rand(1, 3, 9, 32, 32) * 2 - 1
  with torch.no_grad():
    z, z_full = vae.encode(video).mode(), vae.encode_full(video).mode()
    assert z.shape == (1, 6, 3, 2, 2) and torch.allclose(z, z_full, atol=1e-5)
    out, out_full = vae.decode(z), vae.decode_full(z)
  assert out.shape == (1, 3, 9, 32, 32) and torch.allclose(out, out_full, atol=1e-5)


def test_channels_last_decoder_orchestration_matches_the_ncdhw_path():
  """The channels-last walk over the decoder (history tensors instead of concatenated caches, channel halves written
  into even / odd frames, nearest-2x folded into the convolution call) against the plain NCDHW modules, both in fp32
  on the CPU, chunked and whole-clip."""
  torch.manual_seed(0)
  vae = AutoencoderKLWan(WanVAEConfig(base_dim=8)).eval()
  for p in vae.parameters():
    torch.nn.init.normal_(p, std=0.2)
  z = torch.randn(1, 16, 3, 4, 6)
  from maxdiffusion_b200.models.wan.vae_channels_last import ChannelsLastDecoder

  cl = ChannelsLastDecoder(vae)
  with torch.no_grad():
    want = vae.decode(z, chunk=1)
    got = cl.decode(z, chunk=1)
    assert got.shape == want.shape == (1, 3, 9, 32, 48)
    assert (got - want).abs().max() < 1e-4 * (1 + want.abs().max())
    got2 = cl.decode(z, chunk=2)
    assert (got2 - want).abs().max() < 1e-4 * (1 + want.abs().max())
    whole = cl.decode(z, whole_clip=True)
    assert (whole - vae.decode_full(z)).abs().max() < 1e-4 * (1 + want.abs().max())


def test_channels_last_decoder_walks_the_wan_2p2_vae_like_the_ncdhw_path():
  """Wan 2.2 VAE on the channels-last decoder: up blocks with the resampler inside the layer list, the parameter-free
  channel-duplicating shortcut around every up block, and the 2 x 2 pixel patches unfolded at the end; fp32 on the CPU
  against the NCDHW modules, chunked and whole-clip."""
  from maxdiffusion_b200.models.wan.autoencoder_kl_wan_2p2 import AutoencoderKLWan2p2, WanVAE2p2Config
  from maxdiffusion_b200.models.wan.vae_channels_last import ChannelsLastDecoder

  torch.manual_seed(0)
  cfg = WanVAE2p2Config(base_dim=8, base_dec_dim=8, z_dim=16, latents_mean=[0.0] * 16, latents_std=[1.0] * 16)
  vae = AutoencoderKLWan2p2(cfg).eval()
  for p in vae.parameters():
    torch.nn.init.normal_(p, std=0.2)
  z = torch.randn(1, 16, 3, 2, 3)
  cl = ChannelsLastDecoder(vae)
  with torch.no_grad():
    want = vae.decode(z, chunk=1)
    got = cl.decode(z, chunk=1)
    assert got.shape == want.shape == (1, 3, 9, 32, 48)
    tol = 1e-4 * (1 + want.abs().max())
    assert (got - want).abs().max() < tol
    assert (cl.decode(z, chunk=2) - want).abs().max() < tol
    assert (cl.decode(z, whole_clip=True) - vae.decode_full(z)).abs().max() < tol


def test_channels_last_encoder_orchestration_matches_the_ncdhw_path():
  """The encoder on the channels-last walk: stride-2 convolutions padded on the far side, the strided time convolution
  as every second output of the causal one with the remembered frame as history, chunked (first frame alone, then
  chunks of 4 or 8: the two strided time convolutions need a multiple of 4) and whole-clip; fp32 on the CPU against the NCDHW modules."""
  from maxdiffusion_b200.models.wan.vae_channels_last import ChannelsLastDecoder

  torch.manual_seed(0)
  vae = AutoencoderKLWan(WanVAEConfig(base_dim=8)).eval()
  for p in vae.parameters():
    torch.nn.init.normal_(p, std=0.2)
  x = torch.randn(1, 3, 9, 16, 24)
  cl = ChannelsLastDecoder(vae)
  with torch.no_grad():
    want = vae.encode(x, chunk=4).mean
    for chunk in (4, 8):
      got = cl.encode(x, chunk=chunk).chunk(2, dim=1)[0]
      assert got.shape == want.shape == (1, 16, 3, 2, 3)
      assert (got - want).abs().max() < 1e-4 * (1 + want.abs().max())
    whole = cl.encode(x, whole_clip=True).chunk(2, dim=1)[0]
    assert (whole - vae.encode_full(x).mean).abs().max() < 1e-4 * (1 + want.abs().max())


def test_check_inputs_of_the_wan_pipelines():
  import types

  import pytest

  pipe = WanPipeline2_1.__new__(WanPipeline2_1)
  pipe.transformer = types.SimpleNamespace(cfg=types.SimpleNamespace(patch_size=(1, 2, 2)))
  pipe.vae_scale_factor_spatial = 8
  pipe.check_inputs("a cat", None, 480, 832, 81)
  pipe.check_inputs(None, None, 480, 832, 81, prompt_embeds=torch.zeros(1, 4, 8))
  for args, kw, match in ((("a", None, 480, 832, 81), {"prompt_embeds": torch.zeros(1, 4, 8)}, "not both"),
                          ((None, "b", 480, 832, 81), {"negative_prompt_embeds": torch.zeros(1, 4, 8)}, "not both"),
                          ((3, None, 480, 832, 81), {}, "str or a list"), (("a", None, 488, 832, 81), {}, "divisible by 16"),
                          (("a", None, 480, 832, 0), {}, "positive")):
    with pytest.raises(ValueError, match=match):
      pipe.check_inputs(*args, **kw)


def test_cfg_cache_needs_guidance_and_the_two_expert_schedule_spares_the_high_noise_expert():
  """The argument rule and the schedules asserted by the reference's src/maxdiffusion/tests/wan/wan_cfg_cache_test.py:
  `use_cfg_cache` without classifier-free guidance is an error (one scale for 2.1, both for 2.2); with two experts no
  high-noise step is a cache step and the first low-noise step is a full one."""
  for cls, kw in ((WanPipeline2_1, {"guidance_scale": 1.0}), (WanPipeline2_1, {"guidance_scale": 0.0}),
                  (WanPipeline2_2, {"guidance_scale_low": 1.0, "guidance_scale_high": 1.0}),
                  (WanPipeline2_2, {"guidance_scale_low": 0.5, "guidance_scale_high": 4.0}),
                  (WanPipeline2_2, {"guidance_scale_low": 3.0, "guidance_scale_high": 1.0})):
    with pytest.raises(ValueError, match="use_cfg_cache"):
      cls.__new__(cls)(prompt=["test"], use_cfg_cache=True, **kw)
  for policy in ("use_magcache", "use_sen_cache"):
    with pytest.raises(ValueError, match=policy):
      WanPipeline2_2.__new__(WanPipeline2_2)(prompt=["test"], guidance_scale_low=0.5, guidance_scale_high=4.0, **{policy: True})
  for pair in (("use_cfg_cache", "use_magcache"), ("use_sen_cache", "use_magcache"), ("use_cfg_cache", "use_sen_cache")):
    with pytest.raises(ValueError, match="mutually exclusive"):
      WanPipeline2_2.__new__(WanPipeline2_2)(prompt=["test"], guidance_scale_low=3.0, guidance_scale_high=4.0,
                                             **{pair[0]: True, pair[1]: True})
  for cls, kw, cache in ((WanPipeline2_1, {"guidance_scale": 5.0}, True), (WanPipeline2_1, {"guidance_scale": 1.0}, False),
                         (WanPipeline2_2, {"guidance_scale_low": 3.0, "guidance_scale_high": 4.0}, True),
                         (WanPipeline2_2, {"guidance_scale_low": 1.0, "guidance_scale_high": 1.0}, False)):
    try:   # passes the rule and fails later, on the components a bare instance does not have
      cls.__new__(cls)(prompt=["test"], use_cfg_cache=cache, **kw)
    except ValueError as e:
      assert "use_cfg_cache" not in str(e)
    except Exception:
      pass

  def two(n, ratio=0.875, height=720):
    ts = np.linspace(999, 0, n, dtype=np.int32)
    high = [bool(t >= ratio * 1000) for t in ts]
    return CP.cfg_cache_schedule_two_experts(n, height, high), high

  cache, high = two(50)
  assert not any(c for c, h in zip(cache, high) if h)
  first_low = high.index(False)
  assert not cache[first_low] and sum(cache) > 0
  assert sum(two(50, 0.5)[1]) > sum(two(50, 0.9)[1])
  assert sum(two(50, height=480)[0]) > sum(two(50, height=720)[0])
  c480, h480 = two(50, height=480)
  assert all(not c480[s] for s in range(16, 49) if not h480[s] and (s - 16) % 5 == 0) and not c480[49] and c480[48]
  assert sum(two(3)[0]) == 0 and sum(two(50, 0.0)[0]) == 0 and all(two(50, 0.0)[1])
  # one expert: starts at a third of the steps, ends 2 steps (480p) or 10 % (720p) before the last, every 5th step full
  s480, s720 = CP.cfg_cache_schedule(50, 480), CP.cfg_cache_schedule(50, 720)
  assert not any(s480[:16]) and not any(s480[48:]) and not any(s720[45:]) and sum(s480) > sum(s720) > 0
  assert all(not s480[s] for s in range(16, 48, 5)) and sum(CP.cfg_cache_schedule(3, 480)) == 0


def test_magcache_two_phase_forced_zones_and_skip_rules():
  """The host-side MagCache schedule as the reference's src/maxdiffusion/tests/wan/wan2_2_magcache_test.py pins it:
  a forced (retention) zone at the start of each expert's phase, a forced step where the expert changes, at most K
  skips in a row, and a skip only when BOTH branches stay under the error budget."""
  def phases(n, ratio=0.875):
    return [bool(t >= ratio * 1000) for t in np.linspace(999, 0, n, dtype=np.int32)]

  for n in (20, 40, 80):
    high = phases(n)
    hn = sum(high)
    forced = CP.magcache_forced_steps(n, 0.2, high)
    assert all(forced[:int(hn * 0.2)]) and all(forced[hn:hn + int((n - hn) * 0.2)])
    boundaries = [s for s in range(1, n) if high[s] != high[s - 1]]
    assert len(boundaries) == 1 and forced[boundaries[0]]
    sched = CP.magcache_schedule(n, list(np.ones(2 * n)), 1.0, 99, 0.2, high)
    assert not sched[0] and not any(s for s, f in zip(sched, forced) if f) and sum(sched) > 0
  assert CP.magcache_forced_steps(40, 0.2) == [s < 8 for s in range(40)]
  # at most K skips in a row even when the error is zero
  run = best = 0
  for skip in CP.magcache_schedule(20, list(np.ones(40)), 1.0, 2, 0.0):
    run = run + 1 if skip else 0
    best = max(best, run)
  assert best == 2
  # a ratio far from 1 in either branch blocks the skip of that step only
  ratios = np.ones(20)
  ratios[3 * 2 + 1] = 0.5
  sched = CP.magcache_schedule(10, list(ratios), 0.04, 99, 0.2)
  assert not sched[3] and sched[2] and sched[4]
  assert not any(CP.magcache_schedule(10, list(np.full(20, 0.5)), 0.04, 99, 0.2))
  # a curve calibrated on another step count is resampled per branch; one of the right length is used as it is
  assert len(CP.nearest_interp(np.linspace(1.0, 0.8, 20), 40)) == 40
  base = np.linspace(1.0, 0.9, 10)
  a = CP.magcache_schedule(5, list(base), 0.2, 3, 0.2)
  b = CP.magcache_schedule(5, list(np.stack([CP.nearest_interp(base[0::2], 5), CP.nearest_interp(base[1::2], 5)], 1).reshape(-1)), 0.2, 3, 0.2)
  assert a == b


def test_sencache_forced_zones_score_and_reuse_limit():
  """The deterministic part of SenCache as src/maxdiffusion/tests/wan/wan_sen_cache_test.py pins it (first step, first
  30 %, last 10 %, expert change are always computed) and the data-dependent part: the score alpha_x * rms(dx) +
  alpha_t * |dt| / 1000 accumulates since the last full step, and at most `max_reuse` reuses follow one another."""
  for n in (20, 25, 50, 100):
    sc = CP.SenCache(n)
    forced = [sc.forced(s) for s in range(n)]
    assert all(forced[:int(n * 0.3)]) and all(forced[int(n * 0.9):]) and forced[0]
    assert sum(not f for f in forced[int(n * 0.3):int(n * 0.9)]) == int(n * 0.9) - int(n * 0.3)
  high = [bool(t >= 875) for t in np.linspace(999, 0, 3, dtype=np.int32)]
  assert all(CP.SenCache(3).forced(s, s > 0 and high[s] != high[s - 1]) for s in range(3))   # too short to cache
  sc = CP.SenCache(50)
  assert sc.forced(20, at_boundary=True) and not sc.forced(20)

  x = torch.zeros(4, 4)
  sc = CP.SenCache(50, threshold=0.1, max_reuse=3)
  assert not sc.should_reuse(20, x, 600.0, False)            # nothing cached yet
  sc.record_full(x, 600.0, torch.ones(1))
  assert sc.should_reuse(21, x + 0.03, 580.0, False)         # 0.03 + 0.02 <= 0.1
  sc.record_reuse()
  assert not sc.should_reuse(22, x + 0.03 + 0.5, 560.0, False)   # drift of the latents
  sc.record_full(x, 560.0, torch.ones(1))
  assert not sc.should_reuse(23, x + 0.01, 60.0, False)      # drift of the timestep: 0.01 + 0.5
  sc.record_full(x, 500.0, torch.ones(1))
  reused = 0
  for s in range(24, 34):
    if sc.should_reuse(s, x, 500.0, False):
      sc.record_reuse()
      reused += 1
    else:
      break
  assert reused == 3


def test_vae_encode_chunk_comes_from_the_configuration():
  import types

  pipe = WanPipeline2_1.__new__(WanPipeline2_1)
  pipe.vae_scale_factor_temporal = 4
  for value, frames, want in ((4, 81, 4), (8, 81, 8), (-1, 81, 80), (-1, 1, 4), (-1, 10, 12)):
    pipe.config = types.SimpleNamespace(get=lambda k, d=None, v=value: v if k == "vae_encode_chunk" else d)
    assert pipe.vae_encode_chunk(frames) == want
  for bad in (0, 3, 6):
    pipe.config = types.SimpleNamespace(get=lambda k, d=None, v=bad: v)
    with pytest.raises(ValueError, match="multiple of the temporal stride"):
      pipe.vae_encode_chunk(81)
