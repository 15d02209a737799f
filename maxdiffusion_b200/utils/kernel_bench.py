"""Micro-benchmarks of the hot kernels against the measured roofline (CUDA events, L2 flushed).

  python -m maxdiffusion_b200.utils.kernel_bench [gemm] [flash] [rowwise] [--json out.json]

Each case runs 3 warm-up and `iters` timed launches; between timed launches a buffer larger than the
126 MB L2 is overwritten. Fractions are reported against MEASURED_PEAKS.json when it is present in the
working directory ("of measured"), else against the fallback 1590 TFLOP/s / 6650 GB/s ("of fallback").
"""
from __future__ import annotations

import json
import os
import sys

import torch

from maxdiffusion_b200.ops import kernels as K


def peaks():
  try:
    with open("MEASURED_PEAKS.json") as f:
      p = json.load(f)
    return p["bf16_tflops"], p["hbm_gbs"], "measured"
  except Exception:
    return 1590.0, 6650.0, "fallback"


_FLUSH = None


def flush_l2():
  global _FLUSH
  if _FLUSH is None:
    _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
  _FLUSH.zero_()


def time_ms(fn, iters=10, warmup=3):
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  ts = []
  for _ in range(iters):
    flush_l2()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    ts.append(e0.elapsed_time(e1))
  ts.sort()
  return ts[len(ts) // 2], ts[0]


def bench_gemm(results):
  tf_peak, _, tag = peaks()
  shapes = [(32760, 5120, 5120), (32760, 13824, 5120), (32760, 5120, 13824), (4096, 5120, 5120), (4608, 9216, 3072)]
  for M, N, Kd in shapes:
    a = torch.randn((M, Kd), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((N, Kd), device="cuda", dtype=torch.bfloat16)
    out = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    med, best = time_ms(lambda: K.gemm(a, b, out=out))
    lib_med, _ = time_ms(lambda: torch.matmul(a, b.t(), out=out))
    fl = 2.0 * M * N * Kd
    results.append(dict(kernel="gemm_bf16", shape=[M, N, Kd], ms=med, best_ms=best, tflops=fl / med / 1e9,
                        frac=fl / med / 1e9 / tf_peak, of=tag, cublas_ms=lib_med))
    print(results[-1], flush=True)
    del a, b, out


def bench_gemm_small_m(results):
  """The GEMM shapes of one rank of an 8-way sequence split (4095 tokens), 256- against 128-wide tiles, with the
  default and cuBLAS beside them; forward, dgrad (B stored [K,N]) and wgrad (both operands transposed)."""
  tf_peak, _, tag = peaks()
  cases = [(4095, 5120, 5120, False, False), (4095, 15360, 5120, False, False), (4095, 13824, 5120, False, False),
           (4095, 5120, 13824, False, False), (4095, 5120, 5120, False, True), (5120, 5120, 4095, True, True),
           (13824, 5120, 4095, True, True), (8190, 5120, 5120, False, False)]
  for M, N, Kd, a_mn, b_mn in cases:
    a = torch.randn((Kd, M) if a_mn else (M, Kd), device="cuda", dtype=torch.bfloat16)
    if a_mn and M % 8:
      a = torch.randn((Kd, M + 8 - M % 8), device="cuda", dtype=torch.bfloat16)[:, :M]
    b = torch.randn((Kd, N) if b_mn else (N, Kd), device="cuda", dtype=torch.bfloat16)
    out = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    ms = {}
    for bn in (256, 128, 0):
      K.gemm_force_tile_n(bn)
      ms[bn], _ = time_ms(lambda: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out))
    K.gemm_force_tile_n(0)
    am, bm = (a.t() if a_mn else a), (b if b_mn else b.t())
    lib_med, _ = time_ms(lambda: torch.matmul(am, bm, out=out))
    fl = 2.0 * M * N * Kd
    results.append(dict(kernel="gemm_bf16_small_m", shape=[M, N, Kd], a_mn=a_mn, b_mn=b_mn, ms_tile256=ms[256],
                        ms_tile128=ms[128], ms_auto=ms[0], tflops_auto=fl / ms[0] / 1e9,
                        frac_auto=fl / ms[0] / 1e9 / tf_peak, of=tag, cublas_ms=lib_med))
    print(results[-1], flush=True)
    del a, b, out


def bench_gemm_unet(results):
  """The GEMM shapes of the SDXL UNet's transformer blocks at batch 8 (short contractions: K = 640 / 1280, where the
  epilogue weighs as much as the main loop): plain, with bias, with bias + residual add, dgrad, and the weight
  gradient with and without split-K; cuBLAS (`F.linear` / `torch.matmul` + the separate add) beside each."""
  import torch.nn.functional as F

  tf_peak, _, tag = peaks()
  for M, N, Kd in [(8192, 1280, 1280), (8192, 10240, 1280), (8192, 1280, 5120), (32768, 640, 640), (32768, 5120, 640)]:
    a = torch.randn((M, Kd), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((N, Kd), device="cuda", dtype=torch.bfloat16) * 0.03
    bias = torch.randn((N,), device="cuda", dtype=torch.bfloat16)
    res = torch.randn((M, N), device="cuda", dtype=torch.bfloat16)
    dy = torch.randn((M, N), device="cuda", dtype=torch.bfloat16)
    out = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    fl = 2.0 * M * N * Kd
    row = dict(kernel="gemm_bf16_unet", shape=[M, N, Kd], of=tag)
    row["plain_ms"], _ = time_ms(lambda: K.gemm(a, b, out=out))
    row["bias_ms"], _ = time_ms(lambda: K.gemm(a, b, bias=bias, out=out))
    row["bias_res_ms"], _ = time_ms(lambda: K.gemm(a, b, bias=bias, epi="add_res", residual=res, out=out))
    row["dgrad_ms"], _ = time_ms(lambda: K.gemm(dy, b, b_mn=True))
    row["wgrad_ms"], _ = time_ms(lambda: K.gemm(dy, a, a_mn=True, b_mn=True))
    row["wgrad_nosplit_ms"], _ = time_ms(lambda: K.gemm(dy, a, a_mn=True, b_mn=True, split_k=1))
    row["wgrad_splits"] = K.split_k_for(N, Kd, M)
    row["cublas_plain_ms"], _ = time_ms(lambda: torch.matmul(a, b.t(), out=out))
    row["cublas_bias_ms"], _ = time_ms(lambda: F.linear(a, b, bias))
    row["cublas_bias_res_ms"], _ = time_ms(lambda: F.linear(a, b, bias).add_(res))
    row["cublas_dgrad_ms"], _ = time_ms(lambda: torch.matmul(dy, b))
    row["cublas_wgrad_ms"], _ = time_ms(lambda: torch.matmul(dy.t(), a))
    row["tflops_plain"] = fl / row["plain_ms"] / 1e9
    row["frac_plain"] = row["tflops_plain"] / tf_peak
    results.append(row)
    print(row, flush=True)
    del a, b, res, dy, out


def bench_gemm_fp8(results):
  tf_peak, _, tag = peaks()
  for M, N, Kd in [(32760, 5120, 5120), (32760, 13824, 5120), (4096, 5120, 5120)]:
    a = torch.randn((M, Kd), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((N, Kd), device="cuda", dtype=torch.bfloat16)
    aq, sa = K.quantize_fp8(a)
    bq, sb = K.quantize_fp8(b)
    med, best = time_ms(lambda: K.gemm_fp8(aq, sa, bq, sb))
    qmed, _ = time_ms(lambda: K.quantize_fp8(a))
    fl = 2.0 * M * N * Kd
    results.append(dict(kernel="gemm_fp8", shape=[M, N, Kd], ms=med, best_ms=best, tflops=fl / med / 1e9,
                        frac_of_bf16_peak=fl / med / 1e9 / tf_peak, of=tag, quantize_activation_ms=qmed))
    print(results[-1], flush=True)
    del a, b, aq, bq


def bench_flash(results):
  tf_peak, _, tag = peaks()
  for B, H, Sq, Skv in [(1, 40, 4096, 32768), (1, 40, 8192, 8192), (1, 24, 4608, 4608), (1, 40, 32760, 32760)]:
    q = torch.randn((B, Sq, H, 128), device="cuda", dtype=torch.bfloat16)
    k = torch.randn((B, Skv, H, 128), device="cuda", dtype=torch.bfloat16)
    v = torch.randn((B, Skv, H, 128), device="cuda", dtype=torch.bfloat16)
    med, best = time_ms(lambda: K.flash_fwd(q, k, v), iters=5)
    fl = 4.0 * B * H * Sq * Skv * 128
    results.append(dict(kernel="flash_fwd", shape=[B, H, Sq, Skv], ms=med, best_ms=best, tflops=fl / med / 1e9,
                        frac=fl / med / 1e9 / tf_peak, of=tag))
    print(results[-1], flush=True)
    del q, k, v


def bench_flash_fixed_m(results):
  """Plain against fixed-exponent softmax on the same tensors (all heads eligible), plus the cost of the plan."""
  from ..ops import fixed_m as FM

  tf_peak, _, tag = peaks()
  for B, H, Sq, Skv in [(1, 40, 8192, 8192), (1, 40, 32760, 32760)]:
    q = torch.randn((B, Sq, H, 128), device="cuda", dtype=torch.bfloat16)
    k = FM.smooth_keys(torch.randn((B, Skv, H, 128), device="cuda", dtype=torch.bfloat16))
    v = torch.randn((B, Skv, H, 128), device="cuda", dtype=torch.bfloat16)
    plan = FM.plan(q, k)
    base, _ = time_ms(lambda: K.flash_fwd(q, k, v), iters=5)
    fixed, _ = time_ms(lambda: K.flash_fwd(q, k, v, fixed_m=plan), iters=5)
    plan_ms, _ = time_ms(lambda: FM.plan(q, FM.smooth_keys(k)), iters=5)
    fl = 4.0 * B * H * Sq * Skv * 128
    results.append(dict(kernel="flash_fwd_fixed_m", shape=[B, H, Sq, Skv], eligible_heads=int(plan[1].sum()),
                        plain_ms=base, fixed_ms=fixed, plan_and_smoothing_ms=plan_ms, fixed_tflops=fl / fixed / 1e9,
                        fixed_frac=fl / fixed / 1e9 / tf_peak, of=tag))
    print(results[-1], flush=True)
    del q, k, v, plan


def bench_flash_d64(results):
  """head_dim 64 (SDXL self-attention shapes: batch 8, 10 heads x 4096 tokens and 20 heads x 1024 tokens; LTX-Video
  2B: 32 heads) forward and backward, with PyTorch SDPA on the same tensors for comparison."""
  import torch.nn.functional as F

  tf_peak, _, tag = peaks()
  for B, H, S in [(8, 10, 4096), (8, 20, 1024), (1, 32, 16384)]:
    q, k, v, d_o = (torch.randn((B, S, H, 64), device="cuda", dtype=torch.bfloat16) for _ in range(4))
    out, lse = K.flash_fwd(q, k, v)
    delta = K.flash_delta(out, d_o)
    fwd, _ = time_ms(lambda: K.flash_fwd(q, k, v), iters=5)
    dkv, _ = time_ms(lambda: K.flash_bwd_dkv(q, d_o, k, v, lse, delta), iters=5)
    dq, _ = time_ms(lambda: K.flash_bwd_dq(q, d_o, k, v, lse, delta), iters=5)
    qt, kt, vt = (t.transpose(1, 2) for t in (q, k, v))
    sdpa, _ = time_ms(lambda: F.scaled_dot_product_attention(qt, kt, vt), iters=5)
    fl = 4.0 * B * H * S * S * 64
    results.append(dict(kernel="flash_d64", shape=[B, H, S], fwd_ms=fwd, dkv_ms=dkv, dq_ms=dq, sdpa_fwd_ms=sdpa,
                        fwd_tflops=fl / fwd / 1e9, bwd_tflops_algorithmic=2.5 * fl / (dkv + dq) / 1e9,
                        fwd_frac=fl / fwd / 1e9 / tf_peak, of=tag))
    print(results[-1], flush=True)
    del q, k, v, d_o, out


def bench_flash_bwd(results):
  tf_peak, _, tag = peaks()
  for B, H, Sq, Skv in [(1, 40, 4096, 4096), (1, 40, 8192, 8192), (1, 40, 32760, 32760)]:
    q = torch.randn((B, Sq, H, 128), device="cuda", dtype=torch.bfloat16)
    k = torch.randn((B, Skv, H, 128), device="cuda", dtype=torch.bfloat16)
    v = torch.randn((B, Skv, H, 128), device="cuda", dtype=torch.bfloat16)
    d_o = torch.randn((B, Sq, H, 128), device="cuda", dtype=torch.bfloat16)
    out, lse = K.flash_fwd(q, k, v)
    delta = K.flash_delta(out, d_o)
    med_kv, _ = time_ms(lambda: K.flash_bwd_dkv(q, d_o, k, v, lse, delta), iters=5)
    med_q, _ = time_ms(lambda: K.flash_bwd_dq(q, d_o, k, v, lse, delta), iters=5)
    fl = 10.0 * B * H * Sq * Skv * 128  # algorithmic backward FLOPs (5 GEMMs)
    results.append(dict(kernel="flash_bwd", shape=[B, H, Sq, Skv], dkv_ms=med_kv, dq_ms=med_q,
                        tflops_algorithmic=fl / (med_kv + med_q) / 1e9, frac=fl / (med_kv + med_q) / 1e9 / tf_peak,
                        tflops_issued=14.0 * B * H * Sq * Skv * 128 / (med_kv + med_q) / 1e9, of=tag))
    print(results[-1], flush=True)
    del q, k, v, d_o, out


def bench_rowwise(results):
  _, bw_peak, tag = peaks()
  B, S, C = 1, 32760, 5120
  x = torch.randn((B, S, C), device="cuda", dtype=torch.bfloat16)
  sc = torch.randn((B, C), device="cuda", dtype=torch.float32)
  med, best = time_ms(lambda: K.ln_fwd(x, None, None, sc, sc))
  nbytes = 2 * x.numel() * 2
  results.append(dict(kernel="ln_mod_fwd", shape=[B, S, C], ms=med, gbs=nbytes / med / 1e6,
                      frac=nbytes / med / 1e6 / bw_peak, of=tag))
  print(results[-1], flush=True)
  w = torch.randn((C,), device="cuda", dtype=torch.bfloat16)
  cos = torch.rand((S, 64), device="cuda")
  med, best = time_ms(lambda: K.rms_rope_fwd(x, w, cos, cos, heads=40))
  results.append(dict(kernel="rms_rope_fwd", shape=[B, S, C], ms=med, gbs=nbytes / med / 1e6,
                      frac=nbytes / med / 1e6 / bw_peak, of=tag))
  print(results[-1], flush=True)
  # backward kernels: read dy and x, write dx (3 passes of 2 B/element), column sums folded by a second launch
  dy = torch.randn_like(x)
  _, mean, rstd = K.ln_fwd(x, None, None, sc, sc, save_stats=True)
  med, best = time_ms(lambda: K.ln_bwd(dy, x, mean, rstd, None, sc))
  nb3 = 3 * x.numel() * 2
  results.append(dict(kernel="ln_mod_bwd", shape=[B, S, C], ms=med, gbs=nb3 / med / 1e6,
                      frac=nb3 / med / 1e6 / bw_peak, of=tag))
  print(results[-1], flush=True)
  _, rr = K.rms_rope_fwd(x, w, cos, cos, heads=40, save_stats=True)
  med, best = time_ms(lambda: K.rms_rope_bwd(dy.view(B, S, 40, 128), x, rr, w, cos, cos))
  results.append(dict(kernel="rms_rope_bwd", shape=[B, S, C], ms=med, gbs=nb3 / med / 1e6,
                      frac=nb3 / med / 1e6 / bw_peak, of=tag))
  print(results[-1], flush=True)
  med, best = time_ms(lambda: K.colsum(x.view(S, C)))
  results.append(dict(kernel="colsum", shape=[S, C], ms=med, gbs=x.numel() * 2 / med / 1e6,
                      frac=x.numel() * 2 / med / 1e6 / bw_peak, of=tag))
  print(results[-1], flush=True)


def bench_conv(results):
  """Implicit-GEMM convolutions at the shapes of the Wan VAE decoder (720p: latent 90 x 160, four frames per chunk at
  the top stage) and of the SDXL UNet (batch 8), each beside cuDNN on the same bf16 tensors in its preferred layout
  (`channels_last_3d` / `channels_last`). FLOPs count the taps actually needed (27 or 9 per output)."""
  import torch.nn.functional as F

  from maxdiffusion_b200.ops import conv as OC

  tf_peak, bw_peak, tag = peaks()
  cases3d = [(1, 4, 720, 1280, 64, 64), (1, 4, 720, 1280, 128, 128), (1, 4, 720, 1280, 96, 96), (1, 4, 360, 640, 192, 192), (1, 2, 180, 320, 384, 384), (1, 1, 90, 160, 384, 384),
             (1, 4, 720, 1280, 96, 3)]
  for B, T, H, W, Ci, Co in cases3d:
    x = torch.randn((B, T, H, W, Ci), device="cuda", dtype=torch.bfloat16)
    hist = torch.randn((B, 2, H, W, Ci), device="cuda", dtype=torch.bfloat16)
    w = torch.randn((Co, Ci, 3, 3, 3), device="cuda", dtype=torch.bfloat16) * (27 * Ci) ** -0.5
    b = torch.randn((Co,), device="cuda", dtype=torch.bfloat16)
    pk = OC.pack_conv3d(w, b)
    med, best = time_ms(lambda: OC.conv3d_causal(x, pk, hist=hist), iters=5)
    xn = torch.cat([hist, x], dim=1).permute(0, 4, 1, 2, 3).contiguous(memory_format=torch.channels_last_3d)
    wn = w.contiguous(memory_format=torch.channels_last_3d)
    lib, _ = time_ms(lambda: F.conv3d(F.pad(xn, (1, 1, 1, 1, 0, 0)), wn, b), iters=5)
    fl = 2.0 * B * T * H * W * Co * Ci * 27
    byts = 2.0 * B * T * H * W * (Ci + Co)
    results.append(dict(kernel="conv3d_causal_igemm", shape=[B, T, H, W, Ci, Co], ms=med, best_ms=best, tflops=fl / med / 1e9,
                        frac=fl / med / 1e9 / tf_peak, of=tag, gbs=byts / med / 1e6, cudnn_ms=lib))
    print(results[-1], flush=True)
    del x, hist, xn
  # launch shapes of the narrow-tile convolutions: (units per stage, stage limit, CTAs per SM); (0, 0, 0) is the default
  for Ci in (96, 128):
    x = torch.randn((1, 4, 720, 1280, Ci), device="cuda", dtype=torch.bfloat16)
    pk = OC.pack_conv3d(torch.randn((Ci, Ci, 3, 3, 3), device="cuda", dtype=torch.bfloat16) * 0.02, None)
    for cfg in ((0, 0, 0), (2, 0, 1), (1, 0, 1), (1, 0, 2), (1, 2, 2)):
      OC.tune(*cfg)
      try:
        med, best = time_ms(lambda: OC.conv3d_causal(x, pk), iters=5)
      except Exception as e:  # a launch shape that does not fit the shared-memory budget is rejected by the launcher
        print(dict(kernel="conv3d_causal_igemm_tuning", tune=list(cfg), rejected=str(e)), flush=True)
        continue
      results.append(dict(kernel="conv3d_causal_igemm_tuning", shape=[1, 4, 720, 1280, Ci, Ci], tune=list(cfg), ms=med,
                          tflops=2.0 * 4 * 720 * 1280 * Ci * Ci * 27 / med / 1e9))
      print(results[-1], flush=True)
    OC.tune(0, 0, 0)
    del x
  cases2d = [(8, 128, 128, 320, 320, "s1"), (8, 64, 64, 640, 640, "s1"), (8, 32, 32, 1280, 1280, "s1"),
             (8, 128, 128, 320, 320, "s2"), (4, 360, 640, 192, 96, "up"), (8, 64, 64, 640, 640, "dgrad")]
  for B, H, W, Ci, Co, kind in cases2d:
    x = torch.randn((B, H, W, Ci), device="cuda", dtype=torch.bfloat16)
    w = torch.randn((Co, Ci, 3, 3), device="cuda", dtype=torch.bfloat16) * (9 * Ci) ** -0.5
    b = torch.randn((Co,), device="cuda", dtype=torch.bfloat16)
    xn = x.permute(0, 3, 1, 2)  # NCHW view of channels-last memory
    wn = w.contiguous(memory_format=torch.channels_last)
    if kind == "s1":
      pk = OC.pack_conv2d(w, b)
      fn, lib_fn, fl = (lambda: OC.conv2d(x, pk)), (lambda: F.conv2d(xn, wn, b, padding=1)), 2.0 * B * H * W * Co * Ci * 9
    elif kind == "s2":
      pk = OC.pack_conv2d(w, b, stride=2, pad_top_left=1)
      fn, lib_fn, fl = (lambda: OC.conv2d(x, pk)), (lambda: F.conv2d(xn, wn, b, padding=1, stride=2)), 2.0 * B * H * W * Co * Ci * 9 / 4
    elif kind == "up":
      pk = OC.pack_upsample_conv2d(w, b)
      fn = lambda: OC.upsample2x_conv2d(x, pk)
      lib_fn = lambda: F.conv2d(F.interpolate(xn, scale_factor=2.0, mode="nearest"), wn, b, padding=1)
      fl = 2.0 * B * 4 * H * W * Co * Ci * 9  # what up-sampling first would cost; the fused form runs 4 / 9 of it
    else:
      pk = OC.pack_conv2d_dgrad(w)
      dy = torch.randn((B, H, W, Co), device="cuda", dtype=torch.bfloat16)
      dyn = dy.permute(0, 3, 1, 2)
      fn = lambda: OC.conv2d_dgrad(dy, pk)
      lib_fn = lambda: torch.nn.grad.conv2d_input((B, Ci, H, W), wn, dyn, padding=1)
      fl = 2.0 * B * H * W * Co * Ci * 9
    med, best = time_ms(fn, iters=5)
    lib, _ = time_ms(lib_fn, iters=5)
    results.append(dict(kernel=f"conv2d_igemm_{kind}", shape=[B, H, W, Ci, Co], ms=med, best_ms=best, tflops=fl / med / 1e9,
                        frac=fl / med / 1e9 / tf_peak, of=tag, cudnn_ms=lib))
    print(results[-1], flush=True)
  for B, H, W, Ci, Co, stride in [(8, 128, 128, 320, 320, 1), (8, 64, 64, 640, 640, 1), (8, 32, 32, 1280, 1280, 1), (8, 128, 128, 320, 320, 2)]:
    x = torch.randn((B, H, W, Ci), device="cuda", dtype=torch.bfloat16)
    dy = torch.randn((B, H // stride, W // stride, Co), device="cuda", dtype=torch.bfloat16)
    med, best = time_ms(lambda: OC.conv2d_wgrad(x, dy, 3, stride, 1), iters=5)
    bordered, _ = time_ms(lambda: OC.conv2d_wgrad(x, dy, 3, stride, 1, boxed=False), iters=5)
    xn, dyn = x.permute(0, 3, 1, 2), dy.permute(0, 3, 1, 2)
    lib, _ = time_ms(lambda: torch.nn.grad.conv2d_weight(xn, (Co, Ci, 3, 3), dyn, stride=stride, padding=1), iters=5)
    fl = 2.0 * B * (H // stride) * (W // stride) * Co * Ci * 9
    results.append(dict(kernel=f"conv2d_wgrad_s{stride}", shape=[B, H, W, Ci, Co], ms=med, best_ms=best, tflops=fl / med / 1e9,
                        frac=fl / med / 1e9 / tf_peak, of=tag, cudnn_ms=lib, bordered_ms=bordered,
                        note="boxes of output pixels read from the unpadded tensors, split fold included; bordered_ms = the flat form with its zero-border copies"))
    print(results[-1], flush=True)
  from maxdiffusion_b200.ops import functional as OF

  for N, C, H, W in [(8, 320, 128, 128), (8, 1280, 32, 32)]:
    x = torch.randn((N, C, H, W), device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    g = torch.ones(C, device="cuda", dtype=torch.bfloat16)
    med, best = time_ms(lambda: OF.group_norm(x, 32, g, g, 1e-5, True), iters=5)
    lib, _ = time_ms(lambda: F.silu(F.group_norm(x, 32, g, g, 1e-5)), iters=5)
    results.append(dict(kernel="group_norm_silu_cl_fwd", shape=[N, C, H, W], ms=med, gbs=6.0 * x.numel() / med / 1e6,
                        frac=6.0 * x.numel() / med / 1e6 / bw_peak, of=tag, torch_ms=lib, note="two reads + one write of the activation"))
    print(results[-1], flush=True)
  for C in (96, 384):
    x = torch.randn((4 * 720 * 1280 * 96 // C, C), device="cuda", dtype=torch.bfloat16)
    g = torch.ones(C, device="cuda")
    med, best = time_ms(lambda: OC.rms_act(x, g, None, silu=True), iters=5)
    results.append(dict(kernel="rms_act_cl", shape=list(x.shape), ms=med, gbs=4.0 * x.numel() / med / 1e6,
                        frac=4.0 * x.numel() / med / 1e6 / bw_peak, of=tag))
    print(results[-1], flush=True)


def conv_profile_case():
  """One launch of the causal conv3d on a mid-size case (96 channels, 2 x 360 x 640 output positions) for `ncu`."""
  from maxdiffusion_b200.ops import conv as OC

  x = torch.randn((1, 2, 360, 640, 96), device="cuda", dtype=torch.bfloat16)
  hist = torch.randn((1, 2, 360, 640, 96), device="cuda", dtype=torch.bfloat16)
  w = torch.randn((96, 96, 3, 3, 3), device="cuda", dtype=torch.bfloat16) * 0.02
  pk = OC.pack_conv3d(w, None)
  for _ in range(3):
    OC.conv3d_causal(x, pk, hist=hist)
  torch.cuda.synchronize()
  print("conv profile case done")


def unet_profile_case():
  """The UNet's kernels on one mid-size case each, for `ncu`: the convolution weight gradient (640 channels at 64^2,
  batch 8), the forward convolution and the GEMM with bias + residual epilogue at a short contraction."""
  from ..ops import conv as OC

  x = torch.randn((8, 64, 64, 640), device="cuda", dtype=torch.bfloat16)
  dy = torch.randn((8, 64, 64, 640), device="cuda", dtype=torch.bfloat16)
  w = torch.randn((640, 640, 3, 3), device="cuda", dtype=torch.bfloat16) * 0.02
  pk = OC.pack_conv2d(w, None)
  for _ in range(2):
    OC.conv2d_wgrad(x, dy, 3, 1)
    OC.conv2d(x, pk)
  a = torch.randn((32768, 640), device="cuda", dtype=torch.bfloat16)
  b = torch.randn((5120, 640), device="cuda", dtype=torch.bfloat16) * 0.03
  bias = torch.randn((5120,), device="cuda", dtype=torch.bfloat16)
  res = torch.randn((32768, 5120), device="cuda", dtype=torch.bfloat16)
  for _ in range(2):
    K.gemm(a, b, bias=bias, epi="add_res", residual=res)
  torch.cuda.synchronize()
  print("unet profile case done")


def profile_case():
  """One launch of each hot kernel on a mid-size case (inputs larger than L2, < 1 GB resident) for `ncu`."""
  M, N, Kd = 8192, 5120, 5120
  a = torch.randn((M, Kd), device="cuda", dtype=torch.bfloat16)
  b = torch.randn((N, Kd), device="cuda", dtype=torch.bfloat16)
  K.gemm(a, b)
  B, H, S = 1, 16, 8192
  q = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
  k = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
  v = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
  d_o = torch.randn((B, S, H, 128), device="cuda", dtype=torch.bfloat16)
  out, lse = K.flash_fwd(q, k, v)
  delta = K.flash_delta(out, d_o)
  K.flash_bwd_dkv(q, d_o, k, v, lse, delta)
  K.flash_bwd_dq(q, d_o, k, v, lse, delta)
  x = torch.randn((1, 32760, 5120), device="cuda", dtype=torch.bfloat16)
  sc = torch.randn((1, 5120), device="cuda", dtype=torch.float32)
  K.ln_fwd(x, None, None, sc, sc)
  torch.cuda.synchronize()
  print("profile case done")


def main(argv):
  if "profile" in argv:
    return profile_case()
  if "conv_profile" in argv:
    return conv_profile_case()
  if "unet_profile" in argv:
    return unet_profile_case()
  which = [a for i, a in enumerate(argv) if not a.startswith("--") and (i == 0 or argv[i - 1] != "--json")] or ["gemm", "flash", "rowwise"]
  results = []
  if "gemm" in which:
    bench_gemm(results)
  if "gemm_small_m" in which:
    bench_gemm_small_m(results)
  if "gemm_unet" in which:
    bench_gemm_unet(results)
  if "gemm_fp8" in which:
    bench_gemm_fp8(results)
  if "flash" in which:
    bench_flash(results)
  if "flash_bwd" in which:
    bench_flash_bwd(results)
  if "flash_d64" in which:
    bench_flash_d64(results)
  if "flash_fixed_m" in which:
    bench_flash_fixed_m(results)
  if "rowwise" in which:
    bench_rowwise(results)
  if "conv" in which:
    bench_conv(results)
  if "--json" in argv:
    path = argv[argv.index("--json") + 1]
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
      json.dump(results, f, indent=1)


if __name__ == "__main__":
  main(sys.argv[1:])
