"""Compares the attention implementations on one shape: numerics against an fp32 reference and time per call.

  python -m maxdiffusion_b200.pedagogical_examples.attention_comparison [--seq 4096] [--heads 8] [--dim 128]

On a B200 the candidates are the tcgen05 flash kernel of this package (`ops.functional.attention`) and PyTorch SDPA;
on CPU only the reference and SDPA run (reference script: pedagogical_examples/attention_comparison.py).
"""
from __future__ import annotations

import argparse
import time

import torch
import torch.nn.functional as F


def reference_attention(q, k, v):
  s = (q.float() @ k.float().transpose(-1, -2)) / q.shape[-1] ** 0.5
  return (s.softmax(-1) @ v.float())


def timed(fn, iters: int = 5):
  fn()
  if torch.cuda.is_available():
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
      fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters
  t0 = time.perf_counter()
  for _ in range(iters):
    fn()
  return (time.perf_counter() - t0) / iters * 1e3


def run(seq: int = 1024, heads: int = 4, dim: int = 128, batch: int = 1) -> dict:
  dev = "cuda" if torch.cuda.is_available() else "cpu"
  dtype = torch.bfloat16 if dev == "cuda" else torch.float32
  g = torch.Generator(device=dev).manual_seed(0)
  q, k, v = (torch.randn((batch, heads, seq, dim), generator=g, device=dev, dtype=dtype) for _ in range(3))
  ref = reference_attention(q, k, v)
  flops = 4 * batch * heads * seq * seq * dim
  cands = {"sdpa": lambda: F.scaled_dot_product_attention(q, k, v)}
  if dev == "cuda":
    from ..ops import functional as OF

    cands["flash_tcgen05"] = lambda: OF.attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
  out = {}
  for name, fn in cands.items():
    err = (fn().float() - ref).abs().max().item()
    ms = timed(fn)
    out[name] = {"max_abs_err": err, "ms": ms, "tflops": flops / ms / 1e9}
    print(f"{name:>14}: max|err| {err:.3e}  {ms:8.3f} ms  {out[name]['tflops']:8.1f} TFLOP/s")
  return out


if __name__ == "__main__":
  ap = argparse.ArgumentParser()
  ap.add_argument("--seq", type=int, default=4096)
  ap.add_argument("--heads", type=int, default=8)
  ap.add_argument("--dim", type=int, default=128)
  ap.add_argument("--batch", type=int, default=1)
  a = ap.parse_args()
  run(a.seq, a.heads, a.dim, a.batch)
