"""Helpers for tests: skip decorators keyed on what the machine has, tolerant tensor comparison, seeded inputs
(reference: src/maxdiffusion/utils/testing_utils.py)."""
from __future__ import annotations

import os
import random
import unittest

import numpy as np
import torch

from .import_utils import is_available


def require(package: str):
  return unittest.skipUnless(is_available(package), f"needs {package}")


def require_cuda(fn):
  return unittest.skipUnless(torch.cuda.is_available(), "needs a CUDA device")(fn)


def require_multi_gpu(n: int = 2):
  return unittest.skipUnless(torch.cuda.is_available() and torch.cuda.device_count() >= n, f"needs {n} GPUs")


def slow(fn):
  return unittest.skipUnless(os.environ.get("RUN_SLOW", "0") not in ("0", ""), "slow test: set RUN_SLOW=1")(fn)


def enable_full_determinism(seed: int = 0) -> None:
  random.seed(seed)
  np.random.seed(seed)
  torch.manual_seed(seed)
  torch.backends.cudnn.deterministic = True
  torch.backends.cudnn.benchmark = False
  torch.backends.cuda.matmul.allow_tf32 = False


def floats_tensor(shape, scale: float = 1.0, seed: int = 0, device="cpu", dtype=torch.float32) -> torch.Tensor:
  g = torch.Generator().manual_seed(seed)
  return (torch.rand(tuple(shape), generator=g) * scale).to(device=device, dtype=dtype)


def max_diff(a, b) -> float:
  return (torch.as_tensor(a).float() - torch.as_tensor(b).float()).abs().max().item()


def assert_close(a, b, atol: float = 1e-5, rtol: float = 1e-5, msg: str = "") -> None:
  a, b = torch.as_tensor(a).float(), torch.as_tensor(b).float()
  if not torch.allclose(a, b, atol=atol, rtol=rtol):
    d = (a - b).abs()
    raise AssertionError(f"{msg} max|diff| {d.max().item():.3e} at {tuple(np.unravel_index(int(d.argmax()), d.shape))}, atol {atol}, rtol {rtol}")


def relative_l2(a, b) -> float:
  a, b = torch.as_tensor(a).float(), torch.as_tensor(b).float()
  return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()
