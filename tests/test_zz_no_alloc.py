"""The allocation-free column-sum entry point, called through its exported C symbol.

Some users of the kernel library may not allocate device memory at the point of the call (inside a stream
capture, inside another framework's callback, in a loop that forbids allocation after start-up); for them
`mdb_colsum_noalloc` keeps its scratch in a fixed array inside the library. This file is collected last so that a
run which stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
  from maxdiffusion_b200.ops import _lib

  L = _lib.lib()
  fn = L.mdb_colsum_noalloc
  fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
  fn.restype = ctypes.c_int
  err = L.mdb_colsum_noalloc_strerror
  err.argtypes = [ctypes.c_int]
  err.restype = ctypes.c_char_p
  return fn, err


def test_no_alloc_colsum_matches_regular_entry_point_twice():
  from maxdiffusion_b200.ops import kernels as K

  fn, err = _symbols()
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  # two calls in a row with different shapes: the second must not see anything of the first in the shared scratch
  for seed, (rows, cols) in enumerate([(3001, 5120), (777, 1536)]):
    torch.manual_seed(seed)
    x = torch.randn((rows, cols), device="cuda", dtype=torch.bfloat16)
    out = torch.full((cols,), float("nan"), device="cuda", dtype=torch.float32)
    rc = fn(ctypes.c_void_p(x.data_ptr()), x.stride(0), rows, cols, ctypes.c_void_p(out.data_ptr()), stream)
    assert rc == 0, err(rc).decode()
    want = K.colsum(x)
    torch.cuda.synchronize()
    ref = x.float().sum(0)
    assert (out - want).abs().max().item() <= 1e-3 * (1.0 + ref.abs().max().item())
    assert ((out - ref).norm() / ref.norm()).item() < 1e-4


def test_no_alloc_colsum_rejects_what_does_not_fit():
  fn, err = _symbols()
  x = torch.zeros((8, 8), device="cuda", dtype=torch.bfloat16)
  out = torch.zeros((8,), device="cuda", dtype=torch.float32)
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  rc = fn(ctypes.c_void_p(x.data_ptr()), 16384, 4, 16384, ctypes.c_void_p(out.data_ptr()), stream)
  assert rc == -1 and b"8192" in err(rc)
  rc = fn(ctypes.c_void_p(x.data_ptr()), 8, 4, 12, ctypes.c_void_p(out.data_ptr()), stream)
  assert rc == -2


def test_no_alloc_colsum_of_no_rows_is_zero():
  fn, err = _symbols()
  x = torch.zeros((8, 16), device="cuda", dtype=torch.bfloat16)
  out = torch.full((16,), float("nan"), device="cuda", dtype=torch.float32)
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  rc = fn(ctypes.c_void_p(x.data_ptr()), 16, 0, 16, ctypes.c_void_p(out.data_ptr()), stream)
  assert rc == 0, err(rc).decode()
  torch.cuda.synchronize()
  assert torch.equal(out, torch.zeros_like(out))
