"""A device-side wait that runs out: the kernel returns by itself, the host sees the reason in the status word, the
status clears, and the CUDA context goes on working. The failure is made on the host side only: the kernel waits,
with a budget of 50 ms, for a flag that nothing ever sets. No GPU fault, trap or hang is involved."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_flag_wait_runs_out_and_is_reported_and_cleared():
  from maxdiffusion_b200.ops import _lib
  from maxdiffusion_b200.ops import kernels as K
  from maxdiffusion_b200.parallel import symm  # registers the comm entry points

  assert symm.NUM_FLAG_KINDS > 0
  torch.cuda.synchronize()
  _lib.read_status(clear=True)
  flags = torch.zeros(8, dtype=torch.int32, device="cuda")
  t0 = time.perf_counter()
  rc = _lib.lib().mdb_wait_flags(ctypes.c_void_p(flags.data_ptr()), 2, 1, 1, 0.05, _lib.stream())
  assert rc == 0
  torch.cuda.synchronize()  # the kernel came back by itself
  assert time.perf_counter() - t0 < 5.0
  with pytest.raises(_lib.KernelError, match="flag wait timed out at site 100"):
    _lib.raise_on_device_status()
  assert _lib.read_status(clear=False)[0] == 0  # reading cleared it
  # the context is intact: the next kernel of the library runs and is right
  a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
  b = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
  out = K.gemm(a, b)
  torch.cuda.synchronize()
  want = a.float() @ b.float().t()
  assert (out.float() - want).abs().max() <= 3e-2 * want.abs().max()
  _lib.raise_on_device_status()


def test_flag_wait_that_is_satisfied_reports_nothing():
  from maxdiffusion_b200.ops import _lib
  from maxdiffusion_b200.parallel import symm

  flags = torch.zeros(8, dtype=torch.int32, device="cuda")
  symm.set_flag(flags, 0, 3)
  symm.set_flag(flags, 1, 3)
  rc = _lib.lib().mdb_wait_flags(ctypes.c_void_p(flags.data_ptr()), 2, 1, 3, 0.05, _lib.stream())
  assert rc == 0
  torch.cuda.synchronize()
  _lib.raise_on_device_status()
