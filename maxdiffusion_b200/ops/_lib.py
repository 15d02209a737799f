"""ctypes loader for the sm_100a kernel library (`maxdiffusion_b200/_kernels.so`).

The library is built in-tree by `maxdiffusion_b200.build`. On a machine with a GPU every op in
`maxdiffusion_b200.ops` requires it and raises if it is missing — there is no silent PyTorch
fallback for CUDA tensors. On CPU the ops run their pure-PyTorch reference implementation.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
LIB_PATH = Path(__file__).resolve().parent.parent / "_kernels.so"

# launch counter: every successful kernel-library call increments it (bench.py reports it)
_launches = 0


class KernelError(RuntimeError):
  pass


class CopyPlan(ctypes.Structure):
  """Work list of the copy CTAs of `mdb_flash_fwd` (mirrors `MdbCopyPlan` in csrc/flash_fwd.cu)."""
  _fields_ = [("n_remote", ctypes.c_int), ("n_copy_ctas", ctypes.c_int),
              ("src", (ctypes.c_ulonglong * 2) * 7), ("dst", (ctypes.c_ulonglong * 2) * 7),
              ("nbytes", ctypes.c_longlong), ("ready", ctypes.c_ulonglong * 7), ("epoch", ctypes.c_uint),
              ("counters", ctypes.c_ulonglong), ("seg_flags", ctypes.c_ulonglong), ("ack", ctypes.c_ulonglong * 8),
              ("n_ack", ctypes.c_int), ("n_groups", ctypes.c_int)]


class OutScatter(ctypes.Structure):
  """Destination of the attention epilogue's scattered stores (mirrors `MdbOutScatter` in csrc/flash_fwd.cu)."""
  _fields_ = [("n", ctypes.c_int), ("rows_per_rank", ctypes.c_int), ("head_off", ctypes.c_int), ("ptrs", ctypes.c_ulonglong * 8)]


# layout constants of the copy plan (csrc/flash_fwd.cu): flags are rows of FLAG_STRIDE per KV segment, counters one per
# (remote segment, head group) plus one
COPY_FLAG_STRIDE = 8
COPY_NUM_COUNTERS = 7 * 8 + 1


def lib() -> ctypes.CDLL:
  global _LIB
  if _LIB is not None:
    return _LIB
  with _LOCK:
    if _LIB is None:
      if not LIB_PATH.exists():
        if os.environ.get("MDB200_NO_AUTOBUILD") == "1":
          raise KernelError(f"{LIB_PATH} is missing; run `python -m maxdiffusion_b200.build`")
        from maxdiffusion_b200 import build as _build

        _build.build(verbose=False)
      _LIB = ctypes.CDLL(str(LIB_PATH))
      _declare(_LIB)
  return _LIB


def available() -> bool:
  """True when CUDA tensors can be served by the kernel library."""
  return torch.cuda.is_available()


def use_kernels(*tensors: torch.Tensor) -> bool:
  """Dispatch rule: CUDA bf16 tensors go to the hand-written kernels, everything else to the reference."""
  t = tensors[0]
  return t.is_cuda


def stream() -> ctypes.c_void_p:
  return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
  return ctypes.c_void_p(0 if t is None else t.data_ptr())


def check(rc: int, what: str) -> None:
  global _launches
  if rc != 0:
    raise KernelError(f"{what} failed with code {rc}")
  _launches += 1


def launch_count() -> int:
  return _launches


def read_status(clear: bool = True) -> tuple[int, int, int, int]:
  """Returns (code, where, block, detail) of the device status word; code 0 means no kernel gave up a wait."""
  out = (ctypes.c_uint * 4)()
  rc = lib().mdb_read_status(out, 1 if clear else 0)
  if rc != 0:
    raise KernelError(f"mdb_read_status failed with code {rc}")
  return tuple(int(v) for v in out)


def raise_on_device_status() -> None:
  code, where, block, detail = read_status(clear=True)
  if code != 0:
    names = {1: "mbarrier wait timed out", 2: "flag wait timed out", 3: "bad argument"}
    raise KernelError(f"device status: {names.get(code, code)} at site {where}, block {block}, detail {detail}")


def raise_on_device_status_if_loaded() -> None:
  """The check the training and sampling loops make once per step: a no-op on CPU-only runs (library never loaded)."""
  if _LIB is not None and torch.cuda.is_available():
    raise_on_device_status()


def _declare(L: ctypes.CDLL) -> None:
  c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
  c_ull = ctypes.c_ulonglong
  L.mdb_read_status.argtypes = [ctypes.POINTER(ctypes.c_uint), c_int]
  L.mdb_read_status.restype = c_int
  L.mdb_sm_count.restype = c_int
  L.mdb_gemm_bf16.argtypes = [c_void_p] * 6 + [c_int] * 3 + [c_ll] * 5 + [c_int] * 5 + [c_float, c_void_p]
  L.mdb_gemm_bf16.restype = c_int
  L.mdb_gemm_bf16_splitk.argtypes = [c_void_p] * 3 + [c_int] * 3 + [c_ll] * 3 + [c_int] * 3 + [c_float, c_void_p, c_int, c_void_p]
  L.mdb_gemm_bf16_splitk.restype = c_int
  L.mdb_gemm_epilogue_mode.argtypes = [c_int]
  L.mdb_gemm_epilogue_mode.restype = c_int
  L.mdb_gemm_force_tile_n.argtypes = [c_int]
  L.mdb_gemm_force_tile_n.restype = c_int
  L.mdb_flash_fwd.argtypes = ([c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_void_p, c_void_p]
                              + [c_int] * 4 + [ctypes.POINTER(c_int)] + [c_ll] * 12 + [c_float, c_void_p, ctypes.c_uint,
                                                                                      c_void_p, c_void_p])
  L.mdb_flash_fwd.restype = c_int
  L.mdb_flash_fwd_d64.argtypes = L.mdb_flash_fwd.argtypes
  L.mdb_flash_fwd_d64.restype = c_int
  for name in ("mdb_flash_fwd_fixed_m", "mdb_flash_fwd_fixed_m_d64"):
    getattr(L, name).argtypes = L.mdb_flash_fwd.argtypes + [c_void_p, c_void_p]
    getattr(L, name).restype = c_int
  L.mdb_flash_fwd_scatter.argtypes = ([c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p)] + [c_int] * 4 +
                                      [ctypes.POINTER(c_int)] + [c_ll] * 12 + [c_float, c_void_p, ctypes.c_uint, c_void_p,
                                                                              c_void_p, c_void_p])
  L.mdb_flash_fwd_scatter.restype = c_int
  L.mdb_rms_rope_fwd_scatter.argtypes = [c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                         ctypes.POINTER(c_ull), c_int, c_int, c_int, c_void_p]
  L.mdb_rms_rope_fwd_scatter.restype = c_int
  L.mdb_flash_fwd_tune.argtypes = [c_int, c_int]
  L.mdb_flash_fwd_tune.restype = c_int
  L.mdb_flash_fwd_last_variant.argtypes = [ctypes.POINTER(c_int), ctypes.POINTER(c_int)]
  L.mdb_flash_fwd_last_variant.restype = c_int
  L.mdb_ln_fwd.argtypes = [c_void_p] * 6 + [c_ll, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p]
  L.mdb_ln_fwd.restype = c_int
  L.mdb_ln_bwd.argtypes = [c_void_p] * 6 + [c_ll, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
  L.mdb_ln_bwd.restype = c_int
  L.mdb_rms_rope_fwd.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                 c_int, c_int, c_float, c_void_p, c_int, c_void_p]
  L.mdb_rms_rope_fwd.restype = c_int
  L.mdb_rms_rope_bwd.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_void_p, c_ll, c_void_p, c_void_p, c_int, c_void_p]
  L.mdb_rms_rope_bwd.restype = c_int
  L.mdb_gated_res_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
  L.mdb_gated_res_fwd.restype = c_int
  L.mdb_gated_res_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_void_p, c_void_p,
                                  c_void_p, c_int, c_void_p]
  L.mdb_gated_res_bwd.restype = c_int
  L.mdb_colsum.argtypes = [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
  L.mdb_colsum.restype = c_int
  L.mdb_gelu_fwd.argtypes = [c_void_p, c_void_p, c_ll, c_void_p]
  L.mdb_gelu_fwd.restype = c_int
  L.mdb_gelu_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_void_p]
  L.mdb_gelu_bwd.restype = c_int
  L.mdb_geglu_fwd.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_void_p]
  L.mdb_geglu_fwd.restype = c_int
  L.mdb_geglu_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p]
  L.mdb_geglu_bwd.restype = c_int
  L.mdb_adamw.argtypes = [c_void_p] * 4 + [c_ll] + [c_float] * 9 + [c_ull, c_int, c_int, c_int, c_void_p]
  L.mdb_adamw.restype = c_int
  L.mdb_sumsq_maxabs.argtypes = [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_void_p]
  L.mdb_sumsq_maxabs.restype = c_int
  c_llp = ctypes.POINTER(c_ll)
  L.mdb_flash_delta.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int] + [c_ll] * 6 + [c_void_p]
  L.mdb_flash_delta.restype = c_int
  L.mdb_flash_bwd_dkv.argtypes = [c_void_p] * 8 + [c_int] * 4 + [c_llp] * 6 + [c_float, c_int, c_void_p]
  L.mdb_flash_bwd_dkv.restype = c_int
  L.mdb_flash_bwd_dq.argtypes = ([c_void_p, c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_void_p,
                                  c_void_p, c_void_p] + [c_int] * 4 + [ctypes.POINTER(c_int)] + [c_llp] * 5 +
                                 [c_float, c_int, c_void_p])
  L.mdb_flash_bwd_dq.restype = c_int
  L.mdb_flash_bwd_dkv_stacked.argtypes = L.mdb_flash_bwd_dkv.argtypes + [c_int, ctypes.POINTER(c_int), c_int, c_int, c_ll]
  L.mdb_flash_bwd_dkv_stacked.restype = c_int
  for name in ("mdb_flash_delta", "mdb_flash_bwd_dkv", "mdb_flash_bwd_dkv_stacked", "mdb_flash_bwd_dq"):  # head_dim 64 variants: same signatures
    getattr(L, name + "_d64").argtypes = getattr(L, name).argtypes
    getattr(L, name + "_d64").restype = c_int
  for fn in _EXTRA:
    fn(L)


# modules that own further entry points register a declarer here
_EXTRA: list = []


def register(declare_fn) -> None:
  """Registers a function that sets argtypes/restype of more entry points; applied now if the library is loaded."""
  _EXTRA.append(declare_fn)
  if _LIB is not None:
    declare_fn(_LIB)
