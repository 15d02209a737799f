"""Device introspection used to choose tile alignment and to report memory.

Reference: src/maxdiffusion/tpu_utils.py (chip generation detection that selects 128- vs 256-wide alignment :63-80,
memory-info printers). The analogue here: the CUDA compute capability and SM count select the tile shapes the
tcgen05 kernels were built for, and the memory report reads the caching allocator and the driver.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import max_logging


@dataclass(frozen=True)
class DeviceInfo:
  name: str
  capability: tuple
  sm_count: int
  total_memory_gb: float
  l2_bytes: int

  @property
  def is_blackwell(self) -> bool:
    return self.capability[0] == 10

  @property
  def mma_tile_m(self) -> int:
    """Rows of one tcgen05.mma tile (128 per CTA; 256 when a CTA pair shares the tile)."""
    return 128

  @property
  def sequence_alignment(self) -> int:
    """Token counts are padded to this multiple so that every flash / GEMM tile is full."""
    return 128 if self.is_blackwell else 64


def device_info(device: Optional[int] = None) -> Optional[DeviceInfo]:
  if not torch.cuda.is_available():
    return None
  p = torch.cuda.get_device_properties(torch.cuda.current_device() if device is None else device)
  return DeviceInfo(p.name, (p.major, p.minor), p.multi_processor_count, p.total_memory / 2**30, getattr(p, "L2_cache_size", 0))


def require_blackwell() -> DeviceInfo:
  info = device_info()
  if info is None or not info.is_blackwell:
    raise RuntimeError(f"the CUDA kernels of this package are built for sm_100a only; found {info.name if info else 'no GPU'}")
  return info


def pad_to_alignment(n: int, alignment: Optional[int] = None) -> int:
  a = alignment or (device_info().sequence_alignment if torch.cuda.is_available() else 128)
  return -(-n // a) * a


def print_device_memory(prefix: str = "") -> dict:
  """Per visible GPU: used / free / total from the driver and allocated / reserved from the caching allocator."""
  out = {}
  if not torch.cuda.is_available():
    max_logging.log(f"{prefix}no CUDA device")
    return out
  for d in range(torch.cuda.device_count()):
    free, total = torch.cuda.mem_get_info(d)
    out[d] = {"free_gb": free / 2**30, "total_gb": total / 2**30, "allocated_gb": torch.cuda.memory_allocated(d) / 2**30,
              "reserved_gb": torch.cuda.memory_reserved(d) / 2**30, "peak_allocated_gb": torch.cuda.max_memory_allocated(d) / 2**30}
    max_logging.log(f"{prefix}cuda:{d} " + ", ".join(f"{k}={v:.2f}" for k, v in out[d].items()))
  return out
