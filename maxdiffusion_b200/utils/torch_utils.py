"""Tensor helpers shared by the pipelines (reference: src/maxdiffusion/utils/torch_utils.py)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch


def randn_tensor(shape: Sequence[int], generator: Optional[Union[torch.Generator, List[torch.Generator]]] = None, device=None,
                 dtype=None) -> torch.Tensor:
  """Gaussian noise that is reproducible across devices: a CPU generator draws on the CPU and the result is moved, a
  list of generators draws one sample per batch element."""
  device = torch.device(device) if device is not None else torch.device("cpu")
  if isinstance(generator, (list, tuple)):
    if len(generator) != shape[0]:
      raise ValueError(f"{len(generator)} generators for a batch of {shape[0]}")
    return torch.cat([randn_tensor((1, *shape[1:]), g, device, dtype) for g in generator])
  gdev = generator.device if generator is not None else device
  x = torch.randn(tuple(shape), generator=generator, device=gdev, dtype=torch.float32 if gdev.type == "cpu" else dtype)
  return x.to(device=device, dtype=dtype)


def fourier_filter(x: torch.Tensor, threshold: int, scale: float) -> torch.Tensor:
  """Scales the low-frequency box of radius `threshold` of the last two dims by `scale` (FreeU)."""
  X = torch.fft.fftshift(torch.fft.fftn(x.float(), dim=(-2, -1)), dim=(-2, -1))
  H, W = X.shape[-2:]
  mask = torch.ones_like(X.real)
  ch, cw = H // 2, W // 2
  mask[..., ch - threshold:ch + threshold, cw - threshold:cw + threshold] = scale
  out = torch.fft.ifftn(torch.fft.ifftshift(X * mask, dim=(-2, -1)), dim=(-2, -1)).real
  return out.to(x.dtype)


def is_compiled_module(module) -> bool:
  return hasattr(module, "_orig_mod")


def module_device_dtype(module: torch.nn.Module):
  p = next(module.parameters())
  return p.device, p.dtype
