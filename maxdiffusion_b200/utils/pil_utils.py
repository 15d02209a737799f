"""numpy / torch images <-> PIL, and image grids (reference: src/maxdiffusion/utils/pil_utils.py)."""
from __future__ import annotations

from typing import List

import numpy as np


def numpy_to_pil(images: np.ndarray) -> List:
  """[B,H,W,C] (or [H,W,C]) float in [0,1] or uint8 -> list of PIL images; single-channel images become mode L."""
  from PIL import Image

  a = np.asarray(images)
  if a.ndim == 3:
    a = a[None]
  if a.dtype != np.uint8:
    a = (np.clip(a, 0.0, 1.0) * 255).round().astype(np.uint8)
  if a.shape[-1] == 1:
    return [Image.fromarray(x.squeeze(-1), mode="L") for x in a]
  return [Image.fromarray(x) for x in a]


def pt_to_pil(images) -> List:
  """torch [B,C,H,W] in [-1,1] -> PIL."""
  a = (images.detach().float().cpu() / 2 + 0.5).clamp(0, 1).permute(0, 2, 3, 1).numpy()
  return numpy_to_pil(a)


def make_image_grid(images: List, rows: int, cols: int, resize: int | None = None):
  from PIL import Image

  if len(images) != rows * cols:
    raise ValueError(f"{len(images)} images do not fill a {rows}x{cols} grid")
  if resize is not None:
    images = [im.resize((resize, resize)) for im in images]
  w, h = images[0].size
  grid = Image.new("RGB", (cols * w, rows * h))
  for i, im in enumerate(images):
    grid.paste(im, ((i % cols) * w, (i // cols) * h))
  return grid
