"""`load_image` / `load_video` from local paths (reference: src/maxdiffusion/utils/loading_utils.py:1-138).

Images load through PIL. Videos load through OpenCV when it is installed, else imageio / PyAV; a directory of
image files and a `.npy` array `[T, H, W, 3]` (what `export_to_video` writes without a codec) are also accepted.
URLs are not fetched: inputs must be local files.
"""
from __future__ import annotations

import os
from typing import List

import numpy as np


def load_image(path: str):
  from PIL import Image, ImageOps

  if not os.path.exists(path):
    raise ValueError(f"Incorrect path: {path} is not a local file (remote URLs are not downloaded)")
  return ImageOps.exif_transpose(Image.open(path)).convert("RGB")


def load_video(path: str) -> List:
  """Returns a list of PIL images (RGB)."""
  from PIL import Image

  if os.path.isdir(path):
    names = sorted(n for n in os.listdir(path) if n.lower().endswith((".png", ".jpg", ".jpeg", ".bmp", ".webp")))
    return [load_image(os.path.join(path, n)) for n in names]
  if path.endswith(".npy"):
    return [Image.fromarray(f) for f in np.load(path)]
  if path.lower().endswith(".gif"):
    from PIL import ImageSequence

    return [f.convert("RGB") for f in ImageSequence.Iterator(Image.open(path))]
  try:
    import cv2

    cap = cv2.VideoCapture(path)
    frames = []
    while True:
      ok, frame = cap.read()
      if not ok:
        break
      frames.append(Image.fromarray(cv2.cvtColor(frame, cv2.COLOR_BGR2RGB)))
    cap.release()
    if frames:
      return frames
  except ImportError:
    pass
  try:
    import imageio

    return [Image.fromarray(f) for f in imageio.get_reader(path)]
  except ImportError:
    pass
  import av

  with av.open(path) as container:
    return [f.to_image() for f in container.decode(video=0)]
