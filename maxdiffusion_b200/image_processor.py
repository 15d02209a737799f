"""Image pre/post-processing (resize, crop, flip, [-1,1] normalisation, PIL <-> numpy <-> torch).

Reference: `VaeImageProcessor` (src/maxdiffusion/image_processor.py, 554 lines)."""
from __future__ import annotations

import random
from typing import Optional

import numpy as np
import torch


class VaeImageProcessor:

  def __init__(self, vae_scale_factor: int = 8, do_normalize: bool = True):
    self.vae_scale_factor, self.do_normalize = vae_scale_factor, do_normalize

  @staticmethod
  def pil_to_numpy(image) -> np.ndarray:
    return np.asarray(image.convert("RGB"), dtype=np.float32) / 255.0

  @staticmethod
  def numpy_to_pil(arr: np.ndarray):
    from PIL import Image

    arr = (np.clip(arr, 0, 1) * 255).round().astype(np.uint8)
    return [Image.fromarray(a) for a in (arr if arr.ndim == 4 else arr[None])]

  @staticmethod
  def normalize(x):
    return 2.0 * x - 1.0

  @staticmethod
  def denormalize(x):
    return (x / 2 + 0.5).clamp(0, 1)

  def preprocess(self, image, height: int, width: int, center_crop: bool = False, random_flip: bool = False,
                 rng: Optional[random.Random] = None) -> torch.Tensor:
    """PIL image / HWC array / CHW tensor -> [1,3,height,width] float in [-1,1] (dims rounded down to the VAE factor)."""
    height -= height % self.vae_scale_factor
    width -= width % self.vae_scale_factor
    if isinstance(image, torch.Tensor):
      t = image.float()
      t = t if t.dim() == 4 else t[None]
    else:
      arr = self.pil_to_numpy(image) if hasattr(image, "convert") else np.asarray(image, dtype=np.float32)
      if arr.max() > 1.5:
        arr = arr / 255.0
      t = torch.from_numpy(arr).permute(2, 0, 1)[None]
    _, _, h, w = t.shape
    scale = max(height / h, width / w) if center_crop else None
    if center_crop:
      nh, nw = max(height, round(h * scale)), max(width, round(w * scale))
      t = torch.nn.functional.interpolate(t, size=(nh, nw), mode="bilinear", align_corners=False, antialias=True)
      top, left = (nh - height) // 2, (nw - width) // 2
      t = t[:, :, top:top + height, left:left + width]
    else:
      t = torch.nn.functional.interpolate(t, size=(height, width), mode="bilinear", align_corners=False, antialias=True)
    if random_flip and (rng or random).random() < 0.5:
      t = t.flip(-1)
    return self.normalize(t) if self.do_normalize else t

  def postprocess(self, image: torch.Tensor, output_type: str = "pil"):
    x = self.denormalize(image.float())
    if output_type == "pt":
      return x
    arr = x.permute(0, 2, 3, 1).cpu().numpy()
    return arr if output_type == "np" else self.numpy_to_pil(arr)
