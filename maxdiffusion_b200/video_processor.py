"""Video pre/post-processing on top of `VaeImageProcessor` (reference: src/maxdiffusion/video_processor.py:25)."""
from __future__ import annotations

import torch

from .image_processor import VaeImageProcessor


class VideoProcessor(VaeImageProcessor):

  def preprocess_video(self, video, height: int, width: int) -> torch.Tensor:
    """list of frames / [T,H,W,C] array / [B,T,C,H,W] tensor -> [B,C,T,H,W] in [-1,1]."""
    if isinstance(video, torch.Tensor) and video.dim() == 5:
      frames = [torch.cat([self.preprocess(f, height, width) for f in clip]) for clip in video]
      return torch.stack(frames).permute(0, 2, 1, 3, 4)
    frames = torch.cat([self.preprocess(f, height, width) for f in video])
    return frames.permute(1, 0, 2, 3)[None]

  def postprocess_video(self, video: torch.Tensor, output_type: str = "np"):
    b, c, t, h, w = video.shape
    flat = video.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w)
    out = self.postprocess(flat, "pt" if output_type == "pt" else "np")
    if output_type == "pt":
      return out.reshape(b, t, c, h, w)
    return out.reshape(b, t, h, w, c)
