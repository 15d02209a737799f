"""Codec noise for a conditioning image, computed on the device.

LTX-Video was trained on frames of compressed video, so a clean still is first made to look like one. The reference
does it with a real encoder: one libx264 frame at constant rate factor `crf`, decoded again through PyAV
(src/maxdiffusion/pipelines/ltx_video/crf_compressor.py:43-57). No bitstream is needed for that effect, only the
loss of an intra frame, and that loss is the quantisation of 4x4 transform coefficients. `compress` applies exactly
that part of H.264 to a tensor, wherever it lives:

  RGB -> Y'CbCr (BT.601, studio range) with 4:2:0 chroma -> the 4x4 integer core transform in its orthonormal form
  -> dead-zone scalar quantisation with the standard's step size (0.625 at QP 0, doubling every 6 QP) -> inverse transform
  -> chroma up-sampling -> RGB.

The luma QP of an intra frame under x264's rate factor is crf minus the I-frame offset (6 log2 1.4, about 3); the
chroma QP follows the standard's luma-to-chroma table. Intra prediction, entropy coding and the loop filter are left
out: they change the bit count and smooth block edges, not the size of the quantisation error. `crf = 0` returns the
input itself.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

# H.264 forward core transform; rows scaled to unit norm make it orthonormal, which folds the standard's
# position-dependent scaling factors into one step size per plane
_CORE = torch.tensor([[1.0, 1.0, 1.0, 1.0], [2.0, 1.0, -1.0, -2.0], [1.0, -1.0, -1.0, 1.0], [1.0, -2.0, 2.0, -1.0]])
_CORE = _CORE / _CORE.norm(dim=1, keepdim=True)
# chroma QP for luma QP 30..51 (below 30 they are equal): ITU-T H.264 table 8-15
_CHROMA_QP = (29, 30, 31, 32, 32, 33, 34, 34, 35, 35, 36, 36, 37, 37, 37, 38, 38, 38, 39, 39, 39, 39)
_INTRA_DEADZONE = 1.0 / 3.0  # rounding offset of intra blocks
_I_FRAME_OFFSET = 6.0 * math.log2(1.4)


_QSTEP_BASE = (0.625, 0.6875, 0.8125, 0.875, 1.0, 1.125)  # QP 0..5; the step doubles with every 6 QP


def qstep(qp: int) -> float:
  return _QSTEP_BASE[qp % 6] * 2.0 ** (qp // 6)


def chroma_qp(qp: int) -> int:
  qp = max(0, min(51, qp))
  return qp if qp < 30 else _CHROMA_QP[qp - 30]


def _transform_code(plane: torch.Tensor, step: float) -> torch.Tensor:
  """plane [h, w] (multiples of 4, 0..255 scale) -> its reconstruction after 4x4 transform coding at `step`."""
  h, w = plane.shape
  a = _CORE.to(plane.device, plane.dtype)
  blocks = plane.reshape(h // 4, 4, w // 4, 4).permute(0, 2, 1, 3)  # [h/4, w/4, 4, 4]
  coef = a @ blocks @ a.t()
  level = torch.sign(coef) * torch.floor(coef.abs() / step + _INTRA_DEADZONE)
  rec = a.t() @ (level * step) @ a
  return rec.permute(0, 2, 1, 3).reshape(h, w)


def _pad4(plane: torch.Tensor):
  h, w = plane.shape
  ph, pw = (-h) % 4, (-w) % 4
  if ph or pw:  # an encoder extends the picture to whole blocks by repeating its border
    plane = F.pad(plane[None, None], (0, pw, 0, ph), mode="replicate")[0, 0]
  return plane, h, w


def compress(image: torch.Tensor, crf: int = 29) -> torch.Tensor:
  """image [H, W, 3], float in [0, 1] -> the same picture with the loss of an H.264 intra frame at rate factor `crf`
  (height and width cut to even numbers: 4:2:0 chroma)."""
  if crf == 0:
    return image
  H, W = (image.shape[0] // 2) * 2, (image.shape[1] // 2) * 2
  rgb = (image[:H, :W].float().clamp(0, 1) * 255.0).round()  # the encoder sees 8-bit samples
  r, g, b = rgb.unbind(-1)
  y = 16.0 + (65.481 * r + 128.553 * g + 24.966 * b) / 255.0
  cb = 128.0 + (-37.797 * r - 74.203 * g + 112.0 * b) / 255.0
  cr = 128.0 + (112.0 * r - 93.786 * g - 18.214 * b) / 255.0
  cb, cr = (F.avg_pool2d(c[None, None], 2)[0, 0] for c in (cb, cr))
  qp = int(round(max(0.0, min(51.0, crf - _I_FRAME_OFFSET))))
  planes = []
  for plane, q in ((y, qp), (cb, chroma_qp(qp)), (cr, chroma_qp(qp))):
    padded, h, w = _pad4(plane.round())
    planes.append(_transform_code(padded, qstep(q))[:h, :w].round().clamp(0, 255))
  y, cb, cr = planes
  cb, cr = (F.interpolate(c[None, None], scale_factor=2, mode="bilinear", align_corners=False)[0, 0] for c in (cb, cr))
  y, cb, cr = y - 16.0, cb - 128.0, cr - 128.0
  out = torch.stack([1.164383 * y + 1.596027 * cr, 1.164383 * y - 0.391762 * cb - 0.812968 * cr,
                     1.164383 * y + 2.017232 * cb], dim=-1)
  return (out.round().clamp(0, 255) / 255.0).to(image.dtype)
