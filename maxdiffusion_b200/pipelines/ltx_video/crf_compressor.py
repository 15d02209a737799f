"""H.264 round trip of a conditioning image: the image is encoded as one libx264 frame at constant rate factor `crf`
and decoded again, so that a clean still looks like a frame of compressed video, which is what the model saw in
training (reference: src/maxdiffusion/pipelines/ltx_video/crf_compressor.py:43-57). Needs PyAV; `crf=0` is the
identity and needs nothing."""
from __future__ import annotations

import io

import numpy as np
import torch


def _encode_single_frame(out, image: np.ndarray, crf: int) -> None:
  import av

  container = av.open(out, "w", format="mp4")
  try:
    stream = container.add_stream("libx264", rate=1, options={"crf": str(crf), "preset": "veryfast"})
    stream.height, stream.width = image.shape[0], image.shape[1]
    frame = av.VideoFrame.from_ndarray(image, format="rgb24").reformat(format="yuv420p")
    container.mux(stream.encode(frame))
    container.mux(stream.encode())
  finally:
    container.close()


def _decode_single_frame(src) -> np.ndarray:
  import av

  container = av.open(src)
  try:
    stream = next(s for s in container.streams if s.type == "video")
    frame = next(container.decode(stream))
  finally:
    container.close()
  return frame.to_ndarray(format="rgb24")


def compress(image: torch.Tensor, crf: int = 29) -> torch.Tensor:
  """image: [H,W,3] float in [0,1]. Height and width are cut to even numbers (4:2:0 chroma)."""
  if crf == 0:
    return image
  from ...utils.import_utils import requires_backends

  requires_backends("crf_compressor.compress", ["av"])
  arr = (image[:(image.shape[0] // 2) * 2, :(image.shape[1] // 2) * 2] * 255.0).byte().cpu().numpy()
  with io.BytesIO() as buf:
    _encode_single_frame(buf, arr, crf)
    data = buf.getvalue()
  with io.BytesIO(data) as buf:
    arr = _decode_single_frame(buf)
  return torch.tensor(arr, dtype=image.dtype, device=image.device) / 255.0
