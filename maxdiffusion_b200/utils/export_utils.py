"""Writing results: mp4 through imageio-ffmpeg / PyAV when they are installed, otherwise an animated PNG
sequence folder plus a `.npy` next to it; PNG for single images.

Reference: src/maxdiffusion/utils/export_utils.py:159-232 (`export_to_video`), :322 (`export_to_video_with_audio`).
"""
from __future__ import annotations

import os

import numpy as np


def _to_uint8(frames) -> np.ndarray:
  a = np.asarray(frames)
  if a.dtype != np.uint8:
    a = (np.clip(a, 0.0, 1.0) * 255).round().astype(np.uint8)
  return a


def export_to_video(frames, path: str, fps: int = 16) -> str:
  """frames: [T,H,W,3] uint8 (or float in [0,1]). Returns the path actually written."""
  a = _to_uint8(frames)
  try:
    import imageio

    with imageio.get_writer(path, fps=fps, codec="libx264", quality=8) as w:
      for f in a:
        w.append_data(f)
    return path
  except Exception:
    pass
  try:
    import av

    with av.open(path, mode="w") as container:
      stream = container.add_stream("libx264", rate=fps)
      stream.height, stream.width, stream.pix_fmt = a.shape[1], a.shape[2], "yuv420p"
      for f in a:
        for packet in stream.encode(av.VideoFrame.from_ndarray(f, format="rgb24")):
          container.mux(packet)
      for packet in stream.encode():
        container.mux(packet)
    return path
  except Exception:
    pass
  base = os.path.splitext(path)[0]
  np.save(base + ".npy", a)
  try:
    from PIL import Image

    os.makedirs(base + "_frames", exist_ok=True)
    for i, f in enumerate(a):
      Image.fromarray(f).save(os.path.join(base + "_frames", f"{i:05d}.png"))
  except Exception:
    pass
  return base + ".npy"


def export_to_video_with_audio(frames, audio, path: str, fps: int = 24, sample_rate: int = 24000) -> str:
  """Muxes video and a mono/stereo float waveform with PyAV; without PyAV writes the video and a `.wav`."""
  try:
    import av  # noqa: F401
  except Exception:
    out = export_to_video(frames, path, fps)
    import wave

    wav = os.path.splitext(path)[0] + ".wav"
    pcm = (np.clip(np.asarray(audio, dtype=np.float32), -1, 1) * 32767).astype(np.int16)
    with wave.open(wav, "wb") as w:
      w.setnchannels(1 if pcm.ndim == 1 else pcm.shape[0])
      w.setsampwidth(2)
      w.setframerate(sample_rate)
      w.writeframes(pcm.T.tobytes() if pcm.ndim == 2 else pcm.tobytes())
    return out
  import av

  a = _to_uint8(frames)
  with av.open(path, mode="w") as container:
    vs = container.add_stream("libx264", rate=fps)
    vs.height, vs.width, vs.pix_fmt = a.shape[1], a.shape[2], "yuv420p"
    as_ = container.add_stream("aac", rate=sample_rate)
    for f in a:
      for p in vs.encode(av.VideoFrame.from_ndarray(f, format="rgb24")):
        container.mux(p)
    for p in vs.encode():
      container.mux(p)
    wavef = np.asarray(audio, dtype=np.float32)
    wavef = wavef[None] if wavef.ndim == 1 else wavef
    frame = av.AudioFrame.from_ndarray(wavef, format="fltp", layout="mono" if wavef.shape[0] == 1 else "stereo")
    frame.sample_rate = sample_rate
    for p in as_.encode(frame):
      container.mux(p)
    for p in as_.encode():
      container.mux(p)
  return path


def export_to_png(image, path: str) -> str:
  from PIL import Image

  Image.fromarray(_to_uint8(image)).save(path)
  return path
