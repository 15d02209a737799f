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


def _temp_path(suffix: str) -> str:
  import tempfile

  fd, path = tempfile.mkstemp(suffix=suffix)
  os.close(fd)
  return path


def export_to_gif(images, output_gif_path: str | None = None, fps: float = 10.0) -> str:
  """Looping GIF from PIL images or a [T, H, W, 3] array (uint8, or floats in [0, 1]); 100 ms per frame by default
  (reference: src/maxdiffusion/utils/export_utils.py:48-60)."""
  from PIL import Image

  path = output_gif_path or _temp_path(".gif")
  if not isinstance(images, (list, tuple)) or not isinstance(images[0], Image.Image):
    images = [Image.fromarray(f) for f in _to_uint8(images)]
  images[0].save(path, save_all=True, append_images=list(images[1:]), optimize=False, duration=int(round(1000.0 / fps)), loop=0)
  return path


def _mesh_arrays(mesh):
  """(vertices [V, 3] float32, faces [F, 3] int or None, colours [V, 3] in [0, 1] or None) of a mesh object with `verts`,
  `faces` and optionally `vertex_channels` {"R", "G", "B"} (tensors or arrays)."""
  to_np = lambda t: t.detach().cpu().numpy() if hasattr(t, "detach") else np.asarray(t)
  verts = to_np(mesh.verts).astype(np.float32)
  faces = to_np(mesh.faces).astype(np.int64) if getattr(mesh, "faces", None) is not None else None
  channels = getattr(mesh, "vertex_channels", None)
  rgb = np.stack([to_np(channels[c]) for c in "RGB"], axis=1).astype(np.float32) if channels else None
  return verts, faces, rgb


def export_to_ply(mesh, output_ply_path: str | None = None) -> str:
  """Binary little-endian PLY: x y z as float32 (+ red green blue as uchar when the mesh has vertex colours), faces as
  a uchar count followed by int indices (reference: src/maxdiffusion/utils/export_utils.py:63-112)."""
  path = output_ply_path or _temp_path(".ply")
  verts, faces, rgb = _mesh_arrays(mesh)
  header = ["ply", "format binary_little_endian 1.0", f"element vertex {len(verts)}", "property float x", "property float y",
            "property float z"]
  if rgb is not None:
    header += ["property uchar red", "property uchar green", "property uchar blue"]
  if faces is not None:
    header += [f"element face {len(faces)}", "property list uchar int vertex_index"]
  header.append("end_header")
  with open(path, "wb") as f:
    f.write(("\n".join(header) + "\n").encode("ascii"))
    if rgb is not None:
      rec = np.empty(len(verts), dtype=[("p", "<f4", 3), ("c", "u1", 3)])
      rec["p"], rec["c"] = verts, np.clip((rgb * 255.499).round(), 0, 255).astype(np.uint8)
      f.write(rec.tobytes())
    else:
      f.write(verts.astype("<f4").tobytes())
    if faces is not None:
      rec = np.empty(len(faces), dtype=[("n", "u1"), ("i", "<i4", faces.shape[1])])
      rec["n"], rec["i"] = faces.shape[1], faces
      f.write(rec.tobytes())
  return path


def export_to_obj(mesh, output_obj_path: str | None = None) -> str:
  """Wavefront OBJ with per-vertex colours (`v x y z r g b`) and 1-based triangle indices
  (reference: src/maxdiffusion/utils/export_utils.py:115-130)."""
  path = output_obj_path or _temp_path(".obj")
  verts, faces, rgb = _mesh_arrays(mesh)
  lines = []
  for i, v in enumerate(verts.tolist()):
    lines.append("v " + " ".join(repr(float(x)) for x in (v + rgb[i].tolist() if rgb is not None else v)))
  if faces is not None:
    lines += ["f " + " ".join(str(int(j) + 1) for j in tri) for tri in faces.tolist()]
  with open(path, "w", encoding="ascii") as f:
    f.write("\n".join(lines))
  return path
