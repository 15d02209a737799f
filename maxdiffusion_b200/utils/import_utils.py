"""Optional-dependency probing: `is_<package>_available()`, `requires_backends(obj, [...])`, and `OptionalDependencyNotAvailable`
placeholders that raise on first use (reference: src/maxdiffusion/utils/import_utils.py and the generated
`dummy_*_objects.py` files, which this one class replaces)."""
from __future__ import annotations

import importlib.metadata as md
import importlib.util
from functools import lru_cache
from typing import Iterable, Optional


class OptionalDependencyNotAvailable(ImportError):
  pass


@lru_cache(maxsize=None)
def is_available(package: str, dist_name: Optional[str] = None) -> bool:
  if importlib.util.find_spec(package) is None:
    return False
  try:
    md.version(dist_name or package)
  except md.PackageNotFoundError:
    pass  # importable without metadata (vendored): still usable
  return True


def is_torch_available() -> bool: return is_available("torch")
def is_transformers_available() -> bool: return is_available("transformers")
def is_safetensors_available() -> bool: return is_available("safetensors")
def is_datasets_available() -> bool: return is_available("datasets")
def is_tensorboard_available() -> bool: return is_available("tensorboard")
def is_imageio_available() -> bool: return is_available("imageio")
def is_av_available() -> bool: return is_available("av")
def is_pil_available() -> bool: return is_available("PIL", "pillow")
def is_grain_available() -> bool: return is_available("grain")
def is_sentencepiece_available() -> bool: return is_available("sentencepiece")
def is_scipy_available() -> bool: return is_available("scipy")
def is_cv2_available() -> bool: return is_available("cv2", "opencv-python")


def is_cuda_available() -> bool:
  import torch

  return torch.cuda.is_available()


def get_version(package: str) -> Optional[str]:
  try:
    return md.version(package)
  except md.PackageNotFoundError:
    return None


_HINTS = {"transformers": "text encoders and tokenizers need `transformers`", "datasets": "dataset_type=hf needs `datasets`",
          "av": "muxing audio into mp4 needs `av` (PyAV)", "imageio": "mp4 export needs `imageio` with the ffmpeg plugin",
          "grain": "dataset_type=grain needs `grain`", "PIL": "image IO needs `pillow`"}


def requires_backends(obj, backends: Iterable[str]) -> None:
  name = obj if isinstance(obj, str) else getattr(obj, "__name__", type(obj).__name__)
  missing = [b for b in backends if not is_available(b)]
  if missing:
    raise OptionalDependencyNotAvailable(f"{name} needs {', '.join(missing)}: " + "; ".join(_HINTS.get(b, f"install `{b}`") for b in missing))


class DummyObject(type):
  """Metaclass of placeholders: `class Foo(metaclass=DummyObject): _backends = ["transformers"]` raises a helpful error
  when instantiated or when a class attribute such as `from_pretrained` is touched."""

  def __call__(cls, *a, **k):
    requires_backends(cls, cls._backends)
    return super().__call__(*a, **k)

  def __getattr__(cls, key):
    if key.startswith("_"):
      raise AttributeError(key)
    requires_backends(cls, cls._backends)
    raise AttributeError(key)
