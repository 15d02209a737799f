"""Builds the sm_100a kernel library `maxdiffusion_b200/_kernels.so` with nvcc.

The kernels export a plain C ABI (raw pointers + stream) and are loaded through ctypes, so the
build needs neither the PyTorch headers nor a JIT cache: `python -m maxdiffusion_b200.build`
compiles every `csrc/*.cu` in parallel and links one shared object next to the package.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SRC_DIR = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "csrc" / "build"
LIB_PATH = PKG_DIR / "_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
  nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
  if not os.path.exists(nvcc):
    raise RuntimeError("nvcc not found; the sm_100a kernels cannot be built")
  return nvcc


def _digest(path: Path) -> str:
  h = hashlib.sha256()
  h.update(" ".join(NVCC_FLAGS).encode())
  h.update(path.read_bytes())
  for hdr in sorted(SRC_DIR.glob("*.cuh")) + sorted(SRC_DIR.glob("*.h")):
    h.update(hdr.read_bytes())
  return h.hexdigest()


def _compile_one(src: Path, verbose: bool) -> Path:
  obj = OBJ_DIR / (src.stem + ".o")
  stamp = OBJ_DIR / (src.stem + ".sha")
  digest = _digest(src)
  if obj.exists() and stamp.exists() and stamp.read_text() == digest:
    return obj
  cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(SRC_DIR), "-c", str(src), "-o", str(obj)]
  res = subprocess.run(cmd, capture_output=True, text=True)
  log = OBJ_DIR / (src.stem + ".ptxas.log")
  log.write_text(res.stdout + res.stderr)
  if res.returncode != 0:
    raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
  if verbose:
    print(f"[build] compiled {src.name}")
  stamp.write_text(digest)
  return obj


def sources() -> list[Path]:
  return sorted(SRC_DIR.glob("*.cu"))


def build(verbose: bool = True, force: bool = False) -> Path:
  """Compiles every kernel for sm_100a and links `_kernels.so`. Returns its path."""
  OBJ_DIR.mkdir(parents=True, exist_ok=True)
  if force:
    for f in OBJ_DIR.glob("*.sha"):
      f.unlink()
  srcs = sources()
  with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
    objs = list(pool.map(lambda s: _compile_one(s, verbose), srcs))
  newest = max(o.stat().st_mtime for o in objs)
  if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest:
    cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *[str(o) for o in objs], "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
      raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
      print(f"[build] linked {LIB_PATH}")
  return LIB_PATH


if __name__ == "__main__":
  build(verbose=True, force="--force" in sys.argv)
