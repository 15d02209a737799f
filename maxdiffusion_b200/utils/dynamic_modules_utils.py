"""Custom pipelines and components shipped as Python files next to a checkpoint ("community pipelines").

The reference downloads such files from the Hub into a modules cache and imports them from there
(src/maxdiffusion/utils/dynamic_modules_utils.py:44-456: `get_cached_module_file`, `get_class_from_dynamic_module`).
This code base never touches the network, so a module is resolved from a local file or folder only: the file and
everything it imports relatively is copied into a private cache package (so that two checkpoints may ship files of the
same name) and imported from there.

    cls = get_class_from_dynamic_module("/models/my-pipeline", "pipeline.py")          # the one pipeline class in it
    cls = get_class_from_dynamic_module("/models/my-pipeline", "pipeline.py", "MyPipeline")
"""
from __future__ import annotations

import ast
import hashlib
import importlib
import importlib.util
import os
import shutil
import sys
from typing import List, Optional

MODULES_PACKAGE = "maxdiffusion_b200_modules"


def modules_cache(root: Optional[str] = None) -> str:
  """The cache package (created on first use, on `sys.path` through its parent). `MAXDIFFUSION_MODULES_CACHE`
  overrides the location."""
  parent = root or os.environ.get("MAXDIFFUSION_MODULES_CACHE") or os.path.join(os.path.expanduser("~"), ".cache", "maxdiffusion_b200")
  pkg = os.path.join(parent, MODULES_PACKAGE)
  os.makedirs(pkg, exist_ok=True)
  init = os.path.join(pkg, "__init__.py")
  if not os.path.exists(init):
    open(init, "w").close()
  if parent not in sys.path:
    sys.path.insert(0, parent)
  importlib.invalidate_caches()
  return pkg


def get_relative_imports(module_file: str) -> List[str]:
  """Names of the sibling modules a file imports with `from .x import ...` / `from . import x` / `import .x`."""
  with open(module_file, encoding="utf-8") as f:
    tree = ast.parse(f.read(), module_file)
  names = []
  for node in ast.walk(tree):
    if isinstance(node, ast.ImportFrom) and node.level == 1:
      if node.module:
        names.append(node.module.split(".")[0])
      else:
        names.extend(a.name for a in node.names)
  return sorted(set(names))


def get_relative_import_files(module_file: str) -> List[str]:
  """Every file reachable from `module_file` through relative imports (the file itself excluded)."""
  seen, todo = set(), [module_file]
  while todo:
    cur = todo.pop()
    folder = os.path.dirname(cur)
    for name in get_relative_imports(cur):
      path = os.path.join(folder, name + ".py")
      if os.path.exists(path) and path not in seen:
        seen.add(path)
        todo.append(path)
  return sorted(seen)


def check_imports(module_file: str) -> List[str]:
  """Top-level packages the file needs; raises ImportError naming the missing ones."""
  with open(module_file, encoding="utf-8") as f:
    tree = ast.parse(f.read(), module_file)
  wanted = set()
  for node in ast.walk(tree):
    if isinstance(node, ast.Import):
      wanted.update(a.name.split(".")[0] for a in node.names)
    elif isinstance(node, ast.ImportFrom) and node.level == 0 and node.module:
      wanted.add(node.module.split(".")[0])
  missing = sorted(m for m in wanted if importlib.util.find_spec(m) is None)
  if missing:
    raise ImportError(f"{module_file} needs packages that are not installed: {', '.join(missing)}")
  return get_relative_imports(module_file)


def get_cached_module_file(path_or_folder: str, module_file: str, cache_root: Optional[str] = None) -> str:
  """Copies `module_file` of a local folder (and its relative imports) into the cache package; returns the dotted
  module name to import. The sub-package is named after a hash of the files' contents, so an edited file is a new
  module and an unchanged one is reused."""
  src = os.path.join(path_or_folder, module_file) if os.path.isdir(path_or_folder) else path_or_folder
  if not os.path.isfile(src):
    raise FileNotFoundError(f"no module file {src} (custom pipelines are resolved from local files only)")
  check_imports(src)
  files = [src] + get_relative_import_files(src)
  digest = hashlib.sha256()
  for f in files:
    with open(f, "rb") as fh:
      digest.update(os.path.basename(f).encode() + b"\0" + fh.read())
  sub = "m" + digest.hexdigest()[:16]
  dst = os.path.join(modules_cache(cache_root), sub)
  if not os.path.isdir(dst):
    tmp = dst + f".tmp{os.getpid()}"
    os.makedirs(tmp, exist_ok=True)
    open(os.path.join(tmp, "__init__.py"), "w").close()
    for f in files:
      shutil.copy(f, os.path.join(tmp, os.path.basename(f)))
    try:
      os.replace(tmp, dst)
    except OSError:  # another process won the race
      shutil.rmtree(tmp, ignore_errors=True)
  importlib.invalidate_caches()
  return f"{MODULES_PACKAGE}.{sub}.{os.path.splitext(os.path.basename(src))[0]}"


def get_class_in_module(class_name: str, module_name: str):
  return getattr(importlib.import_module(module_name), class_name)


def find_pipeline_class(module) -> type:
  """The single class of a module that looks like a pipeline: defined in the module itself, callable, and either
  derived from this code base's pipeline base or carrying a `from_pretrained` / `from_config` constructor."""
  import inspect

  from ..pipelines.pipeline_utils import DiffusionPipelineMixin as DiffusionPipeline

  found = []
  for name, cls in inspect.getmembers(module, inspect.isclass):
    if cls.__module__ != module.__name__ or not callable(getattr(cls, "__call__", None)):
      continue
    if issubclass(cls, DiffusionPipeline) or hasattr(cls, "from_pretrained") or hasattr(cls, "from_config"):
      found.append(cls)
  if len(found) != 1:
    raise ValueError(f"expected exactly one pipeline class in {module.__name__}, found {[c.__name__ for c in found]}")
  return found[0]


def get_class_from_dynamic_module(path_or_folder: str, module_file: str = "pipeline.py", class_name: Optional[str] = None,
                                  cache_root: Optional[str] = None) -> type:
  name = get_cached_module_file(path_or_folder, module_file, cache_root)
  if class_name is not None:
    return get_class_in_module(class_name, name)
  return find_pipeline_class(importlib.import_module(name))
