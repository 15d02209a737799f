"""Runtime dependency version check (reference: src/maxdiffusion/dependency_versions_check.py): the required packages
are verified when the package is imported, optional ones on demand with `dep_version_check(name)`."""
from __future__ import annotations

import importlib.metadata as md
import re

from .dependency_versions_table import deps, required


def _tuple(v: str):
  return tuple(int(x) for x in re.findall(r"\d+", v.split("+")[0])[:3])


def require_version(requirement: str, hint: str = "") -> None:
  m = re.fullmatch(r"\s*([A-Za-z0-9_.\-]+)\s*(?:(>=|==|>|<=|<)\s*([\w.+]+))?\s*", requirement)
  if not m:
    raise ValueError(f"cannot parse requirement {requirement!r}")
  name, op, want = m.groups()
  try:
    have = md.version(name)
  except md.PackageNotFoundError:
    raise ImportError(f"{name} is required ({requirement}) but is not installed. {hint}".strip()) from None
  if op is None:
    return
  a, b = _tuple(have), _tuple(want)
  ok = {">=": a >= b, "==": a == b, ">": a > b, "<=": a <= b, "<": a < b}[op]
  if not ok:
    raise ImportError(f"{requirement} is required but {name}=={have} is installed. {hint}".strip())


def dep_version_check(pkg: str, hint: str = "") -> None:
  require_version(deps[pkg], hint)


def check_required() -> None:
  for pkg in required:
    dep_version_check(pkg)
