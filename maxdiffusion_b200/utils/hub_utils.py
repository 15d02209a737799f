"""Model-location resolution without network access: a name is a local directory, a path under the Hugging Face cache
(`models--org--name/snapshots/<rev>`), or an error that says how to provide it
(reference: src/maxdiffusion/utils/hub_utils.py, whose download paths have no counterpart on an offline machine)."""
from __future__ import annotations

import glob
import os
from typing import Optional

from .constants import HF_HOME


def cached_snapshot(repo_id: str, revision: Optional[str] = None, cache_dir: Optional[str] = None) -> Optional[str]:
  root = os.path.join(cache_dir or os.path.join(HF_HOME, "hub"), "models--" + repo_id.replace("/", "--"), "snapshots")
  if not os.path.isdir(root):
    return None
  if revision and os.path.isdir(os.path.join(root, revision)):
    return os.path.join(root, revision)
  snaps = sorted(glob.glob(os.path.join(root, "*")), key=os.path.getmtime)
  return snaps[-1] if snaps else None


def resolve_model_path(name_or_path: str, subfolder: Optional[str] = None, revision: Optional[str] = None,
                       cache_dir: Optional[str] = None) -> str:
  cands = [name_or_path]
  snap = cached_snapshot(name_or_path, revision, cache_dir) if not os.path.isabs(name_or_path) else None
  if snap:
    cands.append(snap)
  for c in cands:
    p = os.path.join(c, subfolder) if subfolder else c
    if os.path.exists(p):
      return p
  raise FileNotFoundError(f"{name_or_path!r} is neither a local directory nor in the Hugging Face cache under "
                          f"{cache_dir or os.path.join(HF_HOME, 'hub')}; copy the repository there (this machine has no network)")


def populate_model_card(folder: str, model_name: str, base_model: str = "", tags=(), text: str = "") -> str:
  path = os.path.join(folder, "README.md")
  os.makedirs(folder, exist_ok=True)
  with open(path, "w") as f:
    f.write("---\n" + (f"base_model: {base_model}\n" if base_model else "") + "tags:\n" + "".join(f"- {t}\n" for t in tags) + "---\n\n")
    f.write(f"# {model_name}\n\n{text}\n")
  return path
