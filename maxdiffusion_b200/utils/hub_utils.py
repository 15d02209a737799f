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


_COMMIT_HASH = __import__("re").compile(r"^[0-9a-f]{40}$")


def extract_commit_hash(resolved_file: Optional[str], commit_hash: Optional[str] = None) -> Optional[str]:
  """The revision a cache file belongs to: `.../snapshots/<40 hex digits>/...` (an explicit hash wins)."""
  if resolved_file is None or commit_hash is not None:
    return commit_hash
  import re

  m = re.search(r"snapshots/([^/]+)/", str(resolved_file).replace(os.sep, "/"))
  return m.group(1) if m and _COMMIT_HASH.match(m.group(1)) else None


def add_variant(weights_name: str, variant: Optional[str] = None) -> str:
  """`model.safetensors` + `fp16` -> `model.fp16.safetensors`."""
  if variant is None:
    return weights_name
  parts = weights_name.split(".")
  return ".".join(parts[:-1] + [variant] + parts[-1:])


def get_model_file(pretrained_model_name_or_path, weights_name: str, subfolder: Optional[str] = None,
                   variant: Optional[str] = None, revision: Optional[str] = None, cache_dir: Optional[str] = None) -> str:
  """Path of a weights file: the argument itself when it is a file, else `weights_name` (with the variant infix) in the
  folder or its sub-folder, the folder being a local directory or a Hugging Face cache entry
  (reference: src/maxdiffusion/utils/hub_utils.py:247-356, without its download branches)."""
  path = os.fspath(pretrained_model_name_or_path)
  if os.path.isfile(path):
    return path
  root = path if os.path.isdir(path) else resolve_model_path(path, revision=revision, cache_dir=cache_dir)
  name = add_variant(weights_name, variant)
  for cand in ([os.path.join(root, subfolder, name)] if subfolder else []) + [os.path.join(root, name)]:
    if os.path.isfile(cand):
      return cand
  raise EnvironmentError(f"Error no file named {name} found in directory {root}.")


def http_user_agent(user_agent=None) -> str:
  """Identification string of this library (nothing is sent anywhere: kept for code that logs it)."""
  import sys

  import torch

  from .. import __version__

  ua = f"maxdiffusion_b200/{__version__}; python/{sys.version.split()[0]}; torch/{torch.__version__}"
  if isinstance(user_agent, dict):
    ua += "; " + "; ".join(f"{k}/{v}" for k, v in user_agent.items())
  elif isinstance(user_agent, str):
    ua += "; " + user_agent
  return ua


class PushToHubMixin:
  """`push_to_hub` of the reference uploads a saved folder. This machine type has no network: the folder is written
  (through the object's own `save_pretrained`, with a model card) and its path returned, ready to be uploaded from a
  machine that has access; asking for the upload itself raises."""

  def push_to_hub(self, repo_id: str, output_dir: Optional[str] = None, commit_message: str = "", upload: bool = False,
                  **save_kwargs) -> str:
    if upload:
      raise EnvironmentError("uploading needs network access, which this installation does not use; copy the folder "
                             "that push_to_hub(..., upload=False) writes to a machine that has it")
    folder = output_dir or os.path.join("hub_export", repo_id.replace("/", "--"))
    os.makedirs(folder, exist_ok=True)
    self.save_pretrained(folder, **save_kwargs)
    if not os.path.exists(os.path.join(folder, "README.md")):
      populate_model_card(folder, repo_id.split("/")[-1], tags=("maxdiffusion_b200",), text=commit_message)
    return folder
