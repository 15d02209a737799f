"""Model persistence in the diffusers folder layout: `config.json` + `diffusion_pytorch_model.safetensors`, sharded
into `…-0000k-of-0000n.safetensors` with an index file above a size limit.

Reference: `FlaxModelMixin.from_pretrained / save_pretrained` (src/maxdiffusion/models/modeling_flax_utils.py:217-524)
and the PyTorch `ModelMixin` (src/maxdiffusion/models/modeling_utils.py). Here a model is any `nn.Module` that keeps
its hyper-parameters in a dataclass at `.cfg`; the functions work on it without a base class so that every model
family of the package is covered, and `ModelMixin` offers the same two calls as methods.
"""
from __future__ import annotations

import dataclasses
import glob
import json
import os
import re
from typing import Dict, Optional

import torch

WEIGHTS_NAME = "diffusion_pytorch_model.safetensors"
INDEX_NAME = WEIGHTS_NAME + ".index.json"
CONFIG_NAME = "config.json"


def _parse_size(limit) -> int:
  if isinstance(limit, int):
    return limit
  m = re.fullmatch(r"\s*([\d.]+)\s*([KMG]i?B)\s*", str(limit), flags=re.I)
  if not m:
    raise ValueError(f"cannot parse shard size {limit!r}")
  unit = m.group(2).upper()
  base = 1024 if "I" in unit else 1000
  return int(float(m.group(1)) * base ** {"K": 1, "M": 2, "G": 3}[unit[0]])


def config_to_dict(cfg) -> dict:
  d = cfg.to_dict() if hasattr(cfg, "to_dict") else dataclasses.asdict(cfg) if dataclasses.is_dataclass(cfg) else dict(cfg)
  return {k: (list(v) if isinstance(v, tuple) else v) for k, v in d.items()}


def config_from_dict(cfg_cls, d: dict):
  """Builds the dataclass from a json dict: unknown keys (diffusers bookkeeping such as `_class_name`) are dropped
  and lists become tuples where the field's default is a tuple."""
  if hasattr(cfg_cls, "from_dict"):
    return cfg_cls.from_dict(d)
  fields = {f.name: f for f in dataclasses.fields(cfg_cls)}
  kw = {}
  for k, v in d.items():
    if k not in fields:
      continue
    default = fields[k].default
    kw[k] = tuple(v) if isinstance(v, list) and isinstance(default, tuple) else v
  return cfg_cls(**kw)


def _config_class_of(model_cls):
  """The dataclass a model takes as its first constructor argument, read from the annotation."""
  import inspect
  import typing

  params = [p for p in inspect.signature(model_cls.__init__).parameters.values() if p.name != "self"]
  hints = typing.get_type_hints(model_cls.__init__)
  hint = hints.get(params[0].name) if params else None
  for cand in (hint, *typing.get_args(hint)):  # `Optional[Config]` unwraps to its members
    if dataclasses.is_dataclass(cand):
      return cand
  raise ValueError(f"{model_cls.__name__} declares no `config_class` and its first argument is not a dataclass: pass cfg_cls")


def save_model(model: torch.nn.Module, folder: str, max_shard_size="10GB", class_name: Optional[str] = None) -> None:
  from safetensors.torch import save_file

  os.makedirs(folder, exist_ok=True)
  if hasattr(model, "cfg"):
    d = config_to_dict(model.cfg)
    d["_class_name"] = class_name or type(model).__name__
    with open(os.path.join(folder, CONFIG_NAME), "w") as f:
      json.dump(d, f, indent=2, sort_keys=True)
  sd = {k: v.detach().cpu().contiguous() for k, v in model.state_dict().items()}
  limit = _parse_size(max_shard_size)
  shards, cur, size = [], {}, 0
  for k, v in sd.items():
    n = v.numel() * v.element_size()
    if cur and size + n > limit:
      shards.append(cur)
      cur, size = {}, 0
    cur[k] = v
    size += n
  shards.append(cur)
  for old in glob.glob(os.path.join(folder, "diffusion_pytorch_model*")):
    os.remove(old)
  if len(shards) == 1:
    save_file(shards[0], os.path.join(folder, WEIGHTS_NAME), metadata={"format": "pt"})
    return
  weight_map, total = {}, 0
  for i, sh in enumerate(shards):
    name = WEIGHTS_NAME.replace(".safetensors", f"-{i + 1:05d}-of-{len(shards):05d}.safetensors")
    save_file(sh, os.path.join(folder, name), metadata={"format": "pt"})
    for k, v in sh.items():
      weight_map[k] = name
      total += v.numel() * v.element_size()
  with open(os.path.join(folder, INDEX_NAME), "w") as f:
    json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2, sort_keys=True)


def read_state_dict(folder: str) -> Dict[str, torch.Tensor]:
  """All tensors of a model folder: single file, sharded with index, or any `*.safetensors` / `*.bin` inside it."""
  from safetensors.torch import load_file

  index = glob.glob(os.path.join(folder, "*.safetensors.index.json"))
  if index:
    with open(index[0]) as f:
      files = sorted(set(json.load(f)["weight_map"].values()))
    paths = [os.path.join(folder, n) for n in files]
  else:
    paths = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
  out: Dict[str, torch.Tensor] = {}
  for p in paths:
    out.update(load_file(p))
  if not paths:
    for p in sorted(glob.glob(os.path.join(folder, "*.bin"))):
      out.update(torch.load(p, map_location="cpu", weights_only=True))
  if not out:
    raise FileNotFoundError(f"no weights under {folder}")
  return out


def load_model(model_cls, folder: str, subfolder: Optional[str] = None, cfg_cls=None, dtype=None, device=None,
               strict: bool = True, key_map=None, **model_kwargs):
  """`model_cls(cfg_cls(**config.json), **model_kwargs)` with the folder's weights; `key_map(state_dict)` converts a
  foreign naming (e.g. diffusers) first."""
  folder = os.path.join(folder, subfolder) if subfolder else folder
  with open(os.path.join(folder, CONFIG_NAME)) as f:
    d = json.load(f)
  cfg_cls = cfg_cls or getattr(model_cls, "config_class", None) or _config_class_of(model_cls)
  with torch.device("meta"):
    model = model_cls(config_from_dict(cfg_cls, d), **model_kwargs)
  sd = read_state_dict(folder)
  if key_map is not None:
    sd = key_map(sd)
  if dtype is not None:
    sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
  missing, unexpected = model.load_state_dict(sd, strict=False, assign=True)
  # buffers that are derived at construction (rope tables, ...) are not in the file: build them for real
  still_meta = [n for n, t in list(model.named_parameters()) + list(model.named_buffers()) if t.is_meta]
  if still_meta:
    real = model_cls(config_from_dict(cfg_cls, d), **model_kwargs)
    ref = dict(list(real.named_parameters()) + list(real.named_buffers()))
    for n in still_meta:
      mod, _, leaf = n.rpartition(".")
      owner = model.get_submodule(mod) if mod else model
      t = ref[n]
      if leaf in owner._parameters:
        owner._parameters[leaf] = torch.nn.Parameter(t.detach(), requires_grad=t.requires_grad)
      else:
        owner._buffers[leaf] = t.detach()
  if strict:
    params = {n for n, _ in model.named_parameters()}
    lost = [k for k in missing if k in params]
    if lost or unexpected:
      raise KeyError(f"weights of {folder} do not match {model_cls.__name__}: missing {lost[:5]}, unexpected {list(unexpected)[:5]}")
  if device is not None:
    model = model.to(device)
  return model


class ModelMixin:
  """`save_pretrained(folder)` / `from_pretrained(folder, subfolder=...)` for modules with a dataclass `.cfg`.
  Subclasses set `config_class`."""
  config_class = None

  def save_pretrained(self, folder: str, max_shard_size="10GB") -> None:
    save_model(self, folder, max_shard_size)

  @classmethod
  def from_pretrained(cls, folder: str, subfolder: Optional[str] = None, dtype=None, device=None, strict: bool = True, **kw):
    return load_model(cls, folder, subfolder, dtype=dtype, device=device, strict=strict, **kw)

  def num_parameters(self, only_trainable: bool = False) -> int:
    return sum(p.numel() for p in self.parameters() if p.requires_grad or not only_trainable)
