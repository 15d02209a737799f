"""Pipeline persistence: a folder with `model_index.json` naming every component and one sub-folder per component.

Reference: `FlaxDiffusionPipeline.save_pretrained / from_pretrained` (src/maxdiffusion/pipelines/pipeline_flax_utils.py).
Components are looked up by attribute name on the pipeline object; `nn.Module`s are written with
`models.modeling_utils.save_model`, schedulers with their own `save_pretrained`, HF tokenizers / text encoders with
theirs.
"""
from __future__ import annotations

import importlib
import json
import os
from typing import Dict, Iterable, Optional

import torch

from ..models.modeling_utils import load_model, save_model

MODEL_INDEX = "model_index.json"
DEFAULT_COMPONENTS = ("transformer", "low_noise_transformer", "high_noise_transformer", "unet", "controlnet", "vae", "audio_vae",
                      "vocoder", "connectors", "latent_upsampler", "scheduler", "text_encoder", "text_encoder_2", "tokenizer",
                      "tokenizer_2", "image_encoder", "image_processor")


def _library_of(obj) -> str:
  mod = type(obj).__module__
  return "transformers" if mod.startswith("transformers") else mod


def save_pipeline(pipe, folder: str, components: Optional[Iterable[str]] = None, max_shard_size="10GB") -> Dict[str, list]:
  os.makedirs(folder, exist_ok=True)
  index: Dict[str, list] = {"_class_name": type(pipe).__name__}
  for name in components or DEFAULT_COMPONENTS:
    obj = getattr(pipe, name, None)
    if obj is None:
      continue
    sub = os.path.join(folder, name)
    if hasattr(obj, "save_pretrained"):
      obj.save_pretrained(sub)
    elif isinstance(obj, torch.nn.Module):
      save_model(obj, sub, max_shard_size)
    else:
      continue
    index[name] = [_library_of(obj), type(obj).__name__]
  with open(os.path.join(folder, MODEL_INDEX), "w") as f:
    json.dump(index, f, indent=2, sort_keys=True)
  return index


def load_components(folder: str, dtype=None, device=None, skip=()) -> Dict[str, object]:
  """Every component `model_index.json` names whose class can be imported; the caller passes them to the pipeline
  class's constructor."""
  with open(os.path.join(folder, MODEL_INDEX)) as f:
    index = json.load(f)
  out: Dict[str, object] = {}
  for name, spec in index.items():
    if name.startswith("_") or name in skip or not isinstance(spec, list):
      continue
    lib, cls_name = spec
    cls = getattr(importlib.import_module(lib), cls_name)
    sub = os.path.join(folder, name)
    if lib == "transformers" or not issubclass(cls, torch.nn.Module):
      out[name] = cls.from_pretrained(sub)
    elif hasattr(cls, "from_pretrained") and getattr(cls, "config_class", None) is None:
      out[name] = cls.from_pretrained(sub)
    else:
      out[name] = load_model(cls, sub, dtype=dtype, device=device)
  return out


class DiffusionPipelineMixin:

  def save_pretrained(self, folder: str, components: Optional[Iterable[str]] = None, max_shard_size="10GB"):
    return save_pipeline(self, folder, components, max_shard_size)
