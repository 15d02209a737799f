"""Adapter bookkeeping on modules that carry runtime LoRA layers (`loaders.lora_loader.LoRALinear`): scaling, enabling,
deleting and fusing adapters, and rank / alpha extraction from a PEFT-layout state dict
(reference: src/maxdiffusion/utils/peft_utils.py)."""
from __future__ import annotations

from typing import Dict, Iterable, Optional

import torch


def _lora_layers(model: torch.nn.Module):
  from ..loaders.lora_loader import LoRALinear

  return [(n, m) for n, m in model.named_modules() if isinstance(m, LoRALinear)]


def get_peft_kwargs(rank_dict: Dict[str, int], alpha_dict: Dict[str, float], sd: Dict[str, torch.Tensor]) -> dict:
  """The most common rank / alpha become the defaults; layers that differ go to `rank_pattern` / `alpha_pattern`."""
  from collections import Counter

  ranks = list(rank_dict.values())
  r = Counter(ranks).most_common(1)[0][0]
  rank_pattern = {k.split(".lora_B")[0]: v for k, v in rank_dict.items() if v != r}
  alpha = r
  alpha_pattern = {}
  if alpha_dict:
    alpha = Counter(alpha_dict.values()).most_common(1)[0][0]
    alpha_pattern = {k.split(".alpha")[0]: v for k, v in alpha_dict.items() if v != alpha}
  targets = sorted({k.split(".lora")[0] for k in sd})
  return {"r": r, "lora_alpha": alpha, "rank_pattern": rank_pattern, "alpha_pattern": alpha_pattern, "target_modules": targets}


def get_rank_dict(sd: Dict[str, torch.Tensor]) -> Dict[str, int]:
  return {k: v.shape[1] for k, v in sd.items() if ".lora_B" in k and v.dim() >= 2}


def set_adapter_scale(model: torch.nn.Module, adapter_name: str, scale: float) -> int:
  n = 0
  for _, m in _lora_layers(model):
    if adapter_name in m.adapters:
      m.scales[adapter_name] = float(scale)
      n += 1
  return n


def set_adapters(model: torch.nn.Module, names: Iterable[str], weights: Optional[Iterable[float]] = None) -> None:
  """Adapters in `names` get their weight; every other adapter is switched off (scale 0) but kept."""
  names = list(names)
  weights = list(weights) if weights is not None else [1.0] * len(names)
  table = dict(zip(names, weights))
  for _, m in _lora_layers(model):
    for n in m.adapters:
      m.scales[n] = float(table.get(n, 0.0))


def delete_adapter(model: torch.nn.Module, adapter_name: str) -> None:
  for _, m in _lora_layers(model):
    if adapter_name in m.adapters:
      del m.adapters[adapter_name]
      m.scales.pop(adapter_name, None)


def fuse_adapters(model: torch.nn.Module) -> int:
  """Folds every adapter into the base weight (W += scale * up @ down) and removes the runtime layers."""
  fused = 0
  for name, m in _lora_layers(model):
    base = m.base
    with torch.no_grad():
      for an, ad in m.adapters.items():
        delta = m.scales[an] * (ad["up"].weight.float() @ ad["down"].weight.float())
        base.weight.add_(delta.reshape(base.weight.shape).to(base.weight))
        fused += 1
    parent_name, _, leaf = name.rpartition(".")
    parent = model.get_submodule(parent_name) if parent_name else model
    if leaf.isdigit():
      parent[int(leaf)] = base
    else:
      setattr(parent, leaf, base)
  return fused
