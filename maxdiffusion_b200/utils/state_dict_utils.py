"""LoRA state-dict naming conversions between the PEFT layout (`…lora_A.weight` / `…lora_B.weight`), the older
diffusers layouts (`…lora.down.weight` / `…lora.up.weight`, `to_q_lora.down`), and kohya (`lora_unet_…lora_down.weight`
with `.alpha`) (reference: src/maxdiffusion/utils/state_dict_utils.py)."""
from __future__ import annotations

import enum
from typing import Dict

import torch


class StateDictType(enum.Enum):
  DIFFUSERS_OLD = "diffusers_old"
  DIFFUSERS = "diffusers"
  PEFT = "peft"
  KOHYA_SS = "kohya_ss"


_TO_PEFT = [(".q_proj.lora_linear_layer.up", ".q_proj.lora_B"), (".q_proj.lora_linear_layer.down", ".q_proj.lora_A"),
            (".k_proj.lora_linear_layer.up", ".k_proj.lora_B"), (".k_proj.lora_linear_layer.down", ".k_proj.lora_A"),
            (".v_proj.lora_linear_layer.up", ".v_proj.lora_B"), (".v_proj.lora_linear_layer.down", ".v_proj.lora_A"),
            (".out_proj.lora_linear_layer.up", ".out_proj.lora_B"), (".out_proj.lora_linear_layer.down", ".out_proj.lora_A"),
            ("to_q_lora.up", "to_q.lora_B"), ("to_q_lora.down", "to_q.lora_A"), ("to_k_lora.up", "to_k.lora_B"),
            ("to_k_lora.down", "to_k.lora_A"), ("to_v_lora.up", "to_v.lora_B"), ("to_v_lora.down", "to_v.lora_A"),
            ("to_out_lora.up", "to_out.0.lora_B"), ("to_out_lora.down", "to_out.0.lora_A"),
            (".lora.up", ".lora_B"), (".lora.down", ".lora_A"), (".lora_linear_layer.up", ".lora_B"), (".lora_linear_layer.down", ".lora_A")]
_TO_DIFFUSERS = [(".lora_B", ".lora.up"), (".lora_A", ".lora.down")]


def detect_state_dict_type(sd: Dict[str, torch.Tensor]) -> StateDictType:
  keys = list(sd)
  if any("lora_down.weight" in k or k.endswith(".alpha") for k in keys):
    return StateDictType.KOHYA_SS
  if any(".lora_A" in k for k in keys):
    return StateDictType.PEFT
  if any("to_out_lora" in k or "to_q_lora" in k for k in keys):
    return StateDictType.DIFFUSERS_OLD
  if any(".lora.up" in k or ".lora.down" in k or "lora_linear_layer" in k for k in keys):
    return StateDictType.DIFFUSERS
  raise ValueError("not a LoRA state dict: no lora_A / lora.up / lora_down keys")


def _apply(sd, table):
  out = {}
  for k, v in sd.items():
    for a, b in table:
      if a in k:
        k = k.replace(a, b)
        break
    out[k] = v
  return out


def convert_state_dict_to_peft(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
  kind = detect_state_dict_type(sd)
  if kind == StateDictType.PEFT:
    return dict(sd)
  if kind == StateDictType.KOHYA_SS:
    return _apply({k: v for k, v in sd.items() if not k.endswith(".alpha")}, [("lora_down", "lora_A"), ("lora_up", "lora_B")])
  return _apply(sd, _TO_PEFT)


def convert_state_dict_to_diffusers(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
  return _apply(convert_state_dict_to_peft(sd), _TO_DIFFUSERS)


def convert_state_dict_to_kohya(sd: Dict[str, torch.Tensor], default_alpha_from_rank: bool = True) -> Dict[str, torch.Tensor]:
  out = {}
  for k, v in convert_state_dict_to_peft(sd).items():
    if ".lora_A" in k or ".lora_B" in k:
      base, _, tail = k.partition(".lora_")
      name = base.replace(".", "_")
      name = name if name.startswith("lora_") else "lora_unet_" + name.removeprefix("unet_")
      out[f"{name}.lora_{'down' if tail.startswith('A') else 'up'}.weight"] = v
      if default_alpha_from_rank and tail.startswith("A"):
        out[f"{name}.alpha"] = torch.tensor(float(v.shape[0]))
    else:
      out[k] = v
  return out
