"""LoRA files in the styles they are published in, resolved onto this repository's modules.

`lora_loader.parse_lora_dict` turns a file into {module path: {down, up, alpha, ...}} whatever its tensor suffixes
are; this module deals with the module PATHS, which is where the styles really differ
(reference: src/maxdiffusion/loaders/lora_conversion_utils.py:22-705, models/lora_nnx.py:279-505):

  * UNet (SD / SDXL): Kohya flattens paths with underscores (`lora_unet_down_blocks_1_attentions_0_..._attn1_to_q`)
    and, when trained on the original SGM code base, numbers blocks as `input_blocks_4_1` / `middle_block_1` /
    `output_blocks_3_1` with SGM's layer names (`in_layers_2`, `emb_layers_1`, `skip_connection`, `op`). Text-encoder
    entries (`lora_te_`, `lora_te1_`, `lora_te2_`) are split off. Convolution entries (LoCon: k x k down, 1 x 1 up)
    resolve like the linear ones.
  * Flux: this repository keeps BFL's fused projections, so BFL / Kohya names map module to module
    (`double_blocks_3_img_attn_qkv` -> `transformer_blocks.3.to_qkv`); XLabs files name the attention processors
    (`double_blocks.3.processor.qkv_lora1` = image stream, `qkv_lora2` = text stream); diffusers / PEFT files have
    separate `to_q / to_k / to_v / proj_mlp` adapters, which become row slices of the fused matrices.

Flattened names are resolved against the target model's own module table, never by guessing where the dots were.
"""
from __future__ import annotations

import re
from typing import Dict, Iterable, Optional, Tuple

import torch

from .lora_loader import parse_lora_dict

RowSlice = Optional[Tuple[int, int]]  # (first row, rows) of the target weight an adapter writes to; None = all

_SGM_RESNET = {"in_layers_0": "norm1", "in_layers_2": "conv1", "emb_layers_1": "time_emb_proj", "out_layers_0": "norm2",
               "out_layers_3": "conv2", "skip_connection": "conv_shortcut"}


def sgm_block_to_diffusers(flat: str, layers_per_block: int = 2) -> str:
  """`input_blocks_4_1_transformer_blocks_0_attn1_to_q` -> `down_blocks_1_attentions_0_transformer_blocks_0_attn1_to_q`
  (still underscore-flattened). SGM numbers the UNet's stages in execution order: input block 0 is the stem, then
  per level `layers_per_block` (resnet [, attention]) entries and one down-sampler; output blocks have
  `layers_per_block + 1` entries per level, the last of which carries the up-sampler as its final sub-module."""
  per_down, per_up = layers_per_block + 1, layers_per_block + 1
  m = re.match(r"input_blocks_(\d+)_(\d+)_?(.*)", flat)
  if m:
    i, sub, rest = int(m.group(1)), int(m.group(2)), m.group(3)
    if i == 0:
      return "conv_in" + (f"_{rest}" if rest else "")
    level, j = (i - 1) // per_down, (i - 1) % per_down
    if j == layers_per_block:  # the level's down-sampler: `op` is its convolution
      return f"down_blocks_{level}_downsamplers_0_conv"
    kind = "resnets" if sub == 0 else "attentions"
    return f"down_blocks_{level}_{kind}_{j}_{_sgm_inner(rest, kind)}"
  m = re.match(r"middle_block_(\d+)_?(.*)", flat)
  if m:
    sub, rest = int(m.group(1)), m.group(2)
    kind, idx = ("attentions", 0) if sub == 1 else ("resnets", sub // 2)
    return f"mid_block_{kind}_{idx}_{_sgm_inner(rest, kind)}"
  m = re.match(r"output_blocks_(\d+)_(\d+)_?(.*)", flat)
  if m:
    i, sub, rest = int(m.group(1)), int(m.group(2)), m.group(3)
    level, j = i // per_up, i % per_up
    if rest.startswith("conv") and sub > 0 and not rest.startswith("conv_"):  # `<i>_<sub>_conv`: the up-sampler
      return f"up_blocks_{level}_upsamplers_0_conv"
    kind = "resnets" if sub == 0 else "attentions"
    return f"up_blocks_{level}_{kind}_{j}_{_sgm_inner(rest, kind)}"
  return flat


def _sgm_inner(rest: str, kind: str) -> str:
  if kind == "resnets":
    for a, b in _SGM_RESNET.items():
      if rest == a or rest.startswith(a + "_"):
        return b + rest[len(a):]
  return rest


def module_table(model: torch.nn.Module) -> Dict[str, str]:
  """underscore-flattened module path -> dotted module path, for every module of the model."""
  return {name.replace(".", "_"): name for name, _ in model.named_modules() if name}


def convert_unet_lora(sd: Dict[str, torch.Tensor], unet: torch.nn.Module, layers_per_block: int = 2):
  """-> ({unet module path: entry}, {text encoder index: {flattened path: entry}}, [unresolved keys])."""
  table = module_table(unet)
  names = set(table.values())
  unet_out, te_out, missed = {}, {}, []
  for path, entry in parse_lora_dict(sd).items():
    m = re.match(r"lora_te(\d?)_(.*)", path)
    if m:
      te_out.setdefault(int(m.group(1) or 1) - 1, {})[m.group(2)] = entry
      continue
    if path in names:  # diffusers / PEFT: already dotted
      unet_out[path] = entry
      continue
    flat = path.replace(".", "_")
    if re.match(r"(input_blocks|middle_block|output_blocks)_", flat):
      flat = sgm_block_to_diffusers(flat, layers_per_block)
    if flat in table:
      unet_out[table[flat]] = entry
    else:
      missed.append(path)
  return unet_out, te_out, missed


# ---- Flux -------------------------------------------------------------------------------------------------------
_FLUX_DOUBLE = {"img_mod_lin": "norm1", "txt_mod_lin": "norm1_context", "img_attn_qkv": "to_qkv", "txt_attn_qkv": "add_qkv_proj",
                "img_attn_proj": "to_out", "txt_attn_proj": "to_add_out", "img_mlp_0": "ff_in", "img_mlp_2": "ff_out",
                "txt_mlp_0": "ff_context_in", "txt_mlp_2": "ff_context_out"}
_FLUX_SINGLE = {"modulation_lin": "norm", "linear1": "qkv_mlp", "linear2": "proj_out"}
_XLABS_DOUBLE = {"qkv_lora1": "to_qkv", "proj_lora1": "to_out", "qkv_lora2": "add_qkv_proj", "proj_lora2": "to_add_out"}
_DIFFUSERS_DOUBLE = {"attn.to_q": ("to_qkv", 0), "attn.to_k": ("to_qkv", 1), "attn.to_v": ("to_qkv", 2),
                     "attn.add_q_proj": ("add_qkv_proj", 0), "attn.add_k_proj": ("add_qkv_proj", 1), "attn.add_v_proj": ("add_qkv_proj", 2),
                     "attn.to_out.0": ("to_out", None), "attn.to_add_out": ("to_add_out", None), "ff.net.0.proj": ("ff_in", None),
                     "ff.net.2": ("ff_out", None), "ff_context.net.0.proj": ("ff_context_in", None), "ff_context.net.2": ("ff_context_out", None),
                     "norm1.linear": ("norm1", None), "norm1_context.linear": ("norm1_context", None)}
_DIFFUSERS_SINGLE = {"attn.to_q": ("qkv_mlp", 0), "attn.to_k": ("qkv_mlp", 1), "attn.to_v": ("qkv_mlp", 2), "proj_mlp": ("qkv_mlp", 3),
                     "proj_out": ("proj_out", None), "norm.linear": ("norm", None)}


def flux_lora_target(path: str, hidden: int) -> Tuple[Optional[str], RowSlice]:
  """One adapter's module path (any published style, prefixes already stripped by `parse_lora_dict`) -> (module of
  `FluxTransformer2DModel`, row slice). `hidden` = heads * head_dim: the fused `to_qkv` is (q | k | v) rows of
  `hidden` each and the single blocks' `qkv_mlp` is (q | k | v | mlp)."""
  flat = path.replace(".", "_")
  m = re.match(r"double_blocks_(\d+)_(.*)", flat)
  if m:
    i, rest = m.groups()
    if rest.startswith("processor_"):  # XLabs
      return (f"transformer_blocks.{i}.{_XLABS_DOUBLE[rest[10:]]}", None) if rest[10:] in _XLABS_DOUBLE else (None, None)
    return (f"transformer_blocks.{i}.{_FLUX_DOUBLE[rest]}", None) if rest in _FLUX_DOUBLE else (None, None)
  m = re.match(r"single_blocks_(\d+)_(.*)", flat)
  if m:
    i, rest = m.groups()
    if rest == "processor_qkv_lora":  # XLabs adapts q, k, v of the fused first projection only
      return f"single_transformer_blocks.{i}.qkv_mlp", (0, 3 * hidden)
    if rest == "processor_proj_lora":
      return f"single_transformer_blocks.{i}.proj_out", None
    return (f"single_transformer_blocks.{i}.{_FLUX_SINGLE[rest]}", None) if rest in _FLUX_SINGLE else (None, None)
  m = re.match(r"(single_transformer_blocks|transformer_blocks)\.(\d+)\.(.*)", path)
  if m:
    kind, i, rest = m.groups()
    hit = (_DIFFUSERS_SINGLE if kind.startswith("single") else _DIFFUSERS_DOUBLE).get(rest)
    if hit is None:
      return None, None
    name, part = hit
    if part is None:
      return f"{kind}.{i}.{name}", None
    if part == 3:  # the mlp rows of `qkv_mlp`: everything after q, k, v
      return f"{kind}.{i}.{name}", (3 * hidden, -1)
    return f"{kind}.{i}.{name}", (part * hidden, hidden)
  top = {"img_in": "x_embedder", "txt_in": "context_embedder", "final_layer_linear": "proj_out", "x_embedder": "x_embedder",
         "context_embedder": "context_embedder", "proj_out": "proj_out"}
  return (top[flat], None) if flat in top else (None, None)


def convert_flux_lora(sd: Dict[str, torch.Tensor], hidden: int):
  """-> ([(module path, row slice, entry)], [unresolved paths])."""
  out, missed = [], []
  for path, entry in parse_lora_dict(sd).items():
    target, rows = flux_lora_target(path, hidden)
    if target is None:
      missed.append(path)
    else:
      out.append((target, rows, entry))
  return out, missed
