"""LoRA: parsing of the common file styles, merge-into-weights (Wan, LTX-2) and run-time adapters (SD / SDXL / Flux).

Two mechanisms as in the reference:
  * merge: W += scale * (alpha / rank) * up @ down (+ `.diff` weight deltas, `.diff_b` bias deltas), applied once
    after loading (src/maxdiffusion/models/lora_nnx.py:31-245; loaders/wan_lora_nnx_loader.py:25-111);
  * run-time adapters: extra low-rank branches evaluated next to the wrapped Linear, several adapters at once
    (src/maxdiffusion/models/lora.py:31-125; loaders/lora_pipeline.py:136-170, flux_lora_pipeline.py:57-94).
Key styles understood by `parse_lora_dict`: diffusers-PEFT (`lora_A` / `lora_B`), Kohya / XLabs / SGM
(`lora_down` / `lora_up`, `.alpha`), with `diffusion_model.` / `transformer.` / `lora_unet_` prefixes
(src/maxdiffusion/loaders/lora_conversion_utils.py:22-705).
"""
from __future__ import annotations

import os
import re
from typing import Dict, Optional

import torch
import torch.nn as nn

_PREFIXES = ("diffusion_model.", "transformer.", "model.diffusion_model.", "unet.", "lora_unet_", "lora_transformer_")


def parse_lora_dict(sd: Dict[str, torch.Tensor]) -> Dict[str, dict]:
  """module path -> {down, up, alpha, diff, diff_b}."""
  out: Dict[str, dict] = {}
  for key, t in sd.items():
    k = key
    for p in _PREFIXES:
      if k.startswith(p):
        k = k[len(p):]
    m = re.match(r"(.*)\.(lora_A|lora_down|down)(?:\.default)?\.weight$", k)  # `.down.weight`: XLabs
    if m:
      out.setdefault(m.group(1), {})["down"] = t
      continue
    m = re.match(r"(.*)\.(lora_B|lora_up|up)(?:\.default)?\.weight$", k)
    if m:
      out.setdefault(m.group(1), {})["up"] = t
      continue
    m = re.match(r"(.*)\.alpha$", k)
    if m:
      out.setdefault(m.group(1), {})["alpha"] = float(t)
      continue
    m = re.match(r"(.*)\.diff_b$", k)
    if m:
      out.setdefault(m.group(1), {})["diff_b"] = t
      continue
    m = re.match(r"(.*)\.diff$", k)
    if m:
      out.setdefault(m.group(1), {})["diff"] = t
  return out


def lora_delta(entry: dict, scale: float = 1.0) -> Optional[torch.Tensor]:
  if "down" not in entry or "up" not in entry:
    return None
  down, up = entry["down"].float(), entry["up"].float()
  rank = down.shape[0]
  alpha = entry.get("alpha", rank)
  if down.dim() == 4:  # LoCon: conv k x k down, 1 x 1 up
    delta = torch.einsum("or,rikl->oikl", up.flatten(1), down)
  else:
    delta = up @ down
  return delta * (scale * alpha / rank)


# diffusers Wan module path -> (our parameter, row slice of a fused matrix as (index, parts))
def _wan_target(path: str):
  m = re.match(r"blocks\.(\d+)\.(attn[12])\.(to_q|to_k|to_v|to_out\.0|add_k_proj|add_v_proj)$", path)
  if m:
    i, attn, proj = m.groups()
    if proj == "to_out.0":
      return f"blocks.{i}.{attn}.to_out", None
    if attn == "attn1":
      return f"blocks.{i}.attn1.to_qkv", (("to_q", "to_k", "to_v").index(proj), 3)
    if proj == "to_q":
      return f"blocks.{i}.attn2.to_q", None
    if proj in ("to_k", "to_v"):
      return f"blocks.{i}.attn2.to_kv", (("to_k", "to_v").index(proj), 2)
    return f"blocks.{i}.attn2.add_kv_proj", (("add_k_proj", "add_v_proj").index(proj), 2)
  m = re.match(r"blocks\.(\d+)\.ffn\.net\.(0\.proj|2)$", path)
  if m:
    return f"blocks.{m.group(1)}.{'ffn_in' if m.group(2) != '2' else 'ffn_out'}", None
  m = re.match(r"blocks\.(\d+)\.(self_attn|cross_attn)\.(q|k|v|o|k_img|v_img)$", path)  # original Wan repo naming
  if m:
    i, attn, proj = m.groups()
    mapped = {"q": "to_q", "k": "to_k", "v": "to_v", "o": "to_out.0", "k_img": "add_k_proj", "v_img": "add_v_proj"}[proj]
    return _wan_target(f"blocks.{i}.{'attn1' if attn == 'self_attn' else 'attn2'}.{mapped}")
  m = re.match(r"blocks\.(\d+)\.ffn\.(0|2)$", path)
  if m:
    return f"blocks.{m.group(1)}.{'ffn_in' if m.group(2) == '0' else 'ffn_out'}", None
  return None, None


# modules outside the blocks: original Wan name (and the diffusers name) -> module of this package
_WAN_ROOT_MODULES = {
    "text_embedding.0": "condition_embedder.text_in", "text_embedding.2": "condition_embedder.text_out",
    "time_embedding.0": "condition_embedder.time_in", "time_embedding.2": "condition_embedder.time_out",
    "time_projection.1": "condition_embedder.time_proj", "patch_embedding": "patch_embedding", "head.head": "proj_out",
    "img_emb.proj.0": "condition_embedder.image_embedder.norm1", "img_emb.proj.1": "condition_embedder.image_embedder.ff_in",
    "img_emb.proj.3": "condition_embedder.image_embedder.ff_out", "img_emb.proj.4": "condition_embedder.image_embedder.norm2",
    "condition_embedder.text_embedder.linear_1": "condition_embedder.text_in",
    "condition_embedder.text_embedder.linear_2": "condition_embedder.text_out",
    "condition_embedder.time_embedder.linear_1": "condition_embedder.time_in",
    "condition_embedder.time_embedder.linear_2": "condition_embedder.time_out",
    "condition_embedder.time_proj": "condition_embedder.time_proj",
    "condition_embedder.image_embedder.norm1": "condition_embedder.image_embedder.norm1",
    "condition_embedder.image_embedder.ff.net.0.proj": "condition_embedder.image_embedder.ff_in",
    "condition_embedder.image_embedder.ff.net.2": "condition_embedder.image_embedder.ff_out",
    "condition_embedder.image_embedder.norm2": "condition_embedder.image_embedder.norm2", "proj_out": "proj_out",
}


def _wan_plain_parameter(path: str):
  """LoRA paths whose target is a bare parameter (a `.diff` adds to it): q/k norm weights, the affine norm of a block
  and the modulation tables. Returns (parameter for `.diff`, parameter for `.diff_b`)."""
  if path in ("head.modulation", "head", "scale_shift_table"):      # `head.diff_m` arrives as `head.modulation.diff`
    return "scale_shift_table", None
  m = re.match(r"blocks\.(\d+)\.(.+)$", path)
  if not m:
    return None, None
  i, rest = m.groups()
  names = {"self_attn.norm_q": "attn1.norm_q", "self_attn.norm_k": "attn1.norm_k", "cross_attn.norm_q": "attn2.norm_q",
           "cross_attn.norm_k": "attn2.norm_k", "cross_attn.norm_k_img": "attn2.norm_added_k", "attn1.norm_q": "attn1.norm_q",
           "attn1.norm_k": "attn1.norm_k", "attn2.norm_q": "attn2.norm_q", "attn2.norm_k": "attn2.norm_k",
           "attn2.norm_added_k": "attn2.norm_added_k", "modulation": "scale_shift_table", "scale_shift_table": "scale_shift_table"}
  if rest in names:
    return f"blocks.{i}.{names[rest]}", None
  if rest in ("norm3", "norm2"):                                     # the affine LayerNorm before cross-attention
    return f"blocks.{i}.norm2_weight", f"blocks.{i}.norm2_bias"
  return None, None


def preprocess_wan_lora_dict(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
  """`<module>.diff_m` (a delta of the module's modulation table) becomes `<module>.modulation.diff`
  (reference: src/maxdiffusion/loaders/lora_conversion_utils.py:613-624)."""
  return {(k[:-len(".diff_m")] + ".modulation.diff" if k.endswith(".diff_m") else k): v for k, v in sd.items()}


@torch.no_grad()
def merge_lora_into_wan(model, lora_sd: Dict[str, torch.Tensor], scale: float = 1.0) -> int:
  """Adds the LoRA deltas to the (fused) Wan weights in place. Returns the number of merged modules.

  Targets: the attention and FFN projections of every block (low-rank pairs, `.diff`, `.diff_b`), the embedders, the
  time projection, the patch embedding and the output head, and the `.diff` deltas of bare parameters: q/k norm
  weights, the affine norm of a block, the modulation tables of the blocks and of the head
  (reference: src/maxdiffusion/loaders/lora_conversion_utils.py:627-705)."""
  params = dict(model.named_parameters())
  merged = 0
  for path, entry in parse_lora_dict(preprocess_wan_lora_dict(lora_sd)).items():
    target, part = _wan_target(path)
    if target is None and path in _WAN_ROOT_MODULES:
      target = _WAN_ROOT_MODULES[path]
    if target is None or target + ".weight" not in params:
      p_diff, p_bias = _wan_plain_parameter(path)
      done = False
      if p_diff in params and "diff" in entry:
        params[p_diff] += entry["diff"].to(params[p_diff].device, params[p_diff].dtype).reshape(params[p_diff].shape) * scale
        done = True
      if p_bias in params and "diff_b" in entry:
        params[p_bias] += entry["diff_b"].to(params[p_bias].device, params[p_bias].dtype).reshape(params[p_bias].shape) * scale
        done = True
      merged += int(done)
      continue
    w = params[target + ".weight"]
    rows = slice(None)
    if part is not None:
      n = w.shape[0] // part[1]
      rows = slice(part[0] * n, (part[0] + 1) * n)
    done = False
    delta = lora_delta(entry, scale)
    if delta is not None:
      w[rows] += delta.to(w.device, w.dtype).reshape(w[rows].shape)     # the patch embedding is a flattened conv kernel
      done = True
    if "diff" in entry:
      w[rows] += entry["diff"].to(w.device, w.dtype).reshape(w[rows].shape) * scale
      done = True
    if "diff_b" in entry and target + ".bias" in params:
      params[target + ".bias"][rows] += entry["diff_b"].to(w.device, w.dtype) * scale
      done = True
    merged += int(done)
  return merged


# first component of a module path in the original LTX-2 checkpoint (the namespace LoRA files use) -> this package's
# (diffusers-named) module; everything else -- `transformer_blocks.N.*`, the caption projections, `proj_out` -- has the
# same name on both sides (reference: src/maxdiffusion/loaders/lora_conversion_utils.py:708-823)
_LTX2_ROOTS = {
    "patchify_proj": "proj_in", "audio_patchify_proj": "audio_proj_in", "adaln_single": "time_embed",
    "audio_adaln_single": "audio_time_embed", "av_ca_a2v_gate_adaln_single": "av_cross_attn_video_a2v_gate",
    "av_ca_v2a_gate_adaln_single": "av_cross_attn_audio_v2a_gate",
    "av_ca_audio_scale_shift_adaln_single": "av_cross_attn_audio_scale_shift",
    "av_ca_video_scale_shift_adaln_single": "av_cross_attn_video_scale_shift", "prompt_adaln_single": "prompt_adaln",
    "audio_prompt_adaln_single": "audio_prompt_adaln",
}
_LTX2_CONNECTOR_PREFIX = "text_embedding_projection."


def _ltx2_target(path: str) -> str:
  head, _, rest = path.partition(".")
  return (_LTX2_ROOTS[head] + ("." + rest if rest else "")) if head in _LTX2_ROOTS else path


@torch.no_grad()
def _merge_entry(params: dict, target: str, entry: dict, scale: float) -> bool:
  w = params.get(target + ".weight")
  if w is None:
    return False
  delta = lora_delta(entry, scale)
  if delta is not None:
    if delta.shape != w.shape:
      raise ValueError(f"LoRA delta of {target} has shape {tuple(delta.shape)}, the weight {tuple(w.shape)}")
    w += delta.to(w.device, w.dtype)
  if "diff" in entry:
    w += entry["diff"].to(w.device, w.dtype) * scale
  if "diff_b" in entry and target + ".bias" in params:
    params[target + ".bias"] += entry["diff_b"].to(w.device, w.dtype) * scale
  return delta is not None or "diff" in entry or "diff_b" in entry


@torch.no_grad()
def merge_lora_into_ltx2(transformer, lora_sd: Dict[str, torch.Tensor], scale: float = 1.0, connectors=None) -> dict:
  """Adds the deltas of an LTX-2 LoRA file to the transformer (keys under `diffusion_model.`, original module names or
  diffusers names) and to the text connectors (keys under `text_embedding_projection.`: `aggregate_embed` is the feature
  extractor's projection). Returns {"transformer": merged modules, "connectors": merged modules, "unmatched": [paths]}
  (reference: src/maxdiffusion/loaders/ltx2_lora_nnx_loader.py:32-83)."""
  t_params = dict(transformer.named_parameters())
  c_params = dict(connectors.named_parameters()) if connectors is not None else {}
  report = {"transformer": 0, "connectors": 0, "unmatched": []}
  for path, entry in parse_lora_dict(lora_sd).items():
    if path.startswith(_LTX2_CONNECTOR_PREFIX):
      inner = path[len(_LTX2_CONNECTOR_PREFIX):]
      names = ["feature_extractor.linear", "feature_extractor.video_linear"] if inner == "aggregate_embed" else [inner]
      done = any(_merge_entry(c_params, n, entry, scale) for n in names)
      report["connectors" if done else "unmatched"] = (report["connectors"] + 1) if done else report["unmatched"] + [path]
      continue
    done = _merge_entry(t_params, _ltx2_target(path), entry, scale)
    if done:
      report["transformer"] += 1
    else:
      report["unmatched"].append(path)
  return report


def merge_ltx2_loras(pipe, config) -> list:
  """Merges every file of `lora_config` (`lora_model_name_or_path`, `weight_name`, `scale`) into the pipeline."""
  from safetensors.torch import load_file

  from .. import max_logging

  lc = config.lora_config
  paths = lc["lora_model_name_or_path"]
  reports = []
  for path, name, scale in zip(paths, lc.get("weight_name", [None] * len(paths)), lc.get("scale", [1.0] * len(paths))):
    file = os.path.join(path, name) if (name and os.path.isdir(path)) else path
    rep = merge_lora_into_ltx2(pipe.transformer, load_file(file), float(scale), getattr(pipe, "connectors", None))
    max_logging.log(f"LoRA {file}: {rep['transformer']} transformer and {rep['connectors']} connector modules merged"
                    + (f", {len(rep['unmatched'])} key(s) routed to no module: {rep['unmatched'][:8]}" if rep["unmatched"] else ""))
    reports.append(rep)
  return reports


def merge_wan_loras(pipe, config) -> None:
  """Merges every entry of `lora_config`. Wan 2.1: `weight_name[i]` goes into the transformer. Wan 2.2 (two experts):
  `high_noise_weight_name[i]` into the high-noise expert and `low_noise_weight_name[i]` into the low-noise one; an entry
  that only has `weight_name` goes into both (reference: src/maxdiffusion/loaders/wan_lora_nnx_loader.py:25-111)."""
  from safetensors.torch import load_file

  lc = config.lora_config
  paths = lc["lora_model_name_or_path"]
  pick = lambda key, i: (lc.get(key) or [None] * (i + 1))[i] if i < len(lc.get(key) or []) else None
  for i, path in enumerate(paths):
    scale = float((lc.get("scale") or [1.0] * len(paths))[i])
    resolve = lambda name: os.path.join(path, name) if (name and os.path.isdir(path)) else path
    high, low, both = pick("high_noise_weight_name", i), pick("low_noise_weight_name", i), pick("weight_name", i)
    if pipe.transformer_2 is not None and (high or low):
      if high:
        merge_lora_into_wan(pipe.transformer, load_file(resolve(high)), scale)
      if low:
        merge_lora_into_wan(pipe.transformer_2, load_file(resolve(low)), scale)
      continue
    sd = load_file(resolve(both))
    for m in filter(None, (pipe.transformer, pipe.transformer_2)):
      merge_lora_into_wan(m, sd, scale)


class LoRALinear(nn.Module):
  """Run-time adapter around a Linear-like module: y = base(x) + sum_a scale_a * up_a(down_a(x)). An adapter may
  write to a row range of the output only (`rows` = (first, count), count -1 = to the end): separate q / k / v adapters
  on a fused projection."""

  def __init__(self, base: nn.Module):
    super().__init__()
    self.base = base
    self.adapters = nn.ModuleDict()
    self.scales: Dict[str, float] = {}
    self.rows: Dict[str, Optional[tuple]] = {}

  def add_adapter(self, name: str, down: torch.Tensor, up: torch.Tensor, scale: float, rows: Optional[tuple] = None):
    key = name if name not in self.adapters else f"{name}#{len(self.adapters)}"  # q, k and v of one adapter share a name
    a = nn.ModuleDict({"down": nn.Linear(down.shape[1], down.shape[0], bias=False), "up": nn.Linear(up.shape[1], up.shape[0], bias=False)})
    w = self.base.weight
    a["down"].weight.data = down.to(w.device, w.dtype)
    a["up"].weight.data = up.to(w.device, w.dtype)
    self.adapters[key] = a
    self.scales[key] = scale
    if rows is not None:
      first, count = rows
      count = w.shape[0] - first if count < 0 else count
      if up.shape[0] != count:
        raise ValueError(f"adapter {name}: {up.shape[0]} output rows for a slice of {count}")
      rows = (first, count)
    elif up.shape[0] != w.shape[0]:
      raise ValueError(f"adapter {name}: {up.shape[0]} output rows for a weight of {w.shape[0]}")
    self.rows[key] = rows

  @property
  def weight(self):
    return self.base.weight

  @property
  def bias(self):
    return self.base.bias

  def forward(self, x, activation: Optional[str] = None, residual=None):
    y = self.base(x)
    for name, a in self.adapters.items():
      d = self.scales[name] * a["up"](a["down"](x))
      if self.rows[name] is None:
        y = y + d
      else:
        first, count = self.rows[name]
        y = torch.cat([y[..., :first], y[..., first:first + count] + d, y[..., first + count:]], dim=-1)
    # the adapters act on the pre-activation, so an activation / residual the base would have fused comes after them
    if activation == "gelu_tanh":
      y = nn.functional.gelu(y, approximate="tanh")
    elif activation == "silu":
      y = nn.functional.silu(y)
    elif activation is not None:
      raise ValueError(f"unknown activation {activation}")
    return y if residual is None else residual + y


class LoRAConv2d(nn.Module):
  """LoCon run-time adapter around a convolution: a k x k down convolution to `rank` channels (with the base's stride
  and padding) followed by a 1 x 1 up convolution (reference: src/maxdiffusion/models/lora_nnx.py:90-147)."""

  def __init__(self, base: nn.Module):
    super().__init__()
    self.base = base
    self.adapters = nn.ModuleDict()
    self.scales: Dict[str, float] = {}

  def add_adapter(self, name: str, down: torch.Tensor, up: torch.Tensor, scale: float, rows=None):
    w = self.base.weight
    if down.dim() == 2:
      down = down[:, :, None, None]
    if up.dim() == 2:
      up = up[:, :, None, None]
    if tuple(down.shape[2:]) not in ((1, 1), tuple(w.shape[2:])) or up.shape[0] != w.shape[0] or down.shape[1] != w.shape[1]:
      raise ValueError(f"adapter {name}: down {tuple(down.shape)} / up {tuple(up.shape)} do not fit a weight of {tuple(w.shape)}")
    a = nn.ParameterDict({"down": nn.Parameter(down.to(w.device, w.dtype), requires_grad=False),
                          "up": nn.Parameter(up.to(w.device, w.dtype), requires_grad=False)})
    self.adapters[name] = a
    self.scales[name] = scale

  @property
  def weight(self):
    return self.base.weight

  @property
  def bias(self):
    return self.base.bias

  def forward(self, x, *args, **kw):
    import torch.nn.functional as F

    y = self.base(x, *args, **kw)
    if kw.get("upsample") or (args and args[0]):
      x = F.interpolate(x, scale_factor=2.0, mode="nearest")  # the base folded a nearest-2x into its convolution
    stride = self.base.stride
    for name, a in self.adapters.items():
      k = a["down"].shape[-1]
      pad = tuple(p if k > 1 else 0 for p in (self.base.padding if not isinstance(self.base.padding, str) else (k // 2, k // 2)))
      h = F.conv2d(x, a["down"].to(x.dtype), None, stride, pad)
      y = y + self.scales[name] * F.conv2d(h, a["up"].to(x.dtype))
    return y


def _wrap(model: nn.Module, modules: dict, target: str):
  """Replaces module `target` of `model` by its adapter wrapper (once) and returns the wrapper."""
  mod = modules[target]
  if isinstance(mod, (LoRALinear, LoRAConv2d)):
    return mod
  parent_name, _, leaf = target.rpartition(".")
  parent = modules[parent_name] if parent_name else model
  wrapped = LoRAConv2d(mod) if isinstance(mod, nn.Conv2d) else LoRALinear(mod)
  if leaf.isdigit():
    parent[int(leaf)] = wrapped
  else:
    setattr(parent, leaf, wrapped)
  modules[target] = wrapped
  return wrapped


def add_runtime_adapters(model: nn.Module, lora_sd: Dict[str, torch.Tensor], adapter_name: str, scale: float = 1.0,
                         rename=lambda p: p) -> int:
  """Wraps every targeted Linear of `model` with a `LoRALinear` (or adds one more adapter to an existing wrapper)."""
  modules = dict(model.named_modules())
  n = 0
  for path, entry in parse_lora_dict(lora_sd).items():
    target = rename(path.replace("_", ".") if path not in modules and path.replace("_", ".") in modules else path)
    if target not in modules or "down" not in entry:
      continue
    mod = _wrap(model, modules, target)
    rank = entry["down"].shape[0]
    down, up = (entry["down"], entry["up"]) if isinstance(mod, LoRAConv2d) else (entry["down"].flatten(1), entry["up"].flatten(1))
    mod.add_adapter(adapter_name, down, up, scale * entry.get("alpha", rank) / rank)
    n += 1
  return n


def add_unet_adapters(unet: nn.Module, lora_sd: Dict[str, torch.Tensor], adapter_name: str, scale: float = 1.0,
                      text_encoders=()) -> dict:
  """SD / SDXL: a LoRA file in any published naming (diffusers / PEFT, Kohya, Kohya on SGM block numbers; linear and
  convolution adapters) as run-time adapters on the UNet and, for `lora_te*` entries, on the text encoders.
  Returns counts: {"unet": n, "text_encoder": n, "unresolved": [paths]}."""
  from .lora_conversion_utils import convert_unet_lora, module_table

  cfg = getattr(unet, "cfg", None)
  unet_map, te_map, missed = convert_unet_lora(lora_sd, unet, getattr(cfg, "layers_per_block", 2))
  modules = dict(unet.named_modules())
  counts = {"unet": 0, "text_encoder": 0, "unresolved": missed}
  for target, entry in unet_map.items():
    if "down" not in entry:
      continue
    mod = _wrap(unet, modules, target)
    rank = entry["down"].shape[0]
    down, up = (entry["down"], entry["up"]) if isinstance(mod, LoRAConv2d) else (entry["down"].flatten(1), entry["up"].flatten(1))
    mod.add_adapter(adapter_name, down, up, scale * entry.get("alpha", rank) / rank)
    counts["unet"] += 1
  for index, entries in te_map.items():
    if index >= len(text_encoders) or text_encoders[index] is None:
      counts["unresolved"].extend(f"lora_te{index + 1}_{k}" for k in entries)
      continue
    enc = text_encoders[index]
    table, mods = module_table(enc), dict(enc.named_modules())
    for flat, entry in entries.items():
      target = table.get(flat.replace(".", "_"))
      if target is None or "down" not in entry or not hasattr(mods[target], "weight"):
        counts["unresolved"].append(f"lora_te{index + 1}_{flat}")
        continue
      rank = entry["down"].shape[0]
      _wrap(enc, mods, target).add_adapter(adapter_name, entry["down"].flatten(1), entry["up"].flatten(1),
                                           scale * entry.get("alpha", rank) / rank)
      counts["text_encoder"] += 1
  return counts


def add_flux_adapters(model: nn.Module, lora_sd: Dict[str, torch.Tensor], adapter_name: str, scale: float = 1.0) -> dict:
  """Flux: BFL / Kohya, XLabs and diffusers / PEFT files onto the fused projections of `FluxTransformer2DModel`
  (separate q / k / v adapters become row slices). Returns {"adapters": n, "unresolved": [paths]}."""
  from .lora_conversion_utils import convert_flux_lora

  cfg = model.cfg
  items, missed = convert_flux_lora(lora_sd, cfg.num_attention_heads * cfg.attention_head_dim)
  modules = dict(model.named_modules())
  n = 0
  for target, rows, entry in items:
    if target not in modules or "down" not in entry:
      missed.append(target)
      continue
    rank = entry["down"].shape[0]
    _wrap(model, modules, target).add_adapter(adapter_name, entry["down"].flatten(1), entry["up"].flatten(1),
                                              scale * entry.get("alpha", rank) / rank, rows=rows)
    n += 1
  return {"adapters": n, "unresolved": missed}


def apply_flux_loras(pipe, config) -> None:
  from safetensors.torch import load_file

  lc = config.lora_config
  for path, name, adapter, scale in zip(lc["lora_model_name_or_path"], lc["weight_name"], lc["adapter_name"], lc.get("scale", [1.0] * 99)):
    sd = load_file(os.path.join(path, name) if os.path.isdir(path) else path)
    add_flux_adapters(pipe.transformer, sd, adapter, float(scale))


def apply_unet_loras(pipe, config) -> None:
  """SD / SDXL pipelines (reference: loaders/lora_pipeline.py:136-170)."""
  from safetensors.torch import load_file

  lc = config.lora_config
  encoders = [e for e in (getattr(pipe, "text_encoder", None), getattr(pipe, "text_encoder_2", None))]
  for path, name, adapter, scale in zip(lc["lora_model_name_or_path"], lc["weight_name"], lc["adapter_name"], lc.get("scale", [1.0] * 99)):
    sd = load_file(os.path.join(path, name) if os.path.isdir(path) else path)
    add_unet_adapters(pipe.unet, sd, adapter, float(scale), text_encoders=encoders)
