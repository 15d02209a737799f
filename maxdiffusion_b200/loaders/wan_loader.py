"""diffusers-format Wan weights <-> this framework's parameters, and the reference's flax parameter tree.

Three layouts are involved:
  * diffusers safetensors (`blocks.N.attn1.to_q.weight` [out,in], ...): what `from_pretrained` reads / exports;
  * ours: the same orientation with q,k,v (and cross-attention k,v) fused into one matrix so that the projection
    is one GEMM, and flattened names for the embedders;
  * the reference's flax tree (`blocks.attn1.query.kernel` [L, in, out], ...) used as tree paths of the
    Orbax-layout checkpoints (key renames: src/maxdiffusion/models/wan/wan_utils.py:133-160,391-524; generic
    torch->flax rules src/maxdiffusion/models/modeling_flax_pytorch_utils.py:89-172).

A converted-weights cache (one `.npy` per tensor + `manifest.json`, bf16 stored as uint16 bit views, written to a
temporary directory and renamed) avoids re-converting on every start (reference: wan_utils.py:321-388).
"""
from __future__ import annotations

import glob
import json
import os
import re
import shutil
import tempfile
from typing import Dict, Optional

import numpy as np
import torch

_EMBEDDER = {
    "condition_embedder.time_embedder.linear_1": "condition_embedder.time_in",
    "condition_embedder.time_embedder.linear_2": "condition_embedder.time_out",
    "condition_embedder.time_proj": "condition_embedder.time_proj",
    "condition_embedder.text_embedder.linear_1": "condition_embedder.text_in",
    "condition_embedder.text_embedder.linear_2": "condition_embedder.text_out",
    "condition_embedder.image_embedder.norm1": "condition_embedder.image_embedder.norm1",
    "condition_embedder.image_embedder.ff.net.0.proj": "condition_embedder.image_embedder.ff_in",
    "condition_embedder.image_embedder.ff.net.2": "condition_embedder.image_embedder.ff_out",
    "condition_embedder.image_embedder.norm2": "condition_embedder.image_embedder.norm2",
}


def diffusers_to_ours(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
  out: Dict[str, torch.Tensor] = {}
  fuse: Dict[str, Dict[str, torch.Tensor]] = {}
  for key, t in sd.items():
    if key.startswith("patch_embedding.") or key.startswith("vace_patch_embedding."):
      out[key] = t.reshape(t.shape[0], -1) if key.endswith("weight") else t
      continue
    hit = False
    for src, dst in _EMBEDDER.items():
      if key.startswith(src + "."):
        out[dst + key[len(src):]] = t
        hit = True
        break
    if hit:
      continue
    if key == "condition_embedder.image_embedder.pos_embed":
      out[key] = t
      continue
    m = re.match(r"((?:vace_)?blocks)\.(\d+)\.(.*)", key)
    if not m:
      out[key] = t  # proj_out.*, scale_shift_table
      continue
    i, rest = m.group(2), m.group(3)
    pre = f"{m.group(1)}.{i}."
    m2 = re.match(r"(attn[12])\.(to_q|to_k|to_v|add_k_proj|add_v_proj)\.(weight|bias)", rest)
    if m2:
      attn, proj, kind = m2.groups()
      if attn == "attn2" and proj == "to_q":
        out[pre + f"attn2.to_q.{kind}"] = t
      else:
        group = "to_qkv" if attn == "attn1" else ("to_kv" if proj in ("to_k", "to_v") else "add_kv_proj")
        fuse.setdefault(pre + f"{attn}.{group}.{kind}", {})[proj] = t
      continue
    rest = rest.replace("to_out.0.", "to_out.")
    rest = re.sub(r"^(attn[12])\.(norm_q|norm_k|norm_added_k)\.weight$", r"\1.\2", rest)
    rest = rest.replace("ffn.net.0.proj.", "ffn_in.").replace("ffn.net.2.", "ffn_out.")
    rest = rest.replace("norm2.weight", "norm2_weight").replace("norm2.bias", "norm2_bias")
    out[pre + rest] = t
  order = {"to_qkv": ("to_q", "to_k", "to_v"), "to_kv": ("to_k", "to_v"), "add_kv_proj": ("add_k_proj", "add_v_proj")}
  for name, parts in fuse.items():
    group = name.split(".")[-2]
    out[name] = torch.cat([parts[p] for p in order[group]], dim=0)
  return out


def ours_to_diffusers(sd: Dict[str, torch.Tensor], in_channels: int = 16, patch=(1, 2, 2)) -> Dict[str, torch.Tensor]:
  out: Dict[str, torch.Tensor] = {}
  inv = {v: k for k, v in _EMBEDDER.items()}
  for key, t in sd.items():
    if key == "patch_embedding.weight":
      out[key] = t.reshape(t.shape[0], in_channels, *patch)
      continue
    if key == "vace_patch_embedding.weight":
      out[key] = t.reshape(t.shape[0], -1, *patch)
      continue
    hit = False
    for src, dst in inv.items():
      if key.startswith(src + "."):
        out[dst + key[len(src):]] = t
        hit = True
        break
    if hit:
      continue
    m = re.match(r"((?:vace_)?blocks)\.(\d+)\.(.*)", key)
    if not m:
      out[key] = t
      continue
    pre, rest = f"{m.group(1)}.{m.group(2)}.", m.group(3)
    m2 = re.match(r"(attn[12])\.(to_qkv|to_kv|add_kv_proj)\.(weight|bias)", rest)
    if m2:
      attn, group, kind = m2.groups()
      names = {"to_qkv": ("to_q", "to_k", "to_v"), "to_kv": ("to_k", "to_v"), "add_kv_proj": ("add_k_proj", "add_v_proj")}[group]
      for n, part in zip(names, t.chunk(len(names), dim=0)):
        out[pre + f"{attn}.{n}.{kind}"] = part.contiguous()
      continue
    rest = re.sub(r"^(attn[12])\.(norm_q|norm_k|norm_added_k)$", r"\1.\2.weight", rest)
    rest = rest.replace("to_out.", "to_out.0.").replace("ffn_in.", "ffn.net.0.proj.").replace("ffn_out.", "ffn.net.2.")
    rest = rest.replace("norm2_weight", "norm2.weight").replace("norm2_bias", "norm2.bias")
    out[pre + rest] = t
  return out


def diffusers_to_flax_tree(sd: Dict[str, torch.Tensor], scan_layers: bool = True) -> Dict[str, np.ndarray]:
  """Flat dict of '/'-joined flax paths -> arrays in the reference's orientation ([in,out] kernels, [L,...] stacks)."""
  def rename(k: str) -> str:
    k = k.replace("condition_embedder.time_embedder.linear_1", "condition_embedder.time_embedder.linear_1")
    k = k.replace("condition_embedder.text_embedder.linear_1", "condition_embedder.text_embedder.linear_1")
    k = k.replace(".scale_shift_table", ".adaln_scale_shift_table") if k.startswith(("blocks.", "vace_blocks.")) else k
    k = k.replace("to_out.0", "proj_attn").replace("ffn.net.0.proj", "ffn.act_fn.proj").replace("ffn.net.2", "ffn.proj_out")
    k = k.replace("to_q.", "query.").replace("to_k.", "key.").replace("to_v.", "value.")
    k = re.sub(r"norm2\.(weight|bias)$", r"norm2.layer_norm.\1", k)
    return k

  flat: Dict[str, np.ndarray] = {}
  stacks: Dict[str, Dict[int, np.ndarray]] = {}
  for key, t in sd.items():
    k = rename(key)
    a = t.float().cpu().numpy() if t.dtype == torch.bfloat16 else t.cpu().numpy()
    if k.endswith(".weight"):
      if a.ndim == 2:
        a, k = a.T, k[:-6] + "kernel"
      elif a.ndim == 5:
        a, k = a.transpose(2, 3, 4, 1, 0), k[:-6] + "kernel"
      else:
        k = k[:-6] + "scale"
    m = re.match(r"blocks\.(\d+)\.(.*)", k)
    if m and scan_layers:
      stacks.setdefault("blocks/" + m.group(2).replace(".", "/"), {})[int(m.group(1))] = a
    else:
      flat[k.replace(".", "/")] = a
  for name, layers in stacks.items():
    flat[name] = np.stack([layers[i] for i in sorted(layers)], axis=0)
  return flat


# ---------------------------------------------------------------------------------------------- IO
def read_safetensors_dir(folder: str) -> Dict[str, torch.Tensor]:
  from safetensors.torch import load_file

  files = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
  if not files:
    raise FileNotFoundError(f"no .safetensors file under {folder}")
  sd: Dict[str, torch.Tensor] = {}
  for f in files:
    sd.update(load_file(f))
  return sd


def _cache_key_ok(manifest: dict, keys, dtype: str) -> bool:
  return manifest.get("dtype") == dtype and sorted(manifest.get("tensors", {})) == sorted(keys)


def save_converted_cache(folder: str, sd: Dict[str, torch.Tensor], dtype: str) -> None:
  tmp = tempfile.mkdtemp(prefix=".tmp_", dir=os.path.dirname(os.path.abspath(folder)) or ".")
  manifest = {"dtype": dtype, "tensors": {}}
  for k, t in sd.items():
    a = t.detach().cpu()
    if a.dtype == torch.bfloat16:
      arr, stored = a.view(torch.int16).numpy().view(np.uint16), "bfloat16"
    else:
      arr, stored = a.numpy(), str(a.dtype).replace("torch.", "")
    np.save(os.path.join(tmp, k + ".npy"), arr)
    manifest["tensors"][k] = {"shape": list(a.shape), "dtype": stored}
  with open(os.path.join(tmp, "manifest.json"), "w") as f:
    json.dump(manifest, f)
  if os.path.isdir(folder):
    shutil.rmtree(folder)
  os.replace(tmp, folder)


def load_converted_cache(folder: str, expected_keys=None, dtype: Optional[str] = None) -> Optional[Dict[str, torch.Tensor]]:
  path = os.path.join(folder, "manifest.json")
  if not os.path.exists(path):
    return None
  with open(path) as f:
    manifest = json.load(f)
  if expected_keys is not None and not _cache_key_ok(manifest, expected_keys, dtype):
    return None  # stale: the key set or the dtype policy changed
  out = {}
  for k, meta in manifest["tensors"].items():
    arr = np.load(os.path.join(folder, k + ".npy"))
    t = torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16) if meta["dtype"] == "bfloat16" else torch.from_numpy(arr)
    out[k] = t.reshape(meta["shape"])
  return out


def load_wan_transformer(model, folder: str, converted_weights_dir: str = "", dtype=torch.bfloat16):
  """Loads diffusers safetensors from `folder` into a `WanModel` (through the converted-weights cache if given)."""
  want = list(model.state_dict().keys())
  sd = load_converted_cache(converted_weights_dir, want, str(dtype)) if converted_weights_dir else None
  if sd is None:
    sd = {k: v.to(dtype) for k, v in diffusers_to_ours(read_safetensors_dir(folder)).items()}
    if converted_weights_dir:
      save_converted_cache(converted_weights_dir, sd, str(dtype))
  missing, unexpected = model.load_state_dict(sd, strict=False)
  if missing or unexpected:
    raise ValueError(f"weight mapping does not cover the model: missing {missing[:5]}..., unexpected {unexpected[:5]}...")
  return model


def load_wan_pipeline_components(config, model_name: str, device=None, load_transformer: bool = True) -> dict:
  """transformer(s), VAE, scheduler, tokenizer and UMT5 text encoder from a local diffusers directory
  (`load_transformer=False`: dataset preprocessing only needs the VAE and the text encoder)."""
  from ..models.wan.autoencoder_kl_wan import AutoencoderKLWan, WanVAEConfig
  from ..models.wan.transformer_wan import WanConfig, WanModel
  from ..schedulers.scheduling_unipc_multistep import UniPCMultistepScheduler

  root = config.pretrained_model_name_or_path
  if not os.path.isdir(root):
    raise FileNotFoundError(f"{root} is not a local directory (no network access: download the diffusers repo first)")
  device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
  dtype = config.weights_dtype if device.type == "cuda" else torch.float32

  def build(sub):
    with open(os.path.join(root, sub, "config.json")) as f:
      cfg = WanConfig.from_dict(json.load(f))
    m = WanModel(cfg).to(dtype)
    load_wan_transformer(m, os.path.join(root, sub), config.get("converted_weights_dir", "") and
                         os.path.join(config.converted_weights_dir, sub), dtype)
    return m.to(device)

  out = {"transformer": build("transformer") if load_transformer else None}
  if load_transformer and model_name == "wan2.2" and os.path.isdir(os.path.join(root, "transformer_2")):
    out["transformer_2"] = build("transformer_2")
  with open(os.path.join(root, "vae", "config.json")) as f:
    vae = AutoencoderKLWan(WanVAEConfig.from_dict(json.load(f)))
  from .vae_loader import load_wan_vae

  load_wan_vae(vae, os.path.join(root, "vae"))
  out["vae"] = vae.to(device=device, dtype=config.get("vae_dtype", torch.float32) if device.type == "cuda" else torch.float32)
  out["scheduler"] = UniPCMultistepScheduler.from_pretrained(root, subfolder="scheduler", flow_shift=float(config.flow_shift))
  try:
    from transformers import AutoTokenizer, UMT5EncoderModel

    out["tokenizer"] = AutoTokenizer.from_pretrained(os.path.join(root, "tokenizer"))
    out["text_encoder"] = UMT5EncoderModel.from_pretrained(os.path.join(root, "text_encoder"),
                                                            torch_dtype=config.get("text_encoder_dtype", torch.float32))
  except Exception as e:  # the pipeline still works with pre-computed prompt_embeds
    from .. import max_logging

    max_logging.log(f"text encoder not loaded ({e}); pass prompt_embeds to the pipeline")
  return out


def flax_tree_to_diffusers(flat: Dict[str, np.ndarray], num_layers: Optional[int] = None) -> Dict[str, torch.Tensor]:
  """Inverse of `diffusers_to_flax_tree` (accepts stacked `[L, ...]` or per-layer `blocks/N/...` entries)."""
  out: Dict[str, torch.Tensor] = {}

  def back(path: str, a: np.ndarray):
    k = path.replace("/", ".")
    if k.endswith(".kernel"):
      k = k[:-6] + "weight"
      a = a.T if a.ndim == 2 else (a.transpose(4, 3, 0, 1, 2) if a.ndim == 5 else a)
    elif k.endswith(".scale"):
      k = k[:-5] + "weight"
    k = k.replace("norm2.layer_norm.", "norm2.")
    k = k.replace("query.", "to_q.").replace("key.", "to_k.").replace("value.", "to_v.")
    k = k.replace("proj_attn", "to_out.0").replace("ffn.act_fn.proj", "ffn.net.0.proj").replace("ffn.proj_out", "ffn.net.2")
    k = k.replace(".adaln_scale_shift_table", ".scale_shift_table")
    out[k] = torch.from_numpy(np.ascontiguousarray(a))

  for path, a in flat.items():
    if path.startswith("blocks/") and not re.match(r"blocks/\d+/", path):
      for i in range(a.shape[0]):
        back(f"blocks/{i}/" + path[len("blocks/"):], a[i])
    else:
      back(path, a)
  return out
