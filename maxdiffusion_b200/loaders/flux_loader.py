"""Flux weights: the BFL single-file checkpoint (`flux1-dev.safetensors`: `double_blocks.N.*`, `single_blocks.N.*`,
`img_in`, `txt_in`, `time_in`, `vector_in`, `guidance_in`, `final_layer`) and the diffusers layout, both mapped onto
`models.flux.transformer_flux.FluxTransformer2DModel` (q/k/v fused; single-block qkv || mlp fused).

Reference: src/maxdiffusion/models/flux/util.py:57-281 (BFL loader; the reference does not read the diffusers layout).
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict

import torch

from .wan_loader import read_safetensors_dir


def bfl_to_ours(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
  out = {}
  top = {"img_in": "x_embedder", "txt_in": "context_embedder", "time_in.in_layer": "time_embedder.linear_1",
         "time_in.out_layer": "time_embedder.linear_2", "vector_in.in_layer": "text_embedder.linear_1",
         "vector_in.out_layer": "text_embedder.linear_2", "guidance_in.in_layer": "guidance_embedder.linear_1",
         "guidance_in.out_layer": "guidance_embedder.linear_2", "final_layer.linear": "proj_out"}
  dbl = {"img_mod.lin": "norm1", "txt_mod.lin": "norm1_context", "img_attn.qkv": "to_qkv", "txt_attn.qkv": "add_qkv_proj",
         "img_attn.proj": "to_out", "txt_attn.proj": "to_add_out", "img_mlp.0": "ff_in", "img_mlp.2": "ff_out",
         "txt_mlp.0": "ff_context_in", "txt_mlp.2": "ff_context_out"}
  dbl_norm = {"img_attn.norm.query_norm.scale": "norm_q", "img_attn.norm.key_norm.scale": "norm_k",
              "txt_attn.norm.query_norm.scale": "norm_added_q", "txt_attn.norm.key_norm.scale": "norm_added_k"}
  sgl = {"modulation.lin": "norm", "linear1": "qkv_mlp", "linear2": "proj_out"}
  for k, t in sd.items():
    m = re.match(r"double_blocks\.(\d+)\.(.*)", k)
    if m:
      i, rest = m.groups()
      if rest in dbl_norm:
        out[f"transformer_blocks.{i}.{dbl_norm[rest]}"] = t
        continue
      for src, dst in dbl.items():
        if rest.startswith(src + "."):
          out[f"transformer_blocks.{i}.{dst}{rest[len(src):]}"] = t
      continue
    m = re.match(r"single_blocks\.(\d+)\.(.*)", k)
    if m:
      i, rest = m.groups()
      if rest == "norm.query_norm.scale":
        out[f"single_transformer_blocks.{i}.norm_q"] = t
      elif rest == "norm.key_norm.scale":
        out[f"single_transformer_blocks.{i}.norm_k"] = t
      else:
        for src, dst in sgl.items():
          if rest.startswith(src + "."):
            out[f"single_transformer_blocks.{i}.{dst}{rest[len(src):]}"] = t
      continue
    if k.startswith("final_layer.adaLN_modulation.1."):
      # BFL emits (shift, scale); AdaLayerNormContinuous expects (scale, shift)
      a, b = t.chunk(2, dim=0)
      out["norm_out" + k[len("final_layer.adaLN_modulation.1"):]] = torch.cat([b, a], dim=0)
      continue
    for src, dst in top.items():
      if k.startswith(src + "."):
        out[dst + k[len(src):]] = t
  return out


def diffusers_to_ours(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
  out, fuse = {}, {}
  ren = {"time_text_embed.timestep_embedder": "time_embedder", "time_text_embed.guidance_embedder": "guidance_embedder",
         "time_text_embed.text_embedder": "text_embedder", "norm_out.linear": "norm_out"}
  for k, t in sd.items():
    for a, b in ren.items():
      if k.startswith(a + "."):
        k = b + k[len(a):]
    m = re.match(r"(transformer_blocks|single_transformer_blocks)\.(\d+)\.(.*)", k)
    if not m:
      out[k] = t
      continue
    kind, i, rest = m.groups()
    pre = f"{kind}.{i}."
    rest = rest.replace("norm1.linear", "norm1").replace("norm1_context.linear", "norm1_context").replace("norm.linear", "norm")
    rest = rest.replace("ff.net.0.proj", "ff_in").replace("ff.net.2", "ff_out")
    rest = rest.replace("ff_context.net.0.proj", "ff_context_in").replace("ff_context.net.2", "ff_context_out")
    rest = rest.replace("attn.to_out.0", "to_out").replace("attn.to_add_out", "to_add_out")
    mm = re.match(r"attn\.(norm_q|norm_k|norm_added_q|norm_added_k)\.weight", rest)
    if mm:
      out[pre + mm.group(1)] = t
      continue
    mm = re.match(r"attn\.(to_q|to_k|to_v|add_q_proj|add_k_proj|add_v_proj)\.(weight|bias)", rest)
    if mm:
      proj, wb = mm.groups()
      grp = "add_qkv_proj" if proj.startswith("add_") else ("qkv_mlp" if kind.startswith("single") else "to_qkv")
      fuse.setdefault(pre + grp + "." + wb, {})[proj] = t
      continue
    if kind.startswith("single") and rest.startswith("proj_mlp."):
      fuse.setdefault(pre + "qkv_mlp." + rest.split(".")[-1], {})["proj_mlp"] = t
      continue
    out[pre + rest] = t
  for name, parts in fuse.items():
    order = [p for p in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj", "proj_mlp") if p in parts]
    out[name] = torch.cat([parts[p] for p in order], dim=0)
  return out


def load_flux_transformer(model, path: str, dtype=torch.bfloat16):
  """`path`: a BFL single file or a diffusers `transformer/` directory."""
  if os.path.isfile(path):
    from safetensors.torch import load_file

    sd = bfl_to_ours(load_file(path))
  else:
    sd = diffusers_to_ours(read_safetensors_dir(path))
  missing, unexpected = model.load_state_dict({k: v.to(dtype) for k, v in sd.items()}, strict=False)
  if missing or unexpected:
    raise ValueError(f"Flux weight mapping: missing {missing[:4]}, unexpected {unexpected[:4]}")
  return model


def load_flux_pipeline(config, device=None):
  from ..models.flux.transformer_flux import FluxConfig, FluxTransformer2DModel
  from ..models.vae import AutoencoderKL, VAEConfig
  from ..pipelines.flux.flux_pipeline import FluxPipeline

  root = config.pretrained_model_name_or_path
  device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
  dtype = config.weights_dtype if device.type == "cuda" else torch.float32
  if os.path.isfile(root):
    tcfg, tpath = FluxConfig(guidance_embeds="schnell" not in os.path.basename(root)), root
    vae = None
  else:
    with open(os.path.join(root, "transformer", "config.json")) as f:
      tcfg = FluxConfig.from_dict(json.load(f))
    tpath = os.path.join(root, "transformer")
    with open(os.path.join(root, "vae", "config.json")) as f:
      vae = AutoencoderKL(VAEConfig.from_dict(json.load(f)))
    vae.load_state_dict(read_safetensors_dir(os.path.join(root, "vae")), strict=False)
    vae = vae.to(device, dtype)
  model = load_flux_transformer(FluxTransformer2DModel(tcfg).to(dtype), tpath, dtype).to(device)
  kw = {}
  try:
    from transformers import CLIPTextModel, CLIPTokenizer, T5EncoderModel, T5TokenizerFast

    kw = dict(clip=CLIPTextModel.from_pretrained(os.path.join(root, "text_encoder")),
              clip_tokenizer=CLIPTokenizer.from_pretrained(os.path.join(root, "tokenizer")),
              t5=T5EncoderModel.from_pretrained(os.path.join(root, "text_encoder_2")),
              t5_tokenizer=T5TokenizerFast.from_pretrained(os.path.join(root, "tokenizer_2")))
  except Exception:
    pass
  pipe = FluxPipeline(config, model, vae, device=device, **kw)
  pipe.maybe_shard_weights()
  return pipe
