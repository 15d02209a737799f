"""diffusers-format SD / SDXL checkpoints (UNet, VAE, CLIP text encoders, ControlNet) from a local directory.

The module trees mirror diffusers', so the UNet / VAE / ControlNet safetensors load by name (1x1 convolution
attention projections of old VAE files are reshaped to Linear). Reference: `FlaxModelMixin.from_pretrained`
(src/maxdiffusion/models/modeling_flax_utils.py:217-457) with `from_pt=True` key conversion
(modeling_flax_pytorch_utils.py:89-172), which is unnecessary here because the layout already is PyTorch's.
"""
from __future__ import annotations

import json
import os

import torch

from .wan_loader import read_safetensors_dir


def load_by_name(module, folder: str, dtype=None):
  sd = read_safetensors_dir(folder)
  own = module.state_dict()
  fixed = {}
  for k, v in sd.items():
    k2 = k.replace(".query.", ".to_q.").replace(".key.", ".to_k.").replace(".value.", ".to_v.").replace(".proj_attn.", ".to_out.0.")
    if k2 in own:
      fixed[k2] = v.reshape(own[k2].shape).to(dtype or own[k2].dtype)
  missing = [k for k in own if k not in fixed]
  if missing:
    raise ValueError(f"{folder}: {len(missing)} tensors are not covered, e.g. {missing[:4]}")
  module.load_state_dict(fixed)
  return module


def load_sd_pipeline(config, pipeline_cls, device=None):
  from ..models.controlnet import ControlNetModel
  from ..models.unet_2d_condition import UNet2DConditionModel, UNetConfig
  from ..models.vae import AutoencoderKL, VAEConfig
  from ..pipelines.stable_diffusion.pipeline_stable_diffusion import create_scheduler

  root = config.pretrained_model_name_or_path
  if not os.path.isdir(root):
    raise FileNotFoundError(f"{root} is not a local diffusers directory (no network access)")
  device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
  dtype = config.weights_dtype if device.type == "cuda" else torch.float32
  with open(os.path.join(root, "unet", "config.json")) as f:
    unet = UNet2DConditionModel(UNetConfig.from_dict(json.load(f)))
  unet = load_by_name(unet, config.get("unet_checkpoint", "") or os.path.join(root, "unet"), dtype).to(device, dtype)
  with open(os.path.join(root, "vae", "config.json")) as f:
    vae = load_by_name(AutoencoderKL(VAEConfig.from_dict(json.load(f))), os.path.join(root, "vae"), dtype).to(device, dtype)
  encs, toks = [], []
  try:
    from transformers import CLIPTextModel, CLIPTextModelWithProjection, CLIPTokenizer

    for sub, tsub, cls in (("text_encoder", "tokenizer", CLIPTextModel), ("text_encoder_2", "tokenizer_2", CLIPTextModelWithProjection)):
      if os.path.isdir(os.path.join(root, sub)):
        encs.append(cls.from_pretrained(os.path.join(root, sub)).to(device))
        toks.append(CLIPTokenizer.from_pretrained(os.path.join(root, tsub)))
  except Exception:
    encs, toks = [], []
  controlnet = None
  cn_path = config.get("controlnet_model_name_or_path", "")
  if cn_path and os.path.isdir(cn_path):
    controlnet = load_by_name(ControlNetModel(unet.cfg), cn_path, dtype).to(device, dtype)
  return pipeline_cls(config, unet, vae, create_scheduler(config), encs, toks, controlnet, device=device)
