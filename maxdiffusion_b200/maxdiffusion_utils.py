"""Helpers shared by the Stable Diffusion family and model-agnostic dummy-input / FLOP utilities.

Reference: src/maxdiffusion/maxdiffusion_utils.py — `load_sdxllightning_unet` :34, `maybe_load_sdxl_lora` :44,
`vae_apply` :66, `transform_images` :94, `get_add_time_ids` :143, `override_scheduler_config` / `create_scheduler`
:149-191, `rescale_noise_cfg` :194, dummy inputs :208-386, `calculate_*_tflops` :247,389,401, `tokenize_captions{,_xl}`
:428-461, `get_shaped_batch` :464, `encode{,_xl}` :493-509.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Sequence

import numpy as np
import torch

from . import max_logging
from .max_utils import calculate_model_tflops
from .pipelines.stable_diffusion.pipeline_stable_diffusion import create_scheduler, rescale_noise_cfg  # noqa: F401
from .trainers.stable_diffusion_trainer import get_add_time_ids  # noqa: F401


# ---- SDXL extras ------------------------------------------------------------------------------------------------
def load_sdxllightning_unet(config, unet) -> None:
  """Overwrites the UNet with the distilled Lightning weights named by `lightning_repo` / `lightning_ckpt` (a local
  folder + file name here: there is no hub access)."""
  repo, ckpt = str(config.get("lightning_repo", "")), str(config.get("lightning_ckpt", ""))
  if not repo or not ckpt:
    return
  path = os.path.join(repo, ckpt)
  if not os.path.exists(path):
    raise FileNotFoundError(f"{path}: the Lightning checkpoint must be a local safetensors file")
  from safetensors.torch import load_file

  dtype = next(unet.parameters()).dtype
  unet.load_state_dict({k: v.to(dtype) for k, v in load_file(path).items()})
  max_logging.log(f"loaded SDXL-Lightning UNet weights from {path}")


def maybe_load_sdxl_lora(config, pipe) -> int:
  """Merges every adapter of `lora_config` into the SDXL UNet; returns the number of merged matrices."""
  lc = config.get("lora_config", None) or {}
  paths = list(lc.get("lora_model_name_or_path", []) or [])
  if not paths:
    return 0
  from safetensors.torch import load_file

  from .loaders.lora_loader import lora_delta, parse_lora_dict

  names = list(lc.get("weight_name", []) or [])
  scales = list(lc.get("scale", []) or [])
  merged = 0
  params = dict(pipe.unet.named_parameters())
  for i, p in enumerate(paths):
    f = os.path.join(p, names[i]) if i < len(names) and names[i] else p
    entries = parse_lora_dict(load_file(f))
    scale = float(scales[i]) if i < len(scales) else 1.0
    for key, entry in entries.items():
      target = key.replace("unet.", "", 1).replace("lora_unet_", "") + ".weight"
      if target in params:
        delta = lora_delta(entry, scale)
        if delta is not None:
          with torch.no_grad():
            params[target].add_(delta.reshape(params[target].shape).to(params[target]))
          merged += 1
  max_logging.log(f"merged {merged} LoRA matrices into the UNet")
  return merged


# ---- dataset transforms -----------------------------------------------------------------------------------------
def vae_apply(images: torch.Tensor, vae, generator: Optional[torch.Generator] = None) -> torch.Tensor:
  """Pixels [B,3,H,W] in [-1,1] -> scaled latents sampled from the posterior."""
  with torch.no_grad():
    posterior = vae.encode(images.to(next(vae.parameters()).device, next(vae.parameters()).dtype))
    return vae.scale_latents(posterior.sample(generator))


def transform_images(examples: Dict[str, list], image_column: str, image_resolution: int, vae=None,
                     generator: Optional[torch.Generator] = None, batch_size: int = 8) -> Dict[str, list]:
  """HF-dataset `map` function: PIL images -> resized / centre-cropped float pixels, and VAE latents when a VAE is
  passed (`cache_latents_text_encoder_outputs`)."""
  from .image_processor import VaeImageProcessor

  proc = VaeImageProcessor()
  pix = []
  for img in examples[image_column]:
    img = img.convert("RGB") if hasattr(img, "convert") else img
    w, h = img.size
    s = image_resolution / min(w, h)
    img = img.resize((max(image_resolution, round(w * s)), max(image_resolution, round(h * s))))
    w, h = img.size
    l, t = (w - image_resolution) // 2, (h - image_resolution) // 2
    pix.append(proc.preprocess(img.crop((l, t, l + image_resolution, t + image_resolution)), image_resolution, image_resolution)[0])
  pixels = torch.stack(pix)
  if vae is None:
    examples["pixel_values"] = [p.numpy() for p in pixels]
    return examples
  lat = torch.cat([vae_apply(pixels[i:i + batch_size], vae, generator).float().cpu() for i in range(0, len(pixels), batch_size)])
  examples["pixel_values"] = [x.numpy() for x in lat]
  return examples


def tokenize_captions(examples: Dict[str, list], caption_column: str, tokenizer, input_ids_key: str = "input_ids",
                      text_encoder=None) -> Dict[str, list]:
  caps = [c if isinstance(c, str) else c[0] for c in examples[caption_column]]
  ids = tokenizer(caps, max_length=tokenizer.model_max_length, padding="max_length", truncation=True, return_tensors="pt").input_ids
  if text_encoder is not None:
    with torch.no_grad():
      examples[input_ids_key] = list(encode(ids, text_encoder).float().cpu().numpy())
  else:
    examples[input_ids_key] = list(ids.numpy())
  return examples


def tokenize_captions_xl(examples: Dict[str, list], caption_column: str, tokenizers: Sequence, text_encoders: Sequence = ()):
  caps = [c if isinstance(c, str) else c[0] for c in examples[caption_column]]
  ids = [t(caps, max_length=t.model_max_length, padding="max_length", truncation=True, return_tensors="pt").input_ids for t in tokenizers]
  if text_encoders:
    with torch.no_grad():
      prompt, pooled = encode_xl(ids, text_encoders)
    examples["prompt_embeds"] = list(prompt.float().cpu().numpy())
    examples["text_embeds"] = list(pooled.float().cpu().numpy())
  else:
    examples["input_ids"] = list(np.stack([i.numpy() for i in ids], axis=1))
  return examples


def encode(input_ids: torch.Tensor, text_encoder) -> torch.Tensor:
  return text_encoder(input_ids.to(next(text_encoder.parameters()).device)).last_hidden_state


def encode_xl(input_ids: Sequence[torch.Tensor], text_encoders: Sequence):
  """SDXL conditioning: penultimate hidden states of both encoders concatenated, pooled output of the second."""
  hs, pooled = [], None
  for ids, enc in zip(input_ids, text_encoders):
    o = enc(ids.to(next(enc.parameters()).device), output_hidden_states=True)
    hs.append(o.hidden_states[-2])
    pooled = getattr(o, "text_embeds", pooled)
  return torch.cat(hs, dim=-1), pooled


def override_scheduler_config(scheduler_config: dict, config) -> dict:
  """Applies the non-empty entries of `diffusion_scheduler_config` over a pretrained scheduler config. The four keys the
  pipelines rely on always come out defined: an override wins, else the checkpoint's value, else a safe default
  (`prediction_type` epsilon, `timestep_spacing` leading, `rescale_zero_terminal_snr` False) -- older scheduler files,
  the SD 1.5 PNDM one for instance, omit some of them (reference: src/maxdiffusion/maxdiffusion_utils.py:149-174)."""
  out = dict(scheduler_config)
  over = {k: v for k, v in dict(config.get("diffusion_scheduler_config", {}) or {}).items() if v != "" and v is not None}
  out.update(over)
  for key, default in (("_class_name", ""), ("prediction_type", "epsilon"), ("timestep_spacing", "leading"),
                       ("rescale_zero_terminal_snr", False)):
    out.setdefault(key, default)
  return out


def create_scheduler(scheduler_config: dict, config):
  """(scheduler, state) of the class the (overridden) scheduler config names, with or without the reference's `Flax`
  prefix (reference: src/maxdiffusion/maxdiffusion_utils.py:177-191)."""
  from . import schedulers

  cfg = override_scheduler_config(scheduler_config, config)
  name = str(cfg.get("_class_name", ""))
  cls = getattr(schedulers, name, None) or getattr(schedulers, name[4:] if name.startswith("Flax") else "Flax" + name, None)
  if cls is None:
    raise ValueError(f"unknown scheduler class {name!r}")
  scheduler = cls.from_config({k: v for k, v in cfg.items() if not k.startswith("_")})
  return scheduler, scheduler.create_state()


def rescale_noise_cfg(noise_cfg: torch.Tensor, noise_pred_text: torch.Tensor, guidance_rescale: float = 0.0) -> torch.Tensor:
  """Pulls the per-sample standard deviation of the guided prediction towards that of the conditional one by the
  factor `guidance_rescale` (Lin et al., "Common Diffusion Noise Schedules and Sample Steps are Flawed", 3.4;
  reference: src/maxdiffusion/maxdiffusion_utils.py:194-205)."""
  dims = list(range(1, noise_cfg.dim()))
  rescaled = noise_cfg * (noise_pred_text.std(dim=dims, keepdim=True, unbiased=False) / noise_cfg.std(dim=dims, keepdim=True, unbiased=False))
  return guidance_rescale * rescaled + (1.0 - guidance_rescale) * noise_cfg


def get_add_time_ids(original_size, crops_coords_top_left, target_size, bs: int, dtype=torch.float32) -> torch.Tensor:
  """SDXL micro-conditioning rows [bs, 6]: (original h, w, crop top, left, target h, w)."""
  return torch.tensor([list(original_size) + list(crops_coords_top_left) + list(target_size)] * bs, dtype=dtype)


def convert_dict_to_pil(image):
  """A dataset image stored as {"bytes": ..., "path": ...} becomes a PIL image; anything else passes through."""
  if isinstance(image, dict):
    import io

    from PIL import Image

    return Image.open(io.BytesIO(image["bytes"]))
  return image


# ---- dummy inputs and FLOPs -------------------------------------------------------------------------------------
def get_dummy_unet_inputs(config, unet, batch_size: Optional[int] = None, device="cpu", dtype=torch.float32):
  cfg = unet.cfg
  B = batch_size or max(1, int(float(config.get("per_device_batch_size", 1))))
  lat = int(config.get("resolution", 1024)) // 8
  added = None
  if cfg.addition_embed_type == "text_time":
    added = {"text_embeds": torch.zeros(B, cfg.projection_class_embeddings_input_dim - 6 * cfg.addition_time_embed_dim, device=device, dtype=dtype),
             "time_ids": torch.zeros(B, 6, device=device, dtype=dtype)}
  return (torch.zeros(B, cfg.in_channels, lat, lat, device=device, dtype=dtype), torch.zeros(B, dtype=torch.long, device=device),
          torch.zeros(B, 77, cfg.cross_attention_dim, device=device, dtype=dtype), added)


def get_dummy_flux_inputs(config, model, batch_size: Optional[int] = None, device="cpu", dtype=torch.float32):
  cfg = model.cfg
  B = batch_size or max(1, int(float(config.get("per_device_batch_size", 1))))
  h = w = int(config.get("resolution", 1024)) // 16
  T = int(config.get("max_sequence_length", 512))
  return (torch.zeros(B, h * w, cfg.in_channels, device=device, dtype=dtype), torch.zeros(B, T, cfg.joint_attention_dim, device=device, dtype=dtype),
          torch.zeros(B, cfg.pooled_projection_dim, device=device, dtype=dtype), torch.zeros(B, device=device),
          torch.zeros(B, h * w, 3, device=device), torch.zeros(B, T, 3, device=device), torch.zeros(B, device=device))


def get_dummy_wan_inputs(config, model, batch_size: Optional[int] = None, device="cpu", dtype=torch.float32):
  cfg = model.cfg
  B = batch_size or max(1, int(float(config.get("per_device_batch_size", 1))))
  F = (int(config.get("num_frames", 81)) - 1) // 4 + 1
  H, W = int(config.get("height", 480)) // 8, int(config.get("width", 832)) // 8
  return (torch.zeros(B, cfg.in_channels, F, H, W, device=device, dtype=dtype), torch.zeros(B, device=device),
          torch.zeros(B, int(config.get("max_sequence_length", 512)), cfg.text_dim, device=device, dtype=dtype))


def get_dummy_ltx2_inputs(config, model, batch_size: Optional[int] = None, device="cpu", dtype=torch.float32) -> dict:
  cfg = model.cfg
  B = batch_size or max(1, int(float(config.get("per_device_batch_size", 1))))
  F = (int(config.get("num_frames", 121)) - 1) // 8 + 1
  H, W = int(config.get("height", 512)) // 32, int(config.get("width", 768)) // 32
  Fa = max(1, round(int(config.get("num_frames", 121)) / float(config.get("fps", 24.0)) * 25))
  T = int(config.get("max_sequence_length", 1024))
  return dict(hidden_states=torch.zeros(B, F * H * W, cfg.in_channels, device=device, dtype=dtype),
              audio_hidden_states=torch.zeros(B, Fa, cfg.audio_in_channels, device=device, dtype=dtype),
              encoder_hidden_states=torch.zeros(B, T, cfg.caption_channels, device=device, dtype=dtype),
              audio_encoder_hidden_states=torch.zeros(B, T, cfg.caption_channels, device=device, dtype=dtype),
              timestep=torch.zeros(B, device=device), num_frames=F, height=H, width=W, audio_num_frames=Fa)


def calculate_unet_tflops(config, unet, batch_size: Optional[int] = None, train: bool = True) -> float:
  return calculate_model_tflops(unet, *get_dummy_unet_inputs(config, unet, batch_size, next(unet.parameters()).device,
                                                             next(unet.parameters()).dtype), train=train)


def calculate_flux_tflops(config, model, batch_size: Optional[int] = None, train: bool = True) -> float:
  p = next(model.parameters())
  return calculate_model_tflops(model, *get_dummy_flux_inputs(config, model, batch_size, p.device, p.dtype), train=train)


def calculate_wan_tflops(config, model, batch_size: Optional[int] = None, train: bool = True) -> float:
  """Analytic count (the attention term of a 75k-token sequence is too large to trace on CPU): per token, every block
  does 2 FLOPs per weight of its matrices, self attention adds 4*S*dim and cross attention 4*T*dim."""
  cfg = model.cfg
  B = batch_size or max(1, int(float(config.get("per_device_batch_size", 1))))
  pt, ph, pw = cfg.patch_size
  F = ((int(config.get("num_frames", 81)) - 1) // 4 + 1) // pt
  S = F * (int(config.get("height", 480)) // 8 // ph) * (int(config.get("width", 832)) // 8 // pw)
  T = int(config.get("max_sequence_length", 512))
  d, ffn = cfg.dim, cfg.ffn_dim
  per_token = cfg.num_layers * (2 * (4 * d * d + 2 * d * d + 2 * d * ffn) + 4 * S * d + 4 * T * d)
  text = cfg.num_layers * 2 * (2 * d * d) * T  # cross-attention K/V projections of the text tokens
  text += 2 * T * (cfg.text_dim * d + d * d)  # text embedder MLP
  patch = cfg.in_channels * pt * ph * pw
  ends = 2 * S * d * (patch + cfg.out_channels * pt * ph * pw) + 2 * (cfg.freq_dim * d + d * d + 6 * d * d)  # patchify, head, time MLP
  flops = B * (S * per_token + text + ends)
  return (3 if train else 1) * flops / 1e12


def get_shaped_batch(config, pipeline=None) -> Dict[str, torch.Tensor]:
  """A batch of zeros with the shapes and dtypes of the training dataset (used to warm kernels / graphs before the
  first real batch)."""
  B = max(1, int(float(config.get("per_device_batch_size", 1))))
  res = int(config.get("resolution", 1024))
  cached = bool(config.get("cache_latents_text_encoder_outputs", True))
  xl = "xl" in str(config.get("pretrained_model_name_or_path", "")).lower() or "xl" in str(config.get("model_name", "")).lower()
  batch = {"pixel_values": torch.zeros(B, 4, res // 8, res // 8) if cached else torch.zeros(B, 3, res, res)}
  if not cached:
    batch["input_ids"] = torch.zeros((B, 2, 77) if xl else (B, 77), dtype=torch.long)
  elif xl:
    batch["prompt_embeds"] = torch.zeros(B, 77, 2048)
    batch["text_embeds"] = torch.zeros(B, 1280)
  else:
    batch["input_ids"] = torch.zeros(B, 77, 1024 if "2" in str(config.get("pretrained_model_name_or_path", "")) else 768)
  return batch
