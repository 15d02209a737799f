"""Loads (and saves) the Z-Image components: DiT, Flux-format VAE, Qwen3 text encoder, tokenizer.

Sources, in order (reference: src/maxdiffusion/checkpointing/z_image_checkpointer.py): an Orbax-layout step
directory written by `save_checkpoint` (items `transformer_state`, `z_image_config`), else a Hugging Face folder
`pretrained_model_name_or_path` with `transformer/`, `vae/`, `text_encoder/`, `tokenizer/` sub-folders of
safetensors shards. With `random_init: True` the architecture is built from the preset without weights (benchmarks).
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict
from typing import Optional

import torch

from .. import max_logging
from ..models.qwen3 import QWEN3_PRESETS, Qwen3Model
from ..models.vae import VAE_PRESETS, AutoencoderKL, VAEConfig
from ..models.z_image.transformer_z_image import ZIMAGE_PRESETS, ZImageConfig, ZImageTransformer2DModel
from ..pipelines.z_image.z_image_pipeline import ZImagePipeline
from .checkpointing_utils import Z_IMAGE_CHECKPOINT, CheckpointManager, item_names_for

Z_IMAGE_ITEMS = item_names_for(Z_IMAGE_CHECKPOINT)


def _read_dir(folder: str) -> dict:
  from safetensors.torch import load_file

  out = {}
  for name in sorted(os.listdir(folder)):
    if name.endswith(".safetensors"):
      out.update(load_file(os.path.join(folder, name)))
  return out


class ZImageCheckpointer:

  def __init__(self, config):
    self.config = config
    directory = config.get("checkpoint_dir", "") or ""
    self.manager = CheckpointManager(directory, Z_IMAGE_ITEMS, enable_async=False) if directory else None

  def _device_dtype(self):
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    return device, (self.config.weights_dtype if device.type == "cuda" else torch.float32)

  def load_transformer(self, device, dtype) -> ZImageTransformer2DModel:
    cfg = self.config
    root = cfg.pretrained_model_name_or_path
    step = self.manager.latest_step() if self.manager is not None else None
    if step is not None:
      zcfg = ZImageConfig(**self.manager.restore_json(step, "z_image_config"))
      model = ZImageTransformer2DModel(zcfg).to(dtype)
      model.load_state_dict(self.manager.restore_state(step, "transformer_state"))
      max_logging.log(f"restored Z-Image transformer from step {step}")
      return model.to(device)
    if cfg.get("random_init", False) or not os.path.isdir(os.path.join(root, "transformer")):
      preset = dict(asdict(ZIMAGE_PRESETS[cfg.get("zimage_preset", "z-image-turbo")]))
      preset.update(cfg.get("zimage_config_overrides", {}) or {})
      return ZImageTransformer2DModel(ZImageConfig(**preset)).to(device, dtype)
    with open(os.path.join(root, "transformer", "config.json")) as f:
      raw = json.load(f)
    names = ZImageConfig.__dataclass_fields__.keys()
    model = ZImageTransformer2DModel(ZImageConfig(**{k: v for k, v in raw.items() if k in names})).to(dtype)
    sd = {k: v.to(dtype) for k, v in _read_dir(os.path.join(root, "transformer")).items()}
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if missing or unexpected:
      raise ValueError(f"Z-Image weight mapping: missing {missing[:4]}, unexpected {unexpected[:4]}")
    return model.to(device)

  def load_vae(self, device, dtype) -> AutoencoderKL:
    root = self.config.pretrained_model_name_or_path
    folder = os.path.join(root, "vae")
    if self.config.get("random_init", False) or not os.path.isdir(folder):
      over = dict(VAE_PRESETS["flux"])
      over.update(self.config.get("vae_config_overrides", {}) or {})
      return AutoencoderKL(VAEConfig(**over)).to(device, dtype)
    with open(os.path.join(folder, "config.json")) as f:
      vae = AutoencoderKL(VAEConfig.from_dict(json.load(f)))
    vae.load_state_dict(_read_dir(folder), strict=False)
    return vae.to(device, dtype)

  def load_text_encoder(self, device, dtype):
    root = self.config.pretrained_model_name_or_path
    folder = os.path.join(root, "text_encoder")
    if not os.path.isdir(folder):
      return None, None
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(os.path.join(root, "tokenizer"))
    enc = Qwen3Model.from_pretrained(folder, dtype=dtype, device="cpu" if self.config.get("offload_encoders", False) else device)
    return tok, enc

  def load_pipeline(self) -> ZImagePipeline:
    device, dtype = self._device_dtype()
    transformer = self.load_transformer(device, dtype).eval()
    vae = self.load_vae(device, dtype).eval()
    tok, enc = self.load_text_encoder(device, dtype)
    return ZImagePipeline(transformer, vae, tok, enc, dtype=dtype, device=device,
                          flow_shift=float(self.config.get("flow_shift", 3.0)),
                          offload_encoders=bool(self.config.get("offload_encoders", False)))

  def save_checkpoint(self, step: int, pipeline: ZImagePipeline) -> None:
    if self.manager is None:
      raise ValueError("checkpoint_dir is not set")
    state = {k: v.detach().cpu() for k, v in pipeline.transformer.state_dict().items()}
    cfg = asdict(pipeline.transformer.cfg)
    cfg = {k: (list(v) if isinstance(v, tuple) else v) for k, v in cfg.items()}
    self.manager.save(step, {"transformer_state": state, "z_image_config": cfg})
    self.manager.wait_until_finished()
