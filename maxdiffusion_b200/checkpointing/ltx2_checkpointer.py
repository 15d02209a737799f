"""Builds / restores the LTX-2 pipeline components (reference: src/maxdiffusion/checkpointing/ltx2_checkpointer.py and
the loaders of src/maxdiffusion/pipelines/ltx2/ltx2_pipeline.py:566-955).

Order of sources: an Orbax-layout step under `checkpoint_dir` (items `ltx2_state`, `ltx2_config`, written by
`save_checkpoint`), else the diffusers folder `pretrained_model_name_or_path` (`transformer/`, `vae/`, `audio_vae/`,
`vocoder/`, `connectors/`, `latent_upsampler/`, `text_encoder/`, `tokenizer/`), else — with `random_init: True` —
random weights of the configured architecture (benchmarks, tests).
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

from .. import max_logging
from ..models.ltx2.autoencoder_kl_ltx2 import LTX2VAEConfig, LTX2VideoAutoencoderKL
from ..models.ltx2.autoencoder_kl_ltx2_audio import AutoencoderKLLTX2Audio, LTX2AudioVAEConfig
from ..models.ltx2.latent_upsampler_ltx2 import LTX2LatentUpsamplerModel
from ..models.ltx2.text_encoders_ltx2 import GemmaTextEncoder, LTX2AudioVideoGemmaTextEncoder
from ..models.ltx2.transformer_ltx2 import LTX2_PRESETS, LTX2Config, LTX2VideoTransformer3DModel
from ..models.ltx2.vocoder_ltx2 import LTX2Vocoder, LTX2VocoderWithBWE
from ..pipelines.ltx2.ltx2_pipeline import LTX2Pipeline
from .checkpointing_utils import LTX2_CHECKPOINT, CheckpointManager, item_names_for


def _read_dir(folder: str) -> dict:
  from safetensors.torch import load_file

  out = {}
  for n in sorted(os.listdir(folder)):
    if n.endswith(".safetensors"):
      out.update(load_file(os.path.join(folder, n)))
  return out


def _json(folder: str) -> dict:
  with open(os.path.join(folder, "config.json")) as f:
    return json.load(f)


def upsampler_kind_from_filename(filename: str) -> dict:
  """Constructor arguments of the latent up-sampler that its weights file name implies: which axes it doubles and by
  what factor (`...spatial-upscaler-x2...`, `...temporal-upscaler...`, `...x1.5...`)."""
  kw = {}
  name = filename.lower()
  if "temporal" in name:
    kw.update(spatial_upsample=False, temporal_upsample=True)
  elif "spatial" in name:
    kw.update(spatial_upsample=True, temporal_upsample=False)
  if "x1.5" in name:
    kw["rational_spatial_scale"] = 1.5
  elif "x2" in name:
    kw["rational_spatial_scale"] = 2.0
  return kw


class LTX2Checkpointer:

  def __init__(self, config):
    self.config = config
    d = config.get("checkpoint_dir", "") or ""
    self.manager = CheckpointManager(d, item_names_for(LTX2_CHECKPOINT), enable_async=False) if d else None

  def resolve_transformer_config(self) -> LTX2Config:
    c = self.config
    cfg = dict(LTX2_PRESETS[str(c.get("ltx2_preset", "ltx2-19b"))])
    stg = c.get("spatio_temporal_guidance_blocks", None)
    if stg:
      cfg["spatio_temporal_guidance_blocks"] = tuple(stg)
    cfg.update(c.get("ltx2_config_overrides", {}) or {})
    return LTX2Config(**cfg)

  def _load(self, module, folder, dtype, strict=False):
    module.load_state_dict({k: v.to(dtype) if v.is_floating_point() else v for k, v in _read_dir(folder).items()}, strict=strict)
    return module

  def load_pipeline(self, device=None) -> LTX2Pipeline:
    c = self.config
    device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dtype = c.weights_dtype if device.type == "cuda" else torch.float32
    root = str(c.pretrained_model_name_or_path)
    over = c.get("ltx2_component_overrides", {}) or {}
    have = lambda sub: os.path.isdir(os.path.join(root, sub)) and not c.get("random_init", False)
    step = self.manager.latest_step() if self.manager is not None else None

    if step is not None:
      tcfg = LTX2Config.from_dict(self.manager.restore_json(step, "ltx2_config"))
      transformer = LTX2VideoTransformer3DModel(tcfg).to(dtype)
      transformer.load_state_dict(self.manager.restore_state(step, "ltx2_state"))
      max_logging.log(f"restored the LTX-2 transformer from step {step}")
    elif have("transformer"):
      raw = _json(os.path.join(root, "transformer"))
      transformer = self._load(LTX2VideoTransformer3DModel(LTX2Config.from_dict(raw)).to(dtype), os.path.join(root, "transformer"), dtype)
    else:
      transformer = LTX2VideoTransformer3DModel(self.resolve_transformer_config()).to(dtype)
    tcfg = transformer.cfg

    vae = LTX2VideoAutoencoderKL(LTX2VAEConfig.from_dict(_json(os.path.join(root, "vae"))) if have("vae") else LTX2VAEConfig(**over.get("vae", {})))
    if have("vae"):
      self._load(vae, os.path.join(root, "vae"), torch.float32)
    if c.get("enable_vae_tiling", False):
      vae.enable_tiling()
    audio_vae = AutoencoderKLLTX2Audio(LTX2AudioVAEConfig.from_dict(_json(os.path.join(root, "audio_vae"))) if have("audio_vae")
                                       else LTX2AudioVAEConfig(**over.get("audio_vae", {})))
    if have("audio_vae"):
      self._load(audio_vae, os.path.join(root, "audio_vae"), torch.float32)
    if c.get("use_bwe", False):
      vocoder = LTX2VocoderWithBWE(**over.get("vocoder", {}))
    else:
      vocoder = LTX2Vocoder(**({"in_channels": tcfg.audio_in_channels} | over.get("vocoder", {})))
    if have("vocoder"):
      self._load(vocoder, os.path.join(root, "vocoder"), torch.float32)
    ck = dict(caption_channels=tcfg.caption_channels)
    ck.update(_json(os.path.join(root, "connectors")) if have("connectors") else over.get("connectors", {}))
    names = LTX2AudioVideoGemmaTextEncoder.__init__.__code__.co_varnames
    connectors = LTX2AudioVideoGemmaTextEncoder(**{k: v for k, v in ck.items() if k in names})
    if have("connectors"):
      self._load(connectors, os.path.join(root, "connectors"), dtype)
    upsampler = None
    if c.get("run_latent_upsampler", False):
      up_root = str(c.get("upsampler_model_path", root))
      folder = os.path.join(up_root, "latent_upsampler")
      kw = dict(in_channels=tcfg.in_channels, rational_spatial_scale=float(c.get("upsampler_rational_spatial_scale", 2.0)))
      kw.update(over.get("latent_upsampler", {}))
      if os.path.isdir(folder) and not c.get("random_init", False):
        raw = _json(folder)
        kw.update({k: v for k, v in raw.items() if k in LTX2LatentUpsamplerModel.__init__.__code__.co_varnames})
      # a single weights file beside the components (`upsampler_filename`, the LTX-2.3 layout) names what it does:
      # "spatial" / "temporal" and the factor (reference: src/maxdiffusion/pipelines/ltx2/ltx2_pipeline.py:876-908)
      filename = str(c.get("upsampler_filename", "") or "")
      single = os.path.join(up_root, filename) if filename else ""
      if filename:
        kw.update(upsampler_kind_from_filename(filename))
      upsampler = LTX2LatentUpsamplerModel(**kw)
      if not c.get("random_init", False):
        if single and os.path.isfile(single):
          from safetensors.torch import load_file

          upsampler.load_state_dict({k: v.float() for k, v in load_file(single).items()}, strict=False)
        elif os.path.isdir(folder):
          self._load(upsampler, folder, torch.float32)
      upsampler = upsampler.to(device).eval()
    text_encoder = None
    if have("text_encoder"):
      text_encoder = GemmaTextEncoder(os.path.join(root, "text_encoder"), device=device, dtype=c.get("text_encoder_dtype", dtype))
    pipe = LTX2Pipeline(transformer.to(device).eval(), vae.to(device).eval(), audio_vae.to(device).eval(),
                        vocoder.to(device).eval(), connectors.to(device, dtype).eval(), text_encoder, upsampler,
                        config=c, device=device)
    from ..models.quantizations import get_quantization_mode, quantize_model

    mode = get_quantization_mode(c)
    if mode is not None:
      n = quantize_model(pipe.transformer, mode, lambda name, m: "transformer_blocks." in name and m.in_features % 16 == 0 and m.out_features % 16 == 0)
      max_logging.log(f"quantization={mode}: {n} linear layers run on the fp8 tensor-core path")
    return pipe

  def save_checkpoint(self, step: int, pipeline: LTX2Pipeline) -> None:
    if self.manager is None:
      raise ValueError("checkpoint_dir is not set")
    state = {k: v.detach().cpu() for k, v in pipeline.transformer.state_dict().items()}
    self.manager.save(step, {"ltx2_state": state, "ltx2_config": pipeline.transformer.cfg.to_dict()})
    self.manager.wait_until_finished()
