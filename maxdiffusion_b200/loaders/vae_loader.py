"""diffusers AutoencoderKLWan safetensors -> `models.wan.autoencoder_kl_wan.AutoencoderKLWan`.

The module tree mirrors the diffusers one, so only a few names differ (`mid_block.resnets/attentions`,
`up_blocks.N.resnets/upsamplers` already match). Reference loader: src/maxdiffusion/models/wan/wan_utils.py:622-680.
"""
from __future__ import annotations

import torch

from .wan_loader import read_safetensors_dir


def load_wan_vae(vae, folder: str):
  sd = read_safetensors_dir(folder)
  own = vae.state_dict()
  mapped = {}
  for k, v in sd.items():
    if k in own:
      mapped[k] = v.reshape(own[k].shape)
  missing = [k for k in own if k not in mapped]
  if missing:
    raise ValueError(f"VAE weight mapping misses {len(missing)} tensors, e.g. {missing[:5]}")
  vae.load_state_dict(mapped)
  return vae
