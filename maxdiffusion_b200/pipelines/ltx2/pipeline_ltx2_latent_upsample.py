"""Stand-alone latent up-sampling pass for multi-scale LTX-2 generation: video (or latents) in, up-sampled latents out.

reference: src/maxdiffusion/pipelines/ltx2/pipeline_ltx2_latent_upsample.py — encode the low-resolution video when
pixels are given, de-normalise, run the up-sampler, optionally AdaIN-match to the input statistics and tone-map,
re-normalise so that the result can seed a second denoising pass.
"""
from __future__ import annotations

from typing import Optional

import torch

from ...models.ltx2.latent_upsampler_ltx2 import adain_filter_latent, tone_map_latents


class LTX2LatentUpsamplePipeline:

  def __init__(self, vae, latent_upsampler):
    self.vae, self.latent_upsampler = vae, latent_upsampler

  @torch.no_grad()
  def __call__(self, video: Optional[torch.Tensor] = None, latents: Optional[torch.Tensor] = None, latents_normalized: bool = True,
               adain_factor: float = 0.0, tone_map_compression_ratio: float = 0.0, output_type: str = "latent"):
    if (video is None) == (latents is None):
      raise ValueError("pass exactly one of `video` and `latents`")
    if video is not None:
      lat = self.vae.encode(video)[0]
    else:
      lat = self.vae.denormalize_latents(latents) if latents_normalized else latents
    up = self.latent_upsampler(lat.to(next(self.latent_upsampler.parameters()).dtype)).to(lat.dtype)
    if adain_factor > 0.0:
      up = adain_filter_latent(up, lat, adain_factor)
    if tone_map_compression_ratio > 0.0:
      up = tone_map_latents(up, tone_map_compression_ratio)
    if output_type == "latent":
      return self.vae.normalize_latents(up)
    return self.vae.decode(up)
