"""Wan 2.1 VACE pipeline: text + (control video, mask, reference images) -> video.

Behaviour follows the reference (src/maxdiffusion/pipelines/wan/wan_vace_pipeline_2_1.py):
  * `preprocess_conditions` (:171-275): missing video -> zeros, missing mask -> ones; masks mapped to [0, 1];
    reference images are letter-boxed on a white canvas of the video size;
  * `prepare_video_latents` (:649-713): the binarised mask splits the video into `inactive = v * (1 - m)` and
    `reactive = v * m`; both are VAE-encoded (mode), normalised and concatenated on channels (32); every reference
    image contributes one extra leading latent frame `[ref_latent, zeros]`;
  * `prepare_masks` (:277-320): the pixel mask is folded 8x8 into 64 channels and resampled (nearest-exact) to the
    latent frame count; reference frames get an all-zero mask; control = concat(latents 32, mask 64) = 96 channels;
  * the generated latents have `num_reference_images` extra leading frames, which are dropped before decoding.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch
import torch.nn.functional as F

from ...models.wan.transformer_wan_vace import WanVACEModel
from .wan_pipeline import WanPipeline


class WanVACEPipeline2_1(WanPipeline):
  model_name = "wan2.1"
  transformer_cls = WanVACEModel

  @staticmethod
  def resolve_transformer_config(config):
    from ...trainers.wan_vace_trainer import resolve_wan_vace_config

    return resolve_wan_vace_config(config)

  # ---- conditioning ------------------------------------------------------------------------
  def preprocess_conditions(self, video: Optional[torch.Tensor], mask: Optional[torch.Tensor],
                            reference_images: Optional[Sequence[torch.Tensor]], batch: int, height: int, width: int,
                            num_frames: int):
    """video / mask: [B,3,F,H,W] in [-1,1] or None; reference_images: list of [3,h,w] in [-1,1] (shared by the batch)."""
    if video is None:
      video = torch.zeros((batch, 3, num_frames, height, width))
    size = tuple(video.shape[-2:])
    mask = torch.ones_like(video) if mask is None else ((mask.float() + 1) / 2).clamp(0, 1)
    refs = []
    for img in reference_images or []:
      img = img.float()[None]
      ih, iw = img.shape[-2:]
      scale = min(size[0] / ih, size[1] / iw)
      nh, nw = int(ih * scale), int(iw * scale)
      resized = F.interpolate(img, size=(nh, nw), mode="bilinear", align_corners=False)[0]
      canvas = torch.ones((3, *size))
      top, left = (size[0] - nh) // 2, (size[1] - nw) // 2
      canvas[:, top:top + nh, left:left + nw] = resized
      refs.append(canvas)
    return video.float(), mask, refs

  def prepare_masks(self, mask: torch.Tensor, num_reference_images: int) -> torch.Tensor:
    """[B,3,F,H,W] in [0,1] -> [B,64,T',H/8,W/8] (+ leading zero frames for the reference images)."""
    s = self.vae_scale_factor_spatial
    p = int(self.transformer.cfg.patch_size[1])
    out = []
    for m in mask:
      _, Fr, H, W = m.shape
      t_new = (Fr + self.vae_scale_factor_temporal - 1) // self.vae_scale_factor_temporal
      h_new, w_new = H // (s * p) * p, W // (s * p) * p
      m = m[0, :, :h_new * s, :w_new * s].reshape(Fr, h_new, s, w_new, s).permute(2, 4, 0, 1, 3).flatten(0, 1)
      m = F.interpolate(m[None], size=(t_new, h_new, w_new), mode="nearest-exact")[0]
      if num_reference_images:
        m = torch.cat([torch.zeros_like(m[:, :num_reference_images]), m], dim=1)
      out.append(m)
    return torch.stack(out)

  @torch.no_grad()
  def prepare_video_latents(self, video: torch.Tensor, mask: torch.Tensor, refs: List[torch.Tensor]) -> torch.Tensor:
    vae_dtype = next(self.vae.parameters()).dtype
    video, mask = video.to(self.device, vae_dtype), (mask > 0.5).to(self.device, vae_dtype)
    enc = lambda v: self.vae.normalize_latents(self.vae.encode(v, self.vae_encode_chunk(v.shape[2])).mode())
    latents = torch.cat([enc(video * (1 - mask)), enc(video * mask)], dim=1)  # [B,32,T',h,w]
    for img in refs:
      ref = enc(img.to(self.device, vae_dtype)[None, :, None])  # one frame
      ref = torch.cat([ref, torch.zeros_like(ref)], dim=1).expand(latents.shape[0], -1, -1, -1, -1)
      latents = torch.cat([ref, latents], dim=2)
    return latents

  # ---- call --------------------------------------------------------------------------------
  @torch.no_grad()
  def __call__(self, video=None, mask=None, reference_images=None, conditioning_scale: Union[float, Sequence[float]] = 1.0,
               prompt=None, height: Optional[int] = None, width: Optional[int] = None, num_frames: Optional[int] = None,
               conditioning_latents: Optional[torch.Tensor] = None, output_type: str = "uint8", **kw):
    c = self.config
    height, width = height or int(c.get("height", 480)), width or int(c.get("width", 832))
    num_frames = num_frames or int(c.get("num_frames", 81))
    if mask is not None and video is None:
      raise ValueError("`mask` can only be passed if `video` is passed as well.")
    if video is not None and mask is not None and video.shape[2] != mask.shape[2]:
      raise ValueError(f"Length of `video` {video.shape[2]} and `mask` {mask.shape[2]} do not match.")
    if num_frames % self.vae_scale_factor_temporal != 1:
      num_frames = max(1, num_frames // self.vae_scale_factor_temporal * self.vae_scale_factor_temporal + 1)
    layers = self.transformer.cfg.vace_layers
    scales = [float(conditioning_scale)] * len(layers) if isinstance(conditioning_scale, (int, float)) else list(conditioning_scale)
    if len(scales) != len(layers):
      raise ValueError(f"Length of `conditioning_scale` {len(scales)} does not match number of layers {len(layers)}.")
    embeds = kw.get("prompt_embeds")
    batch = embeds.shape[0] if embeds is not None else (1 if isinstance(prompt, str) or prompt is None else len(prompt))
    n_ref = 0
    if conditioning_latents is None:
      if self.vae is None:
        raise ValueError("a VAE is needed to encode the control video; pass `conditioning_latents` instead")
      v, m, refs = self.preprocess_conditions(video, mask, reference_images, batch, height, width, num_frames)
      n_ref = len(refs)
      lat = self.prepare_video_latents(v, m, refs)
      msk = self.prepare_masks(m, n_ref).to(lat.device, lat.dtype)
      conditioning_latents = torch.cat([lat, msk], dim=1)
    tl = (num_frames - 1) // self.vae_scale_factor_temporal + 1 + n_ref
    if conditioning_latents.shape[2] != tl:
      raise ValueError("The number of frames in the conditioning latents does not match the number of frames to be "
                       f"generated: {conditioning_latents.shape[2]} != {tl}")
    self.extra_model_kwargs = {"control_hidden_states": conditioning_latents.to(self.device, self.dtype),
                               "control_hidden_states_scale": scales}
    try:
      # reference frames extend the latent video; the base pipeline sizes latents from the frame count
      out = super().__call__(prompt=prompt, height=height, width=width,
                             num_frames=num_frames + n_ref * self.vae_scale_factor_temporal, output_type="latent", **kw)
    finally:
      self.extra_model_kwargs = {}
    trace = None
    if isinstance(out, tuple):
      out, trace = out
    latents = out[:, :, n_ref:]
    if output_type != "latent" and self.vae is not None:
      from ...models.wan.autoencoder_kl_wan import postprocess_video

      video_out = self.decode_latents(latents)
      latents = postprocess_video(video_out) if output_type == "uint8" else video_out
    return (latents, trace) if trace is not None else latents
