"""Wan-Animate pipeline: a reference character image driven by a pose video and a face video, generated
segment by segment with the tail of each segment conditioning the next.

Behaviour follows the reference (src/maxdiffusion/pipelines/wan/wan_pipeline_animate.py):
  * the driving videos are padded by reflection to a whole number of segments (`pad_video_frames` :416-436);
    a segment has `segment_frame_length` frames of which the first `prev_segment_conditioning_frames` repeat
    the previous segment's last decoded frames (:758-764, :895-1040);
  * conditioning latents per segment (:568-641): VAE latents of [previous frames | zeros] (replace mode:
    the background video) with a 4-channel I2V mask (1 = known frame; replace mode: the inverted character
    mask), preceded by the reference-image latents with mask 1 (:513-543);
  * model input = concat(noisy latents 16, mask 4 + conditioning latents 16) with one extra leading latent frame
    for the reference image; pose latents enter through the pose patch embedding; face crops are encoded once per
    segment by the motion encoder (`encode_face_motion`), with an all -1 face video for the unconditional branch;
  * CFG: `uncond + g * (cond - uncond)`; UniPC steps; the reference frame is dropped before decoding (:1026).
Videos are tensors [B, 3, T, H, W] in [-1, 1] (masks [B, 1, T, H, W] in [0, 1]).
"""
from __future__ import annotations

from typing import Optional

import torch

from ...models.wan.autoencoder_kl_wan import postprocess_video
from ...models.wan.transformer_wan_animate import WAN_ANIMATE_PRESETS, WanAnimateConfig, WanAnimateModel
from ...ops import functional as OF
from .wan_pipeline import WanPipeline


def resolve_wan_animate_config(config) -> WanAnimateConfig:
  preset = str(config.get("wan_preset", "") or "")
  cfg = dict(WAN_ANIMATE_PRESETS[preset if preset in WAN_ANIMATE_PRESETS else "wan2.2-animate-14b"])
  cfg.update(config.get("wan_config_overrides", None) or {})
  return WanAnimateConfig(**cfg)


def pad_video_frames(video: torch.Tensor, num_target_frames: int) -> torch.Tensor:
  """Reflect-style padding along time: [1,2,3,4,5] -> [1,2,3,4,5,4,3,2,1,2] for 10 frames."""
  T = video.shape[2]
  idx, flip, order = 0, False, []
  while len(order) < num_target_frames:
    order.append(idx)
    idx += -1 if flip else 1
    if idx == 0 or idx == T - 1:
      flip = not flip
    if T == 1:
      idx = 0
  return video[:, :, order]


class WanAnimatePipeline(WanPipeline):
  model_name = "wan2.1"  # single expert
  transformer_cls = WanAnimateModel
  resolve_transformer_config = staticmethod(resolve_wan_animate_config)

  # ---- conditioning ------------------------------------------------------------------------
  def get_i2v_mask(self, batch, latent_t, latent_h, latent_w, mask_len=1, mask_pixel_values=None, dtype=torch.float32):
    """[B, 4, latent_t, h, w]: 1 = known frame. `mask_pixel_values`: [B,1,T_pixel,h,w] at pixel frame rate."""
    s = self.vae_scale_factor_temporal
    pixel_frames = (latent_t - 1) * s + 1
    m = torch.zeros((batch, 1, pixel_frames, latent_h, latent_w), dtype=dtype, device=self.device) \
        if mask_pixel_values is None else mask_pixel_values.to(self.device, dtype).clone()
    m[:, :, :mask_len] = 1.0
    m = torch.cat([m[:, :, :1].repeat(1, 1, s, 1, 1), m[:, :, 1:]], dim=2)
    return m.reshape(batch, latent_t, s, latent_h, latent_w).permute(0, 2, 1, 3, 4)

  @torch.no_grad()
  def _encode(self, video):
    vae_dtype = next(self.vae.parameters()).dtype
    return self.vae.normalize_latents(self.vae.encode(video.to(self.device, vae_dtype), self.vae_encode_chunk(video.shape[2])).mode())

  def prepare_reference_image_latents(self, image, batch):
    lat = self._encode(image[:, :, None] if image.dim() == 4 else image)
    if lat.shape[0] == 1 and batch > 1:
      lat = lat.expand(batch, -1, -1, -1, -1)
    mask = self.get_i2v_mask(batch, 1, lat.shape[3], lat.shape[4], 1, dtype=lat.dtype)
    return torch.cat([mask, lat], dim=1)

  @staticmethod
  def _resize_mask(mask, h, w):
    H, W = mask.shape[-2:]
    if (H, W) == (h, w):
      return mask
    hi = torch.floor(torch.arange(h) * (H / h)).long()
    wi = torch.floor(torch.arange(w) * (W / w)).long()
    return mask[..., hi, :][..., wi]

  def prepare_prev_segment_cond_latents(self, prev_video, background, mask_video, batch, seg_len, start, height, width,
                                        prev_frames, task):
    lh, lw = height // self.vae_scale_factor_spatial, width // self.vae_scale_factor_spatial
    lt = (seg_len - 1) // self.vae_scale_factor_temporal + 1
    if prev_video is None:
      prev_video = background[:, :, :prev_frames] if (task == "replace" and background is not None) else \
          torch.zeros((batch, 3, prev_frames, height, width))
    remaining = background[:, :, prev_frames:] if (task == "replace" and background is not None) else \
        torch.zeros((batch, 3, seg_len - prev_frames, height, width))
    cond = self._encode(torch.cat([prev_video.float().cpu(), remaining.float().cpu()], dim=2))
    mpv = None
    if task == "replace" and mask_video is not None:
      mpv = self._resize_mask(1.0 - mask_video.float(), lh, lw)
    mask = self.get_i2v_mask(batch, lt, lh, lw, prev_frames if start > 0 else 0, mpv, dtype=cond.dtype)
    return torch.cat([mask, cond], dim=1)

  # ---- call --------------------------------------------------------------------------------
  def check_inputs(self, image, pose_video, face_video, background_video, mask_video, prompt, negative_prompt, height,
                   width, prompt_embeds=None, negative_prompt_embeds=None, image_embeds=None, mode="animate",
                   prev_segment_conditioning_frames=5) -> None:
    """The user-facing argument rules (reference: src/maxdiffusion/pipelines/wan/wan_pipeline_animate.py:338-413):
    a prompt or its embedding but not both, the reference image, both driving videos present and non-empty with as many frames as each
    other, background + mask in replace mode, sizes divisible by 16, 1 or 5 conditioning frames."""
    def one_of(a, b, name):
      if a is not None and b is not None:
        raise ValueError(f"pass `{name}` or `{name}_embeds`, not both")
    one_of(prompt, prompt_embeds, "prompt")
    one_of(negative_prompt, negative_prompt_embeds, "negative_prompt")
    if image is None:
      raise ValueError("provide `image`: the reference latents are encoded from it (`image_embeds` only replaces the "
                       "image encoder's output)")
    for name, v in (("pose_video", pose_video), ("face_video", face_video)):
      if v is None:
        raise ValueError(f"provide `{name}`")
      if not torch.is_tensor(v) or v.dim() != 5 or v.shape[2] == 0:
        raise ValueError(f"`{name}` must be a [B, 3, T, H, W] tensor with at least one frame")
    if pose_video.shape[2] != face_video.shape[2]:
      raise ValueError(f"`pose_video` has {pose_video.shape[2]} frames and `face_video` {face_video.shape[2]}")
    if mode not in ("animate", "replace"):
      raise ValueError(f"mode must be 'animate' or 'replace', got {mode!r}")
    if mode == "replace":
      for name, v in (("background_video", background_video), ("mask_video", mask_video)):
        if v is None:
          raise ValueError("`background_video` and `mask_video` are required for replace mode")
        if not torch.is_tensor(v) or v.dim() != 5 or v.shape[2] != pose_video.shape[2]:
          raise ValueError(f"`{name}` must be a 5-D tensor with the {pose_video.shape[2]} frames of `pose_video`")
    if height % 16 or width % 16:
      raise ValueError(f"`height` and `width` have to be divisible by 16 but are {height} and {width}")
    for name, v in (("prompt", prompt), ("negative_prompt", negative_prompt)):
      if v is not None and not isinstance(v, (str, list)):
        raise ValueError(f"`{name}` has to be a str or a list but is {type(v)}")
    if not isinstance(prev_segment_conditioning_frames, int) or prev_segment_conditioning_frames not in (1, 5):
      raise ValueError(f"`prev_segment_conditioning_frames` has to be 1 or 5, got {prev_segment_conditioning_frames!r}")

  @torch.no_grad()
  def __call__(self, image: torch.Tensor, pose_video: torch.Tensor, face_video: torch.Tensor,
               background_video: Optional[torch.Tensor] = None, mask_video: Optional[torch.Tensor] = None, prompt=None,
               negative_prompt=None, height: Optional[int] = None, width: Optional[int] = None,
               segment_frame_length: int = 77, prev_segment_conditioning_frames: int = 5,
               num_inference_steps: Optional[int] = None, guidance_scale: float = 1.0, mode: str = "animate",
               prompt_embeds=None, negative_prompt_embeds=None, image_embeds=None, generator=None,
               motion_encode_batch_size: Optional[int] = None, output_type: str = "uint8"):
    c = self.config
    height, width = height or int(c.get("height", 720)), width or int(c.get("width", 1280))
    steps = num_inference_steps or int(c.get("num_inference_steps", 20))
    self.check_inputs(image, pose_video, face_video, background_video, mask_video, prompt, negative_prompt, height, width,
                      prompt_embeds, negative_prompt_embeds, image_embeds, mode, prev_segment_conditioning_frames)
    s = self.vae_scale_factor_temporal
    if segment_frame_length % s != 1:
      segment_frame_length = max(1, segment_frame_length // s * s + 1)
    do_cfg = guidance_scale > 1.0
    if prompt_embeds is None:
      prompt_embeds = self.encode_prompt(prompt or c.get("prompt", ""), int(c.get("max_sequence_length", 512)))
    if do_cfg and negative_prompt_embeds is None:
      negative_prompt_embeds = self.encode_prompt(negative_prompt or c.get("negative_prompt", ""), int(c.get("max_sequence_length", 512)))
    prompt_embeds = prompt_embeds.to(self.device, self.dtype)
    B = prompt_embeds.shape[0]
    if image_embeds is None:
      image_embeds = self.encode_image(image) if self.image_encoder is not None else None
    embeds = torch.cat([prompt_embeds, negative_prompt_embeds.to(self.device, self.dtype)]) if do_cfg else prompt_embeds
    img_embeds = image_embeds
    if image_embeds is not None:
      image_embeds = image_embeds.to(self.device, self.dtype)
      img_embeds = torch.cat([image_embeds, image_embeds]) if do_cfg else image_embeds

    n_frames = pose_video.shape[2]
    eff = segment_frame_length - prev_segment_conditioning_frames
    last = (n_frames - prev_segment_conditioning_frames) % eff
    target = n_frames + (0 if last == 0 else eff - last)
    n_seg = max(1, target // eff)
    pose_video, face_video = pad_video_frames(pose_video, target), pad_video_frames(face_video, target)
    if mode == "replace":
      background_video, mask_video = pad_video_frames(background_video, target), pad_video_frames(mask_video, target)
    ref_latents = self.prepare_reference_image_latents(image, B)

    start, end, outs, prev_out = 0, segment_frame_length, [], None
    lt = (segment_frame_length - 1) // s + 1
    lh, lw = height // self.vae_scale_factor_spatial, width // self.vae_scale_factor_spatial
    z = self.vae.cfg.z_dim if self.vae is not None else 16
    for _ in range(n_seg):
      lat = torch.randn((B, z, lt + 1, lh, lw), generator=generator, dtype=torch.float32).to(self.device)
      pose_lat = self._encode(pose_video[:, :, start:end])
      if pose_lat.shape[0] == 1 and B > 1:
        pose_lat = pose_lat.expand(B, -1, -1, -1, -1)
      face_seg = face_video[:, :, start:end].to(self.device, self.dtype)
      if face_seg.shape[0] == 1 and B > 1:
        face_seg = face_seg.expand(B, -1, -1, -1, -1)
      prev = prev_out[:, :, -prev_segment_conditioning_frames:] if (start > 0 and prev_out is not None) else None
      bg = background_video[:, :, start:end] if mode == "replace" else None
      mk = mask_video[:, :, start:end] if mode == "replace" else None
      cond = self.prepare_prev_segment_cond_latents(prev, bg, mk, B, segment_frame_length, start, height, width,
                                                    prev_segment_conditioning_frames, mode)
      reference = torch.cat([ref_latents, cond], dim=2).to(self.dtype)           # [B, 20, lt+1, h, w]
      face_b = torch.cat([face_seg, face_seg * 0 - 1]) if do_cfg else face_seg
      motion = self.transformer.encode_face_motion(face_b, face_b.shape[0], motion_encode_batch_size)
      state = self.scheduler.set_timesteps(self.scheduler.create_state(), steps, lat.shape, device=self.device)
      for t in state.timesteps.tolist():
        x = torch.cat([lat.to(self.dtype), reference], dim=1)
        if do_cfg:
          x = torch.cat([x, x])
        ts = torch.full((x.shape[0],), float(t), device=self.device)
        pose_b = torch.cat([pose_lat, pose_lat]) if do_cfg else pose_lat
        out = self.transformer(x, ts, embeds, img_embeds, pose_hidden_states=pose_b.to(self.dtype),
                               face_motion_vec=motion).float()
        noise = OF.lincomb([out[:B], out[B:]], [guidance_scale, 1.0 - guidance_scale]) if do_cfg else out
        lat, state = self.scheduler.step(state, noise, t, lat)
      if output_type == "latent" and n_seg == 1:
        return lat
      prev_out = self.decode_latents(lat[:, :, 1:]).float().cpu()                   # [B, 3, T, H, W] in [-1, 1]
      outs.append(prev_out[:, :, prev_segment_conditioning_frames:] if start > 0 else prev_out)
      start, end = start + eff, end + eff
    video = torch.cat(outs, dim=2)[:, :, :n_frames]
    return postprocess_video(video) if output_type == "uint8" else video
