"""LTX-Video pipeline: T5 text conditioning, rectified-flow sampling with per-step CFG / STG schedules, timestep
conditioned VAE decode, and the two-pass multi-scale wrapper.

Behaviour follows the reference (src/maxdiffusion/pipelines/ltx_video/ltx_video_pipeline.py):
  * latents [B,128,F',H/32,W/32] are patchified with patch 1 into tokens; positions are the latent coordinates scaled
    to pixels / seconds: frame index * 8 (causal: the first frame counts once) / frame_rate, y * 32, x * 32
    (`get_latent_spatial_position`, :533-579; `prepare_latents` :408-444);
  * `guidance_timesteps` maps every sampling step to an entry of the per-phase lists `guidance_scale`, `stg_scale`,
    `rescaling_scale`, `skip_block_list` (:700-770); conditions are batched [uncond?, cond, perturbed?];
  * one step (`run_inference` :959-1062): optional CFG-star rescale of the unconditional branch by
    <cond, uncond> / |uncond|^2, CFG, `+ stg * (cond - perturbed)`, std-rescaling towards the conditional branch,
    rectified-flow Euler step; `skip_initial/final_inference_steps` trim the schedule (:640-700);
  * decode with `decode_timestep` / `decode_noise_scale` noise injection (:850-890);
  * `LTXMultiScalePipeline` (:1140-1296): first pass at `downscale_factor`, latent up-sampler + AdaIN, second pass at
    2x the first-pass resolution starting from the up-sampled latents at a late timestep, bilinear resize to the target.
"""
from __future__ import annotations

from dataclasses import dataclass

import time
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from ...models.ltx2.latent_upsampler_ltx2 import adain_filter_latent
from ...models.ltx_video.transformer3d import SkipLayerStrategy
from ...ops import functional as OF
from ...schedulers.scheduling_rectified_flow import RectifiedFlowMultistepScheduler

STG_MODES = {"attention_values": SkipLayerStrategy.AttentionValues, "attention_skip": SkipLayerStrategy.AttentionSkip,
             "residual": SkipLayerStrategy.Residual, "transformer_block": SkipLayerStrategy.TransformerBlock,
             "stg_av": SkipLayerStrategy.AttentionValues, "stg_as": SkipLayerStrategy.AttentionSkip,
             "stg_r": SkipLayerStrategy.Residual, "stg_t": SkipLayerStrategy.TransformerBlock}


def _per_step(values, guidance_timesteps, timesteps):
  """Picks, for every sampling timestep, the entry of the phase whose `guidance_timesteps` value is nearest above."""
  if not isinstance(values, (list, tuple)):
    return [values] * len(timesteps)
  if guidance_timesteps is None or len(values) == 1:
    return [values[0]] * len(timesteps) if len(values) == 1 else list(values)
  gt = torch.tensor(list(guidance_timesteps), dtype=torch.float64)
  out = []
  for t in timesteps:
    idx = int(torch.argmin((gt - float(t)).abs()))
    out.append(values[idx])
  return out


@dataclass
class ConditioningItem:
  """A frame or clip the generated video must contain: `media_item` [B,3,F,H,W] in [-1,1] (F = 1 + 8k), the frame
  number it starts at, the strength (1 = keep exactly), and an optional top-left position when it is smaller than the
  frame (reference: src/maxdiffusion/pipelines/ltx_video/ltx_video_pipeline.py:72-88)."""
  media_item: torch.Tensor
  media_frame_number: int = 0
  conditioning_strength: float = 1.0
  media_x: Optional[int] = None
  media_y: Optional[int] = None


class LTXVideoPipeline:

  def __init__(self, transformer, vae, text_encoder=None, tokenizer=None, scheduler=None, device=None):
    self.transformer, self.vae, self.text_encoder, self.tokenizer = transformer, vae, text_encoder, tokenizer
    self.scheduler = scheduler or RectifiedFlowMultistepScheduler(shifting="SD3")
    self.device = torch.device(device) if device is not None else next(transformer.parameters()).device
    self.dtype = next(transformer.parameters()).dtype
    self.spatial_ratio = vae.cfg.spatial_compression_ratio if vae is not None else 32
    self.temporal_ratio = vae.cfg.temporal_compression_ratio if vae is not None else 8

  @torch.no_grad()
  def encode_prompt(self, prompt, negative_prompt="", max_sequence_length: int = 512):
    if self.text_encoder is None:
      raise ValueError("no text encoder loaded: pass prompt_embeds")
    def enc(texts):
      tok = self.tokenizer(texts, padding="max_length", max_length=max_sequence_length, truncation=True, return_tensors="pt")
      dev = next(self.text_encoder.parameters()).device
      h = self.text_encoder(tok.input_ids.to(dev), attention_mask=tok.attention_mask.to(dev))[0]
      return h.to(self.device, self.dtype), tok.attention_mask.to(self.device)
    prompts = [prompt] if isinstance(prompt, str) else list(prompt)
    e, m = enc(prompts)
    ne, nm = enc([negative_prompt] * len(prompts) if isinstance(negative_prompt, str) else list(negative_prompt))
    return e, m, ne, nm

  def latent_positions(self, batch, lf, lh, lw, frame_rate: float):
    """indices_grid [B, 3, N]: seconds, pixel rows, pixel columns of every latent token."""
    f, y, x = torch.meshgrid(torch.arange(lf), torch.arange(lh), torch.arange(lw), indexing="ij")
    t_pix = (f * self.temporal_ratio + 1 - self.temporal_ratio).clamp(min=0).float() / frame_rate
    grid = torch.stack([t_pix, y.float() * self.spatial_ratio, x.float() * self.spatial_ratio]).reshape(3, -1)
    return grid[None].repeat(batch, 1, 1).to(self.device)

  def latent_spatial_position(self, latents, item: ConditioningItem, height: int, width: int, strip_latent_border: bool = True):
    """Where the item's latents go in the latent frame; latent borders that do not coincide with a frame border are
    dropped, because they were computed from padding (reference: `get_latent_spatial_position` :533-579)."""
    r = self.spatial_ratio
    h, w = item.media_item.shape[-2:]
    if h > height or w > width or h % r or w % r:
      raise ValueError(f"conditioning item {h}x{w} must fit {height}x{width} and be a multiple of {r}")
    x0 = (width - w) // 2 if item.media_x is None else item.media_x
    y0 = (height - h) // 2 if item.media_y is None else item.media_y
    if strip_latent_border:
      xs, xe = (1 if x0 > 0 else 0), (-1 if x0 + w < width else None)
      ys, ye = (1 if y0 > 0 else 0), (-1 if y0 + h < height else None)
      latents = latents[..., ys:ye, xs:xe]
      x0, y0 = x0 + (r if x0 > 0 else 0), y0 + (r if y0 > 0 else 0)
    return latents, x0 // r, y0 // r

  @torch.no_grad()
  def prepare_conditioning(self, init_latents, items: Sequence[ConditioningItem], height: int, width: int, num_frames: int,
                           generator=None):
    """Blends the VAE latents of every item into `init_latents` [B,C,lf,lh,lw] and returns them with the conditioning
    mask [B,lf,lh,lw] holding each token's strength (0 = free). Items start at frame 0 (the reference handles no
    other case either: `prepare_conditioning` :446-531)."""
    mask = torch.zeros_like(init_latents[:, 0])
    vp = next(self.vae.parameters())
    for item in items:
      m = item.media_item
      n = m.shape[2]
      if n % self.temporal_ratio != 1:
        raise ValueError(f"a conditioning item needs 1 + {self.temporal_ratio}k frames, got {n}")
      if item.media_frame_number != 0:
        raise NotImplementedError("conditioning items must start at frame 0")
      if item.media_frame_number + n > num_frames:
        raise ValueError("the conditioning item does not fit into the video")
      if m.shape[-2:] != (height, width) and item.media_x is None and item.media_y is None:
        flat = m.permute(0, 2, 1, 3, 4).reshape(-1, m.shape[1], *m.shape[-2:])
        flat = torch.nn.functional.interpolate(flat.float(), size=(height, width), mode="bilinear", align_corners=False)
        m = flat.reshape(m.shape[0], n, m.shape[1], height, width).permute(0, 2, 1, 3, 4)
        item = ConditioningItem(m, item.media_frame_number, item.conditioning_strength)
      mean, _ = self.vae.encode(m.to(vp.device, vp.dtype))
      z = self.vae.normalize_latents(mean).to(init_latents)
      z, lx, ly = self.latent_spatial_position(z, item, height, width)
      _, _, fl, hl, wl = z.shape
      s = float(item.conditioning_strength)
      sl = (slice(None), slice(None), slice(0, fl), slice(ly, ly + hl), slice(lx, lx + wl))
      init_latents[sl] = (1 - s) * init_latents[sl] + s * z
      mask[:, :fl, ly:ly + hl, lx:lx + wl] = s
    return init_latents, mask

  @torch.no_grad()
  def __call__(self, prompt=None, negative_prompt="", height: int = 512, width: int = 704, num_frames: int = 121,
               frame_rate: float = 30.0, num_inference_steps: int = 30, guidance_scale=3.0, stg_scale=0.0,
               rescaling_scale=1.0, guidance_timesteps: Optional[Sequence[float]] = None, skip_block_list=None,
               skip_layer_strategy: Optional[SkipLayerStrategy] = None, skip_initial_inference_steps: int = 0,
               skip_final_inference_steps: int = 0, cfg_star_rescale: bool = False, latents=None, seed: int = 0,
               prompt_embeds=None, prompt_attention_mask=None, negative_prompt_embeds=None,
               negative_prompt_attention_mask=None, decode_timestep: float = 0.05, decode_noise_scale: float = 0.025,
               output_type: str = "uint8", max_sequence_length: int = 512, return_trace: bool = False,
               conditioning_items: Optional[Sequence[ConditioningItem]] = None, image_cond_noise_scale: float = 0.0,
               per_token_timestep: bool = False):
    r, rt = self.spatial_ratio, self.temporal_ratio
    if height % r or width % r:
      raise ValueError(f"`height` and `width` have to be divisible by {r} but are {height} and {width}.")
    trace, t0 = {}, time.perf_counter()
    if prompt_embeds is None:
      prompt_embeds, prompt_attention_mask, negative_prompt_embeds, negative_prompt_attention_mask = self.encode_prompt(
          prompt, negative_prompt, max_sequence_length)
    B = prompt_embeds.shape[0]
    lf, lh, lw = (num_frames - 1) // rt + 1, height // r, width // r
    C = self.transformer.cfg.in_channels
    g = torch.Generator().manual_seed(int(seed))
    noise = torch.randn((B, C, lf, lh, lw), generator=g, dtype=torch.float32)
    state = self.scheduler.set_timesteps(self.scheduler.create_state(), num_inference_steps, samples_shape=(B, lf * lh * lw, C))
    timesteps = state.timesteps.tolist()
    if skip_initial_inference_steps or skip_final_inference_steps:
      timesteps = timesteps[skip_initial_inference_steps:len(timesteps) - skip_final_inference_steps]
      state = self.scheduler.set_timesteps(self.scheduler.create_state(), len(timesteps), timesteps=timesteps)
    if latents is not None:  # second pass: the given latents are noised to the first retained timestep
      t_start = float(timesteps[0])
      x = (1 - t_start) * latents.float() + t_start * noise.to(latents.device)
    else:
      x = noise
    cond_mask = init_tokens = None
    if conditioning_items:
      x, cm = self.prepare_conditioning(x.clone(), conditioning_items, height, width, num_frames)
      cond_mask = cm.reshape(B, lf * lh * lw).to(self.device)
    tokens = x.to(self.device).permute(0, 2, 3, 4, 1).reshape(B, lf * lh * lw, C).contiguous()
    if cond_mask is not None:
      init_tokens = tokens.clone()
    grid = self.latent_positions(B, lf, lh, lw, frame_rate)

    gs = _per_step(guidance_scale, guidance_timesteps, timesteps)
    ss = _per_step(stg_scale, guidance_timesteps, timesteps)
    rs = _per_step(rescaling_scale, guidance_timesteps, timesteps)
    if skip_block_list and isinstance(skip_block_list[0], (list, tuple)):
      sb = _per_step(list(skip_block_list), guidance_timesteps, timesteps)
    else:
      sb = [skip_block_list] * len(timesteps)
    do_cfg, do_stg = any(v > 1.0 for v in gs), any(v > 0.0 for v in ss)
    num_conds = 1 + int(do_cfg) + int(do_stg)
    e, m = prompt_embeds.to(self.device, self.dtype), prompt_attention_mask
    embeds = ([negative_prompt_embeds.to(self.device, self.dtype)] if do_cfg else []) + [e] + ([e] if do_stg else [])
    masks = None
    if m is not None:
      masks = torch.cat(([negative_prompt_attention_mask] if do_cfg else []) + [m] + ([m] if do_stg else [])).to(self.device)
    embeds = torch.cat(embeds)
    trace["conditioning"] = time.perf_counter() - t0
    t1 = time.perf_counter()
    for i, t in enumerate(timesteps):
      if cond_mask is not None and image_cond_noise_scale > 0.0:
        # fully conditioned tokens get a little timestep-dependent noise so that motion can start from them
        # (reference: `add_noise_to_image_conditioning_latents_jax` :918-935)
        hard = (cond_mask > 1.0 - 1e-6)[..., None]
        n = torch.randn(tokens.shape, generator=g).to(tokens)
        tokens = torch.where(hard, init_tokens + image_cond_noise_scale * n * float(t) ** 2, tokens)
      x_in = tokens.repeat(num_conds, 1, 1).to(self.dtype)
      sm = None
      if do_stg and sb[i]:
        # the perturbed condition is the last of the `num_conds` groups
        sm = torch.ones((self.transformer.cfg.num_layers, B * num_conds))
        for blk in sb[i]:
          sm[blk, (num_conds - 1) * B:] = 0
      ts = torch.full((B * num_conds,), float(t), device=self.device)
      if cond_mask is not None and per_token_timestep:
        # conditioned tokens are presented at their own (lower) noise level; the reference keeps one scalar per sample
        ts = torch.minimum(ts[:, None], (1.0 - cond_mask).repeat(num_conds, 1))
      pred = self.transformer(x_in, grid.repeat(num_conds, 1, 1), embeds, ts, masks, sm, skip_layer_strategy).float()
      chunks = pred.chunk(num_conds)
      cond = chunks[1] if do_cfg else chunks[0]
      out = cond
      if do_cfg:
        uncond = chunks[0]
        if cfg_star_rescale:
          pf, nf = cond.reshape(B, -1), uncond.reshape(B, -1)
          alpha = ((pf * nf).sum(1, keepdim=True) / ((nf ** 2).sum(1, keepdim=True) + 1e-8)).view(B, 1, 1)
          uncond = alpha * uncond
        out = uncond + gs[i] * (cond - uncond)
      if do_stg:
        out = out + ss[i] * (cond - chunks[-1])
        if ss[i] > 0.0 and rs[i] != 1.0:
          factor = cond.reshape(B, -1).std(dim=1, keepdim=True) / out.reshape(B, -1).std(dim=1, keepdim=True)
          out = out * (rs[i] * factor + (1 - rs[i])).view(B, 1, 1)
      new_tokens, state = self.scheduler.step(state, out, t, tokens)
      if cond_mask is not None:  # a token is only denoised once the schedule has passed its conditioning level
        free = (float(t) - 1e-6 < (1.0 - cond_mask))[..., None]
        new_tokens = torch.where(free, new_tokens, tokens)
      tokens = new_tokens
    if self.device.type == "cuda":
      torch.cuda.synchronize()
    trace["denoise"] = time.perf_counter() - t1
    lat = tokens.reshape(B, lf, lh, lw, C).permute(0, 4, 1, 2, 3)
    if output_type == "latent" or self.vae is None:
      return (lat, trace) if return_trace else lat
    vdtype = next(self.vae.parameters()).dtype
    z = self.vae.denormalize_latents(lat.to(vdtype))
    temb = None
    if self.vae.cfg.timestep_conditioning:
      z = (1 - decode_noise_scale) * z + decode_noise_scale * torch.randn(z.shape, generator=g).to(z)
      temb = torch.full((B,), float(decode_timestep), device=self.device, dtype=vdtype)
    video = self.vae.decode(z, temb)
    if output_type == "uint8":
      video = ((video.float() / 2 + 0.5).clamp(0, 1) * 255).round().to(torch.uint8).permute(0, 2, 3, 4, 1)
    return (video, trace) if return_trace else video


class LTXMultiScalePipeline:

  def __init__(self, video_pipeline: LTXVideoPipeline, latent_upsampler):
    self.video_pipeline, self.latent_upsampler = video_pipeline, latent_upsampler

  @torch.no_grad()
  def __call__(self, height, width, num_frames, first_pass: dict, second_pass: dict, downscale_factor: float = 2 / 3,
               output_type: str = "uint8", **common):
    vp = self.video_pipeline
    r = vp.spatial_ratio
    h1 = int(height * downscale_factor) // r * r
    w1 = int(width * downscale_factor) // r * r
    lat = vp(height=h1, width=w1, num_frames=num_frames, output_type="latent", **{**common, **first_pass})
    z = vp.vae.denormalize_latents(lat.float())
    up = self.latent_upsampler(z.to(next(self.latent_upsampler.parameters()).dtype)).float()
    up = vp.vae.normalize_latents(adain_filter_latent(up, z))
    video = vp(height=h1 * 2, width=w1 * 2, num_frames=num_frames, latents=up, output_type="float" if output_type != "latent" else "latent",
               **{**common, **second_pass})
    if output_type == "latent":
      return video
    B, C, Fr = video.shape[:3]
    v = F.interpolate(video.permute(0, 2, 1, 3, 4).reshape(B * Fr, C, *video.shape[3:]).float(), size=(height, width),
                      mode="bilinear", align_corners=False).reshape(B, Fr, C, height, width).permute(0, 2, 1, 3, 4)
    if output_type == "uint8":
      return ((v / 2 + 0.5).clamp(0, 1) * 255).round().to(torch.uint8).permute(0, 2, 3, 4, 1)
    return v
