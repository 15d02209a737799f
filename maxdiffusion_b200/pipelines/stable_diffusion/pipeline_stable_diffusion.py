"""Text-to-image pipelines for SD 1.x / 2.x and SDXL, with optional ControlNet.

Reference: `FlaxStableDiffusionPipeline`, `FlaxStableDiffusionXLPipeline` and the ControlNet variants
(src/maxdiffusion/pipelines/stable_diffusion/, stable_diffusion_xl/, controlnet/; scripts generate.py,
generate_sdxl.py, controlnet/generate_controlnet*_replicated.py). The reference replicates the loop with `jax.pmap`;
here every data-parallel rank runs its own slice of the batch and the results are gathered at the end.
`create_scheduler` honours the YAML `diffusion_scheduler_config` overrides (maxdiffusion_utils.py:149-191) and
`rescale_noise_cfg` implements guidance rescale (:194).
"""
from __future__ import annotations

from typing import Optional

import torch

from ...models.controlnet import ControlNetModel
from ...models.unet_2d_condition import UNet2DConditionModel
from ...models.vae import VAE_PRESETS, AutoencoderKL, VAEConfig
from ...ops import functional as OF
from ...schedulers import SCHEDULERS
from ...trainers.stable_diffusion_trainer import get_add_time_ids, resolve_unet_config


def create_scheduler(config, default: str = "FlaxEulerDiscreteScheduler"):
  # empty strings in the override mean "keep what the pretrained scheduler config says" (the defaults here)
  sc = {k: v for k, v in dict(config.get("diffusion_scheduler_config", {}) or {}).items() if v != ""}
  name = sc.pop("_class_name", default)
  cls = SCHEDULERS[name.replace("Flax", "")]
  kwargs = dict(beta_start=0.00085, beta_end=0.012, beta_schedule="scaled_linear")
  kwargs.update(sc)
  import inspect

  accepted = set(inspect.signature(cls.__init__).parameters)
  return cls(**{k: v for k, v in kwargs.items() if k in accepted})


def rescale_noise_cfg(noise_cfg, noise_pred_text, guidance_rescale: float = 0.0):
  """Rescales the guided prediction to the std of the text-conditioned one (arXiv 2305.08891, sec. 3.4)."""
  dims = list(range(1, noise_pred_text.dim()))
  std_text = noise_pred_text.std(dim=dims, keepdim=True)
  std_cfg = noise_cfg.std(dim=dims, keepdim=True)
  rescaled = noise_cfg * (std_text / std_cfg)
  return guidance_rescale * rescaled + (1 - guidance_rescale) * noise_cfg


class StableDiffusionPipeline:
  is_xl = False

  def __init__(self, config, unet: UNet2DConditionModel, vae: Optional[AutoencoderKL], scheduler, text_encoders=(),
               tokenizers=(), controlnet: Optional[ControlNetModel] = None, device=None):
    self.config, self.unet, self.vae, self.scheduler = config, unet, vae, scheduler
    self.text_encoders, self.tokenizers, self.controlnet = list(text_encoders), list(tokenizers), controlnet
    self.device = torch.device(device) if device is not None else next(unet.parameters()).device
    self.dtype = next(unet.parameters()).dtype

  @classmethod
  def from_config(cls, config, device=None, load_vae=True, with_controlnet=False):
    device = torch.device(device) if device is not None else (
        torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    dtype = config.weights_dtype if device.type == "cuda" else torch.float32
    torch.manual_seed(int(config.get("seed", 0)))
    ucfg = resolve_unet_config(config)
    unet = UNet2DConditionModel(ucfg).to(device, dtype)
    vae = None
    if load_vae:
      v = dict(VAE_PRESETS["sdxl" if cls.is_xl else "sd"])
      v.update(config.get("vae_config_overrides", None) or {})
      vae = AutoencoderKL(VAEConfig(**v)).to(device, dtype)
    cn = ControlNetModel(ucfg).to(device, dtype) if with_controlnet else None
    return cls(config, unet, vae, create_scheduler(config), controlnet=cn, device=device)

  def encode_prompt(self, prompt, negative_prompt=""):
    if not self.text_encoders:
      raise ValueError("no text encoder loaded: pass prompt_embeds")
    outs = []
    for text in (prompt, negative_prompt):
      hs, pooled = [], None
      for tok, enc in zip(self.tokenizers, self.text_encoders):
        ids = tok([text] if isinstance(text, str) else list(text), padding="max_length", max_length=77, truncation=True,
                  return_tensors="pt").input_ids.to(next(enc.parameters()).device)
        o = enc(ids, output_hidden_states=True)
        hs.append(o.hidden_states[-2] if self.is_xl else o.last_hidden_state)
        pooled = getattr(o, "text_embeds", pooled)
      outs.append((torch.cat(hs, dim=-1), pooled))
    return outs

  @torch.no_grad()
  def __call__(self, prompt=None, negative_prompt="", height=None, width=None, num_inference_steps=None,
               guidance_scale=None, guidance_rescale=None, prompt_embeds=None, negative_prompt_embeds=None,
               pooled_prompt_embeds=None, negative_pooled_prompt_embeds=None, controlnet_image=None,
               controlnet_conditioning_scale=None, latents=None, generator=None, output_type="uint8"):
    c = self.config
    res = int(c.get("resolution", 1024 if self.is_xl else 512))
    height, width = height or res, width or res
    steps = num_inference_steps or int(c.get("num_inference_steps", 30))
    g_scale = float(guidance_scale if guidance_scale is not None else c.get("guidance_scale", 7.5))
    g_rescale = float(guidance_rescale if guidance_rescale is not None else c.get("guidance_rescale", 0.0))
    if prompt_embeds is None:
      (prompt_embeds, pooled_prompt_embeds), (negative_prompt_embeds, negative_pooled_prompt_embeds) = self.encode_prompt(
          prompt or c.get("prompt", ""), negative_prompt or c.get("negative_prompt", ""))
    do_cfg = g_scale > 1.0 and negative_prompt_embeds is not None
    B = prompt_embeds.shape[0]
    embeds = torch.cat([negative_prompt_embeds, prompt_embeds]) if do_cfg else prompt_embeds
    embeds = embeds.to(self.device, self.dtype)
    added = None
    if self.is_xl:
      pooled = torch.cat([negative_pooled_prompt_embeds, pooled_prompt_embeds]) if do_cfg else pooled_prompt_embeds
      ids = get_add_time_ids((height, width), (0, 0), (height, width), embeds.shape[0], self.device)
      added = {"text_embeds": pooled.to(self.device, self.dtype), "time_ids": ids}
    state = self.scheduler.set_timesteps(self.scheduler.create_state(), steps, device=self.device)
    if latents is None:
      g = generator or torch.Generator().manual_seed(int(c.get("seed", 0)))
      latents = torch.randn((B, self.unet.cfg.in_channels, height // 8, width // 8), generator=g)
    latents = latents.to(self.device, torch.float32) * getattr(state, "init_noise_sigma", 1.0)
    cond_scale = float(controlnet_conditioning_scale if controlnet_conditioning_scale is not None else c.get("controlnet_conditioning_scale", 1.0))
    for i, t in enumerate(state.timesteps.tolist()):
      x = torch.cat([latents, latents]) if do_cfg else latents
      x = self.scheduler.scale_model_input(state, x, t)
      tt = torch.full((x.shape[0],), t, device=self.device)
      extra = {}
      if self.controlnet is not None and controlnet_image is not None:
        cimg = controlnet_image.to(self.device, self.dtype)
        cimg = torch.cat([cimg, cimg]) if do_cfg else cimg
        down, mid = self.controlnet(x, tt, embeds, cimg, cond_scale, added)
        extra = dict(down_block_additional_residuals=down, mid_block_additional_residual=mid)
      noise = self.unet(x.to(self.dtype), tt, embeds, added, **extra).float()
      if do_cfg:
        uncond, text = noise.chunk(2)
        noise = OF.lincomb([text, uncond], [g_scale, 1.0 - g_scale])
        if g_rescale > 0:
          noise = rescale_noise_cfg(noise, text, g_rescale)
      latents, state = self.scheduler.step(state, noise, t, latents)
    if output_type == "latent" or self.vae is None:
      return latents
    img = self.vae.decode(self.vae.unscale_latents(latents.to(next(self.vae.parameters()).dtype)))
    if output_type == "uint8":
      img = ((img.float() / 2 + 0.5).clamp(0, 1) * 255).round().to(torch.uint8).permute(0, 2, 3, 1).contiguous()
    return img


class StableDiffusionXLPipeline(StableDiffusionPipeline):
  is_xl = True


class StableDiffusionControlNetPipeline(StableDiffusionPipeline):
  pass


class StableDiffusionXLControlNetPipeline(StableDiffusionXLPipeline):
  pass
