"""Flux text-to-image pipeline (dev: 28 guided Euler steps, schnell: 4 steps).

Reference flow (src/maxdiffusion/generate_flux.py:80-172,277-490, pipelines/flux/flux_pipeline.py): CLIP pooled +
T5 embeddings -> packed 2x2 latents and position ids -> timesteps linspace(1, 0, N+1) shifted by the
resolution-dependent mu (:128-135,431-439) -> Euler loop `latents += (t_prev - t_curr) * v` -> unpack -> VAE decode.
Data parallelism replicates the loop per rank on its own batch slice; with `ici_fsdp_parallelism > 1` the weights
are sharded per block and gathered one block ahead (`parallel.fsdp.FSDPEngine` in inference mode).
"""
from __future__ import annotations

import math
import time
from typing import Optional

import torch

from ...models.flux.transformer_flux import (FLUX_PRESETS, FluxConfig, FluxTransformer2DModel, pack_latents,
                                             prepare_latent_image_ids, unpack_latents)
from ...models.vae import VAE_PRESETS, AutoencoderKL, VAEConfig
from ...parallel.mesh import create_device_mesh


def time_shift(mu: float, sigma: float, t: torch.Tensor) -> torch.Tensor:
  return math.exp(mu) / (math.exp(mu) + (1.0 / t - 1.0) ** sigma)


def compute_mu(seq_len: int, base_seq: int = 256, max_seq: int = 4096, base_shift: float = 0.5, max_shift: float = 1.15) -> float:
  """Linear interpolation of the shift in the image sequence length (reference: compute_empirical_mu / get_lin_function)."""
  m = (max_shift - base_shift) / (max_seq - base_seq)
  return m * seq_len + (base_shift - m * base_seq)


def flux_timesteps(num_steps: int, seq_len: int, shift: bool = True, base_shift: float = 0.5, max_shift: float = 1.15):
  t = torch.linspace(1.0, 0.0, num_steps + 1, dtype=torch.float64)
  if shift:
    mu = compute_mu(seq_len, base_shift=base_shift, max_shift=max_shift)
    t = torch.where(t > 0, time_shift(mu, 1.0, t.clamp_min(1e-12)), torch.zeros_like(t))
  return t.float()


class FluxPipeline:

  def __init__(self, config, transformer: FluxTransformer2DModel, vae: Optional[AutoencoderKL], clip=None, t5=None,
               clip_tokenizer=None, t5_tokenizer=None, mesh=None, device=None):
    self.config, self.transformer, self.vae = config, transformer, vae
    self.clip, self.t5, self.clip_tokenizer, self.t5_tokenizer = clip, t5, clip_tokenizer, t5_tokenizer
    self.mesh = mesh if mesh is not None else create_device_mesh(config)
    self.device = torch.device(device) if device is not None else next(transformer.parameters()).device
    self.dtype = next(transformer.parameters()).dtype
    self.engine = None
    # `offload_encoders`: CLIP and T5 wait in host memory and visit the GPU only while a prompt is encoded, so that
    # their 10 GB do not sit beside the transformer during the denoising loop (reference: src/maxdiffusion/generate_flux.py:384-386)
    self.offload_encoders = bool(config.get("offload_encoders", False)) and self.device.type == "cuda"
    if self.device.type == "cuda" and not self.offload_encoders:
      self.clip = self.clip.to(self.device) if self.clip is not None else None
      self.t5 = self.t5.to(self.device) if self.t5 is not None else None

  @classmethod
  def from_config(cls, config, device=None, load_vae: bool = True, **kw):
    device = torch.device(device) if device is not None else (
        torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    dtype = config.weights_dtype if device.type == "cuda" else torch.float32
    preset = dict(FLUX_PRESETS[str(config.get("flux_preset", "") or ("flux-schnell" if "schnell" in str(config.get("flux_name", "")) else "flux-dev"))])
    preset.update(config.get("flux_config_overrides", None) or {})
    torch.manual_seed(int(config.get("seed", 0)))
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
      with torch.device(device):
        transformer = FluxTransformer2DModel(FluxConfig(**preset))
    finally:
      torch.set_default_dtype(prev)
    vae = None
    if load_vae:
      vcfg = dict(VAE_PRESETS["flux"])
      vcfg.update(config.get("vae_config_overrides", None) or {})
      vae = AutoencoderKL(VAEConfig(**vcfg)).to(device=device, dtype=dtype)
    pipe = cls(config, transformer, vae, device=device, **kw)
    pipe.maybe_shard_weights()
    return pipe

  def maybe_shard_weights(self):
    """FSDP weight shard for inference: block weights live sharded and are gathered one block ahead."""
    group = self.mesh.group("fsdp")
    if group is None:
      return
    from ...parallel.fsdp import AdamWConfig, FSDPEngine

    blocks = self.transformer.blocks
    ids = {id(p) for b in blocks for p in b.parameters()}
    root = [p for p in self.transformer.parameters() if id(p) not in ids]
    self.engine = FSDPEngine(blocks, root, AdamWConfig(), group=group, device=self.device, param_dtype=self.dtype,
                             train=False)
    self.transformer.block_hook = self.engine.block_hook

  def encode_prompt(self, prompt, prompt_2=None, max_sequence_length: int = 512):
    if self.clip is None or self.t5 is None:
      raise ValueError("no text encoders loaded: pass prompt_embeds and pooled_prompt_embeds")
    prompts = [prompt] if isinstance(prompt, str) else list(prompt)
    p2 = prompts if prompt_2 is None else ([prompt_2] if isinstance(prompt_2, str) else list(prompt_2))
    if self.offload_encoders:
      self.clip, self.t5 = self.clip.to(self.device), self.t5.to(self.device)
    with torch.no_grad():
      ids = self.clip_tokenizer(prompts, padding="max_length", max_length=77, truncation=True, return_tensors="pt").input_ids
      pooled = self.clip(ids.to(next(self.clip.parameters()).device)).pooler_output
      ids2 = self.t5_tokenizer(p2, padding="max_length", max_length=max_sequence_length, truncation=True, return_tensors="pt").input_ids
      embeds = self.t5(ids2.to(next(self.t5.parameters()).device)).last_hidden_state
    embeds, pooled = embeds.to(self.device, self.dtype), pooled.to(self.device, self.dtype)
    if self.offload_encoders:
      self.clip, self.t5 = self.clip.to("cpu"), self.t5.to("cpu")
      if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return embeds, pooled

  @torch.no_grad()
  def __call__(self, prompt=None, prompt_2=None, height: Optional[int] = None, width: Optional[int] = None,
               num_inference_steps: Optional[int] = None, guidance_scale: Optional[float] = None, prompt_embeds=None,
               pooled_prompt_embeds=None, latents=None, generator=None, output_type: str = "uint8",
               return_trace: bool = False):
    c = self.config
    height = height or int(c.get("resolution", 1024))
    width = width or int(c.get("resolution", 1024))
    steps = num_inference_steps or int(c.get("num_inference_steps", 28))
    guidance_scale = float(guidance_scale if guidance_scale is not None else c.get("guidance_scale", 3.5))
    if prompt_embeds is None:
      prompt_embeds, pooled_prompt_embeds = self.encode_prompt(prompt or c.get("prompt", ""), prompt_2,
                                                               int(c.get("max_sequence_length", 512)))
    B = prompt_embeds.shape[0]
    lh, lw = height // 8, width // 8
    ch = self.transformer.cfg.in_channels // 4
    if latents is None:
      g = generator or torch.Generator().manual_seed(int(c.get("seed", 0)))
      latents = torch.randn((B, ch, lh, lw), generator=g, dtype=torch.float32, device=g.device)
    x = pack_latents(latents.to(self.device))
    img_ids = prepare_latent_image_ids(lh // 2, lw // 2, self.device)
    txt_ids = torch.zeros((prompt_embeds.shape[1], 3), device=self.device)
    ts = flux_timesteps(steps, x.shape[1], shift=bool(c.get("time_shift", True)), base_shift=float(c.get("base_shift", 0.5)),
                        max_shift=float(c.get("max_shift", 1.15))).to(self.device)
    guidance = torch.full((B,), guidance_scale, device=self.device) if self.transformer.cfg.guidance_embeds else None
    pe, pp = prompt_embeds.to(self.device, self.dtype), pooled_prompt_embeds.to(self.device, self.dtype)
    trace = {}
    ev = None
    if self.device.type == "cuda":
      torch.cuda.synchronize()
      ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
      ev[0].record()  # the loop is timed on the device, by events on the launching stream
    t0 = time.perf_counter()
    for i in range(steps):
      t_vec = ts[i].expand(B)
      v = self.transformer(x.to(self.dtype), pe, pp, t_vec, img_ids, txt_ids, guidance)
      x = x + (ts[i + 1] - ts[i]) * v.float()
    if ev is not None:
      ev[1].record()
      torch.cuda.synchronize()
    trace["denoise_total"] = ev[0].elapsed_time(ev[1]) / 1e3 if ev is not None else time.perf_counter() - t0
    lat = unpack_latents(x, lh, lw)
    if output_type == "latent" or self.vae is None:
      return (lat, trace) if return_trace else lat
    img = self.vae.decode(self.vae.unscale_latents(lat.to(next(self.vae.parameters()).dtype)))
    if output_type == "uint8":
      img = ((img.float() / 2 + 0.5).clamp(0, 1) * 255).round().to(torch.uint8).permute(0, 2, 3, 1).contiguous()
    return (img, trace) if return_trace else img
