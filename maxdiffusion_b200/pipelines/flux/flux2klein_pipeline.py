"""Flux.2-Klein text-to-image pipeline (4B / 9B).

Behaviour follows the reference (src/maxdiffusion/pipelines/flux/flux2klein_pipeline.py):
  * prompts are wrapped in the Qwen3 chat template with an empty think block and padded to `max_sequence_length`;
    the conditioning is the concatenation of the hidden states of Qwen3 layers 9, 18 and 27 (:115-125, :452-460);
  * noise is drawn in the unpacked 32-channel latent space [B,32,H/8,W/8] and packed 2x2 into 128-channel tokens
    (:328-350); image ids (0, h, w, 0), text ids (0, 0, 0, i) (models/flux/util.py:353-378);
  * sigmas = linspace(1, 1/steps, steps) with exponential dynamic shift mu = compute_empirical_mu(seq, steps)
    (:413-421); Euler: latents += (sigma_next - sigma) * prediction, last sigma_next = 0 (:161-188);
  * decode: tokens * bn_std + bn_mean (the VAE's BatchNorm statistics over the 128 packed channels), unpack to
    32 channels, VAE decode, clip((x + 1) * 127.5) (:127-145, :603).
The Euler update is one launch of the fused linear-combination kernel.
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence, Union

import torch

from ...ops import functional as OF
from ...schedulers.scheduling_flow_match import FlowMatchScheduler, compute_empirical_mu

QWEN3_LAYERS = (9, 18, 27)


def prepare_text_ids(seq_len: int, device=None) -> torch.Tensor:
  ids = torch.zeros((seq_len, 4), device=device)
  ids[:, 3] = torch.arange(seq_len, device=device)
  return ids


def prepare_latent_image_ids(height: int, width: int, device=None) -> torch.Tensor:
  ids = torch.zeros((height, width, 4), device=device)
  ids[..., 1] = torch.arange(height, device=device)[:, None]
  ids[..., 2] = torch.arange(width, device=device)[None, :]
  return ids.reshape(-1, 4)


def pack_latents(x: torch.Tensor) -> torch.Tensor:
  """[B,32,H,W] -> tokens [B,(H/2)(W/2),128]; channel index = c*4 + dh*2 + dw."""
  B, C, H, W = x.shape
  x = x.reshape(B, C, H // 2, 2, W // 2, 2).permute(0, 1, 3, 5, 2, 4).reshape(B, C * 4, (H // 2) * (W // 2))
  return x.transpose(1, 2)


def unpack_latents(tokens: torch.Tensor, h_latent: int, w_latent: int) -> torch.Tensor:
  B = tokens.shape[0]
  x = tokens.reshape(B, h_latent // 2, w_latent // 2, 32, 2, 2).permute(0, 3, 1, 4, 2, 5)
  return x.reshape(B, 32, h_latent, w_latent)


class Flux2KleinPipeline:

  def __init__(self, transformer, vae, text_encoder=None, tokenizer=None, scheduler: Optional[FlowMatchScheduler] = None,
               vae_bn_mean: Optional[torch.Tensor] = None, vae_bn_std: Optional[torch.Tensor] = None, device=None,
               max_sequence_length: int = 512):
    self.transformer, self.vae, self.text_encoder, self.tokenizer = transformer, vae, text_encoder, tokenizer
    self.scheduler = scheduler or FlowMatchScheduler(num_train_timesteps=1000, shift=1.0, sigma_max=1.0, sigma_min=0.001,
                                                     use_dynamic_shifting=True, time_shift_type="exponential")
    self.device = torch.device(device) if device is not None else next(transformer.parameters()).device
    self.dtype = next(transformer.parameters()).dtype
    self.vae_bn_mean = vae_bn_mean if vae_bn_mean is not None else torch.zeros(128)
    self.vae_bn_std = vae_bn_std if vae_bn_std is not None else torch.ones(128)
    self.max_sequence_length = max_sequence_length

  @torch.no_grad()
  def encode_prompt(self, prompts: Sequence[str]) -> torch.Tensor:
    if self.text_encoder is None or self.tokenizer is None:
      raise ValueError("no text encoder loaded: pass `prompt_embeds`")
    if self.text_encoder.cfg.num_hidden_layers < max(QWEN3_LAYERS):
      raise ValueError("Flux.2-Klein conditions on Qwen3 layers 9, 18 and 27: the text encoder needs >= 27 layers")
    texts = [f"<|im_start|>user\n{p}<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n" for p in prompts]
    enc = self.tokenizer(texts, return_tensors="pt", padding="max_length", truncation=True, max_length=self.max_sequence_length)
    _, hidden = self.text_encoder(enc["input_ids"].to(self.device), enc["attention_mask"].to(self.device))
    out = torch.stack([hidden[i] for i in QWEN3_LAYERS], dim=1)                  # [B,3,T,D]
    return out.permute(0, 2, 1, 3).reshape(out.shape[0], out.shape[2], -1)

  @torch.no_grad()
  def __call__(self, prompt: Union[str, List[str], None] = None, height: int = 1024, width: int = 1024,
               num_inference_steps: int = 4, batch_size: int = 1, latents: Optional[torch.Tensor] = None, seed: int = 0,
               prompt_embeds: Optional[torch.Tensor] = None, output_type: str = "uint8", return_trace: bool = False):
    trace, t0 = {}, time.perf_counter()
    sync = (lambda: torch.cuda.synchronize()) if self.device.type == "cuda" else (lambda: None)
    if prompt_embeds is None:
      prompts = [prompt] * batch_size if isinstance(prompt, str) else list(prompt)
      prompt_embeds = self.encode_prompt(prompts)
    prompt_embeds = prompt_embeds.to(self.device, self.dtype)
    B = prompt_embeds.shape[0]
    sync()
    trace["prompt_encoding"] = time.perf_counter() - t0
    h_lat, w_lat = height // 8, width // 8
    if latents is None:
      g = torch.Generator().manual_seed(int(seed))
      latents = torch.randn((B, 32, h_lat, w_lat), generator=g, dtype=torch.float32)
    tokens = (pack_latents(latents) if latents.dim() == 4 else latents).to(self.device, torch.float32).contiguous()
    img_ids = prepare_latent_image_ids(h_lat // 2, w_lat // 2, self.device)
    txt_ids = prepare_text_ids(prompt_embeds.shape[1], self.device)
    mu = compute_empirical_mu(tokens.shape[1], num_inference_steps)
    sig = torch.linspace(1.0, 1.0 / num_inference_steps, num_inference_steps)
    state = self.scheduler.set_timesteps_ltx2(self.scheduler.create_state(), num_inference_steps, shift=mu, sigmas=sig)
    sigmas = torch.cat([state.sigmas.float().cpu(), torch.zeros(1)])
    t1 = time.perf_counter()
    for i in range(num_inference_steps):
      t = torch.full((B,), float(state.timesteps[i]) / 1000.0, device=self.device)
      pred = self.transformer(tokens.to(self.dtype), prompt_embeds, t, img_ids, txt_ids)
      tokens = OF.lincomb([tokens, pred], [1.0, float(sigmas[i + 1] - sigmas[i])], out_dtype=torch.float32)
    sync()
    trace["denoise_loop"] = time.perf_counter() - t1
    if output_type == "latent" or self.vae is None:
      return (tokens, trace) if return_trace else tokens
    t2 = time.perf_counter()
    z = tokens * self.vae_bn_std.to(tokens).view(1, 1, -1) + self.vae_bn_mean.to(tokens).view(1, 1, -1)
    z = unpack_latents(z, h_lat, w_lat)
    img = self.vae.decode(z.to(next(self.vae.parameters()).dtype)).float()
    img = ((img + 1.0) * 127.5).clamp(0, 255).to(torch.uint8).permute(0, 2, 3, 1)
    sync()
    trace["vae_decode"] = time.perf_counter() - t2
    return (img, trace) if return_trace else img
