"""Z-Image text-to-image pipeline: Qwen3 text encoder -> flow-matching Euler loop over the DiT -> VAE decode.

Behaviour follows the reference (src/maxdiffusion/pipelines/z_image/z_image_pipeline.py):
  * prompts go through the tokenizer's chat template with thinking enabled, padded to `max_sequence_length`; the
    conditioning is the penultimate hidden state of Qwen3 with the padded positions dropped (:34-43, :147-195);
  * sigmas = shift * s / (1 + (shift - 1) s), s = linspace(1, 0, steps + 1); the model sees timestep 1 - sigma;
    update `latents += (sigma_next - sigma) * (-prediction)` with fp32 latents (:45-57, :197-200, :262-276);
  * decode `latents / scaling_factor + shift_factor` in chunks of `vae_decode_chunk` images (:104-117, :281-289).

The Euler update is one launch of the fused linear-combination kernel.
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence, Union

import torch

from ...ops import functional as OF


def shifted_sigmas(num_inference_steps: int, shift: float) -> torch.Tensor:
  s = torch.linspace(1.0, 0.0, num_inference_steps + 1, dtype=torch.float32)
  return shift * s / (1.0 + (shift - 1.0) * s)


class ZImagePipeline:

  def __init__(self, transformer, vae, tokenizer=None, text_encoder=None, dtype=torch.bfloat16, device=None,
               flow_shift: float = 3.0, offload_encoders: bool = False):
    self.transformer, self.vae, self.tokenizer, self.text_encoder = transformer, vae, tokenizer, text_encoder
    self.dtype = dtype
    self.device = torch.device(device) if device is not None else next(transformer.parameters()).device
    self.flow_shift = flow_shift
    self.offload_encoders = offload_encoders
    self.vae_scale_factor = 2 ** (len(vae.cfg.block_out_channels) - 1) if vae is not None else 8

  @torch.no_grad()
  def encode_prompt(self, prompt: Union[str, Sequence[str]], max_sequence_length: int = 512) -> List[torch.Tensor]:
    if self.tokenizer is None or self.text_encoder is None:
      raise ValueError("no text encoder loaded: pass `prompt_embeds`")
    prompts = [prompt] if isinstance(prompt, str) else list(prompt)
    chats = [self.tokenizer.apply_chat_template([{"role": "user", "content": p}], tokenize=False,
                                                add_generation_prompt=True, enable_thinking=True) for p in prompts]
    enc = self.tokenizer(chats, padding="max_length", max_length=max_sequence_length, truncation=True, return_tensors="pt")
    if self.offload_encoders:
      self.text_encoder.to(self.device)
    ids, mask = enc["input_ids"].to(self.device), enc["attention_mask"].to(self.device)
    _, hidden = self.text_encoder(ids, mask)
    if self.offload_encoders:
      self.text_encoder.to("cpu")
    emb = hidden[-2]
    return [emb[i][mask[i].bool()].to(self.dtype) for i in range(len(prompts))]

  @torch.no_grad()
  def denoise_step(self, latents, timestep, prompt_embeds, sigma_delta: float):
    """One Euler step; `latents` [B, C, H, W] fp32."""
    samples = [s[:, None] for s in latents.to(self.dtype)]
    preds = self.transformer(samples, timestep, prompt_embeds)
    pred = torch.stack([p[:, 0] for p in preds])
    return OF.lincomb([latents, pred], [1.0, -float(sigma_delta)], out_dtype=torch.float32)

  @torch.no_grad()
  def __call__(self, prompt=None, height: int = 1024, width: int = 1024, num_inference_steps: int = 9,
               guidance_scale: float = 0.0, seed: int = 0, max_sequence_length: int = 512, vae_decode_chunk: int = 1,
               output_type: str = "np", return_timings: bool = False, prompt_embeds: Optional[List[torch.Tensor]] = None,
               latents: Optional[torch.Tensor] = None):
    del guidance_scale  # the published configurations run without classifier-free guidance
    vae_scale = self.vae_scale_factor * 2
    if height % vae_scale or width % vae_scale:
      raise ValueError(f"height and width must be divisible by {vae_scale}")
    trace, t0 = {}, time.perf_counter()

    def stage(name):
      nonlocal t0
      if return_timings:
        if self.device.type == "cuda":
          torch.cuda.synchronize()
        trace[name] = time.perf_counter() - t0
        t0 = time.perf_counter()

    if prompt_embeds is None:
      prompt_embeds = self.encode_prompt(prompt, max_sequence_length)
    prompt_embeds = [e.to(self.device, self.dtype) for e in prompt_embeds]
    stage("text_encode")
    B = len(prompt_embeds)
    lh, lw = 2 * (height // vae_scale), 2 * (width // vae_scale)
    if latents is None:
      g = torch.Generator().manual_seed(int(seed))
      latents = torch.randn((B, self.transformer.cfg.in_channels, lh, lw), generator=g, dtype=torch.float32)
    latents = latents.to(self.device, torch.float32)
    sigmas = shifted_sigmas(num_inference_steps, self.flow_shift)
    for i in range(num_inference_steps):
      t = torch.full((B,), 1.0 - float(sigmas[i]), dtype=torch.float32, device=self.device)
      latents = self.denoise_step(latents, t, prompt_embeds, float(sigmas[i + 1] - sigmas[i]))
    stage("denoise")
    if output_type == "latent" or self.vae is None:
      return (latents, trace) if return_timings else latents
    chunk = max(1, int(vae_decode_chunk))
    vdtype = next(self.vae.parameters()).dtype
    decoded = torch.cat([self.vae.decode(self.vae.unscale_latents(latents[s:s + chunk]).to(vdtype))
                         for s in range(0, B, chunk)])
    stage("vae_decode")
    images = (decoded.float().permute(0, 2, 3, 1) / 2 + 0.5).clamp(0, 1)
    images = (images * 255).round().to(torch.uint8)
    stage("host_post")
    return (images, trace) if return_timings else images
