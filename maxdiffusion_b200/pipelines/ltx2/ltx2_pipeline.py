"""LTX-2 joint audio + video generation pipeline.

Behaviour follows the reference (src/maxdiffusion/pipelines/ltx2/ltx2_pipeline.py):
  * prompts -> Gemma-3 hidden states of all layers -> feature extractor -> video / audio connectors (:1143-1363);
  * video latents [B,128,F',H/32,W/32] packed to tokens, audio latents [B,8,T_a,mel/4] packed to [B,T_a,8*mel/4];
    T_a = round(num_frames / fps * sample_rate / hop / 4) (:1420-1773, :1879-1900);
  * sigmas = linspace(1, 1/steps, steps) through the exponential dynamic shift with
    mu = calculate_shift(min(6144, video tokens)) and the terminal stretch (:1901-1921);
  * guidance (`apply_ltx2_guidance`, :166-251): plain CFG on two branches, or — with spatio-temporal guidance — a
    four-way batch [uncond, cond, perturbed, isolated] combined in x0 space:
        x0 = x0_text + (g - 1)(x0_text - x0_uncond) + stg (x0_text - x0_perturbed) + (m - 1)(x0_text - x0_isolated)
    optionally rescaled towards the std of x0_text (`rescale_noise_cfg`, :131-147); audio uses its own scales;
    the perturbed branch carries `perturbation_mask = 0`, the isolated branch `modality_mask = 0` (:2460-2470);
  * the loop reuses the text K/V cache, the rotary tables and the per-step time embeddings (:2380-2415, :2499-2688);
  * decode: un-pack, de-normalise, optional latent up-sampler + AdaIN / tone-map filters, video VAE (timestep
    conditioned when the VAE asks for it), audio VAE -> mel -> vocoder -> waveform (:1488-1570, :2300-2380).
The per-step latent update is the fused linear-combination kernel.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Sequence, Union

import torch

from ...models.ltx2.latent_upsampler_ltx2 import adain_filter_latent, tone_map_latents
from ...ops import functional as OF
from ...schedulers.scheduling_flow_match import FlowMatchScheduler


@dataclass
class LTX2PipelineOutput:
  frames: torch.Tensor
  audio: Optional[torch.Tensor] = None
  timings: Optional[dict] = None


def calculate_shift(image_seq_len, base_seq_len: int = 256, max_seq_len: int = 4096, base_shift: float = 0.5, max_shift: float = 1.15):
  m = (max_shift - base_shift) / (max_seq_len - base_seq_len)
  return image_seq_len * m + (base_shift - m * base_seq_len)


def rescale_noise_cfg(noise_cfg, noise_pred_text, guidance_rescale: float = 0.0):
  dims = list(range(1, noise_pred_text.dim()))
  std_text = noise_pred_text.std(dim=dims, keepdim=True, unbiased=False)
  std_cfg = noise_cfg.std(dim=dims, keepdim=True, unbiased=False).clamp_min(1e-5)
  return guidance_rescale * (noise_cfg * (std_text / std_cfg)) + (1 - guidance_rescale) * noise_cfg


def apply_ltx2_guidance(noise_pred, noise_pred_audio, latents, audio_latents, sigma_t: float, guidance_scale, stg_scale,
                        modality_scale, guidance_rescale, audio_guidance_scale=None, audio_stg_scale=None,
                        audio_modality_scale=None, audio_guidance_rescale: float = 0.0, do_cfg=True, do_stg=False):
  if not do_cfg:
    return noise_pred, noise_pred_audio
  if not do_stg:
    u, t = noise_pred.chunk(2)
    au, at = noise_pred_audio.chunk(2)
    return OF.lincomb([t, u], [guidance_scale, 1 - guidance_scale]), OF.lincomb([at, au], [guidance_scale, 1 - guidance_scale])

  def combine(pred, x, g, s, m, rescale):
    u, t, p, iso = (x - v * sigma_t for v in pred.chunk(4))  # x0 of the four branches
    x0 = t + (g - 1) * (t - u) + s * (t - p) + (m - 1) * (t - iso)
    if rescale > 0:
      x0 = rescale_noise_cfg(x0, t, rescale)
    return (x - x0) / sigma_t

  ag = guidance_scale if audio_guidance_scale is None else audio_guidance_scale
  as_ = stg_scale if audio_stg_scale is None else audio_stg_scale
  am = modality_scale if audio_modality_scale is None else audio_modality_scale
  return (combine(noise_pred, latents, guidance_scale, stg_scale, modality_scale, guidance_rescale),
          combine(noise_pred_audio, audio_latents, ag, as_, am, audio_guidance_rescale))


class LTX2Pipeline:

  def __init__(self, transformer, vae, audio_vae, vocoder, connectors, text_encoder=None, latent_upsampler=None,
               scheduler: Optional[FlowMatchScheduler] = None, config=None, device=None):
    self.transformer, self.vae, self.audio_vae, self.vocoder = transformer, vae, audio_vae, vocoder
    self.connectors, self.text_encoder, self.latent_upsampler, self.config = connectors, text_encoder, latent_upsampler, config
    self.scheduler = scheduler or FlowMatchScheduler(num_train_timesteps=1000, shift=1.0, use_dynamic_shifting=True,
                                                     time_shift_type="exponential", shift_terminal=0.1)
    self.schedule_shift = dict(base_image_seq_len=1024, max_image_seq_len=4096, base_shift=0.95, max_shift=2.05)
    self.device = torch.device(device) if device is not None else next(transformer.parameters()).device
    self.dtype = next(transformer.parameters()).dtype
    self.vae_spatial_compression_ratio = vae.cfg.spatial_compression_ratio if vae is not None else 32
    self.vae_temporal_compression_ratio = vae.cfg.temporal_compression_ratio if vae is not None else 8
    tc = transformer.cfg
    self.patch, self.patch_t = tc.patch_size, tc.patch_size_t
    self.audio_sampling_rate, self.audio_hop_length = tc.audio_sampling_rate, tc.audio_hop_length
    self.audio_temporal_ratio = audio_vae.latent_downsample_factor if audio_vae is not None else 4
    self.audio_mel_ratio = audio_vae.latent_downsample_factor if audio_vae is not None else 4

  # ---- latent layouts ------------------------------------------------------------------------
  @staticmethod
  def pack_latents(x, p: int = 1, pt: int = 1):
    B, C, Fr, H, W = x.shape
    x = x.reshape(B, C, Fr // pt, pt, H // p, p, W // p, p).permute(0, 2, 4, 6, 1, 3, 5, 7)
    return x.reshape(B, (Fr // pt) * (H // p) * (W // p), -1)

  @staticmethod
  def unpack_latents(tokens, Fr, H, W, p: int = 1, pt: int = 1):
    B = tokens.shape[0]
    x = tokens.reshape(B, Fr // pt, H // p, W // p, -1, pt, p, p).permute(0, 4, 1, 5, 2, 6, 3, 7)
    return x.reshape(B, -1, Fr, H, W)

  @staticmethod
  def pack_audio_latents(x):
    B, C, T, M = x.shape
    return x.permute(0, 2, 1, 3).reshape(B, T, C * M)

  @staticmethod
  def unpack_audio_latents(tokens, T, mel_bins):
    B = tokens.shape[0]
    return tokens.reshape(B, T, -1, mel_bins).permute(0, 2, 1, 3)

  # ---- conditioning --------------------------------------------------------------------------
  @torch.no_grad()
  def encode_prompt(self, prompt, negative_prompt=None, do_cfg: bool = True, max_sequence_length: int = 1024):
    if self.text_encoder is None:
      raise ValueError("no text encoder loaded: pass `prompt_embeds` / `prompt_attention_mask`")
    prompts = [prompt] if isinstance(prompt, str) else list(prompt)
    embeds, mask = self.text_encoder(prompts, max_sequence_length)
    neg = neg_mask = None
    if do_cfg:
      negs = [negative_prompt or ""] * len(prompts) if not isinstance(negative_prompt, (list, tuple)) else list(negative_prompt)
      neg, neg_mask = self.text_encoder(negs, max_sequence_length)
    return embeds, mask, neg, neg_mask

  def check_inputs(self, prompt, height: int, width: int, prompt_embeds=None, negative_prompt_embeds=None,
                   prompt_attention_mask=None, negative_prompt_attention_mask=None) -> None:
    """Argument rules (reference: src/maxdiffusion/pipelines/ltx2/ltx2_pipeline.py:1365-1417): a frame size the VAE's
    spatial stride divides, a prompt or its embedding (not both, not neither), a mask with every embedding, and
    positive / negative embeddings and masks of equal shape when both are passed."""
    r = self.vae_spatial_compression_ratio
    if height % r or width % r:
      raise ValueError(f"`height` and `width` have to be divisible by {r} but are {height} and {width}.")
    if prompt is not None and prompt_embeds is not None:
      raise ValueError("pass `prompt` or `prompt_embeds`, not both")
    if prompt is None and prompt_embeds is None:
      raise ValueError("provide either `prompt` or `prompt_embeds`")
    if prompt is not None and not isinstance(prompt, (str, list)):
      raise ValueError(f"`prompt` has to be a str or a list but is {type(prompt)}")
    if prompt_embeds is not None and prompt_attention_mask is None:
      raise ValueError("`prompt_attention_mask` is required with `prompt_embeds`")
    if negative_prompt_embeds is not None and negative_prompt_attention_mask is None:
      raise ValueError("`negative_prompt_attention_mask` is required with `negative_prompt_embeds`")
    if prompt_embeds is not None and negative_prompt_embeds is not None:
      if prompt_embeds.shape != negative_prompt_embeds.shape:
        raise ValueError(f"`prompt_embeds` {tuple(prompt_embeds.shape)} and `negative_prompt_embeds` "
                         f"{tuple(negative_prompt_embeds.shape)} must have the same shape")
      if prompt_attention_mask.shape != negative_prompt_attention_mask.shape:
        raise ValueError(f"`prompt_attention_mask` {tuple(prompt_attention_mask.shape)} and `negative_prompt_attention_mask` "
                         f"{tuple(negative_prompt_attention_mask.shape)} must have the same shape")

  @staticmethod
  def _noised(x: torch.Tensor, noise_scale: float, generator) -> torch.Tensor:
    noise = torch.randn(x.shape, generator=generator, dtype=torch.float32).to(x.device)
    return noise_scale * noise + (1.0 - noise_scale) * x.float()

  def prepare_latents(self, batch: int, lf: int, lh: int, lw: int, generator, latents=None,
                      noise_scale: Optional[float] = None) -> torch.Tensor:
    """Packed fp32 video tokens [B, N, C] the loop starts from (reference: ltx2_pipeline.py:1678-1727).

    Without `latents`: unit noise. With `latents` and `noise_scale=None` they are the start state as given (5-D
    tensors are packed). With a number, the reference's re-noising applies: 5-D latents are VAE latents and are
    normalised with the VAE's statistics first, then start = noise_scale * noise + (1 - noise_scale) * latents --
    how a second, higher-resolution pass continues from up-sampled latents."""
    if latents is None:
      z = torch.randn((batch, self.transformer.cfg.in_channels, lf, lh, lw), generator=generator, dtype=torch.float32)
      return self.pack_latents(z, self.patch, self.patch_t).to(self.device)
    if latents.dim() == 5:
      if noise_scale is not None and self.vae is not None:
        latents = self.vae.normalize_latents(latents.float())
      latents = self.pack_latents(latents.float(), self.patch, self.patch_t)
    if latents.dim() != 3:
      raise ValueError(f"`latents` must be [B, C, F, H, W] or packed [B, N, C], got {tuple(latents.shape)}")
    latents = latents.to(self.device, torch.float32)
    return latents if noise_scale is None else self._noised(latents, float(noise_scale), generator)

  def prepare_audio_latents(self, batch: int, channels: int, frames: int, mel_bins: int, generator, latents=None,
                            noise_scale: Optional[float] = None) -> torch.Tensor:
    """The audio counterpart (reference: ltx2_pipeline.py:1729-1772): 4-D [B, C, T, mel] latents are packed, normalised
    with the audio VAE's statistics and re-noised when `noise_scale` is a number."""
    if latents is None:
      z = torch.randn((batch, channels, frames, mel_bins), generator=generator, dtype=torch.float32)
      return self.pack_audio_latents(z).to(self.device)
    if latents.dim() == 4:
      latents = self.pack_audio_latents(latents.float())
    if latents.dim() != 3:
      raise ValueError(f"`audio_latents` must be [B, C, T, mel] or packed [B, T, C * mel], got {tuple(latents.shape)}")
    latents = latents.to(self.device, torch.float32)
    if noise_scale is None:
      return latents
    if self.audio_vae is not None:
      latents = self.audio_vae.normalize_latents(latents)
    return self._noised(latents, float(noise_scale), generator)

  # ---- call ----------------------------------------------------------------------------------
  @torch.no_grad()
  def __call__(self, prompt=None, negative_prompt=None, height: int = 512, width: int = 768, num_frames: int = 121,
               frame_rate: float = 24.0, num_inference_steps: int = 40, sigmas: Optional[Sequence[float]] = None,
               timesteps: Optional[Sequence[float]] = None, noise_scale: Optional[float] = None,
               num_videos_per_prompt: int = 1, guidance_scale: float = 3.0, guidance_rescale: float = 0.0, stg_scale: float = 1.0,
               modality_scale: float = 1.0, audio_guidance_scale=None, audio_guidance_rescale: float = 0.0,
               audio_stg_scale=None, audio_modality_scale=None, generator: Optional[torch.Generator] = None,
               latents=None, audio_latents=None, prompt_embeds=None, negative_prompt_embeds=None,
               prompt_attention_mask=None, negative_prompt_attention_mask=None, decode_timestep: float = 0.0,
               decode_noise_scale: Optional[float] = None, max_sequence_length: int = 1024, output_type: str = "uint8",
               use_cross_timestep: bool = False, use_kv_cache: bool = True):
    r, rt = self.vae_spatial_compression_ratio, self.vae_temporal_compression_ratio
    self.check_inputs(prompt, height, width, prompt_embeds, negative_prompt_embeds, prompt_attention_mask,
                      negative_prompt_attention_mask)
    if stg_scale > 0.0 and guidance_scale <= 1.0:
      raise ValueError("Spatio-temporal guidance requires guidance_scale > 1.0.")
    timings, t0 = {}, time.perf_counter()
    sync = (lambda: torch.cuda.synchronize()) if self.device.type == "cuda" else (lambda: None)
    do_cfg, do_stg = guidance_scale > 1.0, stg_scale > 0.0
    if prompt_embeds is None:
      prompt_embeds, prompt_attention_mask, negative_prompt_embeds, negative_prompt_attention_mask = self.encode_prompt(
          prompt, negative_prompt, do_cfg, max_sequence_length)
    if prompt_attention_mask is None:
      prompt_attention_mask = torch.ones(prompt_embeds.shape[:2], dtype=torch.long)
    if do_cfg and negative_prompt_embeds is not None and negative_prompt_attention_mask is None:
      negative_prompt_attention_mask = torch.ones(negative_prompt_embeds.shape[:2], dtype=torch.long)
    if num_videos_per_prompt > 1:
      # every prompt's embeddings and mask are repeated in place: videos [i * n, (i + 1) * n) belong to prompt i
      rep = lambda t: None if t is None else t.repeat_interleave(int(num_videos_per_prompt), dim=0)
      prompt_embeds, prompt_attention_mask = rep(prompt_embeds), rep(prompt_attention_mask)
      negative_prompt_embeds, negative_prompt_attention_mask = rep(negative_prompt_embeds), rep(negative_prompt_attention_mask)
    B = prompt_embeds.shape[0]
    if do_cfg:
      if negative_prompt_embeds is None:
        raise ValueError("classifier-free guidance needs `negative_prompt_embeds`")
      if negative_prompt_attention_mask is None:
        negative_prompt_attention_mask = torch.ones(negative_prompt_embeds.shape[:2], dtype=torch.long)
      reps = 3 if do_stg else 1
      embeds = torch.cat([negative_prompt_embeds] + [prompt_embeds] * reps)
      mask = torch.cat([negative_prompt_attention_mask] + [prompt_attention_mask] * reps)
    else:
      embeds, mask = prompt_embeds, prompt_attention_mask
    n_branch = embeds.shape[0] // B
    cdtype = next(self.connectors.parameters()).dtype
    video_text, audio_text, text_mask = self.connectors(embeds.to(self.device, cdtype), mask.to(self.device))
    text_mask = None if bool(text_mask.all()) else text_mask.bool()
    sync()
    timings["text_encode"] = time.perf_counter() - t0

    lh, lw, lf = height // r, width // r, (num_frames - 1) // rt + 1
    g = generator if generator is not None else torch.Generator().manual_seed(int(self.config.get("seed", 1)) if self.config is not None else 1)
    tc = self.transformer.cfg
    tokens = self.prepare_latents(B, lf, lh, lw, g, latents, noise_scale)
    audio_lps = self.audio_sampling_rate / self.audio_hop_length / float(self.audio_temporal_ratio)
    audio_frames = round(num_frames / frame_rate * audio_lps)
    mel_bins = (self.audio_vae.cfg.mel_bins if self.audio_vae is not None else 64) // self.audio_mel_ratio
    a_ch = self.audio_vae.cfg.latent_channels if self.audio_vae is not None else tc.audio_in_channels // mel_bins
    a_tokens = self.prepare_audio_latents(B, a_ch, audio_frames, mel_bins, g, audio_latents, noise_scale)

    if timesteps is not None and sigmas is not None:
      raise ValueError("only one of `timesteps` and `sigmas` can be passed")
    if timesteps is not None:
      # custom timesteps are sigmas on the scheduler's 0..num_train_timesteps axis
      sigmas = [float(t) / float(self.scheduler.config.num_train_timesteps) for t in timesteps]
    sig = torch.linspace(1.0, 1.0 / num_inference_steps, num_inference_steps) if sigmas is None else torch.as_tensor(sigmas, dtype=torch.float32)
    s = self.schedule_shift
    mu = calculate_shift(min(6144, lf * lh * lw), s["base_image_seq_len"], s["max_image_seq_len"], s["base_shift"], s["max_shift"])
    state = self.scheduler.set_timesteps_ltx2(self.scheduler.create_state(), len(sig), shift=mu, sigmas=sig)
    timesteps, sched_sigmas = state.timesteps.float(), state.sigmas.float()

    # loop constants: rotary tables, text K/V, per-step time embeddings
    rope = self.transformer.rope_tables(1, lf, lh, lw, audio_frames, frame_rate, self.device)
    # with per-timestep prompt modulation (LTX-2.3) only the caption projections are cached, not the keys / values
    kv = self.transformer.compute_kv_cache(video_text, audio_text) if use_kv_cache else None
    ones = torch.ones((B, 1, 1), device=self.device)
    modality_mask = perturbation_mask = None
    if do_cfg and do_stg:
      modality_mask = torch.cat([ones, ones, ones, ones * 0])
      perturbation_mask = torch.cat([ones, ones, ones * 0, ones])
    sync()
    t1 = time.perf_counter()
    for i in range(len(timesteps)):
      t = float(timesteps[i])
      tt = torch.full((1,), t, device=self.device)
      te = self.transformer.time_embeds(tt, sigma=tt, audio_sigma=tt, use_cross_timestep=use_cross_timestep)
      x_in = tokens.repeat(n_branch, 1, 1).to(self.dtype)
      a_in = a_tokens.repeat(n_branch, 1, 1).to(self.dtype)
      rc = {k: (v[0].expand(x_in.shape[0], *v[0].shape[1:]), v[1].expand(x_in.shape[0], *v[1].shape[1:])) for k, v in rope.items()}
      pred, a_pred = self.transformer(
          x_in, a_in, None if kv is not None else video_text, None if kv is not None else audio_text,
          tt.expand(x_in.shape[0]), encoder_attention_mask=text_mask, audio_encoder_attention_mask=text_mask,
          modality_mask=modality_mask, perturbation_mask=perturbation_mask, cached_kv=kv, rope_cache=rc, time_embed_cache=te)
      sigma_t = float(sched_sigmas[i])
      pred, a_pred = apply_ltx2_guidance(pred.float(), a_pred.float(), tokens, a_tokens, sigma_t, guidance_scale, stg_scale,
                                         modality_scale, guidance_rescale, audio_guidance_scale, audio_stg_scale,
                                         audio_modality_scale, audio_guidance_rescale, do_cfg, do_stg)
      sigma_next = float(sched_sigmas[i + 1]) if i + 1 < len(timesteps) else 0.0
      tokens = OF.lincomb([tokens, pred.contiguous()], [1.0, sigma_next - sigma_t], out_dtype=torch.float32)
      a_tokens = OF.lincomb([a_tokens, a_pred.contiguous()], [1.0, sigma_next - sigma_t], out_dtype=torch.float32)
    sync()
    timings["denoise"] = time.perf_counter() - t1

    lat = self.unpack_latents(tokens, lf, lh, lw, self.patch, self.patch_t)
    if output_type == "latent" or self.vae is None:
      return LTX2PipelineOutput(frames=lat, audio=self.unpack_audio_latents(a_tokens, audio_frames, mel_bins), timings=timings)
    t2 = time.perf_counter()
    vdtype = next(self.vae.parameters()).dtype
    lat = self.vae.denormalize_latents(lat.to(vdtype))
    cfg = self.config
    if cfg is not None and cfg.get("run_latent_upsampler", False) and self.latent_upsampler is not None:
      up = self.latent_upsampler(lat.to(next(self.latent_upsampler.parameters()).dtype)).to(vdtype)
      f = float(cfg.get("upsampler_adain_factor", 0.0))
      lat = adain_filter_latent(up, lat, f) if f > 0.0 else up
      c = float(cfg.get("upsampler_tone_map_compression_ratio", 0.0))
      lat = tone_map_latents(lat, c) if c > 0.0 else lat
    temb = None
    if self.vae.cfg.timestep_conditioning:
      noise = torch.randn(lat.shape, generator=g, dtype=torch.float32).to(lat)
      # a number applies to the whole batch, a list gives one value per video
      per_video = lambda v: torch.as_tensor(list(v) if isinstance(v, (list, tuple)) else [float(v)] * B, dtype=torch.float32)
      dt = per_video(decode_timestep)
      ns = dt if decode_noise_scale is None else per_video(decode_noise_scale)
      if dt.numel() != B or ns.numel() != B:
        raise ValueError(f"`decode_timestep` / `decode_noise_scale` lists need one value per video ({B})")
      ns = ns.to(lat).view(B, 1, 1, 1, 1)
      lat = (1 - ns) * lat + ns * noise
      temb = dt.to(self.device, vdtype)
    video = self.vae.decode(lat, temb)
    sync()
    timings["vae_decode"] = time.perf_counter() - t2
    t3 = time.perf_counter()
    audio = None
    if self.audio_vae is not None and self.vocoder is not None:
      adtype = next(self.audio_vae.parameters()).dtype
      a_lat = self.unpack_audio_latents(self.audio_vae.denormalize_latents(a_tokens.to(adtype)), audio_frames, mel_bins)
      mel = self.audio_vae.decode(a_lat)
      audio = self.vocoder(mel.to(next(self.vocoder.parameters()).dtype)).float()
    sync()
    timings["audio_decode"] = time.perf_counter() - t3
    if output_type == "uint8":
      video = ((video.float() / 2 + 0.5).clamp(0, 1) * 255).round().to(torch.uint8).permute(0, 2, 3, 4, 1)
    return LTX2PipelineOutput(frames=video, audio=audio, timings=timings)
