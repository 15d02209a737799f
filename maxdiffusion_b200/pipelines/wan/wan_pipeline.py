"""Wan text-to-video / image-to-video pipelines (2.1 and 2.2) for inference.

Public surface of the reference (src/maxdiffusion/pipelines/wan/*.py): `WanPipeline2_1`, `WanPipeline2_2`,
`WanPipelineI2V_2_1`, `WanPipelineI2V_2_2` with `from_pretrained(config)` / `from_checkpoint(config)` /
`__call__(prompt, negative_prompt, height, width, num_frames, num_inference_steps, guidance_scale, ...)`.

One denoising step = [transformer on cond (+ uncond) latents] -> CFG combine -> UniPC step, all on device without
host synchronisation; the cache policies (`cache_policies.py`) are decided on the host before / between steps.
Classifier-free guidance runs as one batch of two (`[cond; uncond]`, reference: wan_pipeline.py:1395-1433); when
the `data` mesh axis is 2 each half goes to one data-parallel rank (CFG as data parallelism, README.md:703).
Sequence parallelism is delegated to `parallel.context.ContextParallel` through the model's `pctx` argument.
Stage timings are returned in a `trace` dict like the reference's (wan_pipeline_2_1.py:149-211).
"""
from __future__ import annotations

import os
import time
from typing import List, Optional, Sequence, Union

import torch
import torch.distributed as dist

from ... import max_logging
from ...models.wan.autoencoder_kl_wan import AutoencoderKLWan, WanVAEConfig, postprocess_video
from ...models.wan.transformer_wan import WAN_PRESETS, WanConfig, WanModel, wan_rope_tables
from ...ops import _lib
from ...ops import functional as OF
from ...parallel.context import ContextParallel
from ...parallel.mesh import DeviceMesh, create_device_mesh
from ...schedulers.scheduling_unipc_multistep import UniPCMultistepScheduler
from . import cache_policies as CP


class PromptCache:
  """Last `size` prompt embeddings (the reference keeps 16, wan_pipeline.py:734-804)."""

  def __init__(self, size: int = 16):
    self.size, self.items = size, {}

  def get(self, key):
    return self.items.get(key)

  def put(self, key, value):
    if len(self.items) >= self.size:
      self.items.pop(next(iter(self.items)))
    self.items[key] = value


class WanPipeline:
  model_name = "wan2.1"
  is_i2v = False
  transformer_cls = WanModel

  @staticmethod
  def resolve_transformer_config(config):
    from ...trainers.wan_trainer import resolve_wan_config

    return resolve_wan_config(config)

  def __init__(self, config, transformer: WanModel, vae: Optional[AutoencoderKLWan], scheduler: UniPCMultistepScheduler,
               tokenizer=None, text_encoder=None, transformer_2: Optional[WanModel] = None,
               image_encoder=None, mesh: Optional[DeviceMesh] = None, device=None):
    self.config = config
    self.transformer, self.transformer_2 = transformer, transformer_2  # 2.2: high-noise, low-noise experts
    self.vae, self.scheduler = vae, scheduler
    self.tokenizer, self.text_encoder, self.image_encoder = tokenizer, text_encoder, image_encoder
    self.mesh = mesh if mesh is not None else create_device_mesh(config)
    anchor = transformer if transformer is not None else vae  # preprocessing pipelines carry no transformer
    self.device = torch.device(device) if device is not None else next(anchor.parameters()).device
    self.dtype = next(anchor.parameters()).dtype
    self.pctx = None
    fixed_m = bool(config.get("fixed_m_softmax", False))
    if self.mesh.size("context") > 1 or fixed_m:
      # a one-rank context still goes through ContextParallel when the fixed-exponent softmax is selected
      self.pctx = ContextParallel(self.mesh, str(config.get("context_strategy", "ring")),
                                  peer_memory=bool(config.get("peer_memory_transport", True)) and self.device.type == "cuda",
                                  fixed_m=fixed_m, ulysses_chunks=int(config.get("ulysses_attention_chunks", 1)),
                                  kv_transport=str(config.get("ring_kv_transport", "dma")))
    if self.mesh.size("tensor") > 1:
      from ...parallel.tensor import apply_tensor_parallel_wan

      for m in filter(None, (self.transformer, self.transformer_2)):
        if getattr(m, "tp_group", None) is None:
          apply_tensor_parallel_wan(m, self.mesh.group("tensor"))
    # VAE spatial parallelism: the ranks that hold the same latents (the context axis, else the tensor axis) each
    # decode a vertical strip of the frame (reference: the `vae_spatial` mesh axis, wan_pipeline.py:560-640).
    # vae_spatial: -1 = over that whole axis, 1 = off.
    self.vae_spatial = None
    axis = "context" if self.mesh.size("context") > 1 else "tensor"
    want = int(config.get("vae_spatial", -1))
    if vae is not None and self.mesh.size(axis) > 1 and want != 1:
      if want not in (-1, 0, self.mesh.size(axis)):
        raise ValueError(f"vae_spatial={want}: the VAE is split over the whole {axis} axis ({self.mesh.size(axis)} ranks) or not at all")
      from ...parallel.spatial import HaloExchange

      self.vae_spatial = HaloExchange(self.mesh.group(axis),
                                      peer_memory=bool(config.get("peer_memory_transport", True)) and self.device.type == "cuda")
    self.prompt_cache = PromptCache()
    from ...models.quantizations import get_quantization_mode, quantize_model

    mode = get_quantization_mode(config)
    if mode is not None:
      # reference: qwix rules applied to the transformer(s) at pipeline construction (wan_pipeline.py:569-651)
      for m in filter(None, (self.transformer, self.transformer_2)):
        n = quantize_model(m, mode)
        max_logging.log(f"quantization={mode}: {n} linear layers run on the fp8 tensor-core path")
    self.vae_scale_factor_temporal, self.vae_scale_factor_spatial = 4, 8
    self.extra_model_kwargs: dict = {}  # set by subclasses for the duration of a call (control latents, ...)

  # ------------------------------------------------------------------ construction
  @classmethod
  def from_config(cls, config, device=None, dtype=None, load_vae: bool = True, **kw):
    """Random-initialised pipeline of the configured architecture (benchmarks, tests)."""
    device = torch.device(device) if device is not None else (
        torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    dtype = dtype or (config.weights_dtype if device.type == "cuda" else torch.float32)
    wcfg = cls.resolve_transformer_config(config)
    torch.manual_seed(int(config.get("seed", 0)))
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
      with torch.device(device):
        transformer = cls.transformer_cls(wcfg)
        transformer_2 = cls.transformer_cls(wcfg) if cls.model_name == "wan2.2" else None
    finally:
      torch.set_default_dtype(prev)
    vae = None
    if load_vae:
      vae_cfg = WanVAEConfig(**(config.get("vae_config_overrides", None) or {}))
      vae = AutoencoderKLWan(vae_cfg).to(device=device, dtype=config.get("vae_dtype", torch.float32) if device.type == "cuda" else torch.float32)
    scheduler = UniPCMultistepScheduler(prediction_type="flow_prediction", use_flow_sigmas=True,
                                        flow_shift=float(config.get("flow_shift", 5.0)), solver_order=2)
    return cls(config, transformer, vae, scheduler, transformer_2=transformer_2, device=device, **kw)

  @classmethod
  def from_pretrained(cls, config, device=None, load_transformer: bool = True, **kw):
    """Loads diffusers-format weights from `pretrained_model_name_or_path` (a local directory)."""
    from ...loaders.wan_loader import load_wan_pipeline_components

    comps = load_wan_pipeline_components(config, cls.model_name, device=device, load_transformer=load_transformer)
    return cls(config, device=device, **comps, **kw)

  @classmethod
  def from_checkpoint(cls, config, device=None, **kw):
    from ...checkpointing.wan_checkpointer import WanCheckpointer

    pipe = cls.from_config(config, device=device, **kw)
    WanCheckpointer(config).restore_into_pipeline(pipe)
    return pipe

  # ------------------------------------------------------------------ prompt / latents
  def encode_prompt(self, prompt: Union[str, List[str]], max_sequence_length: int = 512):
    """UMT5 embeddings, zero-padded beyond the true length (reference: wan_pipeline.py:696-732)."""
    prompts = [prompt] if isinstance(prompt, str) else list(prompt)
    key = (tuple(prompts), max_sequence_length)
    hit = self.prompt_cache.get(key)
    if hit is not None:
      return hit
    if self.text_encoder is None or self.tokenizer is None:
      raise ValueError("no text encoder is loaded: pass prompt_embeds / negative_prompt_embeds instead of prompts")
    tok = self.tokenizer(prompts, padding="max_length", max_length=max_sequence_length, truncation=True,
                         add_special_tokens=True, return_attention_mask=True, return_tensors="pt")
    enc_device = next(self.text_encoder.parameters()).device
    with torch.no_grad():
      hidden = self.text_encoder(tok.input_ids.to(enc_device), tok.attention_mask.to(enc_device)).last_hidden_state
    lens = tok.attention_mask.sum(dim=1)
    out = torch.zeros_like(hidden)
    for i, n in enumerate(lens.tolist()):
      out[i, :n] = hidden[i, :n]
    out = out.to(self.device, self.dtype)
    self.prompt_cache.put(key, out)
    return out

  def prepare_latents(self, batch: int, height: int, width: int, num_frames: int, generator=None, latents=None):
    shape = (batch, self.transformer.cfg.in_channels if not self.is_i2v else 16,
             (num_frames - 1) // self.vae_scale_factor_temporal + 1, height // self.vae_scale_factor_spatial,
             width // self.vae_scale_factor_spatial)
    if latents is not None:
      return latents.to(self.device, torch.float32)
    g = generator
    if g is None:
      g = torch.Generator(device="cpu").manual_seed(int(self.config.get("seed", 0)))
    return torch.randn(shape, generator=g, dtype=torch.float32, device=g.device).to(self.device)

  # ------------------------------------------------------------------ experts / guidance
  def _expert(self, t: float, boundary: Optional[float], scale_low: Optional[float] = None, scale_high: Optional[float] = None):
    """(model, guidance scale, is the high-noise expert) for timestep t; a scale passed to the call wins over the
    configuration's `guidance_scale_low` / `guidance_scale_high`."""
    if self.transformer_2 is None or boundary is None:
      return self.transformer, float(self.config.get("guidance_scale", 5.0)), False
    if t >= boundary:
      high = scale_high if scale_high is not None else self.config.get("guidance_scale_high", self.config.get("guidance_scale", 5.0))
      return self.transformer, float(high), True
    low = scale_low if scale_low is not None else self.config.get("guidance_scale_low", self.config.get("guidance_scale", 5.0))
    return self.transformer_2, float(low), False

  def vae_encode_chunk(self, num_frames: int) -> int:
    """Frames per VAE encoder pass after the first frame: `vae_encode_chunk` of the configuration, a multiple of the
    temporal stride (4); -1 takes the rest of the clip in one pass (reference:
    src/maxdiffusion/models/wan/autoencoder_kl_wan.py:1063-1077,1144-1149)."""
    stride = self.vae_scale_factor_temporal
    chunk = int(self.config.get("vae_encode_chunk", stride)) if self.config is not None else stride
    if chunk == -1:
      return max(stride, -(-max(1, num_frames - 1) // stride) * stride)
    if chunk < 1 or chunk % stride:
      raise ValueError(f"vae_encode_chunk ({chunk}) must be -1 or a positive multiple of the temporal stride ({stride})")
    return chunk

  def _cfg_split(self):
    """With data axis 2 and CFG on, rank coordinate 0 runs cond and 1 runs uncond (CFG as data parallelism)."""
    return self.mesh.size("data") == 2

  def _forward(self, model, latents, t, embeds, image_embeds=None, kv_cache=None, rope=None, **kw):
    ts = torch.full((latents.shape[0],), float(t), device=self.device, dtype=torch.float32)
    for name, val in self.extra_model_kwargs.items():
      if torch.is_tensor(val) and val.dim() > 1 and val.shape[0] != latents.shape[0]:
        val = val.repeat(latents.shape[0] // val.shape[0], *([1] * (val.dim() - 1)))  # CFG doubles the batch
      kw[name] = val
    return model(latents.to(self.dtype), ts, embeds, encoder_hidden_states_image=image_embeds, pctx=self.pctx,
                 kv_cache=kv_cache, rope=rope, **kw)

  # ------------------------------------------------------------------ call
  def check_inputs(self, prompt, negative_prompt, height: int, width: int, num_frames: int, prompt_embeds=None,
                   negative_prompt_embeds=None) -> None:
    """Argument rules shared by the Wan pipelines (reference: src/maxdiffusion/pipelines/wan/wan_vace_pipeline_2_1.py:
    387-425): a prompt or its embedding but not both, text as str or list, a frame size the VAE stride times the patch
    size divides, a positive frame count."""
    for name, text, emb in (("prompt", prompt, prompt_embeds), ("negative_prompt", negative_prompt, negative_prompt_embeds)):
      if text is not None and emb is not None:
        raise ValueError(f"pass `{name}` or `{name}_embeds`, not both")
      if text is not None and not isinstance(text, (str, list)):
        raise ValueError(f"`{name}` has to be a str or a list but is {type(text)}")
    patch = tuple(self.transformer.cfg.patch_size) if self.transformer is not None else (1, 2, 2)
    base_h, base_w = self.vae_scale_factor_spatial * patch[1], self.vae_scale_factor_spatial * patch[2]
    if height % base_h or width % base_w:
      raise ValueError(f"`height` and `width` have to be divisible by {base_h} and {base_w} but are {height} and {width}")
    if num_frames < 1:
      raise ValueError(f"`num_frames` must be positive, got {num_frames}")

  @torch.no_grad()
  def __call__(self, prompt=None, negative_prompt=None, height: Optional[int] = None, width: Optional[int] = None,
               num_frames: Optional[int] = None, num_inference_steps: Optional[int] = None,
               guidance_scale: Optional[float] = None, prompt_embeds=None, negative_prompt_embeds=None,
               image_embeds=None, condition=None, latents=None, generator=None, output_type: str = "uint8",
               use_cfg_cache: Optional[bool] = None, use_magcache: Optional[bool] = None,
               use_sen_cache: Optional[bool] = None, use_kv_cache: Optional[bool] = None, return_trace: bool = False,
               guidance_scale_low: Optional[float] = None, guidance_scale_high: Optional[float] = None):
    c = self.config if getattr(self, "config", None) is not None else {}
    height = height or int(c.get("height", 480))
    width = width or int(c.get("width", 832))
    num_frames = num_frames or int(c.get("num_frames", 81))
    steps = num_inference_steps or int(c.get("num_inference_steps", 50))
    guidance_scale = float(guidance_scale if guidance_scale is not None else c.get("guidance_scale", 5.0))
    do_cfg = bool(c.get("do_classifier_free_guidance", True)) and guidance_scale > 1.0
    use_cfg_cache = bool(c.get("use_cfg_cache", False)) if use_cfg_cache is None else use_cfg_cache
    use_magcache = bool(c.get("use_magcache", False)) if use_magcache is None else use_magcache
    use_sen_cache = bool(c.get("use_sen_cache", False)) if use_sen_cache is None else use_sen_cache
    use_kv_cache = bool(c.get("use_kv_cache", False)) if use_kv_cache is None else use_kv_cache
    two_experts = getattr(self, "transformer_2", None) is not None or self.model_name == "wan2.2"
    chosen = [n for n, on in (("use_cfg_cache", use_cfg_cache), ("use_magcache", use_magcache), ("use_sen_cache", use_sen_cache)) if on]
    if len(chosen) > 1:
      raise ValueError(f"{', '.join(chosen)} are mutually exclusive: pick one cache policy")
    # every policy of the two-expert models, and the CFG cache of the others, reuses a guided prediction or rebuilds the
    # unconditional branch: without classifier-free guidance there is nothing to reuse
    if two_experts and chosen:
      low = float(guidance_scale_low if guidance_scale_low is not None else c.get("guidance_scale_low", guidance_scale))
      high = float(guidance_scale_high if guidance_scale_high is not None else c.get("guidance_scale_high", guidance_scale))
      if low <= 1.0 or high <= 1.0:
        raise ValueError(f"{chosen[0]}=True needs guidance_scale_low > 1.0 and guidance_scale_high > 1.0 (got {low}, {high})")
    elif use_cfg_cache and guidance_scale <= 1.0:
      raise ValueError(f"use_cfg_cache=True needs guidance_scale > 1.0 (got {guidance_scale}): the cache skips the "
                       "unconditional pass of classifier-free guidance")
    self.check_inputs(prompt, negative_prompt, height, width, num_frames, prompt_embeds, negative_prompt_embeds)
    if use_sen_cache and self.transformer_2 is None:
      raise ValueError("use_sen_cache is a Wan 2.2 option")
    trace = {}
    sync = (lambda: torch.cuda.synchronize()) if self.device.type == "cuda" else (lambda: None)

    t0 = time.perf_counter()
    if prompt_embeds is None:
      prompt_embeds = self.encode_prompt(prompt or c.get("prompt", ""), int(c.get("max_sequence_length", 512)))
    if do_cfg and negative_prompt_embeds is None:
      neg = negative_prompt if negative_prompt is not None else c.get("negative_prompt", "")
      neg = [neg] * prompt_embeds.shape[0] if isinstance(neg, str) else neg
      negative_prompt_embeds = self.encode_prompt(neg, int(c.get("max_sequence_length", 512)))
    prompt_embeds = prompt_embeds.to(self.device, self.dtype)
    B = prompt_embeds.shape[0]
    latents = self.prepare_latents(B, height, width, num_frames, generator, latents)
    trace["conditioning"] = time.perf_counter() - t0

    state = self.scheduler.set_timesteps(self.scheduler.create_state(), steps, latents.shape, device=self.device)
    timesteps = state.timesteps.tolist()
    boundary = None
    if self.transformer_2 is not None:
      boundary = float(c.get("boundary_ratio", 0.875)) * self.scheduler.config.num_train_timesteps

    cfg_split = do_cfg and self._cfg_split()
    if do_cfg and not cfg_split:
      embeds_all = torch.cat([prompt_embeds, negative_prompt_embeds.to(self.device, self.dtype)], dim=0)
    elif cfg_split:
      embeds_all = prompt_embeds if self.mesh.coords["data"] == 0 else negative_prompt_embeds.to(self.device, self.dtype)
    else:
      embeds_all = prompt_embeds

    # constants of the loop: rotary tables, cross-attention K/V
    grid = (latents.shape[2], latents.shape[3] // 2, latents.shape[4] // 2)
    rope = wan_rope_tables(self.transformer.cfg.attention_head_dim, grid, device=self.device)
    kv_caches = {}
    if use_kv_cache:
      for m in filter(None, (self.transformer, self.transformer_2)):
        kv_caches[id(m)] = m.compute_kv_cache(embeds_all, image_embeds)

    if use_cfg_cache and do_cfg and not cfg_split:
      if self.transformer_2 is not None and boundary is not None:
        cfg_sched = CP.cfg_cache_schedule_two_experts(steps, height, [float(t) >= boundary for t in timesteps])
      else:
        cfg_sched = CP.cfg_cache_schedule(steps, height)
    else:
      cfg_sched = [False] * steps
    phases = [float(t) >= boundary for t in timesteps] if (self.transformer_2 is not None and boundary is not None) else None
    mag_sched = CP.magcache_schedule(steps, c.get("mag_ratios_base", [1.0, 1.0]), float(c.get("magcache_thresh", 0.12)),
                                     int(c.get("magcache_K", 2)), float(c.get("retention_ratio", 0.2)),
                                     phases) if use_magcache else [False] * steps
    sen = CP.SenCache(steps) if use_sen_cache else None
    cached_cond = cached_uncond = cached_residual = None
    prev_high = None

    sync()
    t_loop = time.perf_counter()
    ev = None
    if self.device.type == "cuda":  # the loop is also timed on the device, by events on the launching stream
      ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
      ev[0].record()
    for i, t in enumerate(timesteps):
      model, g_scale, is_high = self._expert(t, boundary, guidance_scale_low, guidance_scale_high)
      if self.transformer_2 is None:
        g_scale = guidance_scale
      at_boundary = prev_high is not None and prev_high != is_high
      prev_high = is_high
      if at_boundary:
        cached_residual = None  # the residual of one expert does not carry over to the other
      lat_in = latents if condition is None else torch.cat([latents, condition.to(latents.dtype)], dim=1)
      kv = kv_caches.get(id(model))

      if sen is not None and sen.should_reuse(i, latents, t, at_boundary):
        noise = sen.record_reuse()
      elif cfg_sched[i] and cached_cond is not None:
        cond = self._forward(model, lat_in, t, prompt_embeds, image_embeds, kv_cache=None, rope=rope).float()
        w1, w2 = CP.cfg_cache_weights(i, steps)
        uncond = CP.fft_compensate(cond, cached_cond, cached_uncond, w1, w2)
        noise = OF.lincomb([cond, uncond], [g_scale, 1.0 - g_scale])
        cached_cond = cond
      else:
        skip = mag_sched[i] and cached_residual is not None
        lat_b = torch.cat([lat_in, lat_in], dim=0) if (do_cfg and not cfg_split) else lat_in
        img_b = image_embeds
        if image_embeds is not None and do_cfg and not cfg_split:
          img_b = torch.cat([image_embeds, image_embeds], dim=0)
        out = self._forward(model, lat_b, t, embeds_all, img_b, kv_cache=kv, rope=rope, skip_blocks=skip,
                            cached_residual=cached_residual if skip else None, return_residual=use_magcache)
        if use_magcache:
          out, res = out
          if not skip:
            cached_residual = res
        out = out.float()
        if do_cfg and not cfg_split:
          cond, uncond = out[:B], out[B:]
          noise = OF.lincomb([cond, uncond], [g_scale, 1.0 - g_scale])
          cached_cond, cached_uncond = cond, uncond
        elif cfg_split:
          both = [torch.empty_like(out) for _ in range(2)]
          dist.all_gather(both, out.contiguous(), group=self.mesh.group("data"))
          noise = OF.lincomb([both[0], both[1]], [g_scale, 1.0 - g_scale])
        else:
          noise = out
        if sen is not None:
          sen.record_full(latents, t, noise)
      latents, state = self.scheduler.step(state, noise, t, latents)
      if self.pctx is not None:
        # kernels of this step waited (bounded) on other ranks: a wait that ran out must not feed the next step
        _lib.raise_on_device_status_if_loaded()
    if ev is not None:
      ev[1].record()
    sync()
    _lib.raise_on_device_status_if_loaded()
    trace["denoise_total"] = ev[0].elapsed_time(ev[1]) / 1e3 if ev is not None else time.perf_counter() - t_loop
    trace["denoise_per_step"] = trace["denoise_total"] / max(1, steps)

    if output_type == "latent" or self.vae is None:
      return (latents, trace) if return_trace else latents
    t_v = time.perf_counter()
    video = self.decode_latents(latents)
    sync()
    trace["vae_decode"] = time.perf_counter() - t_v
    if output_type == "uint8":
      video = postprocess_video(video)
    return (video, trace) if return_trace else video

  def decode_latents(self, latents):
    z = self.vae.denormalize_latents(latents.float())
    if z.is_cuda and bool(self.config.get("vae_kernel_decode", True)):
      # bf16 latents select the channels-last decoder on this repository's convolution kernels (the weights are
      # packed to bf16 whatever dtype the module keeps them in)
      z = z.to(torch.bfloat16)
    else:
      z = z.to(next(self.vae.parameters()).dtype)
    chunk = int(self.config.get("vae_decode_chunk", 1))
    if self.vae_spatial is not None and z.is_cuda and z.dtype == torch.bfloat16 and hasattr(self.vae, "channels_last_decoder"):
      video = self.vae.channels_last_decoder().decode(z, chunk, spatial=self.vae_spatial)
      _lib.raise_on_device_status_if_loaded()  # the halo exchanges waited (bounded) on the neighbours
      return video
    return self.vae.decode(z, chunk=chunk)


class WanPipeline2_1(WanPipeline):
  model_name = "wan2.1"


class WanPipeline2_2(WanPipeline):
  """Two experts (high-noise, low-noise) switched at `boundary_ratio * num_train_timesteps`
  (reference: wan_pipeline_2_2.py:225,368,887-903)."""
  model_name = "wan2.2"


class _I2VMixin:
  is_i2v = True

  def prepare_condition(self, image: torch.Tensor, num_frames: int, height: int, width: int):
    """First-frame conditioning: VAE latents of [image, zeros...] plus a 4-channel frame mask
    (reference: wan_pipeline.py:829-890). image: [B,3,H,W] in [-1,1]. Returns [B,20,T',H',W']."""
    B = image.shape[0]
    video = torch.zeros((B, 3, num_frames, height, width), device=image.device, dtype=image.dtype)
    video[:, :, 0] = image
    vae_dtype = next(self.vae.parameters()).dtype
    if video.is_cuda and bool(self.config.get("vae_kernel_decode", True)) and hasattr(self.vae, "channels_last_decoder"):
      vae_dtype = torch.bfloat16  # bf16 frames select the encoder on this repository's convolution kernels
    lat = self.vae.normalize_latents(self.vae.encode(video.to(vae_dtype), self.vae_encode_chunk(video.shape[2])).mode().float())
    tl = (num_frames - 1) // 4 + 1
    mask = torch.zeros((B, 4, tl, height // 8, width // 8), device=image.device, dtype=lat.dtype)
    mask[:, :, 0] = 1.0
    return torch.cat([mask, lat], dim=1)

  def encode_image(self, image):
    if self.image_encoder is None:
      return None
    with torch.no_grad():
      return self.image_encoder(image).to(self.device, self.dtype)


class WanPipelineI2V_2_1(_I2VMixin, WanPipeline):
  model_name = "wan2.1"


class WanPipelineI2V_2_2(_I2VMixin, WanPipeline):
  model_name = "wan2.2"
