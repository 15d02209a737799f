"""Flux finetuning: flow-matching loss on packed latents with T5 / CLIP conditioning.

Reference: `FluxTrainer` (src/maxdiffusion/trainers/flux_trainer.py:207-519): the input pipeline precomputes T5 / CLIP
embeddings and VAE latents (:207-252,295-353); `_train_step` noises with x_t = t*eps + (1-t)*x and regresses eps - x
(:470-519). Block weights are sharded with `parallel.fsdp.FSDPEngine` (optimizer step inside backward).
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from ..models.gradient_checkpoint import resolve_remat
import torch.distributed as dist

from ..input_pipeline.synthetic_data_iterator import SyntheticFluxIterator
from ..max_utils import create_optimizer
from ..models.flux.transformer_flux import FLUX_PRESETS, FluxConfig, FluxTransformer2DModel
from ..parallel.fsdp import FSDPEngine, lr_schedule
from ..parallel.mesh import create_device_mesh
from ..train_utils import MetricsWriter


class FluxTrainer:

  def __init__(self, config, mesh=None, model: Optional[FluxTransformer2DModel] = None, device=None):
    self.config = config
    self.mesh = mesh if mesh is not None else create_device_mesh(config)
    self.device = torch.device(device) if device is not None else (
        torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    self.dtype = config.weights_dtype if self.device.type == "cuda" else torch.float32
    seed = int(config.get("seed", 0))
    remat = resolve_remat(config.get("remat_policy", "NONE"), config.get("names_which_can_be_saved", []) or [],
                          config.get("names_which_can_be_offloaded", []) or [])
    group = self.mesh.group("fsdp")
    if group is not None and remat == "NONE":
      remat = "SAVE_ATTENTION"
    if model is None:
      preset = dict(FLUX_PRESETS[str(config.get("flux_preset", "flux-dev"))])
      preset.update(config.get("flux_config_overrides", None) or {})
      torch.manual_seed(seed)
      prev = torch.get_default_dtype()
      torch.set_default_dtype(self.dtype)
      try:
        with torch.device(self.device):
          model = FluxTransformer2DModel(FluxConfig(**preset), remat_policy=remat)
      finally:
        torch.set_default_dtype(prev)
    model.remat_policy = remat
    self.model = model.to(self.device, self.dtype)
    blocks = self.model.blocks
    ids = {id(p) for b in blocks for p in b.parameters()}
    root = [p for p in self.model.parameters() if id(p) not in ids]
    self.engine = FSDPEngine(blocks, root, create_optimizer(config), group=group, replica_group=self.mesh.group("replica"),
                             device=self.device, param_dtype=self.dtype, seed=seed,
                             peer_memory=bool(config.get("peer_memory_transport", True)))
    self.model.block_hook = self.engine.block_hook if remat != "NONE" or group is not None else None
    self._no_remat = remat == "NONE"
    self.gen = torch.Generator(device=self.device).manual_seed(seed + 1 + 7919 * self.mesh.rank)
    self.seed = seed
    self.vae, self.text_encoders, self.tokenizers = None, (), ()  # set by `attach_encoders` for raw image / caption data
    self.step = 0
    self.batch_size = max(1, int(float(config.get("per_device_batch_size", 1))))

  def load_dataset(self):
    cfg = self.model.cfg
    if str(self.config.get("dataset_type", "synthetic")) == "synthetic":
      return SyntheticFluxIterator(self.config, self.batch_size, seed=int(self.config.get("seed", 0)) + 17 + self.mesh.rank,
                                   text_dim=cfg.joint_attention_dim, pooled_dim=cfg.pooled_projection_dim, latent_dim=cfg.in_channels)
    from ..input_pipeline.input_pipeline_interface import make_data_iterator

    return make_data_iterator(self.config, self.mesh, self.batch_size)

  def attach_encoders(self, vae, clip, t5, clip_tokenizer, t5_tokenizer) -> None:
    """Frozen VAE and text encoders for datasets of raw images and captions (reference: the encoders are applied in
    the input pipeline, flux_trainer.py:207-353)."""
    self.vae, self.text_encoders, self.tokenizers = vae, (clip, t5), (clip_tokenizer, t5_tokenizer)

  @torch.no_grad()
  def encode_batch(self, batch: dict) -> dict:
    """pixels + captions -> packed latents, T5 embeddings, CLIP pooled vector, position ids (the synthetic layout)."""
    if "pixel_values" in batch and batch["pixel_values"].dim() == 3:
      return batch  # already packed latents
    from ..models.flux.transformer_flux import pack_latents, prepare_latent_image_ids

    if self.vae is None or not self.text_encoders:
      raise ValueError("raw image / caption batches need `attach_encoders(vae, clip, t5, tokenizers)` first")
    vdtype = next(self.vae.parameters()).dtype
    lat = self.vae.scale_latents(self.vae.encode(batch["pixel_values"].to(self.device, vdtype)).sample(self.gen))
    packed = pack_latents(lat.float())
    clip, t5 = self.text_encoders
    ctok, ttok = self.tokenizers
    caps = list(batch["captions"])
    ids = ctok(caps, padding="max_length", max_length=77, truncation=True, return_tensors="pt").input_ids
    pooled = clip(ids.to(next(clip.parameters()).device)).pooler_output
    ids2 = ttok(caps, padding="max_length", max_length=int(self.config.get("max_sequence_length", 512)), truncation=True,
                return_tensors="pt").input_ids
    emb = t5(ids2.to(next(t5.parameters()).device)).last_hidden_state
    B, _, lh, lw = lat.shape
    img_ids = prepare_latent_image_ids(lh // 2, lw // 2, self.device)
    return {"pixel_values": packed, "text_embeds": emb.float(), "prompt_embeds": pooled.float(),
            "img_ids": img_ids[None].expand(B, -1, -1), "txt_ids": torch.zeros((B, emb.shape[1], 3), device=self.device)}

  def train_step(self, batch: dict) -> dict:
    batch = self.encode_batch(batch)
    batch = {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()}
    # the noise / timestep stream is a function of (seed, rank, step): a resumed run continues it exactly
    self.gen.manual_seed(self.seed + 1 + 7919 * self.mesh.rank + 1000003 * self.step)
    lr = lr_schedule(self.step, float(self.config.learning_rate), int(self.config.learning_rate_schedule_steps),
                     float(self.config.warmup_steps_fraction))
    self.engine.begin_step(lr)
    x = batch["pixel_values"].float()  # packed latents [B, S, 64]
    B = x.shape[0]
    t = torch.rand((B,), generator=self.gen, device=self.device)
    noise = torch.randn(x.shape, generator=self.gen, device=self.device)
    tb = t.view(B, 1, 1)
    noisy = tb * noise + (1 - tb) * x
    guidance = torch.full((B,), float(self.config.get("guidance_scale", 3.5)), device=self.device)
    pred = self.model(noisy.to(self.dtype), batch["text_embeds"], batch["prompt_embeds"], t, batch["img_ids"],
                      batch["txt_ids"], guidance)
    loss = ((noise - x) - pred.float()).pow(2).mean()
    loss.backward()
    if self._no_remat:  # gradients of every block are complete only now
      for i in range(len(self.engine.blocks)):
        self.engine.reduce_and_step(i)
    stats = self.engine.finish_step(model_group=None)
    self.step += 1
    return {"learning/loss": loss.detach(), "learning/max_grad_norm": stats["grad_norm"], "learning/current_learning_rate": lr}

  def checkpointer(self):
    from ..checkpointing.flux_checkpointer import FluxCheckpointer

    c = self.config
    if int(c.get("checkpoint_every", -1)) > 0 or c.get("save_final_checkpoint", False):
      return FluxCheckpointer(c)
    return None

  def start_training(self, data=None):
    """Resume -> (cached) data -> steps with metrics -> periodic / final checkpoints (reference: flux_trainer.py:355-468)."""
    from .loop import EncodedBatchCache, run_training_loop

    def build():
      it = data if data is not None else self.load_dataset()
      if self.vae is not None and self.config.get("cache_latents_text_encoder_outputs", True):
        it = EncodedBatchCache(iter(it), self.encode_batch)
      return it

    return run_training_loop(self, build, self.checkpointer())
