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
    self.step = 0
    self.batch_size = max(1, int(float(config.get("per_device_batch_size", 1))))

  def load_dataset(self):
    cfg = self.model.cfg
    return SyntheticFluxIterator(self.config, self.batch_size, seed=int(self.config.get("seed", 0)) + 17,
                                 text_dim=cfg.joint_attention_dim, pooled_dim=cfg.pooled_projection_dim, latent_dim=cfg.in_channels)

  def train_step(self, batch: dict) -> dict:
    batch = {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()}
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

  def start_training(self):
    data = self.load_dataset()
    writer = MetricsWriter(self.config, self.mesh.rank)
    while self.step < int(self.config.max_train_steps):
      t0 = time.perf_counter()
      m = self.train_step(next(data))
      loss = float(m["learning/loss"])
      writer.write(self.step, {**{k: float(v) for k, v in m.items()}, "perf/step_time_seconds": time.perf_counter() - t0})
    writer.close()
    return self
