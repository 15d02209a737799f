"""SD 1.x / 2.x and SDXL UNet training (DDPM noise scheduler, epsilon / v-prediction MSE, optional min-SNR weights and
timestep-bias sampling), and the Dreambooth variant with prior preservation.

Reference: `BaseStableDiffusionTrainer.start_training` (src/maxdiffusion/trainers/base_stable_diffusion_trainer.py:115-197),
SDXL `_train_step` (sdxl_trainer.py:294-391: `add_time_ids`, timestep bias :326-335, min-SNR :371-378), SD `_train_step`
(stable_diffusion_trainer.py:253-358) and Dreambooth prior-preservation loss (dreambooth_trainer.py:252-337).
The batch holds either cached latents + text embeddings (`cache_latents_text_encoder_outputs`) or pixels + token ids
that go through the frozen VAE / text encoders first.
"""
from __future__ import annotations

import time
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import max_logging
from ..max_utils import create_optimizer
from ..models.unet_2d_condition import UNET_PRESETS, UNet2DConditionModel, UNetConfig
from ..parallel.fsdp import FlatShardedOptimizer, lr_schedule
from ..parallel.mesh import create_device_mesh
from ..schedulers.scheduling_ddpm import DDPMScheduler
from ..train_utils import MetricsWriter, compute_snr, generate_timestep_weights


def get_add_time_ids(original_size, crops_coords_top_left, target_size, batch: int, device=None, dtype=torch.float32):
  """SDXL micro-conditioning ids [B, 6] (reference: maxdiffusion_utils.py:143)."""
  ids = torch.tensor(list(original_size) + list(crops_coords_top_left) + list(target_size), device=device, dtype=dtype)
  return ids[None].expand(batch, -1)


def resolve_unet_config(config) -> UNetConfig:
  preset = str(config.get("unet_preset", "") or ("sdxl" if "xl" in str(config.get("pretrained_model_name_or_path", "")).lower() else "sd15"))
  d = dict(UNET_PRESETS[preset])
  d.update(config.get("unet_config_overrides", None) or {})
  return UNetConfig(**d)


class StableDiffusionTrainer:
  is_xl = False

  def __init__(self, config, mesh=None, unet: Optional[UNet2DConditionModel] = None, vae=None, text_encoders=(), device=None,
               tokenizers=()):
    self.config = config
    self.mesh = mesh if mesh is not None else create_device_mesh(config)
    self.device = torch.device(device) if device is not None else (
        torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    self.dtype = config.weights_dtype if self.device.type == "cuda" else torch.float32
    seed = int(config.get("seed", 0))
    if unet is None:
      torch.manual_seed(seed)
      prev = torch.get_default_dtype()
      torch.set_default_dtype(self.dtype)
      try:
        with torch.device(self.device):
          unet = UNet2DConditionModel(resolve_unet_config(config))
      finally:
        torch.set_default_dtype(prev)
    self.unet = unet.to(self.device, self.dtype)
    self.vae, self.text_encoders, self.tokenizers = vae, list(text_encoders), list(tokenizers)
    group = self.mesh.group("replica") if self.mesh.size("fsdp") == 1 else dist.group.WORLD if dist.is_initialized() else None
    # `train_text_encoder`: the (first) text encoder is trained along with the UNet, in the same flat optimizer
    # (reference: src/maxdiffusion/trainers/stable_diffusion_trainer.py:84-117, dreambooth_trainer.py:150-170)
    self.train_text_encoder = bool(config.get("train_text_encoder", False)) and len(self.text_encoders) > 0
    params = list(self.unet.parameters())
    if self.train_text_encoder:
      params += [p for p in self.text_encoders[0].parameters() if p.requires_grad]
    self.optimizer = FlatShardedOptimizer(params, create_optimizer(config), group=group, seed=seed)
    self.seed = seed
    sc = dict(config.get("diffusion_scheduler_config", {}) or {})
    self.prediction_type = sc.get("prediction_type") or "epsilon"  # empty = keep the pretrained scheduler's own
    self.scheduler = DDPMScheduler(beta_start=0.00085, beta_end=0.012, beta_schedule="scaled_linear",
                                   prediction_type=self.prediction_type,
                                   rescale_zero_terminal_snr=bool(sc.get("rescale_zero_terminal_snr", False)))
    self.sched_state = self.scheduler.create_state()
    self.timestep_weights = generate_timestep_weights(config, 1000)
    self.gen = torch.Generator(device=self.device).manual_seed(seed + 1 + 7919 * self.mesh.rank)
    self.step = 0
    # forward + backward as one CUDA graph: only for the plain objective (Dreambooth's two-term loss and a trained
    # text encoder run eagerly) on a GPU
    self._graphed = None
    if (bool(config.get("cuda_graph_train_step", False)) and self.device.type == "cuda" and not self.train_text_encoder
        and type(self).loss is StableDiffusionTrainer.loss):
      from .graphed_step import GraphedObjective

      self._graphed = GraphedObjective(self.objective, list(self.unet.parameters()))
    self.snr_gamma = float(config.get("snr_gamma", -1.0))
    self.batch_size = max(1, int(float(config.get("per_device_batch_size", 1))))

  # ---- conditioning -----------------------------------------------------------------------
  def encode_batch(self, batch: dict) -> dict:
    """Latents and text embeddings from pixels / token ids when they are not cached in the dataset."""
    out = dict(batch)
    if "captions" in out and "input_ids" not in out and "encoder_hidden_states" not in out:
      for i, tok in enumerate(self.tokenizers):
        ids = tok(list(out["captions"]), padding="max_length", max_length=getattr(tok, "model_max_length", 77),
                  truncation=True, return_tensors="pt").input_ids
        out[f"input_ids{'' if i == 0 else '_2'}"] = ids
    if "latents" not in out:
      with torch.no_grad():
        dist_ = self.vae.encode(out["pixel_values"].to(self.device, next(self.vae.parameters()).dtype))
        out["latents"] = self.vae.scale_latents(dist_.sample(self.gen))
    if "encoder_hidden_states" not in out:
      with torch.set_grad_enabled(self.train_text_encoder and torch.is_grad_enabled()):
        hs, pooled = [], None
        for i, enc in enumerate(self.text_encoders):
          o = enc(out[f"input_ids{'' if i == 0 else '_2'}"].to(self.device), output_hidden_states=True)
          hs.append(o.hidden_states[-2] if self.is_xl else o.last_hidden_state)
          pooled = getattr(o, "text_embeds", None) if i == len(self.text_encoders) - 1 else pooled
        out["encoder_hidden_states"] = torch.cat(hs, dim=-1)
        if pooled is not None:
          out["text_embeds"] = pooled
    return out

  # ---- step -------------------------------------------------------------------------------
  def draw(self, batch: dict) -> dict:
    """Everything random or data dependent of a step, as tensors: the noised latents, the timesteps, the regression
    target, the per-sample loss weights and the conditioning. What remains (`objective`) is a fixed sequence of
    kernels on fixed shapes."""
    latents = batch["latents"].to(self.device, torch.float32)
    B = latents.shape[0]
    noise = torch.randn(latents.shape, generator=self.gen, device=self.device)
    w = self.timestep_weights.to(self.device)
    timesteps = torch.multinomial(w, B, replacement=True, generator=self.gen)
    noisy = self.scheduler.add_noise(self.sched_state, latents, noise, timesteps)
    out = {"noisy": noisy.to(self.dtype), "timesteps": timesteps,
           "encoder_hidden_states": batch["encoder_hidden_states"].to(self.device)}
    if self.is_xl:
      res = int(self.config.get("resolution", 1024))
      time_ids = batch.get("time_ids")
      if time_ids is None:
        time_ids = get_add_time_ids((res, res), (0, 0), (res, res), B, self.device)
      out["text_embeds"], out["time_ids"] = batch["text_embeds"].to(self.device), time_ids.to(self.device)
    if self.prediction_type == "epsilon":
      out["target"] = noise
    elif self.prediction_type == "v_prediction":
      out["target"] = self.scheduler.get_velocity(self.sched_state, latents, noise, timesteps)
    else:
      raise ValueError(self.prediction_type)
    if self.snr_gamma > 0:
      snr = compute_snr(self.sched_state.common.alphas_cumprod, timesteps)
      weights = torch.minimum(snr, torch.full_like(snr, self.snr_gamma)) / snr
      if self.prediction_type == "v_prediction":
        weights = weights * snr / (snr + 1)
      out["weights"] = weights
    return out

  def objective(self, noisy, timesteps, encoder_hidden_states, target, text_embeds=None, time_ids=None, weights=None):
    added = {"text_embeds": text_embeds, "time_ids": time_ids} if text_embeds is not None else None
    pred = self.unet(noisy, timesteps, encoder_hidden_states, added).float()
    loss = (target - pred) ** 2
    if weights is not None:
      loss = loss.mean(dim=(1, 2, 3)) * weights
    return loss.mean()

  def loss(self, batch: dict) -> torch.Tensor:
    return self.objective(**self.draw(batch))

  def train_step(self, batch: dict) -> dict:
    batch = self.encode_batch({k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()})
    lr = lr_schedule(self.step, float(self.config.learning_rate), int(self.config.learning_rate_schedule_steps),
                     float(self.config.warmup_steps_fraction))
    # the noise / timestep stream is a function of (seed, rank, step): a resumed run continues it exactly
    self.gen.manual_seed(self.seed + 1 + 7919 * self.mesh.rank + 1000003 * self.step)
    if self._graphed is not None:
      loss = self._graphed(self.draw(batch))  # forward + backward replayed from a CUDA graph
    else:
      loss = self.loss(batch)
      loss.backward()
    stats = self.optimizer.step(lr)
    self.step += 1
    return {"learning/loss": loss.detach(), "learning/grad_norm": stats["grad_norm"], "learning/current_learning_rate": lr}

  def synthetic_batch(self, index: Optional[int] = None) -> dict:
    cfg = self.unet.cfg
    g = torch.Generator().manual_seed((self.step if index is None else index) + 17 + 7919 * self.mesh.rank)
    lat = int(self.config.get("resolution", 1024)) // 8
    b = {"latents": torch.randn((self.batch_size, cfg.in_channels, lat, lat), generator=g),
         "encoder_hidden_states": torch.randn((self.batch_size, 77, cfg.cross_attention_dim), generator=g)}
    if self.is_xl:
      b["text_embeds"] = torch.randn((self.batch_size, cfg.projection_class_embeddings_input_dim - 6 * cfg.addition_time_embed_dim), generator=g)
    return {k: (v.pin_memory() if torch.cuda.is_available() else v) for k, v in b.items()}

  def load_dataset(self):
    """The configured input pipeline (`dataset_type`: synthetic, tfrecord, hf, grain), sharded over the data ranks."""
    if str(self.config.get("dataset_type", "synthetic")) == "synthetic":
      def synthetic(i=self.step):  # batch i is a function of i alone: a resumed run sees the batches it would have seen
        while True:
          yield self.synthetic_batch(i)
          i += 1
      return synthetic()
    from ..input_pipeline.input_pipeline_interface import make_data_iterator

    return make_data_iterator(self.config, self.mesh, self.batch_size)

  def checkpointer(self):
    from ..checkpointing.base_stable_diffusion_checkpointer import BaseStableDiffusionCheckpointer

    c = self.config
    if int(c.get("checkpoint_every", -1)) > 0 or c.get("save_final_checkpoint", False):
      return BaseStableDiffusionCheckpointer(c)
    return None

  def start_training(self, data=None):
    """Resume -> (cached) data -> steps with metrics -> periodic / final checkpoints
    (reference: base_stable_diffusion_trainer.py:115-197)."""
    from .loop import EncodedBatchCache, run_training_loop

    def build():
      it = data if data is not None else self.load_dataset()
      if (self.config.get("cache_latents_text_encoder_outputs", False) and self.vae is not None and not self.train_text_encoder
          and str(self.config.get("dataset_type", "synthetic")) != "synthetic"):
        it = EncodedBatchCache(iter(it), self.encode_batch)
      return it

    return run_training_loop(self, build, self.checkpointer())


class StableDiffusionXLTrainer(StableDiffusionTrainer):
  is_xl = True


class DreamboothTrainer(StableDiffusionTrainer):
  """Instance + class (prior-preservation) batches: the two halves of the batch get separate MSE terms and the
  class term is weighted by `prior_loss_weight`."""

  def generate_class_images(self, pipeline, class_dir: Optional[str] = None) -> int:
    """Fills `class_data_dir` up to `num_class_images` pictures of `class_prompt` sampled from the model being
    fine-tuned, before training starts (reference: dreambooth_trainer.py:94-147). Returns how many were generated."""
    import os

    from PIL import Image

    c = self.config
    class_dir = class_dir or str(c.get("class_data_dir", ""))
    want = int(c.get("num_class_images", 0))
    if not class_dir or want <= 0:  # the reference's Dreambooth always trains with prior preservation
      return 0
    os.makedirs(class_dir, exist_ok=True)
    have = len([f for f in os.listdir(class_dir) if f.lower().endswith((".png", ".jpg", ".jpeg"))])
    made = 0
    bs = max(1, int(c.get("class_images_batch_size", 0) or self.batch_size))
    while have + made < want:
      n = min(bs, want - have - made)
      imgs = pipeline(prompt=[str(c.get("class_prompt", ""))] * n, seed=int(c.get("seed", 0)) + have + made)
      imgs = imgs.cpu().numpy() if torch.is_tensor(imgs) else imgs
      for img in imgs:
        Image.fromarray(img).save(os.path.join(class_dir, f"class_{have + made:05d}.png"))
        made += 1
    return made

  def load_dataset(self):
    """Instance / class image folders when `instance_data_dir` and `class_data_dir` are set (the Dreambooth data set of
    the reference), else the configured input pipeline."""
    c = self.config
    if str(c.get("instance_data_dir", "") or "") and str(c.get("class_data_dir", "") or "") and \
        str(c.get("dataset_type", "synthetic")) != "synthetic":
      from ..input_pipeline.input_pipeline_interface import make_dreambooth_train_iterator

      return make_dreambooth_train_iterator(c, self.mesh, self.batch_size)
    return super().load_dataset()

  def loss(self, batch: dict) -> torch.Tensor:
    if not any(k.startswith("class_") for k in batch):
      return super().loss(batch)
    inst = {k: v for k, v in batch.items() if not k.startswith("class_")}
    cls = {k[len("class_"):]: v for k, v in batch.items() if k.startswith("class_")}
    return super().loss(inst) + float(self.config.get("prior_loss_weight", 1.0)) * super().loss(cls)
