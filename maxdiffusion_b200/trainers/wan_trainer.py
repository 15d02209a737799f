"""Wan 2.1 text-to-video training: flow-matching MSE, per-block remat, FSDP x context parallelism.

Flow of one step (reference: src/maxdiffusion/trainers/wan_trainer.py:136-189 and
src/maxdiffusion/trainers/base_wan_trainer.py:256-374):
  host batch (pinned) -> device, sample shifted timesteps, noise, `apply_flow_match` -> model forward on this
  rank's token shard -> weighted MSE against the sharded target -> backward, during which every block's
  gradients are reduce-scattered and its AdamW update applied (`parallel.fsdp`) -> replicated root parameters ->
  metrics (`learning/loss`, `learning/max_grad_norm`, `learning/max_abs_grad`, step time, TFLOP/s).
"""
from __future__ import annotations

import os
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Optional

import torch
import torch.distributed as dist

from ..models.gradient_checkpoint import resolve_remat
from ..ops import _lib
from ..ops import functional as OF

from .. import max_logging
from ..input_pipeline.synthetic_data_iterator import make_synthetic_iterator
from ..models.wan.transformer_wan import WAN_PRESETS, WanConfig, WanModel
from ..parallel.context import ContextParallel
from ..parallel.fsdp import AdamWConfig, FSDPEngine, lr_schedule
from ..parallel.mesh import DeviceMesh, create_device_mesh
from ..schedulers.scheduling_flow_match import FlowMatchScheduler


def wan_train_tflops(cfg: WanConfig, seq_len: int, batch: float, text_len: int = 512) -> float:
  """Analytic training TFLOPs per step (3x forward), the reference's own model
  (src/maxdiffusion/trainers/base_wan_trainer.py:107-155)."""
  d = cfg.dim
  attn = (3 * 2 * seq_len * d * d + 2 * 2 * seq_len * seq_len * d + 3 * 2 * text_len * d * d + 2 * seq_len * d * d +
          2 * 2 * seq_len * text_len * d + 2 * 2 * seq_len * d * d)
  ffn = 2 * 2 * seq_len * d * cfg.ffn_dim
  return 3 * batch * (attn + ffn) * cfg.num_layers / 1e12


def resolve_wan_config(config) -> WanConfig:
  preset = str(config.get("wan_preset", "") or "")
  if not preset:
    name = str(config.get("pretrained_model_name_or_path", "")).lower()
    preset = "wan2.1-t2v-1.3b" if "1.3b" in name else ("wan2.1-i2v-14b" if "i2v" in name else "wan2.1-t2v-14b")
  cfg = dict(WAN_PRESETS[preset])
  override = config.get("wan_config_overrides", None)
  if override:
    cfg.update(override)
  return WanConfig(**cfg)


class WanTrainer:
  model_cls = WanModel
  resolve_config = staticmethod(resolve_wan_config)

  def model_kwargs(self, batch: dict) -> dict:
    """Extra keyword arguments of the model call taken from the batch (subclasses: control latents)."""
    return {}

  def __init__(self, config, mesh: Optional[DeviceMesh] = None, model: Optional[WanModel] = None, device=None):
    self.config = config
    self.device = torch.device(device) if device is not None else torch.device(
        "cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    self.mesh = mesh if mesh is not None else create_device_mesh(config)
    self.dtype = config.weights_dtype if self.device.type == "cuda" else torch.float32
    self.wan_cfg = model.cfg if model is not None else self.resolve_config(config)
    seed = int(config.get("seed", 0))
    remat = resolve_remat(config.get("remat_policy", "NONE"), config.get("names_which_can_be_saved", []) or [],
                          config.get("names_which_can_be_offloaded", []) or [])
    if self.mesh.world_size > 1 and remat == "NONE":
      remat = "SAVE_ATTENTION"  # sharded weights are only resident around a block's (re)computation
    if model is None:
      torch.manual_seed(seed)
      prev = torch.get_default_dtype()
      torch.set_default_dtype(self.dtype)
      try:
        with torch.device(self.device):
          model = self.model_cls(self.wan_cfg, remat_policy=remat)
      finally:
        torch.set_default_dtype(prev)
    else:
      model = model.to(device=self.device, dtype=self.dtype)
      model.remat_policy = remat
    model.remat_keep_blocks = int(config.get("remat_keep_blocks", 0) or 0)
    if self.mesh.size("tensor") > 1:
      # every rank built the same full model (same seed): keep this rank's heads and FFN units of every block
      from ..parallel.tensor import apply_tensor_parallel_wan

      apply_tensor_parallel_wan(model, self.mesh.group("tensor"))
    self.model = model

    opt = AdamWConfig(
        lr=float(config.get("learning_rate", 1e-5)), b1=float(config.get("adam_b1", 0.9)),
        b2=float(config.get("adam_b2", 0.999)), eps=float(config.get("adam_eps", 1e-8)),
        weight_decay=float(config.get("adam_weight_decay", 0.0)),
        clip_value=float(config.get("max_grad_value", 1.0)) if config.get("opt_enable_grad_clipping", False) else 0.0,
        clip_global_norm=float(config.get("max_grad_norm", 1.0)) if config.get("opt_enable_grad_global_norm_clipping", False) else 0.0,
        state_dtype=config.get("opt_state_dtype", self.dtype) if self.device.type == "cuda" else torch.float32,
        stochastic_rounding=bool(config.get("stochastic_rounding", True)))
    block_param_ids = {id(p) for b in model.blocks for p in b.parameters()}
    root_params = [p for p in model.parameters() if id(p) not in block_param_ids]
    shard_group = self.mesh.group("shard")
    replica_group = self.mesh.group("replica")
    self.engine = FSDPEngine(model.blocks, root_params, opt, group=shard_group, replica_group=replica_group,
                             device=self.device, param_dtype=self.dtype, seed=seed,
                             peer_memory=bool(config.get("peer_memory_transport", True)))
    model.block_hook = self.engine.block_hook
    self.pctx = None
    fixed_m = bool(config.get("fixed_m_softmax", False))
    if self.mesh.size("context") > 1 or fixed_m:
      # a one-rank context still goes through ContextParallel when the fixed-exponent softmax is selected
      self.pctx = ContextParallel(self.mesh, str(config.get("context_strategy", "ring")),
                                  peer_memory=bool(config.get("peer_memory_transport", True)) and self.device.type == "cuda",
                                  fixed_m=fixed_m, save_remote_kv=bool(config.get("ring_save_remote_kv", True)), ulysses_chunks=int(config.get("ulysses_attention_chunks", 1)),
                                  kv_transport=str(config.get("ring_kv_transport", "dma")))

    self.scheduler = FlowMatchScheduler(num_train_timesteps=1000, shift=float(config.get("flow_shift", 3.0)))
    self.scheduler_state = self.scheduler.set_timesteps(self.scheduler.create_state(), 1000, training=True, device=self.device)
    self.gen = torch.Generator(device=self.device).manual_seed(seed + 1 + 7919 * (self.mesh.coords.get('data', 0) * self.mesh.size('fsdp') + self.mesh.coords.get('fsdp', 0)))
    self.step = 0
    self.base_lr = opt.lr
    self.schedule_steps = int(config.get("learning_rate_schedule_steps", 0) or config.get("max_train_steps", 1))
    self.warmup_fraction = float(config.get("warmup_steps_fraction", 0.0))
    self.use_weights = not bool(config.get("disable_training_weights", False))
    # samples per (data, fsdp) replica: the context x tensor ranks of a replica work on the same samples
    self.batch_size = max(1, int(round(float(config.get("per_device_batch_size", 1)) * self.mesh.size("context") *
                                       self.mesh.size("tensor"))))

  # ------------------------------------------------------------------ data
  def load_dataset(self):
    dataset_type = str(self.config.get("dataset_type", "synthetic"))
    if dataset_type == "synthetic":
      # ranks along `data` x `fsdp` draw different samples; the context / tensor ranks of a replica draw the same ones
      return make_synthetic_iterator(self.config, self.batch_size,
                                     seed=int(self.config.get("seed", 0)) + 17 + 1009 * self.batch_index())
    from ..input_pipeline.input_pipeline_interface import make_data_iterator

    return make_data_iterator(self.config, self.mesh, self.batch_size)

  def batch_index(self) -> int:
    """Index of this rank's replica among the `data` x `fsdp` ranks that hold different samples."""
    return self.mesh.coords.get("data", 0) * self.mesh.size("fsdp") + self.mesh.coords.get("fsdp", 0)

  def to_device(self, batch: dict) -> dict:
    out = {}
    for k, v in batch.items():
      if torch.is_tensor(v):
        out[k] = v.to(self.device, non_blocking=True)
      else:
        out[k] = v
    return out

  # ------------------------------------------------------------------ step
  def train_step(self, batch: dict, host_inputs: bool = True) -> dict:
    """One optimizer step. `batch` holds host (pinned) or device tensors; returns device-side metrics."""
    cfg = self.wan_cfg
    if host_inputs:
      batch = self.to_device(batch)
    latents = batch["latents"].to(self.dtype)
    text = batch["encoder_hidden_states"].to(self.dtype)
    B = latents.shape[0]
    lr = lr_schedule(self.step, self.base_lr, self.schedule_steps, self.warmup_fraction)
    self.engine.begin_step(lr)

    # a batch may bring its own timesteps and noise (evaluation at fixed timesteps, reproducible comparisons)
    timesteps = batch.get("timesteps")
    if timesteps is None:
      timesteps = self.scheduler.sample_timesteps(B, generator=self.gen, device=self.device)
    noise = batch.get("noise")
    if noise is None:
      noise = torch.randn(latents.shape, generator=self.gen, device=self.device, dtype=torch.float32)
    noise = noise.to(self.dtype)
    noisy, target, weights = self.scheduler.apply_flow_match(noise.float(), latents.float(), timesteps, self.scheduler_state)

    pred = self.model(noisy.to(self.dtype), timesteps, text, pctx=self.pctx, return_tokens=True,
                      **self.model_kwargs(batch))  # [B,S_loc,P]
    tgt_tokens, _ = self.model.patchify(target, channel_last=True)
    total = tgt_tokens.numel()
    if self.pctx is not None:
      full_len = tgt_tokens.shape[1]
      tgt_tokens = self.pctx.shard_sequence(tgt_tokens)
      valid = self.pctx.valid_lengths(self.pctx.size, tgt_tokens.shape[1])[self.pctx.rank]
      pred_all = pred
      pred, tgt_tokens = pred[:, :valid], tgt_tokens[:, :valid]
    # weighted squared error and its gradient in one fused pass; normalised by the global element count so that
    # the per-rank losses of a sequence-sharded step add up to the mean
    if pred.numel() == 0:
      # a rank whose shard is padding only (tiny sequences on many ranks): no loss, but the graph still runs so that
      # every rank takes part in the collectives of the backward pass
      local = pred_all.float().sum() * 0.0
    else:
      local = OF.weighted_mse(pred, tgt_tokens, weights.tolist() if self.use_weights else None)
    # Ranks along `data` and `fsdp` hold different samples and their gradients are summed by the reduce-scatter and
    # the replica all-reduce, so each rank's share is divided by the number of batch replicas: the applied gradient,
    # the logged norm and the clipping thresholds then refer to the mean over the global batch, as in the reference
    # (src/maxdiffusion/trainers/wan_trainer.py:150-168, a mean over the batch axis of the global array).
    replicas = self.mesh.size("data") * self.mesh.size("fsdp")
    loss = local * (pred.numel() / total / replicas)
    loss.backward()
    # replicated (root) parameters see different tokens / samples on the ranks of the shard group; the tensor ranks of a
    # replica compute identical gradients for them, so the tensor axis is not summed over
    stats = self.engine.finish_step(model_group=self.mesh.group("shard"))
    loss_value = loss.detach()
    if self.mesh.world_size > 1:
      loss_value = loss_value.clone()
      for name in ("model", "replica"):
        if self.mesh.group(name) is not None:
          dist.all_reduce(loss_value, group=self.mesh.group(name))
      loss_value = loss_value / self.mesh.size("tensor")  # tensor ranks of a replica repeat the same partial loss
    self.step += 1
    return {"learning/loss": loss_value, "learning/max_grad_norm": stats["grad_norm"],
            "learning/max_abs_grad": stats["max_abs_grad"], "learning/current_learning_rate": lr}

  # ------------------------------------------------------------------ evaluation
  @torch.no_grad()
  def eval_step(self, batch: dict, host_inputs: bool = True) -> torch.Tensor:
    """Per-sample loss [B] of a batch that brings its own `timesteps`, without touching the weights: the training
    objective (flow-matching target, timestep weights unless `disable_training_weights`) averaged over everything but
    the batch axis (reference: src/maxdiffusion/trainers/wan_trainer.py:192-243, `eval_step`)."""
    if host_inputs:
      batch = self.to_device(batch)
    latents = batch["latents"].to(self.dtype)
    text = batch["encoder_hidden_states"].to(self.dtype)
    timesteps = batch["timesteps"].to(self.device)
    noise = batch.get("noise")
    if noise is None:
      noise = torch.randn(latents.shape, generator=self.gen, device=self.device, dtype=torch.float32)
    noisy, target, weights = self.scheduler.apply_flow_match(noise.float(), latents.float(), timesteps, self.scheduler_state)
    was_training = self.model.training
    self.model.eval()
    try:
      pred = self.model(noisy.to(self.dtype), timesteps, text, pctx=self.pctx, return_tokens=True, **self.model_kwargs(batch))
    finally:
      self.model.train(was_training)
    tgt, _ = self.model.patchify(target, channel_last=True)
    total = tgt[0].numel()
    if self.pctx is not None:
      tgt = self.pctx.shard_sequence(tgt)
      valid = self.pctx.valid_lengths(self.pctx.size, tgt.shape[1])[self.pctx.rank]
      pred, tgt = pred[:, :valid], tgt[:, :valid]
    err = (pred.float() - tgt.float()).pow(2).flatten(1).sum(dim=1) / total   # this rank's share of every sample's mean
    if self.use_weights:
      err = err * weights.to(err)
    if self.mesh.world_size > 1 and self.mesh.group("model") is not None:
      dist.all_reduce(err, group=self.mesh.group("model"))                 # the sequence / tensor shards of a sample
      err = err / self.mesh.size("tensor")
    return err

  def eval(self, step: int, writer=None) -> Optional[float]:
    """Evaluation pass over the evaluation split: the per-sample losses are grouped by timestep, every group is cut to
    `eval_max_number_of_samples_in_bucket` samples and averaged, and the mean of the group means is logged as
    `learning/eval_loss` (reference: src/maxdiffusion/trainers/base_wan_trainer.py:209-255)."""
    from ..input_pipeline.input_pipeline_interface import make_data_iterator

    data = make_data_iterator(self.config, self.mesh, self.batch_size, eval_mode=True)
    by_t: dict = {}
    for batch in data:
      t0 = time.perf_counter()
      losses, ts = self.eval_step(batch), batch["timesteps"].to(self.device)
      replicas = self.mesh.group("replica")
      if self.mesh.world_size > 1 and replicas is not None:
        n = dist.get_world_size(replicas)
        all_l = [torch.empty_like(losses) for _ in range(n)]
        all_t = [torch.empty_like(ts) for _ in range(n)]
        dist.all_gather(all_l, losses, group=replicas)
        dist.all_gather(all_t, ts, group=replicas)
        losses, ts = torch.cat(all_l), torch.cat(all_t)
      for t, l in zip(ts.flatten().tolist(), losses.flatten().tolist()):
        by_t.setdefault(int(t), []).append(float(l))
      max_logging.log(f"Eval time: {time.perf_counter() - t0:.2f} seconds.")
    if not by_t:
      return None
    cap = int(self.config.get("eval_max_number_of_samples_in_bucket", 60))
    means = []
    for t, values in sorted(by_t.items()):
      values = values[:min(cap, len(values))] if cap > 0 else values
      means.append(sum(values) / len(values))
      max_logging.log(f"  Mean eval loss for timestep {t}: {means[-1]:.4f}")
    final = sum(means) / len(means)
    max_logging.log(f"Step {step}, Final Average Eval loss: {final:.4f}")
    if writer is not None:
      writer.write(step, {"learning/eval_loss": final})
    return final

  def _save(self, checkpointer, monitor) -> None:
    """Checkpoint write bracketed by a device-status check and a host-side barrier: saving is a rank-asymmetric host
    phase (rank 0 writes for seconds), and the peers' next kernels must not start their bounded waits on a rank
    that is still writing."""
    _lib.raise_on_device_status_if_loaded()
    checkpointer.save(self.step, self)
    if monitor is not None:
      monitor.barrier()
    elif self.mesh.world_size > 1:
      dist.barrier()

  # ------------------------------------------------------------------ loop
  def seq_len(self) -> int:
    c = self.config
    pt, ph, pw = self.wan_cfg.patch_size
    return ((int(c.get("num_frames", 81)) - 1) // 4 + 1) // pt * (int(c.get("height", 480)) // 8 // ph) * (int(c.get("width", 832)) // 8 // pw)

  def start_training(self):
    from ..train_utils import MetricsWriter, load_next_batch

    config = self.config
    data = self.load_dataset()
    writer = MetricsWriter(config, self.mesh.rank)
    tflops = wan_train_tflops(self.wan_cfg, self.seq_len(), float(self.batch_size) * self.mesh.size("data") * self.mesh.size("fsdp"))
    per_device = tflops / self.mesh.world_size
    max_logging.log(f"Calculated TFLOPs per pass: {tflops:.4f} ({per_device:.4f} per device)")
    max_steps = int(config.get("max_train_steps", 1))
    pool = ThreadPoolExecutor(max_workers=1)
    reuse = {"batch": None}   # `reuse_example_batch`: the first batch is served for every step

    def fetch():
      reuse["batch"] = load_next_batch(data, reuse["batch"], config)
      return reuse["batch"]

    nxt = pool.submit(fetch)
    checkpointer = None
    if int(config.get("checkpoint_every", -1)) > 0 or config.get("save_final_checkpoint", False):
      from ..checkpointing.wan_checkpointer import WanCheckpointer

      checkpointer = WanCheckpointer(config)
      restored = checkpointer.maybe_restore(self)
      if restored is not None:
        self.step = restored
    profiler = None
    if config.get("enable_profiler", False):
      from ..max_utils import Profiler

      profiler = Profiler(config)
    monitor = None
    if self.mesh.world_size > 1 and config.get("enable_health_monitor", True):
      from ..parallel.health import HealthMonitor

      monitor = HealthMonitor(timeout_s=float(config.get("health_timeout_seconds", 600.0))).start()
    from ..parallel.health import guarded_step

    while self.step < max_steps:
      batch = nxt.result()
      nxt = pool.submit(fetch)
      if profiler is not None:
        profiler.maybe_start(self.step)
      t0 = time.perf_counter()
      with guarded_step(monitor, self.step):  # peers are checked on the host before this step's first launch
        metrics = self.train_step(batch)
        loss = float(metrics["learning/loss"])  # device -> host, ends the step
        # a device-side wait that ran out (a peer that stopped signalling) left stale data behind: raise here, inside
        # the guard, so that the peers learn of it and nothing of this step reaches a checkpoint
        _lib.raise_on_device_status_if_loaded()
      dt = time.perf_counter() - t0
      if profiler is not None:
        profiler.maybe_stop(self.step)
      scalars = {k: float(v) for k, v in metrics.items()}
      scalars.update({"perf/step_time_seconds": dt, "perf/per_device_tflops": per_device,
                      "perf/per_device_tflops_per_sec": per_device / dt})
      writer.write(self.step, scalars)
      eval_every = int(config.get("eval_every", -1))
      if eval_every > 0 and self.step % eval_every == 0 and str(config.get("dataset_type", "synthetic")) != "synthetic":
        self.eval(self.step, writer)
      if checkpointer is not None and int(config.get("checkpoint_every", -1)) > 0 and self.step % int(config.checkpoint_every) == 0:
        self._save(checkpointer, monitor)
    if checkpointer is not None and config.get("save_final_checkpoint", False):
      self._save(checkpointer, monitor)
    writer.close()
    if monitor is not None:
      monitor.stop()
    pool.shutdown(wait=False, cancel_futures=True)
    return self
