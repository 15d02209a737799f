"""Flux and Stable Diffusion families on CPU: training steps, checkpoint round trips, and every generate entry point
on tiny random-init configurations."""
import os

import pytest
import torch

from maxdiffusion_b200 import pyconfig
from maxdiffusion_b200.parallel.mesh import create_device_mesh

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs")
TINY_VAE = '{"block_out_channels":[32,32],"layers_per_block":1,"norm_num_groups":8}'
FLUX = ["random_init=True", "flux_preset=tiny", f"vae_config_overrides={TINY_VAE}", "resolution=64", "max_sequence_length=8",
        "num_inference_steps=2", "log_config=false", "write_metrics=false", "dataset_type=synthetic"]
SD = ["random_init=True", 'vae_config_overrides={"block_out_channels":[32,32],"layers_per_block":1,"norm_num_groups":8,"latent_channels":4}',
      "resolution=32", "num_inference_steps=2", "log_config=false", "write_metrics=false", "dataset_type=synthetic",
      "per_device_batch_size=2"]


def _cfg(name, extra, tmp):
  if "flux" not in name and not any(e.startswith("unet_preset") for e in extra):
    extra = list(extra) + ["unet_preset=" + ("tiny" if "xl" in name else "tiny_sd")]
  return pyconfig.initialize(["x", os.path.join(CFG, name), f"output_dir={tmp}/out", f"checkpoint_dir={tmp}/ckpt", *extra], unittest=True)


def test_flux_train_step_and_checkpoint_round_trip(tmp_path):
  from maxdiffusion_b200.checkpointing.flux_checkpointer import FluxCheckpointer
  from maxdiffusion_b200.trainers.flux_trainer import FluxTrainer

  config = _cfg("base_flux_dev.yml", FLUX + ["save_optimizer=true", "learning_rate=1e-3"], tmp_path)
  tr = FluxTrainer(config, mesh=create_device_mesh(config), device="cpu")
  data = tr.load_dataset()
  b0, b1 = next(data), next(data)
  l0 = float(tr.train_step(b0)["learning/loss"])
  assert l0 == l0
  ck = FluxCheckpointer(config)
  ck.save(1, tr)
  ck.manager.wait_until_finished()
  config2 = _cfg("base_flux_dev.yml", FLUX + ["save_optimizer=true", "learning_rate=1e-3"], tmp_path)
  tr2 = FluxTrainer(config2, mesh=create_device_mesh(config2), device="cpu")
  with torch.no_grad():
    for p in tr2.model.parameters():
      p.add_(0.25)  # everything must come from the checkpoint
  assert FluxCheckpointer(config2).maybe_restore(tr2) == 1
  tr2.step = 1  # what the training loop does after a restore; the noise stream is a function of (seed, step)
  assert float(tr.train_step(b1)["learning/loss"]) == float(tr2.train_step(b1)["learning/loss"])
  pipe = FluxCheckpointer(config2).load_pipeline(device="cpu")
  saved = ck.manager.restore_state(1, "flux_state")
  for n, p in pipe.transformer.state_dict().items():
    assert torch.allclose(p, saved[n].to(p.dtype)), n


def test_flux_generate_entry_points(tmp_path):
  from maxdiffusion_b200 import generate_flux, generate_flux_multi_res, generate_flux_pipeline

  img = generate_flux.run(_cfg("base_flux_schnell.yml", FLUX, tmp_path))
  assert img.shape[0] == 1 and img.dtype == torch.uint8
  img2 = generate_flux_pipeline.run(_cfg("base_flux_dev.yml", FLUX + ["checkpoint_dir="], tmp_path))
  assert img2.shape == img.shape
  res = generate_flux_multi_res.run(_cfg("base_flux_dev_multi_res.yml", FLUX + ["resolutions=[[64,64],[32,64]]"], tmp_path))
  assert len(res) == 2 and os.path.exists(os.path.join(tmp_path, "out", "flux_32x64_0.png"))


@pytest.mark.parametrize("entry,cfg", [("train", "base15.yml"), ("train_sdxl", "base_xl.yml"), ("dreambooth", "base14.yml")])
def test_sd_train_steps_and_checkpoint(entry, cfg, tmp_path):
  from maxdiffusion_b200.checkpointing.base_stable_diffusion_checkpointer import BaseStableDiffusionCheckpointer
  from maxdiffusion_b200.trainers.stable_diffusion_trainer import DreamboothTrainer, StableDiffusionTrainer, StableDiffusionXLTrainer

  cls = {"train": StableDiffusionTrainer, "train_sdxl": StableDiffusionXLTrainer, "dreambooth": DreamboothTrainer}[entry]
  config = _cfg(cfg, SD + ["save_optimizer=true", "learning_rate=1e-3"], tmp_path)
  tr = cls(config, mesh=create_device_mesh(config), device="cpu")
  b = tr.synthetic_batch()
  l0 = float(tr.train_step(b)["learning/loss"])
  assert l0 == l0
  ck = BaseStableDiffusionCheckpointer(config)
  ck.save(1, tr)
  ck.manager.wait_until_finished()
  tr2 = cls(_cfg(cfg, SD + ["save_optimizer=true", "learning_rate=1e-3"], tmp_path), device="cpu")
  with torch.no_grad():
    for p in tr2.unet.parameters():
      p.add_(0.25)  # everything must come from the checkpoint
  assert BaseStableDiffusionCheckpointer(config).maybe_restore(tr2) == 1
  tr2.step = 1
  for (n, p), (_, q) in zip(tr.unet.named_parameters(), tr2.unet.named_parameters()):
    assert torch.equal(p, q), n
  assert tr2.optimizer.step_count == 1 and torch.equal(tr.optimizer.m, tr2.optimizer.m)
  assert float(tr.train_step(b)["learning/loss"]) == float(tr2.train_step(b)["learning/loss"])


def test_sd_generate_entry_points(tmp_path):
  from maxdiffusion_b200 import generate, generate_sdxl, generate_sdxl_replicated
  from maxdiffusion_b200.controlnet import generate_controlnet_replicated, generate_controlnet_sdxl_replicated

  for mod, cfg in ((generate, "base15.yml"), (generate, "base21.yml"), (generate_sdxl, "base_xl.yml"),
                   (generate_sdxl, "base_xl_lightning.yml"), (generate_sdxl_replicated, "base_xl.yml"),
                   (generate_controlnet_replicated, "base14.yml"), (generate_controlnet_sdxl_replicated, "base_xl.yml")):
    img = mod.run(_cfg(cfg, SD + ["per_device_batch_size=1"], tmp_path))
    assert img.shape[0] >= 1 and img.dtype == torch.uint8, (mod.__name__, cfg)


def test_flux_text_encoders_visit_the_device_only_while_a_prompt_is_encoded():
  """`offload_encoders`: CLIP and T5 are moved to the pipeline's device for `encode_prompt` and back to host memory
  after it; with the switch off they are left where they are."""
  import types

  from maxdiffusion_b200.pipelines.flux.flux_pipeline import FluxPipeline

  config = _cfg("base_flux_dev.yml", FLUX, "/tmp/unused")
  pipe = FluxPipeline.from_config(config, device="cpu", load_vae=False)
  moves = []

  class Encoder(torch.nn.Module):
    def __init__(self, name, width, pooled):
      super().__init__()
      self.name, self.pooled, self.w = name, pooled, torch.nn.Parameter(torch.zeros(width))

    def to(self, where, *a, **k):
      moves.append((self.name, str(where)))
      return self

    def forward(self, ids):
      out = torch.ones(ids.shape[0], ids.shape[1], self.w.numel())
      return types.SimpleNamespace(pooler_output=out[:, 0], last_hidden_state=out)

  tok = lambda prompts, **kw: types.SimpleNamespace(input_ids=torch.zeros((len(prompts), kw["max_length"]), dtype=torch.long))
  pipe.clip, pipe.t5, pipe.clip_tokenizer, pipe.t5_tokenizer = Encoder("clip", 6, True), Encoder("t5", 10, False), tok, tok
  assert pipe.offload_encoders is False            # only a CUDA pipeline offloads
  e, p = pipe.encode_prompt(["a", "b"], max_sequence_length=8)
  assert e.shape == (2, 8, 10) and p.shape == (2, 6) and moves == []
  pipe.offload_encoders = True
  pipe.encode_prompt("a", max_sequence_length=8)
  assert moves == [("clip", "cpu"), ("t5", "cpu"), ("clip", "cpu"), ("t5", "cpu")]   # to the (CPU) device, then back to the host
