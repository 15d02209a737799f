"""Wan VACE on CPU: hint injection, conditioning-latent layout, a training step and checkpoint resume."""
import os

import torch

from maxdiffusion_b200 import pyconfig
from maxdiffusion_b200.checkpointing.wan_vace_checkpointer import WanVACECheckpointer2_1
from maxdiffusion_b200.models.wan.transformer_wan_vace import WanVACEConfig, WanVACEModel
from maxdiffusion_b200.parallel.mesh import create_device_mesh
from maxdiffusion_b200.pipelines.wan.wan_vace_pipeline import WanVACEPipeline2_1
from maxdiffusion_b200.trainers.wan_vace_trainer import WanVACETrainer

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs",
                   "base_wan_14b.yml")
TINY = ('{"num_attention_heads": 2, "attention_head_dim": 32, "ffn_dim": 64, "num_layers": 2, "text_dim": 32, '
        '"freq_dim": 32, "vace_layers": [0, 1], "vace_in_channels": 96}')


def _config(tmp, *extra):
  return pyconfig.initialize(
      ["t", CFG, "run_name=vace", f"output_dir={tmp}", "height=32", "width=32", "num_frames=5", "dataset_type=synthetic",
       "wan_preset=tiny", f"wan_config_overrides={TINY}", "warmup_steps_fraction=0.0", "log_config=false",
       "write_metrics=false", "learning_rate=1e-3", "synthetic_override_text_dim=32", "max_sequence_length=8",
       'vae_config_overrides={"base_dim": 8, "z_dim": 16}', "num_inference_steps=2", *extra], unittest=True)


def test_hints_enter_after_the_configured_layers_and_scale_to_zero():
  torch.manual_seed(0)
  cfg = WanVACEConfig(num_attention_heads=2, attention_head_dim=32, ffn_dim=64, num_layers=3, text_dim=32, freq_dim=32,
                      vace_layers=(0, 2), vace_in_channels=20)
  m = WanVACEModel(cfg).eval()
  x, c = torch.randn(1, 16, 2, 8, 8), torch.randn(1, 20, 2, 8, 8)
  t, e = torch.tensor([400.0]), torch.randn(1, 6, 32)
  with torch.no_grad():
    on = m(x, t, e, c)
    off = m(x, t, e, c, control_hidden_states_scale=[0.0, 0.0])
    base = super(WanVACEModel, m).forward(x, t, e)  # the plain Wan stream
    cached = m(x, t, e, c, kv_cache=m.compute_kv_cache(e))
  assert (on - off).abs().max() > 1e-3
  assert torch.allclose(off, base, atol=1e-5)
  assert torch.allclose(on, cached, atol=1e-5)


def test_pipeline_builds_96_channel_control_latents_and_drops_reference_frames(tmp_path):
  pipe = WanVACEPipeline2_1.from_config(_config(str(tmp_path)), device="cpu")
  vid = torch.rand(1, 3, 5, 32, 32) * 2 - 1
  msk = (torch.rand(1, 3, 5, 32, 32) > 0.5).float() * 2 - 1
  v, m, refs = pipe.preprocess_conditions(vid, msk, [torch.rand(3, 20, 24) * 2 - 1], 1, 32, 32, 5)
  assert refs[0].shape == (3, 32, 32) and float(refs[0][:, 0, 0].min()) == 1.0  # letter-boxed on white
  lat = pipe.prepare_video_latents(v, m, refs)
  masks = pipe.prepare_masks(m, 1)
  assert lat.shape == (1, 32, 3, 4, 4) and masks.shape == (1, 64, 3, 4, 4)
  assert float(masks[:, :, 0].abs().max()) == 0.0 and float(lat[:, 16:, 0].abs().max()) == 0.0
  e, ne = torch.randn(1, 8, 32), torch.randn(1, 8, 32)
  out = pipe(video=vid, mask=msk, reference_images=[torch.rand(3, 20, 24) * 2 - 1], prompt_embeds=e,
             negative_prompt_embeds=ne)
  assert out.shape == (1, 5, 32, 32, 3) and out.dtype == torch.uint8


def test_train_step_and_checkpoint_round_trip(tmp_path):
  config = _config(str(tmp_path), "save_optimizer=true")
  tr = WanVACETrainer(config, mesh=create_device_mesh(config), device="cpu")
  data = tr.load_dataset()
  b0, b1 = next(data), next(data)
  l0 = float(tr.train_step(b0)["learning/loss"])
  assert l0 == l0 and tr.model.vace_blocks[0].proj_in is not None
  ck = WanVACECheckpointer2_1(config)
  ck.save(1, tr)
  ck.manager.wait_until_finished()
  config2 = _config(str(tmp_path), "save_optimizer=true", "seed=9")
  tr2 = WanVACETrainer(config2, mesh=create_device_mesh(config2), device="cpu")
  assert WanVACECheckpointer2_1(config2).maybe_restore(tr2) == 1
  for (n, p), (_, q) in zip(tr.model.named_parameters(), tr2.model.named_parameters()):
    assert torch.allclose(p, q, atol=1e-6), n
  tr.gen, tr2.gen = torch.Generator().manual_seed(3), torch.Generator().manual_seed(3)
  assert float(tr.train_step(b1)["learning/loss"]) == float(tr2.train_step(b1)["learning/loss"])
