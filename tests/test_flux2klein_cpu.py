"""Flux.2-Klein on CPU: latent packing, ids, schedule, and a tiny end-to-end generation."""
import os

import pytest
import torch

from maxdiffusion_b200 import pyconfig
from maxdiffusion_b200.models.flux.transformer_flux2_klein import (FLUX2_KLEIN_PRESETS, Flux2KleinConfig,
                                                                    Flux2KleinTransformer2DModel)
from maxdiffusion_b200.pipelines.flux.flux2klein_pipeline import (pack_latents, prepare_latent_image_ids, prepare_text_ids,
                                                                   unpack_latents)
from maxdiffusion_b200.schedulers.scheduling_flow_match import FlowMatchScheduler, compute_empirical_mu


def test_pack_unpack_and_ids():
  x = torch.randn(2, 32, 8, 12)
  t = pack_latents(x)
  assert t.shape == (2, 24, 128)
  assert torch.equal(unpack_latents(t, 8, 12), x)
  # channel index = c*4 + dh*2 + dw of the token at (h, w)
  assert torch.equal(t[0, 1 * 6 + 2, 5 * 4 + 1 * 2 + 0], x[0, 5, 2 * 1 + 1, 2 * 2 + 0])
  ids = prepare_latent_image_ids(4, 6)
  assert ids.shape == (24, 4) and ids[6 + 2].tolist() == [0, 1, 2, 0]
  assert prepare_text_ids(5)[3].tolist() == [0, 0, 0, 3]


def test_schedule_matches_exponential_shift_formula():
  mu = compute_empirical_mu(4096, 4)
  a = (0.00016927 * 4096 + 0.45666666 - (8.73809524e-05 * 4096 + 1.89833333)) / 190.0
  assert abs(mu - (a * 4 + (0.00016927 * 4096 + 0.45666666) - 200 * a)) < 1e-9
  assert abs(compute_empirical_mu(5000, 4) - (0.00016927 * 5000 + 0.45666666)) < 1e-9
  sch = FlowMatchScheduler(num_train_timesteps=1000, shift=1.0, sigma_max=1.0, sigma_min=0.001,
                           use_dynamic_shifting=True, time_shift_type="exponential")
  st = sch.set_timesteps_ltx2(sch.create_state(), 4, shift=mu, sigmas=torch.linspace(1.0, 0.25, 4))
  e = torch.exp(torch.tensor(mu, dtype=torch.float64))
  want = e / (e + (1 / torch.linspace(1.0, 0.25, 4, dtype=torch.float64) - 1))
  assert torch.allclose(st.sigmas.double(), want, atol=1e-6) and float(st.sigmas[0]) == 1.0
  assert torch.allclose(st.timesteps, st.sigmas * 1000)
  # terminal stretch: the last sigma lands on shift_terminal
  sch2 = FlowMatchScheduler(shift=1.0, use_dynamic_shifting=True, time_shift_type="exponential", shift_terminal=0.1)
  st2 = sch2.set_timesteps_ltx2(sch2.create_state(), 8, shift=2.05)
  assert abs(float(st2.sigmas[-1]) - 0.1) < 1e-6


def test_modulation_is_shared_and_text_changes_output():
  torch.manual_seed(0)
  m = Flux2KleinTransformer2DModel(Flux2KleinConfig(**FLUX2_KLEIN_PRESETS["tiny"])).eval()
  names = [n for n, _ in m.named_parameters()]
  assert not any("transformer_blocks.0.norm1" in n for n in names)  # no per-block modulation weights
  assert "double_stream_modulation_img.weight" in names and "single_stream_modulation.weight" in names
  ids, tid = prepare_latent_image_ids(2, 4), prepare_text_ids(6)
  x, e, t = torch.randn(1, 8, 128), torch.randn(1, 6, 48), torch.tensor([0.7])
  with torch.no_grad():
    a, b = m(x, e, t, ids, tid), m(x, e * 0.5, t, ids, tid)
  assert a.shape == (1, 8, 128) and (a - b).abs().max() > 1e-4


def test_generate_tiny(tmp_path):
  from maxdiffusion_b200 import generate_flux2klein as G

  config = pyconfig.initialize(
      ["x", "maxdiffusion_b200/configs/base_flux2klein_9B.yml", "random_init=True", "flux_preset=tiny",
       'vae_config_overrides={"block_out_channels":[32,32],"layers_per_block":1,"norm_num_groups":8}', "resolution=64",
       "max_sequence_length=8", f"output_dir={tmp_path}", "log_config=false", "batch_size=2"], unittest=True)
  assert G.partition_prompts(str(config.prompt), 3)[2].startswith("A detailed vector")
  images = G.run(config)
  assert images.shape == (2, 16, 16, 3) and images.dtype == torch.uint8  # the 2-level test VAE upsamples 2x


def test_repetitions_custom_noise_and_interactive_requests(tmp_path):
  """`num_reps` writes one image per repetition, `latents_path` starts from stored noise (the same file gives the same
  image), and interactive mode serves typed prompts until `exit` (a stand-in text encoder here)."""
  import numpy as np

  from maxdiffusion_b200 import generate_flux2klein as G

  base = ["x", "maxdiffusion_b200/configs/base_flux2klein_9B.yml", "random_init=True", "flux_preset=tiny",
          'vae_config_overrides={"block_out_channels":[32,32],"layers_per_block":1,"norm_num_groups":8}', "resolution=64",
          "max_sequence_length=8", "log_config=false", "batch_size=1"]
  noise = tmp_path / "noise.npy"
  np.save(noise, np.random.default_rng(0).standard_normal((1, 32, 8, 8)).astype(np.float32))
  torch.manual_seed(0)
  c = pyconfig.initialize(base + [f"output_dir={tmp_path}/a", "num_reps=2", f"latents_path={noise}", "seed=1"], unittest=True)
  a = G.run(c)
  assert sorted(os.listdir(tmp_path / "a")) == ["rep_1_flux2klein_generated_image.png", "rep_2_flux2klein_generated_image.png"]
  torch.manual_seed(0)
  c2 = pyconfig.initialize(base + [f"output_dir={tmp_path}/b", f"latents_path={noise}", "seed=1"], unittest=True)
  b = G.run(c2)                       # the same stored noise: the same picture
  assert torch.equal(a, b) and os.listdir(tmp_path / "b") == ["flux2klein_generated_image.png"]
  torch.manual_seed(0)
  drawn = G.run(pyconfig.initialize(base + [f"output_dir={tmp_path}/d", "seed=1"], unittest=True))
  assert not torch.equal(a, drawn)    # without the file the noise is drawn from the seed

  # interactive: needs a text encoder; served requests are numbered, blank lines are skipped, `exit` ends the loop
  c3 = pyconfig.initialize(base + [f"output_dir={tmp_path}/c", "interactive=True"], unittest=True)
  with pytest.raises(ValueError, match="text encoder"):
    G.run(c3)
  pipe = G.load_pipeline(c3)
  dim = pipe.transformer.cfg.joint_attention_dim
  pipe.text_encoder = object()
  pipe.encode_prompt = lambda prompts: torch.randn((len(prompts), 8, dim), generator=torch.Generator().manual_seed(len(prompts[0])))
  lines = iter(["a red car", "", "a cat || a dog", "exit", "never read"])
  kw = dict(height=64, width=64, num_inference_steps=2, batch_size=1, seed=0)
  assert G.interactive_loop(c3, pipe, kw, read=lambda _: next(lines)) == 2
  assert sorted(os.listdir(tmp_path / "c")) == ["generated_001.png", "generated_002.png"]
  assert next(lines) == "never read"

  def ended(_):
    raise EOFError
  assert G.interactive_loop(c3, pipe, kw, read=ended) == 0
