"""Utility surface: shared SD helpers, device info, safety checker, dependency check, dataset preprocessing scripts,
package exports, Wan checkpointer variants."""
import csv
import os

import numpy as np
import pytest
import torch

from maxdiffusion_b200 import pyconfig

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs")


def test_package_exports_resolve():
  import maxdiffusion_b200 as M

  for n in M.__all__:
    assert getattr(M, n) is not None, n
  assert M.FlaxStableDiffusionXLPipeline is M.StableDiffusionXLPipeline
  assert M.VaceWanPipeline2_1.__name__ == "WanVACEPipeline2_1"
  assert M.FlaxUniPCMultistepScheduler is M.UniPCMultistepScheduler
  with pytest.raises(AttributeError):
    M.NoSuchThing


def test_dependency_check():
  from maxdiffusion_b200.dependency_versions_check import dep_version_check, require_version

  dep_version_check("torch")
  require_version("numpy>=1.0")
  with pytest.raises(ImportError):
    require_version("numpy>=999.0")
  with pytest.raises(ImportError):
    require_version("surely_not_a_package_xyz")


def test_gpu_utils_cpu():
  from maxdiffusion_b200 import gpu_utils

  assert gpu_utils.pad_to_alignment(129, 128) == 256 and gpu_utils.pad_to_alignment(128, 128) == 128
  info = gpu_utils.DeviceInfo("NVIDIA B200", (10, 0), 148, 178.0, 126 << 20)
  assert info.is_blackwell and info.sequence_alignment == 128
  if not torch.cuda.is_available():
    assert gpu_utils.device_info() is None and gpu_utils.print_device_memory() == {}
    with pytest.raises(RuntimeError):
      gpu_utils.require_blackwell()


def test_safety_checker_thresholds():
  from maxdiffusion_b200.pipelines.stable_diffusion.safety_checker import StableDiffusionSafetyChecker, run_safety_checker

  class Vision(torch.nn.Module):
    def forward(self, x):  # pooled output = mean colour, repeated
      return None, x.mean(dim=(2, 3)).repeat(1, 4)[:, :8]

  ck = StableDiffusionSafetyChecker(Vision(), hidden_size=8, projection_dim=8)
  with torch.no_grad():
    ck.visual_projection.weight.copy_(torch.eye(8))
    ck.concept_embeds.copy_(torch.randn(17, 8, generator=torch.Generator().manual_seed(0)))
    ck.special_care_embeds.copy_(torch.randn(3, 8, generator=torch.Generator().manual_seed(1)))
    ck.concept_embeds_weights.fill_(2.0)  # cosine similarity never exceeds 1
    ck.special_care_embeds_weights.fill_(2.0)
  imgs = torch.randint(0, 255, (3, 32, 32, 3), dtype=torch.uint8)
  out, flags = run_safety_checker(ck, imgs)
  assert not flags.any() and torch.equal(out, imgs)
  with torch.no_grad():
    ck.concept_embeds_weights.fill_(-2.0)
  out, flags = run_safety_checker(ck, imgs)
  assert flags.all() and int(out.sum()) == 0
  # the special-care adjustment lowers the threshold by exactly 0.01
  with torch.no_grad():
    pooled = Vision()(torch.ones(1, 3, 4, 4))[1]
    ck.concept_embeds[0].copy_(pooled[0])
    ck.concept_embeds_weights.fill_(2.0)
    ck.concept_embeds_weights[0] = 1.005
    ck.special_care_embeds[0].copy_(pooled[0])
  assert not bool(ck(torch.ones(1, 3, 4, 4))[0])
  with torch.no_grad():
    ck.special_care_embeds_weights[0] = 0.5
  assert bool(ck(torch.ones(1, 3, 4, 4))[0])


def test_maxdiffusion_utils(tmp_path):
  from maxdiffusion_b200 import maxdiffusion_utils as U
  from maxdiffusion_b200.models.flux.transformer_flux import FLUX_PRESETS, FluxConfig, FluxTransformer2DModel
  from maxdiffusion_b200.models.unet_2d_condition import UNET_PRESETS, UNet2DConditionModel, UNetConfig
  from maxdiffusion_b200.models.vae import AutoencoderKL, VAEConfig
  from maxdiffusion_b200.models.wan.transformer_wan import WAN_PRESETS, WanConfig, WanModel

  cfg = pyconfig.initialize(["x", os.path.join(CFG, "base_xl.yml"), "resolution=32", "log_config=false", "per_device_batch_size=2"], unittest=True)
  unet = UNet2DConditionModel(UNetConfig(**UNET_PRESETS["tiny"]))
  args = U.get_dummy_unet_inputs(cfg, unet)
  assert args[0].shape == (2, 4, 4, 4) and unet(*args).shape == (2, 4, 4, 4)
  assert U.calculate_unet_tflops(cfg, unet) > 0
  fcfg = pyconfig.initialize(["x", os.path.join(CFG, "base_flux_dev.yml"), "resolution=64", "max_sequence_length=8", "log_config=false"], unittest=True)
  flux = FluxTransformer2DModel(FluxConfig(**FLUX_PRESETS["tiny"]))
  assert flux(*U.get_dummy_flux_inputs(fcfg, flux)).shape == (1, 16, 64)
  assert U.calculate_flux_tflops(fcfg, flux, train=False) > 0
  wcfg = pyconfig.initialize(["x", os.path.join(CFG, "base_wan_14b.yml"), "height=32", "width=32", "num_frames=5", "log_config=false"], unittest=True)
  wan = WanModel(WanConfig(**WAN_PRESETS["tiny"]))
  assert wan(*U.get_dummy_wan_inputs(wcfg, wan)).shape == (1, 16, 2, 4, 4)
  from maxdiffusion_b200.max_utils import calculate_model_tflops

  traced = calculate_model_tflops(wan, *U.get_dummy_wan_inputs(wcfg, wan))
  assert abs(U.calculate_wan_tflops(wcfg, wan, train=False) / traced - 1) < 0.25  # analytic count skips embedders / head
  assert U.override_scheduler_config({"prediction_type": "epsilon", "timestep_spacing": "leading"}, cfg)["timestep_spacing"] in ("leading", "trailing")
  b = U.get_shaped_batch(cfg)
  assert b["pixel_values"].shape == (2, 4, 4, 4) and b["text_embeds"].shape == (2, 1280)
  # dataset transforms
  from PIL import Image

  vae = AutoencoderKL(VAEConfig(block_out_channels=(32, 32), layers_per_block=1, norm_num_groups=8))
  ex = {"image": [Image.fromarray(np.random.randint(0, 255, (40, 56, 3), np.uint8)) for _ in range(3)]}
  out = U.transform_images(dict(ex), "image", 32)
  assert out["pixel_values"][0].shape == (3, 32, 32) and abs(out["pixel_values"][0]).max() <= 1.0
  out = U.transform_images(dict(ex), "image", 32, vae=vae, generator=torch.Generator().manual_seed(0))
  assert out["pixel_values"][0].shape == (4, 16, 16)

  class Tok:
    model_max_length = 6

    def __call__(self, caps, max_length, padding, truncation, return_tensors):
      class R:
        input_ids = torch.tensor([[len(c) % 7] * max_length for c in caps])
      return R

  out = U.tokenize_captions({"text": ["a cat", ["two", "captions"]]}, "text", Tok())
  assert np.asarray(out["input_ids"]).shape == (2, 6)
  out = U.tokenize_captions_xl({"text": ["a", "b"]}, "text", [Tok(), Tok()])
  assert np.asarray(out["input_ids"]).shape == (2, 2, 6)


def test_pusav1_to_tfrecords_and_back(tmp_path):
  from maxdiffusion_b200.data_preprocessing import wan_pusav1_to_tfrecords
  from maxdiffusion_b200.input_pipeline.input_pipeline_interface import TFRecordIterator

  src = tmp_path / "pusa"
  (src / "train").mkdir(parents=True)
  g = torch.Generator().manual_seed(0)
  lat = {}
  with open(src / "metadata.csv", "w", newline="") as f:
    w = csv.writer(f)
    w.writerow(["file_name", "text"])
    for i in range(10):
      name = f"clip{i}.mp4"
      w.writerow([name, f"caption {i}"])
      lat[i] = torch.randn((16, 2, 4, 4), generator=g).to(torch.bfloat16)
      torch.save({"latents": lat[i], "prompt_emb": {"context": torch.randn((1, 8, 32), generator=g).to(torch.bfloat16)}},
                 src / "train" / f"{name}.tensors.pth")
  cfg = pyconfig.initialize(["x", os.path.join(CFG, "base_wan_14b.yml"), f"train_data_dir={src}", f"tfrecords_dir={tmp_path}/rec",
                             "no_records_per_shard=4", "log_config=false"], unittest=True)
  files = wan_pusav1_to_tfrecords.run(cfg)
  assert [os.path.basename(f) for f in files] == ["file_00-4.tfrec", "file_01-8.tfrec", "file_02-10.tfrec"]
  it = TFRecordIterator(f"{tmp_path}/rec", 5, shuffle=False, repeat=False)
  batches = list(it)
  assert len(batches) == 2 and batches[0]["latents"].shape == (5, 16, 2, 4, 4) and batches[0]["encoder_hidden_states"].shape == (5, 8, 32)
  assert torch.equal(batches[0]["latents"][3], lat[3].float())
  # evaluation split: 6 samples over 3 timesteps, nothing after them
  cfg = pyconfig.initialize(["x", os.path.join(CFG, "base_wan_14b.yml"), f"train_data_dir={src}", f"tfrecords_dir={tmp_path}/eval",
                             "no_records_per_shard=100", "enable_eval_timesteps=true", "num_eval_samples=6", "timesteps_list=[100,500,900]",
                             "log_config=false"], unittest=True)
  wan_pusav1_to_tfrecords.run(cfg)
  ev = list(TFRecordIterator(f"{tmp_path}/eval", 6, shuffle=False, repeat=False, with_timesteps=True))
  assert len(ev) == 1 and ev[0]["timesteps"].tolist() == [100, 100, 500, 500, 900, 900]


def test_txt2vid_preprocessing(tmp_path):
  from maxdiffusion_b200.data_preprocessing import wan_txt2vid_data_preprocessing as P
  from maxdiffusion_b200.input_pipeline.input_pipeline_interface import TFRecordIterator
  from maxdiffusion_b200.pipelines.wan.wan_pipeline import WanPipeline

  cfg = pyconfig.initialize(["x", os.path.join(CFG, "base_wan_14b.yml"), "wan_preset=tiny", "random_init=true", "height=32", "width=32",
                             'vae_config_overrides={"base_dim":8}', f"tfrecords_dir={tmp_path}/rec", "no_records_per_shard=2",
                             "max_sequence_length=8", "log_config=false"], unittest=True)
  pipe = WanPipeline.from_config(cfg, device="cpu")
  pipe.transformer = None
  pipe.encode_prompt = lambda prompts, max_len: torch.stack([torch.full((max_len, 16), float(len(p))) for p in prompts])

  class DS:
    rows = [{"text": "a" * (i + 1), "image": np.random.randint(0, 255, (5, 40, 48, 3), np.uint8)} for i in range(3)]

    def __len__(self):
      return len(self.rows)

    def __getitem__(self, s):
      rows = self.rows[s]
      return {"text": [r["text"] for r in rows], "image": [r["image"] for r in rows]}

  files = P.generate_dataset(cfg, pipe, DS(), batch_size=2)
  assert len(files) == 2
  b = next(TFRecordIterator(f"{tmp_path}/rec", 3, shuffle=False, repeat=False))
  assert b["latents"].shape == (3, 16, 2, 4, 4) and b["encoder_hidden_states"][:, 0, 0].tolist() == [1.0, 2.0, 3.0]


def test_wan_checkpointer_variants(tmp_path):
  from maxdiffusion_b200.checkpointing import WanCheckpointer2_1, WanCheckpointer2_2

  args = ["wan_preset=tiny", "random_init=true", f"checkpoint_dir={tmp_path}/ck", 'vae_config_overrides={"base_dim":8}', "log_config=false"]
  cfg = pyconfig.initialize(["x", os.path.join(CFG, "base_wan_14b.yml"), *args], unittest=True)
  ck = WanCheckpointer2_1(cfg)
  pipe, step = ck.load_checkpoint(device="cpu")
  assert step is None and type(pipe).__name__ == "WanPipeline2_1"
  ck.save_pipeline(3, pipe)
  cfg2 = pyconfig.initialize(["x", os.path.join(CFG, "base_wan_14b.yml"), *args, "seed=7"], unittest=True)
  pipe2, step2 = WanCheckpointer2_1(cfg2).load_checkpoint(device="cpu")
  assert step2 == 3
  for (k, a), (_, b) in zip(pipe.transformer.state_dict().items(), pipe2.transformer.state_dict().items()):
    assert torch.equal(a, b), k
  cfg3 = pyconfig.initialize(["x", os.path.join(CFG, "base_wan_27b.yml"), "wan_preset=tiny", "random_init=true", f"checkpoint_dir={tmp_path}/ck22",
                              'vae_config_overrides={"base_dim":8}', "log_config=false"], unittest=True)
  p3, _ = WanCheckpointer2_2(cfg3).load_checkpoint(device="cpu")
  assert type(p3).__name__ == "WanPipeline2_2" and p3.transformer_2 is not None


def test_pedagogical_examples(tmp_path):
  from maxdiffusion_b200.pedagogical_examples import (attention_comparison, checkpoint_params_restore, dataset_tf_cache_to_tfrecord,
                                                      model_flop_calculation, parameter_count, parameter_shardings)

  r = attention_comparison.run(seq=64, heads=2, dim=32)
  assert r["sdpa"]["max_abs_err"] < 1e-4
  c = parameter_count.run("wan2.1-t2v-14b")
  assert 14.0e9 < c["total"] < 14.6e9
  assert checkpoint_params_restore.run(str(tmp_path / "ck"))
  s = parameter_shardings.run("wan2.1-t2v-1.3b", 8)
  assert s["blocks"] == 30 and s["block_shard"] * 8 >= s["block_numel"]
  cfg = pyconfig.initialize(["x", os.path.join(CFG, "base_wan_14b.yml"), "wan_preset=tiny", "height=32", "width=32", "num_frames=5",
                             "max_sequence_length=16", "log_config=false"], unittest=True)
  f = model_flop_calculation.run(cfg)
  assert abs(f["analytic"] / f["traced"] - 1) < 0.25
  # re-sharding keeps every record
  from maxdiffusion_b200.data_preprocessing.tfrecord_shards import ShardedWriter, create_example
  from maxdiffusion_b200.input_pipeline.tfrecord import read_records

  w = ShardedWriter(str(tmp_path / "a"), 100)
  for i in range(7):
    w.write(create_example(np.full((2, 2), i, np.float32), np.zeros((1, 4), np.float32)))
  w.close()
  files = dataset_tf_cache_to_tfrecord.run(str(tmp_path / "a"), str(tmp_path / "b"), 3)
  assert len(files) == 3 and sum(1 for f in files for _ in read_records(f)) == 7


def test_save_sd_checkpoint_example_and_eval_assert(tmp_path):
  import json
  import subprocess
  import sys

  from maxdiffusion_b200.pedagogical_examples import save_sd_checkpoint
  from maxdiffusion_b200.pipelines.pipeline_utils import load_components

  cfg = pyconfig.initialize(["x", os.path.join(CFG, "base15.yml"), "random_init=True", "unet_preset=tiny_sd", f"output_dir={tmp_path}/out",
                             'vae_config_overrides={"block_out_channels":[32,32],"layers_per_block":1,"norm_num_groups":8,"latent_channels":4}',
                             f"checkpoint_dir={tmp_path}/none", "log_config=false"], unittest=True)
  out = save_sd_checkpoint.run(cfg)
  comps = load_components(out)
  assert {"unet", "vae", "scheduler"} <= set(comps)
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  m = tmp_path / "metrics.txt"
  with open(m, "w") as f:
    for i in range(20):
      f.write(json.dumps({"learning/loss": 1.0 / (i + 1), "perf/step_time_seconds": 0.5, "perf/per_device_tflops_per_sec": 700.0}) + "\n")
  script = os.path.join(root, "end_to_end", "gpu", "eval_assert.py")
  assert subprocess.run([sys.executable, script, "final_loss", str(m), "0.1"]).returncode == 0
  assert subprocess.run([sys.executable, script, "final_loss", str(m), "0.01"], capture_output=True).returncode != 0
  assert subprocess.run([sys.executable, script, "avg_tflops", str(m), "600"]).returncode == 0
  assert subprocess.run([sys.executable, script, "avg_step_time", str(m), "0.4"], capture_output=True).returncode != 0


def test_inference_bench_runs_on_tiny_presets(capsys):
  import json

  from maxdiffusion_b200.utils import inference_bench

  assert inference_bench.main(["wan", "--preset", "tiny", "--height", "64", "--width", "64", "--frames", "5", "--steps", "2"]) == 0
  assert inference_bench.main(["flux", "--preset", "tiny", "--resolution", "64", "--steps", "2"]) == 0
  lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
  assert lines[0]["unit"] == "s/step" and lines[0]["value"] > 0 and lines[0]["config"]["tokens"] == 32
  assert lines[1]["unit"] == "images/s" and lines[1]["value"] > 0


def test_names_the_reference_users_import_resolve():
  """The import lines of the reference's src/maxdiffusion/tests/models_import_test.py with the package name changed, and
  the head-group chunk ranges its attention test pins (attention_test.py:261-278)."""
  from maxdiffusion_b200 import (aot_cache, checkpointing, common_types, configuration_utils, max_logging, max_utils,  # noqa: F401
                                 maxdiffusion_utils, multihost_dataloading, pyconfig, tpu_utils, train_utils)
  from maxdiffusion_b200.checkpointing.base_stable_diffusion_checkpointer import BaseStableDiffusionCheckpointer  # noqa: F401
  from maxdiffusion_b200.models import FlaxAutoencoderKL, FlaxControlNetModel, FlaxUNet2DConditionModel
  from maxdiffusion_b200.models.unet_2d_condition import UNet2DConditionModel
  from maxdiffusion_b200.parallel.context import ulysses_head_chunks
  from maxdiffusion_b200.pipelines import FlaxStableDiffusionPipeline, FlaxStableDiffusionXLPipeline  # noqa: F401
  from maxdiffusion_b200.schedulers import FlaxDDIMScheduler, FlaxDDPMScheduler, FlaxDPMSolverMultistepScheduler  # noqa: F401

  assert FlaxUNet2DConditionModel is UNet2DConditionModel and FlaxAutoencoderKL is not None and FlaxControlNetModel is not None
  assert "device_info" in tpu_utils.__all__ and callable(tpu_utils.device_info)
  assert ulysses_head_chunks(40, 8, 2) == [(0, 16), (16, 40)]
  assert ulysses_head_chunks(40, 8, 5) == [(0, 8), (8, 16), (16, 24), (24, 32), (32, 40)]
  assert ulysses_head_chunks(40, 8, 3) == [(0, 8), (8, 16), (16, 40)] and ulysses_head_chunks(40, 8, 1) == [(0, 40)]


def test_gif_ply_and_obj_exporters_round_trip(tmp_path):
  import struct
  import types

  import numpy as np
  from PIL import Image

  from maxdiffusion_b200.utils.export_utils import export_to_gif, export_to_obj, export_to_ply

  frames = (np.random.default_rng(0).random((4, 8, 8, 3)) * 255).astype(np.uint8)
  gif = export_to_gif(frames, str(tmp_path / "a.gif"))
  with Image.open(gif) as im:
    assert im.n_frames == 4 and im.size == (8, 8) and im.info["duration"] == 100 and im.info.get("loop") == 0
  assert os.path.getsize(export_to_gif([Image.fromarray(f) for f in frames])) > 0    # PIL images, temporary file

  verts = torch.tensor([[0.0, 0.0, 0.0], [1.0, 0.0, 0.0], [0.0, 1.0, 0.0], [0.0, 0.0, 1.0]])
  faces = torch.tensor([[0, 1, 2], [0, 2, 3]])
  colour = {c: torch.tensor(v) for c, v in zip("RGB", ([0.0, 1.0, 0.5, 0.25], [1.0, 0.0, 0.5, 0.25], [0.0, 0.0, 1.0, 0.25]))}
  mesh = types.SimpleNamespace(verts=verts, faces=faces, vertex_channels=colour)
  raw = open(export_to_ply(mesh, str(tmp_path / "m.ply")), "rb").read()
  head, body = raw.split(b"end_header\n", 1)
  assert b"element vertex 4" in head and b"element face 2" in head and b"property uchar red" in head
  assert len(body) == 4 * (12 + 3) + 2 * (1 + 12)
  assert struct.unpack_from("<3f3B", body, 15) == (1.0, 0.0, 0.0, 255, 0, 0)
  assert struct.unpack_from("<B3i", body, 4 * 15 + 13) == (3, 0, 2, 3)
  bare = types.SimpleNamespace(verts=verts, faces=None, vertex_channels=None)
  assert open(export_to_ply(bare, str(tmp_path / "b.ply")), "rb").read().endswith(verts.numpy().astype("<f4").tobytes())

  lines = open(export_to_obj(mesh, str(tmp_path / "m.obj"))).read().splitlines()
  assert len(lines) == 6 and lines[1].split() == ["v", "1.0", "0.0", "0.0", "1.0", "0.0", "0.0"] and lines[-1] == "f 1 3 4"


def test_max_utils_helpers(tmp_path):
  import io
  import json
  import types

  import numpy as np
  import pytest

  from maxdiffusion_b200 import max_utils as M

  tree = {"a": torch.full((2, 2), 2.0), "b": [torch.ones(3), {"c": torch.zeros(5)}], "d": None}
  assert abs(M.l2norm_pytree(tree) - (16 + 3) ** 0.5) < 1e-9 and M.calculate_num_params_from_pytree(tree) == 12
  lin = torch.nn.Linear(3, 2)
  assert M.calculate_num_params_from_pytree(lin) == 8
  assert M.get_global_batch_size(0.5) == 0.5 and M.safe_getattr(None, "x", 7) == 7 and M.safe_getattr(lin, "in_features", 0) == 3
  assert M.get_precision({"precision": "HIGHEST"}) == "highest" and M.get_precision({"precision": "DEFAULT"}) == "high"
  assert M.profiler_enabled({"enable_profiler": True}) and M.is_gpu_backend({"hardware": "tpu"})
  assert M.parse_gcs_bucket_and_prefix("gs://bucket/some/prefix") == ("bucket", "some/prefix")
  with pytest.raises(EnvironmentError, match="network"):
    M.upload_blob("gs://b/x", "file")
  h = M.get_git_commit_hash()
  assert h is None or len(h) == 40
  (tmp_path / "x").write_text("1")
  M.delete_file(str(tmp_path / "x"))
  M.delete_file(str(tmp_path / "x"))               # missing: logged, not raised
  assert not (tmp_path / "x").exists()
  cfg = {"output_file": str(tmp_path / "img" / "out.png"), "output_dir": str(tmp_path), "run_name": "r", "seed": 3}
  imgs = [np.zeros((4, 4, 3), np.uint8), torch.full((4, 4, 3), 255, dtype=torch.uint8)]
  assert [os.path.basename(p) for p in M.save_images(cfg, imgs)] == ["out_0.png", "out_1.png"]
  assert os.path.basename(M.save_images({**cfg, "output_file": ""}, imgs[:1])[0]) == "r_output_3.png"
  os.remove("r_output_3.png")
  with pytest.raises(EnvironmentError):
    M.save_images({**cfg, "output_dir": "gs://bucket/x"}, imgs)

  class File(io.StringIO):
    closed_by_writer = False

    def close(self):
      self.closed_by_writer = True

  f = File()
  c = types.SimpleNamespace(get=lambda k, d=None: {"run_name": "r", "max_train_steps": 2}.get(k, d))
  f.write("stale\n")
  M.write_metrics_locally({"scalar": {"learning/loss": torch.tensor(0.5)}}, 0, c, f)
  M.write_metrics_locally({"scalar": {"learning/loss": 0.25}}, 1, c, f)
  lines = [json.loads(x) for x in f.getvalue().splitlines()]
  assert len(lines) == 2 and lines[-1] == {"learning/loss": 0.25, "step": 1.0, "run_name": "r"} and f.closed_by_writer
  M.close_summary_writer(None)


def test_scheduler_creation_from_a_checkpoint_config_and_small_pipeline_helpers():
  """`create_scheduler` as the reference's src/maxdiffusion/tests/maxdiffusion_utils_test.py:73 uses it: overrides from
  `diffusion_scheduler_config` win, keys an old scheduler file omits get safe defaults, the class is found with or
  without the `Flax` prefix."""
  import io
  import types

  from PIL import Image

  from maxdiffusion_b200 import maxdiffusion_utils as U
  from maxdiffusion_b200.schedulers import DDIMScheduler, PNDMScheduler

  over = types.SimpleNamespace(get=lambda k, d=None: {"diffusion_scheduler_config": {
      "prediction_type": "v_prediction", "rescale_zero_terminal_snr": True, "timestep_spacing": "trailing", "_class_name": ""}}.get(k, d))
  ckpt = {"_class_name": "FlaxDDIMScheduler", "_diffusers_version": "0.20", "beta_schedule": "scaled_linear", "beta_start": 0.00085,
          "beta_end": 0.012, "num_train_timesteps": 1000, "prediction_type": "epsilon"}
  sched, state = U.create_scheduler(ckpt, over)
  assert isinstance(sched, DDIMScheduler) and state is not None
  assert (sched.config.prediction_type, sched.config.timestep_spacing, sched.config.rescale_zero_terminal_snr) == ("v_prediction", "trailing", True)
  plain = types.SimpleNamespace(get=lambda k, d=None: d)
  old_file = {"_class_name": "PNDMScheduler", "beta_schedule": "scaled_linear", "beta_start": 0.00085, "beta_end": 0.012,
              "num_train_timesteps": 1000, "skip_prk_steps": True}
  cfg = U.override_scheduler_config(old_file, plain)
  assert (cfg["prediction_type"], cfg["timestep_spacing"], cfg["rescale_zero_terminal_snr"]) == ("epsilon", "leading", False)
  assert isinstance(U.create_scheduler(old_file, plain)[0], PNDMScheduler) and "prediction_type" not in old_file
  import pytest

  with pytest.raises(ValueError, match="unknown scheduler"):
    U.create_scheduler({"_class_name": "NoSuchScheduler"}, plain)

  cfg_noise, text = torch.tensor([[[1.0, 2.0], [3.0, 4.0]]]), torch.ones(1, 2, 2) + torch.tensor([[[0.0, 1.0], [2.0, 3.0]]]) * 0.5
  assert torch.equal(U.rescale_noise_cfg(cfg_noise, text, 0.0), cfg_noise)
  full = U.rescale_noise_cfg(cfg_noise, text, 1.0)
  assert torch.allclose(full.std(unbiased=False), text.std(unbiased=False), atol=1e-6)
  assert U.get_add_time_ids((1024, 1024), (0, 0), (768, 512), 2).tolist() == [[1024, 1024, 0, 0, 768, 512]] * 2
  buf = io.BytesIO()
  Image.new("RGB", (3, 2), (9, 8, 7)).save(buf, format="PNG")
  img = U.convert_dict_to_pil({"bytes": buf.getvalue(), "path": None})
  assert img.size == (3, 2) and U.convert_dict_to_pil(img) is img
