"""`start_training` of the Stable Diffusion / SDXL / Dreambooth / Flux trainers on CPU: periodic checkpoints inside the
loop, and a run that resumes from a checkpoint continues the uninterrupted run (weights, optimizer moments, step
counter, learning-rate schedule and the noise / timestep stream all come back)."""
import os
import shutil

import pytest
import torch

from maxdiffusion_b200 import pyconfig
from maxdiffusion_b200.parallel.mesh import create_device_mesh

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs")
COMMON = ["random_init=True", "log_config=false", "write_metrics=false", "dataset_type=synthetic", "save_optimizer=true",
          "learning_rate=1e-3", "checkpoint_every=2", "enable_async_checkpointing=false", "warmup_steps_fraction=0.5"]
SD = ["resolution=32", "per_device_batch_size=2"]
FLUX = ["flux_preset=tiny", "resolution=64", "max_sequence_length=8"]


def _cfg(name, extra, out):
  return pyconfig.initialize(["x", os.path.join(CFG, name), "run_name=r", f"output_dir={out}", *COMMON, *extra], unittest=True)


def _record(trainer):
  losses = []
  step = trainer.train_step

  def wrapped(batch):
    m = step(batch)
    losses.append(float(m["learning/loss"]))
    return m

  trainer.train_step = wrapped
  return losses


def _only_step(src_ckpt: str, dst_ckpt: str, step: int):
  os.makedirs(dst_ckpt, exist_ok=True)
  shutil.copytree(os.path.join(src_ckpt, str(step)), os.path.join(dst_ckpt, str(step)))


@pytest.mark.parametrize("kind,cfg,preset", [("sd", "base15.yml", "tiny_sd"), ("sdxl", "base_xl.yml", "tiny"), ("dreambooth", "base14.yml", "tiny_sd")])
def test_stable_diffusion_trainers_checkpoint_in_the_loop_and_resume(kind, cfg, preset, tmp_path):
  from maxdiffusion_b200.trainers.stable_diffusion_trainer import DreamboothTrainer, StableDiffusionTrainer, StableDiffusionXLTrainer

  cls = {"sd": StableDiffusionTrainer, "sdxl": StableDiffusionXLTrainer, "dreambooth": DreamboothTrainer}[kind]
  extra = SD + [f"unet_preset={preset}", "max_train_steps=4"]
  ca = _cfg(cfg, extra, tmp_path / "a")
  a = cls(ca, mesh=create_device_mesh(ca), device="cpu")
  la = _record(a)
  a.start_training()
  assert len(la) == 4 and a.step == 4
  ckpt_a = ca.checkpoint_dir
  assert sorted(int(d) for d in os.listdir(ckpt_a) if d.isdigit()) == [2, 4]

  cb = _cfg(cfg, extra, tmp_path / "b")
  _only_step(ckpt_a, cb.checkpoint_dir, 2)
  b = cls(cb, mesh=create_device_mesh(cb), device="cpu")
  with torch.no_grad():
    for p in b.unet.parameters():
      p.add_(0.5)  # whatever the new process starts with is overwritten by the checkpoint
  lb = _record(b)
  b.start_training()
  assert b.step == 4 and len(lb) == 2
  assert lb == pytest.approx(la[2:], rel=1e-5, abs=1e-7)
  for (n, p), (_, q) in zip(a.unet.named_parameters(), b.unet.named_parameters()):
    assert torch.allclose(p, q, atol=1e-6), n


def test_flux_trainer_checkpoint_in_the_loop_and_resume(tmp_path):
  from maxdiffusion_b200.trainers.flux_trainer import FluxTrainer

  extra = FLUX + ["max_train_steps=4"]
  ca = _cfg("base_flux_dev.yml", extra, tmp_path / "a")
  a = FluxTrainer(ca, mesh=create_device_mesh(ca), device="cpu")
  data = a.load_dataset()
  batches = [next(data) for _ in range(6)]
  la = _record(a)
  a.start_training(iter(batches))
  assert len(la) == 4
  cb = _cfg("base_flux_dev.yml", extra, tmp_path / "b")
  _only_step(ca.checkpoint_dir, cb.checkpoint_dir, 2)
  b = FluxTrainer(cb, mesh=create_device_mesh(cb), device="cpu")
  with torch.no_grad():
    for p in b.model.parameters():
      p.add_(0.5)
  lb = _record(b)
  b.start_training(iter(batches[2:]))
  assert b.step == 4 and lb == pytest.approx(la[2:], rel=1e-5, abs=1e-7)


def test_encoded_batch_cache_replays_a_finite_dataset():
  from maxdiffusion_b200.trainers.loop import EncodedBatchCache

  calls = []

  def encode(b):
    calls.append(int(b["pixel_values"][0]))
    return {"latents": b["pixel_values"] * 2, "pixel_values": b["pixel_values"], "captions": ["x"]}

  cache = EncodedBatchCache(iter([{"pixel_values": torch.tensor([float(i)])} for i in range(3)]), encode)
  seen = [float(next(cache)["latents"][0]) for _ in range(8)]
  assert seen == [0.0, 2.0, 4.0, 0.0, 2.0, 4.0, 0.0, 2.0]
  assert calls == [0, 1, 2]  # the encoders ran once per batch
  assert "pixel_values" not in cache.store[0]


def test_dreambooth_class_images_are_generated_up_to_the_requested_count(tmp_path):
  from maxdiffusion_b200.trainers.stable_diffusion_trainer import DreamboothTrainer

  cdir = tmp_path / "class"
  c = _cfg("base14.yml", SD + ["unet_preset=tiny_sd", "max_train_steps=1", f"class_data_dir={cdir}", "num_class_images=5",
                             "class_prompt=a photo of a dog"], tmp_path / "o")
  tr = DreamboothTrainer(c, mesh=create_device_mesh(c), device="cpu")
  prompts = []

  def fake_pipeline(prompt, seed):
    prompts.append((tuple(prompt), seed))
    return torch.zeros((len(prompt), 8, 8, 3), dtype=torch.uint8)

  assert tr.generate_class_images(fake_pipeline) == 5
  assert len(os.listdir(cdir)) == 5 and all(p[0][0] == "a photo of a dog" for p in prompts)
  assert tr.generate_class_images(fake_pipeline) == 0  # already there


def test_graphed_objective_runs_eagerly_without_a_gpu_and_the_objective_split_is_the_loss():
  """`loss(batch)` is `objective(**draw(batch))`; on a CPU the graphed wrapper is the eager forward + backward."""
  from maxdiffusion_b200.trainers.graphed_step import GraphedObjective
  from maxdiffusion_b200.trainers.stable_diffusion_trainer import StableDiffusionXLTrainer

  c = _cfg("base_xl.yml", SD + ["unet_preset=tiny", "max_train_steps=2", "cuda_graph_train_step=true"], "/tmp/unused-output")
  tr = StableDiffusionXLTrainer(c, mesh=create_device_mesh(c), device="cpu")
  assert tr._graphed is None  # no CUDA device: the switch is ignored
  batch = tr.synthetic_batch(0)
  tr.gen.manual_seed(5)
  a = tr.loss(batch)
  tr.gen.manual_seed(5)
  drawn = tr.draw(batch)
  b = tr.objective(**drawn)
  assert torch.equal(a, b)
  g = GraphedObjective(tr.objective, list(tr.unet.parameters()), eager_calls=0)
  got = g(drawn)
  assert torch.allclose(got, a.detach()) and g.replays == 0
  assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in tr.unet.parameters())


def test_phases_around_the_steps_are_timed_into_the_timing_file(tmp_path):
  """`write_timing_metrics` + `timing_metrics_file`: restore, data set, the loop and the final save each leave a
  "Starting" and a "Finished ... Duration" line; without a file name the lines go to the log."""
  from maxdiffusion_b200.trainers.loop import PhaseTimer
  from maxdiffusion_b200.trainers.stable_diffusion_trainer import StableDiffusionTrainer

  log = tmp_path / "timing" / "phases.log"
  c = _cfg("base15.yml", SD + ["unet_preset=tiny_sd", "max_train_steps=3", "save_final_checkpoint=true", "checkpoint_every=2",
                                "write_timing_metrics=true", f"timing_metrics_file={log}"], tmp_path / "t")
  t = StableDiffusionTrainer(c, mesh=create_device_mesh(c), device="cpu")
  t.start_training()
  lines = log.read_text().splitlines()
  for phase in ("restore checkpoint", "load dataset", "training loop", "final checkpoint"):
    assert f"Starting: {phase}..." in lines
    done = [ln for ln in lines if ln.startswith(f"Finished: {phase} - Duration: ") and ln.endswith(" seconds")]
    assert len(done) == 1 and float(done[0].split("Duration: ")[1].split()[0]) >= 0.0
  assert set(t.phase_timer.durations) == {"restore checkpoint", "load dataset", "training loop", "final checkpoint"}
  assert lines.index("Starting: training loop...") > lines.index("Starting: load dataset...")
  # no file named, or the switch off: nothing is written; other ranks stay silent
  off = PhaseTimer({"write_timing_metrics": False, "timing_metrics_file": str(tmp_path / "no.log")})
  assert off("x", lambda: 7) == 7 and not (tmp_path / "no.log").exists() and "x" in off.durations
  quiet = PhaseTimer({"write_timing_metrics": True, "timing_metrics_file": str(tmp_path / "r1.log")}, rank=1)
  quiet("y", lambda: None)
  assert not (tmp_path / "r1.log").exists()


def test_reuse_example_batch_serves_the_first_batch_for_every_step(tmp_path):
  """`reuse_example_batch=True` takes the input pipeline out of the steps: the loop asks the data source once."""
  import datetime

  from maxdiffusion_b200 import train_utils as T
  from maxdiffusion_b200.trainers.stable_diffusion_trainer import StableDiffusionTrainer

  for reuse, want in (("true", 1), ("false", None)):
    c = _cfg("base15.yml", SD + ["unet_preset=tiny_sd", "max_train_steps=3", "checkpoint_every=-1", f"reuse_example_batch={reuse}"],
             tmp_path / reuse)
    t = StableDiffusionTrainer(c, mesh=create_device_mesh(c), device="cpu")
    pulls = []
    source = t.load_dataset()

    class Counting:
      def __iter__(self):
        return self

      def __next__(self):
        pulls.append(1)
        return next(source)

    t.start_training(data=Counting())
    assert t.step == 3 and (len(pulls) == want if want else len(pulls) >= 3)

  # the small helpers around it
  assert T.load_next_batch(iter([1, 2]), None, {"reuse_example_batch": True}) == 1
  assert T.load_next_batch(iter([1, 2]), "kept", {"reuse_example_batch": True}) == "kept"
  assert T.load_next_batch(iter([1, 2]), "kept", {"reuse_example_batch": False}) == 1
  import types

  assert T.get_first_step(types.SimpleNamespace(step=torch.tensor(7))) == 7 and T.get_first_step(3) == 3
  m = {"scalar": {"learning/loss": 0.5}}
  T.record_scalar_metrics(m, datetime.timedelta(seconds=2), 10.0, 1e-4, total_weights=5)
  assert m["scalar"]["perf/per_device_tflops_per_sec"] == 5.0 and m["scalar"]["learning/total_weights"] == 5.0
  assert set(m["scalar"]) - {"perf/per_device_tflops"} <= set(T.METRICS_TO_MANAGED)
  saved = T.get_params_to_save({"a": torch.ones(2, requires_grad=True), "b": [torch.zeros(1)]})
  assert saved["a"].device.type == "cpu" and not saved["a"].requires_grad and isinstance(saved["b"], list)


def test_write_metrics_function_form(tmp_path):
  import json
  import types

  from maxdiffusion_b200 import train_utils as T

  path = tmp_path / "m.jsonl"
  cfg = {"metrics_file": str(path), "write_metrics": True, "log_period": 1}
  w = T.MetricsWriter(types.SimpleNamespace(get=cfg.get), rank=0)
  T.write_metrics(w, {"scalar": {"learning/loss": torch.tensor(0.25)}}, 3)
  w.close()
  assert json.loads(path.read_text().splitlines()[-1]) == {"step": 3, "learning/loss": 0.25}
  with T.transformer_engine_context():
    pass


def test_structural_similarity_matches_a_filter_based_restatement():
  """The clip-level SSIM against a restatement on scipy's uniform filter (window over time, height and width, sample
  covariances, border cropped)."""
  import numpy as np
  from scipy.ndimage import uniform_filter

  from maxdiffusion_b200 import train_utils as T

  rng = np.random.default_rng(0)
  a = rng.integers(0, 256, (9, 12, 10, 3)).astype(np.uint8)
  b = np.clip(a.astype(np.int32) + rng.integers(-40, 41, a.shape), 0, 255).astype(np.uint8)

  def restated(x, y, R=255.0, win=7):
    out = []
    for c in range(x.shape[-1]):
      p, q = x[..., c].astype(np.float64), y[..., c].astype(np.float64)
      f = lambda t: uniform_filter(t, size=win)
      n = win ** p.ndim
      k = n / (n - 1)
      up, uq = f(p), f(q)
      vp, vq, vpq = k * (f(p * p) - up * up), k * (f(q * q) - uq * uq), k * (f(p * q) - up * uq)
      c1, c2 = (0.01 * R) ** 2, (0.03 * R) ** 2
      s = ((2 * up * uq + c1) * (2 * vpq + c2)) / ((up * up + uq * uq + c1) * (vp + vq + c2))
      pad = (win - 1) // 2
      out.append(s[tuple(slice(pad, d - pad) for d in s.shape)].mean())
    return float(np.mean(out))

  got = T.structural_similarity(a, b)
  assert abs(got - restated(a, b)) < 1e-9 and 0.0 < got < 1.0
  assert abs(T.structural_similarity(a, a) - 1.0) < 1e-12
  assert abs(T.structural_similarity(a[0], b[0]) - restated(a[0], b[0])) < 1e-9      # a single image
  assert T.print_ssim(a, b) == got
  with pytest.raises(ValueError, match="win_size"):
    T.structural_similarity(a[:3], b[:3])
