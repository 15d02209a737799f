"""Checkpoint layout, resume (weights + optimizer moments) and the converted-weights cache."""
import json
import os

import torch

from maxdiffusion_b200 import pyconfig
from maxdiffusion_b200.checkpointing.wan_checkpointer import WanCheckpointer
from maxdiffusion_b200.loaders import wan_loader
from maxdiffusion_b200.parallel.mesh import create_device_mesh
from maxdiffusion_b200.trainers.wan_trainer import WanTrainer

CFG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs",
                   "base_wan_14b.yml")
TINY = '{"num_attention_heads": 2, "attention_head_dim": 32, "ffn_dim": 64, "num_layers": 2, "text_dim": 32, "freq_dim": 32}'


def _trainer(tmp, seed=0):
  config = pyconfig.initialize(
      ["t", CFG, "run_name=ck", f"output_dir={tmp}", "height=32", "width=32", "num_frames=5", "dataset_type=synthetic",
       "wan_preset=tiny", f"wan_config_overrides={TINY}", "warmup_steps_fraction=0.0", "log_config=false",
       "write_metrics=false", "learning_rate=1e-3", "synthetic_override_text_dim=32", "max_sequence_length=8",
       "save_optimizer=true", f"seed={seed}"], unittest=True)
  return config, WanTrainer(config, mesh=create_device_mesh(config), device="cpu")


def test_save_layout_and_resume(tmp_path):
  config, tr = _trainer(str(tmp_path))
  data = tr.load_dataset()
  batches = [next(data) for _ in range(4)]
  for b in batches[:2]:
    tr.train_step(b)
  ck = WanCheckpointer(config)
  ck.save(2, tr)
  ck.manager.wait_until_finished()
  step_dir = os.path.join(config.checkpoint_dir, "2")
  assert os.path.exists(os.path.join(step_dir, "_CHECKPOINT_METADATA"))
  assert json.load(open(os.path.join(step_dir, "wan_config", "metadata")))["num_layers"] == 2
  meta = json.load(open(os.path.join(step_dir, "wan_state", "_METADATA")))["tree_metadata"]
  # the reference's tree paths: scanned [L, in, out] kernels under blocks/...
  assert meta["blocks/attn1/query/kernel"]["shape"] == [2, 64, 64]
  assert "condition_embedder/time_embedder/linear_1/kernel" in meta and "blocks/ffn/proj_out/kernel" in meta
  tr.gen = torch.Generator().manual_seed(1)
  ref = [float(tr.train_step(b)["learning/loss"]) for b in batches[2:]]  # the uninterrupted run

  config2, tr2 = _trainer(str(tmp_path), seed=5)  # different init: everything must come from the checkpoint
  assert WanCheckpointer(config2).maybe_restore(tr2) == 2
  tr2.step = 2
  tr2.gen = torch.Generator().manual_seed(1)
  # same RNG stream + same state -> the next steps agree
  config3, tr3 = _trainer(str(tmp_path), seed=7)
  WanCheckpointer(config3).maybe_restore(tr3)
  tr3.gen = torch.Generator().manual_seed(1)
  a = [float(tr2.train_step(b)["learning/loss"]) for b in batches[2:]]
  b_ = [float(tr3.train_step(b)["learning/loss"]) for b in batches[2:]]
  assert a == b_ and tr2.engine.step_count == tr3.engine.step_count == 4
  # resuming continues the uninterrupted run: weights, moments and the step counter all came back
  import pytest

  assert a == pytest.approx(ref, rel=1e-5, abs=1e-7)


def test_converted_weights_cache_round_trip_and_invalidation(tmp_path):
  sd = {"a.weight": torch.randn(4, 3).to(torch.bfloat16), "b": torch.arange(5, dtype=torch.float32)}
  folder = str(tmp_path / "cache")
  wan_loader.save_converted_cache(folder, sd, "torch.bfloat16")
  back = wan_loader.load_converted_cache(folder, list(sd), "torch.bfloat16")
  assert all(torch.equal(back[k], sd[k]) for k in sd)
  assert wan_loader.load_converted_cache(folder, list(sd) + ["c"], "torch.bfloat16") is None   # key set changed
  assert wan_loader.load_converted_cache(folder, list(sd), "torch.float32") is None            # dtype policy changed


def _tiny_pipeline_config(tmp, name="base_wan_14b.yml", **kw):
  extra = [f"{k}={v}" for k, v in kw.items()]
  cfg = os.path.join(os.path.dirname(CFG), name)
  return pyconfig.initialize(
      ["t", cfg, "run_name=pc", f"output_dir={tmp}", "wan_preset=tiny", f"wan_config_overrides={TINY}", "log_config=false",
       "enable_async_checkpointing=false", "height=32", "width=32", "num_frames=5", *extra], unittest=True)


def test_pretrained_weights_cache_hit_miss_and_disabled(tmp_path):
  """`pretrained_orbax_dir`: a miss loads the pretrained weights and writes the cache, a hit restores from it without
  touching the pretrained weights, an empty setting never writes one (the cases of the reference's
  src/maxdiffusion/tests/wan/wan_checkpointer_test.py:38-86)."""
  from maxdiffusion_b200.pipelines.wan.wan_pipeline import WanPipeline2_1

  calls = []

  class Pipe(WanPipeline2_1):
    @classmethod
    def from_pretrained(cls, config, device=None, **kw):
      calls.append("from_pretrained")
      torch.manual_seed(123)
      return cls.from_config(config, device="cpu", load_vae=False)

  cache = str(tmp_path / "cache")
  config = _tiny_pipeline_config(str(tmp_path), pretrained_orbax_dir=cache)
  ck = WanCheckpointer(config)
  first = ck.load_pretrained_pipeline_or_diffusers(Pipe, device="cpu")
  assert calls == ["from_pretrained"] and os.path.exists(os.path.join(cache, "0", "wan_state", "state.safetensors"))
  second = WanCheckpointer(config).load_pretrained_pipeline_or_diffusers(Pipe, device="cpu")
  assert calls == ["from_pretrained"]                                  # hit: the pretrained weights were not read again
  for (n, a), (_, b) in zip(first.transformer.state_dict().items(), second.transformer.state_dict().items()):
    assert torch.equal(a, b), n
  plain = _tiny_pipeline_config(str(tmp_path / "p"), pretrained_orbax_dir="")
  WanCheckpointer(plain).load_pretrained_pipeline_or_diffusers(Pipe, device="cpu")
  assert calls == ["from_pretrained", "from_pretrained"] and not os.path.exists(str(tmp_path / "p" / "cache"))


def test_checkpoint_of_one_expert_does_not_fill_a_two_expert_pipeline(tmp_path):
  """Strict item selection: a Wan 2.1 checkpoint (`wan_state`) restored into a Wan 2.2 pipeline, or the reverse, names
  the item that is absent instead of loading something else."""
  import pytest

  from maxdiffusion_b200.pipelines.wan.wan_pipeline import WanPipeline2_1, WanPipeline2_2

  c1 = _tiny_pipeline_config(str(tmp_path / "one"))
  one = WanPipeline2_1.from_config(c1, device="cpu", load_vae=False)
  WanCheckpointer(c1).save_pipeline(3, one)
  c2 = _tiny_pipeline_config(str(tmp_path / "two"), "base_wan_27b.yml").replace(checkpoint_dir=c1.checkpoint_dir)
  two = WanPipeline2_2.from_config(c2, device="cpu", load_vae=False)
  with pytest.raises(ValueError, match="high_noise_transformer_state"):
    WanCheckpointer(c2).restore_into_pipeline(two)
  c3 = _tiny_pipeline_config(str(tmp_path / "three"), "base_wan_27b.yml")
  WanCheckpointer(c3).save_pipeline(1, two)
  c4 = _tiny_pipeline_config(str(tmp_path / "four")).replace(checkpoint_dir=c3.checkpoint_dir)
  with pytest.raises(ValueError, match="wan_state"):
    WanCheckpointer(c4).restore_into_pipeline(one)
  WanCheckpointer(c2.replace(checkpoint_dir=c3.checkpoint_dir)).restore_into_pipeline(two)   # matching variant: fine


def test_train_wan_loop_checkpoints_resumes_and_can_reuse_one_batch(tmp_path):
  """`train_wan.train`: the loop writes periodic and final checkpoints, a second start in the same output directory
  resumes from the last one, and `reuse_example_batch` asks the data source for one batch only."""
  from maxdiffusion_b200 import train_wan

  def config(steps, *extra):
    return pyconfig.initialize(
        ["t", CFG, "run_name=loop", f"output_dir={tmp_path}", "height=32", "width=32", "num_frames=5", "dataset_type=synthetic",
         "wan_preset=tiny", f"wan_config_overrides={TINY}", "warmup_steps_fraction=0.0", "log_config=false", "write_metrics=false",
         "learning_rate=1e-3", "synthetic_override_text_dim=32", "max_sequence_length=8", "save_optimizer=true",
         "enable_async_checkpointing=false", "checkpoint_every=2", "save_final_checkpoint=true", f"max_train_steps={steps}",
         *extra], unittest=True)

  first = train_wan.train(config(3))
  ckpt = first.config.checkpoint_dir
  assert first.step == 3 and sorted(int(d) for d in os.listdir(ckpt) if d.isdigit()) == [2, 3]
  calls = []
  original = WanTrainer.train_step

  def counted(self, batch):
    calls.append(self.step)
    return original(self, batch)

  WanTrainer.train_step = counted
  try:
    second = train_wan.train(config(5))                     # picks up at step 3: two steps are left
  finally:
    WanTrainer.train_step = original
  assert len(calls) == 2 and second.step == 5 and second.engine.step_count == 5
  assert sorted(int(d) for d in os.listdir(ckpt) if d.isdigit()) == [2, 3, 4, 5]

  pulls = []
  c = config(8, "reuse_example_batch=true", "checkpoint_every=-1", "save_final_checkpoint=false")
  trainer = WanTrainer(c, mesh=create_device_mesh(c), device="cpu")
  source = trainer.load_dataset()

  class Counting:
    def __iter__(self):
      return self

    def __next__(self):
      pulls.append(1)
      return next(source)

  trainer.load_dataset = lambda: Counting()
  trainer.start_training()
  assert trainer.step == 8 and len(pulls) == 1


def test_wan_eval_groups_losses_by_timestep_and_runs_inside_the_loop(tmp_path):
  """`eval_every` with a TFRecord evaluation split: per-sample losses at the records' own timesteps, grouped by
  timestep, every group cut to `eval_max_number_of_samples_in_bucket`, mean of the group means as `learning/eval_loss`."""
  import json

  import numpy as np

  from maxdiffusion_b200.input_pipeline import tfrecord

  rng = np.random.default_rng(0)
  ts = [100, 100, 100, 500, 500, 900]
  recs = [tfrecord.make_example({"latents": [tfrecord.serialize_tensor(rng.standard_normal((16, 2, 4, 4)).astype(np.float32))],
                                 "encoder_hidden_states": [tfrecord.serialize_tensor(rng.standard_normal((8, 32)).astype(np.float32))],
                                 "timesteps": np.array([t], dtype=np.int64)}) for t in ts]
  os.makedirs(tmp_path / "eval")
  tfrecord.write_records(str(tmp_path / "eval" / "e.tfrecord"), recs)
  metrics = tmp_path / "metrics.jsonl"
  config = pyconfig.initialize(
      ["t", CFG, "run_name=ev", f"output_dir={tmp_path}", "height=32", "width=32", "num_frames=5", "dataset_type=tfrecord",
       f"train_data_dir={tmp_path}/eval", f"eval_data_dir={tmp_path}/eval", "wan_preset=tiny", f"wan_config_overrides={TINY}",
       "warmup_steps_fraction=0.0", "log_config=false", "learning_rate=1e-3", "max_sequence_length=8", "per_device_batch_size=2",
       "eval_every=2", "max_train_steps=2", "eval_max_number_of_samples_in_bucket=2", f"metrics_file={metrics}",
       "checkpoint_every=-1", "enable_async_checkpointing=false"], unittest=True)
  tr = WanTrainer(config, mesh=create_device_mesh(config), device="cpu")
  tr.gen = torch.Generator().manual_seed(3)
  got = tr.eval(0)
  # by hand: the same noise stream, one batch of two after another
  from maxdiffusion_b200.input_pipeline.input_pipeline_interface import make_data_iterator

  tr.gen = torch.Generator().manual_seed(3)
  buckets = {}
  for batch in make_data_iterator(config, tr.mesh, tr.batch_size, eval_mode=True):
    for t, l in zip(batch["timesteps"].tolist(), tr.eval_step(batch).tolist()):
      buckets.setdefault(int(t), []).append(l)
  assert sorted(buckets) == [100, 500, 900] and len(buckets[100]) == 3
  want = sum(sum(v[:2]) / len(v[:2]) for v in buckets.values()) / 3      # the 100 bucket is cut to two samples
  assert abs(got - want) < 1e-6 and got > 0
  before = [p.detach().clone() for p in tr.model.parameters()]
  tr.eval(0)
  assert all(torch.equal(a, b) for a, b in zip(before, tr.model.parameters()))   # evaluation leaves the weights alone
  tr.start_training()                                                            # step 2 triggers an evaluation
  lines = [json.loads(x) for x in metrics.read_text().splitlines()]
  assert any("learning/eval_loss" in ln and ln["step"] == 2 for ln in lines)
