"""TFRecord codec (framing + Example + TensorProto), iterators, retry loader, image processor."""
import os

import numpy as np
import pytest
import torch

from maxdiffusion_b200.image_processor import VaeImageProcessor
from maxdiffusion_b200.input_pipeline import tfrecord
from maxdiffusion_b200.input_pipeline.input_pipeline_interface import TFRecordIterator
from maxdiffusion_b200.multihost_dataloading import MultiHostDataLoadIterator
from maxdiffusion_b200.video_processor import VideoProcessor


def test_crc32c_known_vector():
  assert tfrecord.crc32c(b"123456789") == 0xE3069283


def test_example_and_tensor_round_trip(tmp_path):
  rng = np.random.default_rng(0)
  recs = []
  for i in range(5):
    lat = rng.standard_normal((16, 3, 4, 4)).astype(np.float32)
    emb = rng.standard_normal((8, 32)).astype(np.float32)
    recs.append(tfrecord.make_example({"latents": [tfrecord.serialize_tensor(lat)],
                                       "encoder_hidden_states": [tfrecord.serialize_tensor(emb)],
                                       "timesteps": np.array([125 * (i + 1)], dtype=np.int64), "w": np.array([0.5, 1.5], np.float32)}))
  path = str(tmp_path / "a.tfrecord")
  tfrecord.write_records(path, recs)
  back = [tfrecord.parse_example(r) for r in tfrecord.read_records(path, verify=True)]
  assert len(back) == 5 and back[2]["timesteps"][0] == 375 and np.allclose(back[0]["w"], [0.5, 1.5])
  assert tfrecord.parse_tensor(back[0]["latents"][0]).shape == (16, 3, 4, 4)
  it = TFRecordIterator(str(tmp_path), batch_size=2, shuffle=False, repeat=False, with_timesteps=True, pad_to_batch=True)
  batches = list(it)
  assert len(batches) == 3 and batches[0]["latents"].shape == (2, 16, 3, 4, 4) and batches[-1]["timesteps"].tolist() == [625, 625]


def test_retry_loader():
  class Flaky:
    def __init__(self):
      self.n = 0
    def __iter__(self):
      return self
    def __next__(self):
      self.n += 1
      if self.n < 3:
        raise OSError("transient")
      return {"x": torch.ones(1)}
  assert MultiHostDataLoadIterator(Flaky(), sleep_s=0.0).__next__()["x"].item() == 1.0
  with pytest.raises(RuntimeError):
    class Dead:
      def __iter__(self):
        return self
      def __next__(self):
        raise OSError("gone")
    MultiHostDataLoadIterator(Dead(), max_retries=2, sleep_s=0.0).__next__()


def test_image_and_video_processor():
  img = np.random.default_rng(0).integers(0, 255, (50, 70, 3)).astype(np.uint8)
  t = VaeImageProcessor().preprocess(img, 32, 48, center_crop=True)
  assert t.shape == (1, 3, 32, 48) and t.min() >= -1 and t.max() <= 1
  v = VideoProcessor().preprocess_video([img] * 3, 32, 48)
  assert v.shape == (1, 3, 3, 32, 48)
  assert VideoProcessor().postprocess_video(v).shape == (1, 3, 32, 48, 3)


def test_hf_dataset_iterator_shards_shuffles_and_preprocesses(monkeypatch):
  """`dataset_type=hf` against a stand-in for the `datasets` package: the split is sharded over the data ranks, rows wrap
  around with a reshuffle, images come out normalised [-1, 1] at the configured resolution, captions as text."""
  import sys
  import types

  import numpy as np
  from PIL import Image

  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.input_pipeline.input_pipeline_interface import HFDatasetIterator

  class FakeSplit:
    def __init__(self, rows):
      self.rows = rows

    def __len__(self):
      return len(self.rows)

    def __getitem__(self, i):
      return self.rows[i]

    def shard(self, n, i):
      return FakeSplit(self.rows[i::n])

  calls = {}

  def load_dataset(name, **kw):
    calls["args"] = (name, kw)
    rows = [{"image": Image.fromarray(np.full((40, 56, 3), 10 * j, dtype=np.uint8)), "text": f"caption {j}"} for j in range(6)]
    return FakeSplit(rows)

  monkeypatch.setitem(sys.modules, "datasets", types.SimpleNamespace(load_dataset=load_dataset))
  cfg_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs")
  c = pyconfig.initialize(["t", os.path.join(cfg_dir, "base15.yml"), "run_name=t", "dataset_type=hf", "dataset_name=some/set",
                           "resolution=32", "enable_data_shuffling=false", "log_config=false"], unittest=True)
  it = HFDatasetIterator(c, batch_size=2, shard_index=1, num_shards=2)
  assert calls["args"][0] == "some/set" and len(it.ds) == 3
  b1, b2 = next(it), next(it)
  assert b1["pixel_values"].shape == (2, 3, 32, 32) and -1.0 <= b1["pixel_values"].min() and b1["pixel_values"].max() <= 1.0
  assert b1["captions"] == ["caption 1", "caption 3"] and b2["captions"] == ["caption 5", "caption 1"]  # wraps around


def test_grain_iterator_parses_records_and_saves_its_position(monkeypatch, tmp_path):
  """`dataset_type=grain` against a stand-in for `grain.python`: records are `tf.train.Example` bytes parsed by this
  repository's reader, batches are tensors, and the position round-trips through get_state / set_state."""
  import sys
  import types

  import numpy as np

  from maxdiffusion_b200.input_pipeline import _grain, tfrecord

  recs = [tfrecord.make_example({"latents": [tfrecord.serialize_tensor(np.full((2, 3), float(i), np.float32))],
                                      "encoder_hidden_states": [tfrecord.serialize_tensor(np.full((4,), float(-i), np.float32))]})
          for i in range(8)]

  class MapTransform:
    pass

  class Batch:
    def __init__(self, n, drop_remainder=True):
      self.n = n

  class DataLoader:
    def __init__(self, data_source, sampler, operations, worker_count):
      self.src, self.ops = data_source, operations

    def __iter__(self):
      loader = self

      class It:
        pos = 0

        def __next__(self):
          parse, batch = loader.ops
          rows = [parse.map(loader.src[(self.pos + j) % len(loader.src)]) for j in range(batch.n)]
          self.pos += batch.n
          return {k: np.stack([r[k] for r in rows]) for k in rows[0]}

        def get_state(self):
          return {"pos": self.pos}

        def set_state(self, s):
          self.pos = s["pos"]

      return It()

  fake = types.SimpleNamespace(ArrayRecordDataSource=lambda files: recs, MapTransform=MapTransform, Batch=Batch, DataLoader=DataLoader,
                               IndexSampler=lambda *a, **k: None, ShardOptions=lambda *a, **k: None)
  monkeypatch.setitem(sys.modules, "grain", types.SimpleNamespace(python=fake))
  monkeypatch.setitem(sys.modules, "grain.python", fake)
  cfg = types.SimpleNamespace(train_data_dir=str(tmp_path), seed=0, get=lambda k, d=None: d)
  it = _grain.make_grain_iterator(cfg, batch_size=2, shard_index=0, num_shards=1)
  b = next(it)
  assert b["latents"].shape == (2, 2, 3) and float(b["latents"][1, 0, 0]) == 1.0 and float(b["encoder_hidden_states"][1, 0]) == -1.0
  state = it.get_state()
  second = next(it)
  it.set_state(state)
  assert torch.equal(next(it)["latents"], second["latents"])


def test_synthetic_iterators_have_the_shapes_and_keys_the_reference_test_expects():
  """src/maxdiffusion/tests/input_pipeline_interface_test.py:446-549: Wan evaluation batches at the override size with
  `timesteps`, Flux batches with packed latents, T5 / CLIP embeddings and position ids."""
  from maxdiffusion_b200 import pyconfig
  from maxdiffusion_b200.input_pipeline.synthetic_data_iterator import make_synthetic_iterator

  cfg_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "maxdiffusion_b200", "configs")
  c = pyconfig.initialize(["t", os.path.join(cfg_dir, "base_wan_14b.yml"), "log_config=false", "synthetic_override_height=720",
                           "synthetic_override_width=1280", "synthetic_override_num_frames=121"], unittest=True)
  b = next(make_synthetic_iterator(c, batch_size=2, is_training=False))
  assert b["latents"].shape == (2, 16, (121 - 1) // 4 + 1, 720 // 8, 1280 // 8)
  assert b["encoder_hidden_states"].shape == (2, 512, 4096) and b["timesteps"].shape == (2,)
  assert "timesteps" not in next(make_synthetic_iterator(c, batch_size=2))
  f = pyconfig.initialize(["t", os.path.join(cfg_dir, "base_flux_dev.yml"), "log_config=false", "resolution=512",
                           "max_sequence_length=512"], unittest=True)
  b = next(make_synthetic_iterator(f, batch_size=3))
  seq = (512 // 16) ** 2
  assert b["pixel_values"].shape == (3, seq, 64) and b["input_ids"].shape == (3, 512, 3) and b["img_ids"].shape == (3, seq, 3)
  assert b["text_embeds"].shape == (3, 512, 4096) and b["prompt_embeds"].shape == (3, 768) and b["txt_ids"] is b["input_ids"]


def test_dreambooth_iterator_pairs_every_class_image_with_a_cycled_instance_image(tmp_path):
  """Two folders -> batches with an instance half (plain keys) and a class half (`class_` keys): as many pairs as
  class images, instance images cycled; `DreamboothTrainer.loss` weighs the halves separately."""
  import types

  from PIL import Image

  from maxdiffusion_b200.input_pipeline.input_pipeline_interface import DreamboothIterator, make_dreambooth_train_iterator

  for folder, count, base in (("inst", 2, 40), ("cls", 5, 200)):
    os.makedirs(tmp_path / folder)
    for i in range(count):
      Image.new("RGB", (20, 16), (base + 10 * i, 0, 0)).save(tmp_path / folder / f"{i}.png")
  (tmp_path / "cls" / "notes.txt").write_text("not an image")
  cfg = {"instance_data_dir": str(tmp_path / "inst"), "class_data_dir": str(tmp_path / "cls"), "resolution": 8, "seed": 0,
         "instance_prompt": "a photo of sks dog", "class_prompt": "a photo of a dog", "enable_data_shuffling": False,
         "center_crop": True}
  it = DreamboothIterator(types.SimpleNamespace(get=cfg.get), batch_size=2)
  assert len(it.pairs) == 5 and len(it.instance_files) == 2
  red = lambda t: [round((float(x[0].mean()) + 1) * 127.5) for x in t]
  b1, b2, b3 = next(it), next(it), next(it)
  assert b1["pixel_values"].shape == (2, 3, 8, 8) and b1["class_pixel_values"].shape == (2, 3, 8, 8)
  assert b1["captions"] == ["a photo of sks dog"] * 2 and b1["class_captions"] == ["a photo of a dog"] * 2
  assert red(b1["class_pixel_values"]) + red(b2["class_pixel_values"]) + red(b3["class_pixel_values"]) == [200, 210, 220, 230, 240, 200]
  assert red(b1["pixel_values"]) + red(b2["pixel_values"]) + red(b3["pixel_values"]) == [40, 50, 40, 50, 40, 40]   # cycled, then wraps
  mesh = types.SimpleNamespace(size=lambda a: {"data": 2, "fsdp": 1}.get(a, 1), coords={"data": 1, "fsdp": 0})
  sharded = make_dreambooth_train_iterator(types.SimpleNamespace(get=cfg.get), mesh, 1)
  assert sharded.pairs == [1, 3]
  import pytest

  with pytest.raises(FileNotFoundError, match="no instance images"):
    DreamboothIterator(types.SimpleNamespace(get={**cfg, "instance_data_dir": str(tmp_path / "none")}.get), 1)


def test_dreambooth_loss_takes_the_class_half_of_a_pixel_batch(monkeypatch):
  import types

  from maxdiffusion_b200.trainers import stable_diffusion_trainer as T

  seen = []
  monkeypatch.setattr(T.StableDiffusionTrainer, "loss", lambda self, batch: (seen.append(sorted(batch)), torch.tensor(2.0))[1])
  stub = T.DreamboothTrainer.__new__(T.DreamboothTrainer)
  stub.config = {"prior_loss_weight": 0.5}
  batch = {"pixel_values": torch.zeros(1), "captions": ["a"], "class_pixel_values": torch.zeros(1), "class_captions": ["b"]}
  assert float(T.DreamboothTrainer.loss(stub, batch)) == 3.0                 # instance term + 0.5 x class term
  assert seen == [["captions", "pixel_values"], ["captions", "pixel_values"]]
  seen.clear()
  assert float(T.DreamboothTrainer.loss(stub, {"latents": torch.zeros(1)})) == 2.0 and len(seen) == 1
