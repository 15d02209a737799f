"""TFRecord codec (framing + Example + TensorProto), iterators, retry loader, image processor."""
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
