"""`make_data_iterator`: dataset_type in {synthetic, tfrecord, tf, hf, grain} -> iterator of host batches.

Reference: src/maxdiffusion/input_pipeline/input_pipeline_interface.py:47-234 and the per-source modules
(_tfds_data_processing.py:83-166 TFRecord iterator with per-host sharding, shuffle, batch, repeat, prefetch, and the
eval set padded to a batch multiple; _hf_data_processing.py; _grain_data_processing.py). Batches are dicts of pinned
CPU tensors; the trainer copies them to the device asynchronously.
"""
from __future__ import annotations

import glob
import os
import queue
import random
import threading
from typing import Iterator, Optional

import numpy as np
import torch

from .. import max_logging
from . import tfrecord
from .synthetic_data_iterator import make_synthetic_iterator


def _pin(t):
  return t.pin_memory() if torch.cuda.is_available() else t


class TFRecordIterator:
  """Wan latents / text-embedding records. Files are sharded over data-parallel ranks (`ds.shard`), examples are
  shuffled inside a buffer, batched, repeated, and prefetched on a background thread."""

  def __init__(self, directory: str, batch_size: int, shard_index: int = 0, num_shards: int = 1, shuffle: bool = True,
               seed: int = 0, repeat: bool = True, with_timesteps: bool = False, prefetch: int = 2, pad_to_batch: bool = False):
    files = sorted(set(glob.glob(os.path.join(directory, "*.tfrec*"))))
    if not files:
      raise FileNotFoundError(f"no TFRecord files under {directory}")
    self.files = files[shard_index::num_shards] or files
    self.batch_size, self.shuffle, self.repeat = batch_size, shuffle, repeat
    self.with_timesteps, self.pad_to_batch = with_timesteps, pad_to_batch
    self.rng = random.Random(seed + shard_index)
    self.queue: "queue.Queue" = queue.Queue(maxsize=prefetch)
    self.thread = threading.Thread(target=self._produce, daemon=True)
    self.thread.start()

  def _examples(self):
    while True:
      files = list(self.files)
      if self.shuffle:
        self.rng.shuffle(files)
      for f in files:
        for rec in tfrecord.read_records(f):
          ex = tfrecord.parse_example(rec)
          # Wan records name the text states `encoder_hidden_states`, Stable Diffusion ones `hidden_states`
          text_key = "encoder_hidden_states" if "encoder_hidden_states" in ex else "hidden_states"
          item = {"latents": tfrecord.parse_tensor(ex["latents"][0]).astype(np.float32),
                  "encoder_hidden_states": tfrecord.parse_tensor(ex[text_key][0]).astype(np.float32)}
          if self.with_timesteps and "timesteps" in ex:
            item["timesteps"] = np.asarray(ex["timesteps"], dtype=np.int64)[0]
          yield item
      if not self.repeat:
        return

  def _produce(self):
    buf, batch = [], []
    try:
      for ex in self._examples():
        if self.shuffle:
          buf.append(ex)
          if len(buf) < 64:
            continue
          ex = buf.pop(self.rng.randrange(len(buf)))
        batch.append(ex)
        if len(batch) == self.batch_size:
          self.queue.put(self._collate(batch))
          batch = []
      batch.extend(buf)
      while len(batch) >= self.batch_size:
        self.queue.put(self._collate(batch[:self.batch_size]))
        batch = batch[self.batch_size:]
      if batch and self.pad_to_batch:
        batch = batch + [batch[-1]] * (self.batch_size - len(batch))
        self.queue.put(self._collate(batch))
    except Exception as e:
      self.queue.put(e)
    self.queue.put(None)

  @staticmethod
  def _collate(items):
    return {k: _pin(torch.from_numpy(np.stack([it[k] for it in items]))) for k in items[0]}

  def __iter__(self):
    return self

  def __next__(self):
    item = self.queue.get()
    if item is None:
      raise StopIteration
    if isinstance(item, Exception):
      raise item
    return item


class HFDatasetIterator:
  """Hugging Face `datasets` source (local files / cache only: there is no network). Columns are `image_column` and
  `caption_column`; images are resized / cropped / flipped and normalised to [-1, 1], captions are returned as text
  for the trainer's tokenizers."""

  def __init__(self, config, batch_size: int, shard_index: int = 0, num_shards: int = 1):
    import datasets  # optional dependency

    if config.get("train_data_dir", ""):
      ds = datasets.load_dataset("imagefolder", data_dir=config.train_data_dir, split=config.get("train_split", "train"))
    else:
      ds = datasets.load_dataset(config.dataset_name, data_dir=config.get("hf_data_dir", None) or None,
                                 data_files=config.get("hf_train_files", None), split=config.get("train_split", "train"),
                                 token=config.get("hf_access_token", None))
    self.ds = ds.shard(num_shards, shard_index) if num_shards > 1 else ds
    self.config, self.batch_size = config, batch_size
    self.order = list(range(len(self.ds)))
    self.pos, self.rng = 0, random.Random(int(config.get("seed", 0)))

  def __iter__(self):
    return self

  def __next__(self):
    from ..image_processor import VaeImageProcessor

    proc = VaeImageProcessor()
    res = int(self.config.get("resolution", 512))
    imgs, caps = [], []
    for _ in range(self.batch_size):
      if self.pos >= len(self.order):
        self.pos = 0
        if self.config.get("enable_data_shuffling", True):
          self.rng.shuffle(self.order)
      row = self.ds[self.order[self.pos]]
      self.pos += 1
      imgs.append(proc.preprocess(row[self.config.get("image_column", "image")], res, res,
                                  center_crop=bool(self.config.get("center_crop", False)),
                                  random_flip=bool(self.config.get("random_flip", False)), rng=self.rng))
      caps.append(row[self.config.get("caption_column", "text")])
    return {"pixel_values": _pin(torch.cat(imgs)), "captions": caps}


class DreamboothIterator:
  """Instance + class (prior-preservation) batches for Dreambooth from two image folders.

  There are as many pairs as class images; the instance images are cycled to match (few photographs of the subject
  against many pictures of its class). A batch carries the instance half under the plain keys and the class half under
  `class_`-prefixed keys, which is what `DreamboothTrainer.loss` weighs separately
  (reference: src/maxdiffusion/input_pipeline/input_pipeline_interface.py:127-234, `make_dreambooth_train_iterator`)."""

  EXTENSIONS = (".png", ".jpg", ".jpeg", ".webp", ".bmp")

  def __init__(self, config, batch_size: int, shard_index: int = 0, num_shards: int = 1):
    def listing(folder, what):
      files = sorted(f for f in os.listdir(folder) if f.lower().endswith(self.EXTENSIONS)) if os.path.isdir(folder) else []
      if not files:
        raise FileNotFoundError(f"no {what} images under {folder!r}")
      return [os.path.join(folder, f) for f in files]

    self.class_files = listing(str(config.get("class_data_dir", "")), "class")
    self.instance_files = listing(str(config.get("instance_data_dir", "")), "instance")
    self.pairs = list(range(len(self.class_files)))[shard_index::num_shards] or list(range(len(self.class_files)))
    self.config, self.batch_size = config, batch_size
    self.pos, self.rng = 0, random.Random(int(config.get("seed", 0)) + shard_index)

  def __iter__(self):
    return self

  def _load(self, path: str) -> torch.Tensor:
    from PIL import Image

    from ..image_processor import VaeImageProcessor

    res = int(self.config.get("resolution", 512))
    with Image.open(path) as im:
      return VaeImageProcessor().preprocess(im.convert("RGB"), res, res, center_crop=bool(self.config.get("center_crop", False)),
                                            random_flip=bool(self.config.get("random_flip", False)), rng=self.rng)

  def __next__(self) -> dict:
    inst, cls = [], []
    for _ in range(self.batch_size):
      if self.pos >= len(self.pairs):
        self.pos = 0
        if self.config.get("enable_data_shuffling", True):
          self.rng.shuffle(self.pairs)
      i = self.pairs[self.pos]
      self.pos += 1
      inst.append(self._load(self.instance_files[i % len(self.instance_files)]))
      cls.append(self._load(self.class_files[i]))
    n = self.batch_size
    return {"pixel_values": _pin(torch.cat(inst)), "captions": [str(self.config.get("instance_prompt", ""))] * n,
            "class_pixel_values": _pin(torch.cat(cls)), "class_captions": [str(self.config.get("class_prompt", ""))] * n}


def make_dreambooth_train_iterator(config, mesh, batch_size: int):
  """The Dreambooth iterator of this rank: the pairs are split over the ranks that hold different samples."""
  shards = mesh.size("data") * mesh.size("fsdp")
  index = mesh.coords.get("data", 0) * mesh.size("fsdp") + mesh.coords.get("fsdp", 0)
  return DreamboothIterator(config, batch_size, index, shards)


def make_data_iterator(config, mesh, batch_size: int, eval_mode: bool = False):
  kind = str(config.get("dataset_type", "synthetic"))
  dp = mesh.size("data") * mesh.size("fsdp")
  idx = mesh.coords.get("data", 0) * mesh.size("fsdp") + mesh.coords.get("fsdp", 0)
  if kind == "synthetic":
    return make_synthetic_iterator(config, batch_size, seed=int(config.get("seed", 0)) + 17 + idx)
  if kind in ("tfrecord", "tf"):
    directory = config.get("eval_data_dir", "") if eval_mode else config.get("train_data_dir", "") or config.get("tfrecords_dir", "")
    return TFRecordIterator(directory, batch_size, idx, dp, shuffle=bool(config.get("enable_data_shuffling", True)) and not eval_mode,
                            seed=int(config.get("seed", 0)), repeat=not eval_mode, with_timesteps=eval_mode, pad_to_batch=eval_mode)
  if kind == "hf":
    return HFDatasetIterator(config, batch_size, idx, dp)
  if kind == "grain":
    try:
      import grain  # noqa: F401
    except ImportError as e:
      raise ImportError("dataset_type=grain needs the `grain` package (ArrayRecord files); it is not installed") from e
    from ._grain import make_grain_iterator

    return make_grain_iterator(config, batch_size, idx, dp)
  raise ValueError(f"unknown dataset_type {kind}")
