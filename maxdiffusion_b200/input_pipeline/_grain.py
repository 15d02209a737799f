"""Grain (ArrayRecord) source, available when the `grain` package is installed; its iterator state is saved as the
checkpoint item `iter` (reference: src/maxdiffusion/input_pipeline/_grain_data_processing.py)."""
from __future__ import annotations

import glob
import os

import numpy as np
import torch

from . import tfrecord


def make_grain_iterator(config, batch_size: int, shard_index: int, num_shards: int):
  import grain.python as grain

  files = sorted(glob.glob(os.path.join(config.train_data_dir, "*.array_record*")))
  source = grain.ArrayRecordDataSource(files)

  class Parse(grain.MapTransform):

    def map(self, rec):
      ex = tfrecord.parse_example(rec)
      return {"latents": tfrecord.parse_tensor(ex["latents"][0]).astype(np.float32),
              "encoder_hidden_states": tfrecord.parse_tensor(ex["encoder_hidden_states"][0]).astype(np.float32)}

  sampler = grain.IndexSampler(len(source), shuffle=bool(config.get("enable_data_shuffling", True)), seed=int(config.seed),
                               shard_options=grain.ShardOptions(shard_index, num_shards, drop_remainder=True), num_epochs=None)
  loader = grain.DataLoader(data_source=source, sampler=sampler, operations=[Parse(), grain.Batch(batch_size, drop_remainder=True)],
                            worker_count=0)
  it = iter(loader)

  class Wrapped:

    def __iter__(self):
      return self

    def __next__(self):
      return {k: torch.from_numpy(v) for k, v in next(it).items()}

    def get_state(self):
      return it.get_state()

    def set_state(self, s):
      it.set_state(s)

  return Wrapped()
