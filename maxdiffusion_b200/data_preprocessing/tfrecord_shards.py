"""Sharded TFRecord writer shared by the preprocessing scripts.

Shards are named `file_<shard>-<last record index>.tfrec` and hold `no_records_per_shard` examples each; every
example is a `tf.train.Example` with `latents` and `encoder_hidden_states` as serialized float32 tensors and an
optional int64 `timesteps` (reference example layout: src/maxdiffusion/data_preprocessing/wan_pusav1_to_tfrecords.py:58-71).
Records are framed with length + masked CRC32C by `input_pipeline.tfrecord`, so TensorFlow readers accept them.
"""
from __future__ import annotations

import os
from typing import List, Optional

import numpy as np

from ..input_pipeline.tfrecord import make_example, serialize_tensor, write_records


def create_example(latent: np.ndarray, hidden_states: np.ndarray, timestep: Optional[int] = None) -> bytes:
  feats = {"latents": [serialize_tensor(np.asarray(latent, np.float32))],
           "encoder_hidden_states": [serialize_tensor(np.asarray(hidden_states, np.float32))]}
  if timestep is not None:
    feats["timesteps"] = np.array([int(timestep)], np.int64)
  return make_example(feats)


class ShardedWriter:

  def __init__(self, folder: str, records_per_shard: int):
    if records_per_shard <= 0:
      raise ValueError("no_records_per_shard must be positive")
    os.makedirs(folder, exist_ok=True)
    self.folder, self.per_shard = folder, int(records_per_shard)
    self.shard, self.total, self.pending = 0, 0, []
    self.files: List[str] = []

  def write(self, record: bytes) -> None:
    self.pending.append(record)
    self.total += 1
    if len(self.pending) >= self.per_shard:
      self.flush()

  def flush(self) -> None:
    if not self.pending:
      return
    path = os.path.join(self.folder, "file_%.2i-%i.tfrec" % (self.shard, self.total))
    write_records(path, self.pending)
    self.files.append(path)
    self.pending, self.shard = [], self.shard + 1

  def close(self) -> List[str]:
    self.flush()
    return self.files
