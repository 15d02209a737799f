"""PusaV1 (pre-encoded Wan latents + T5 embeddings, one `.tensors.pth` per clip) -> TFRecord shards.

`python -m maxdiffusion_b200.data_preprocessing.wan_pusav1_to_tfrecords configs/base_wan_14b.yml train_data_dir=…
tfrecords_dir=… no_records_per_shard=…`. With `enable_eval_timesteps` the first `num_eval_samples` clips get a fixed
timestep each, `num_eval_samples / len(timesteps_list)` consecutive clips per entry of `timesteps_list`, and nothing
after them is written: that is the evaluation split (reference: wan_pusav1_to_tfrecords.py:73-138).
"""
from __future__ import annotations

import csv
import os
import sys

import torch

from .. import max_logging, pyconfig
from .tfrecord_shards import ShardedWriter, create_example


def generate_dataset(config) -> list:
  writer = ShardedWriter(config.tfrecords_dir, int(config.no_records_per_shard))
  eval_mode = bool(config.get("enable_eval_timesteps", False))
  steps = list(config.get("timesteps_list", []) or [])
  n_eval = int(config.get("num_eval_samples", 0))
  if eval_mode:
    if not steps or n_eval % len(steps) != 0:
      raise ValueError("num_eval_samples must be a multiple of len(timesteps_list)")
    bucket = n_eval // len(steps)
  with open(os.path.join(config.train_data_dir, "metadata.csv"), newline="") as f:
    rows = csv.reader(f)
    next(rows)  # header
    for row in rows:
      if eval_mode and writer.total >= n_eval:
        break
      blob = torch.load(os.path.join(config.train_data_dir, "train", f"{row[0]}.tensors.pth"), map_location="cpu", weights_only=True)
      emb = blob["prompt_emb"]["context"].squeeze().float().numpy()
      lat = blob["latents"].float().numpy()
      t = steps[writer.total // bucket] if eval_mode else None
      writer.write(create_example(lat, emb, t))
  files = writer.close()
  max_logging.log(f"wrote {writer.total} examples to {len(files)} shards under {config.tfrecords_dir}")
  return files


def run(config):
  return generate_dataset(config)


def main(argv=None):
  return run(pyconfig.initialize(list(argv if argv is not None else sys.argv)))


if __name__ == "__main__":
  main()
