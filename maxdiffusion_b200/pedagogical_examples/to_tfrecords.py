"""Image-caption dataset -> TFRecords of VAE latents and text-encoder states for Stable Diffusion training with
`dataset_type=tfrecord` (features `latents`, `hidden_states`; reference: pedagogical_examples/to_tfrecords.py:105-160).

  python -m maxdiffusion_b200.pedagogical_examples.to_tfrecords configs/base15.yml dataset_name=/data/pokemon \
      tfrecords_dir=/data/pokemon_tfrec no_records_per_shard=512
"""
from __future__ import annotations

import sys

import numpy as np
import torch

from .. import max_logging, pyconfig
from ..data_preprocessing.tfrecord_shards import ShardedWriter
from ..input_pipeline.tfrecord import make_example, serialize_tensor
from ..maxdiffusion_utils import encode, transform_images


def create_example(latent: np.ndarray, hidden_states: np.ndarray) -> bytes:
  return make_example({"latents": [serialize_tensor(np.asarray(latent, np.float32))],
                       "hidden_states": [serialize_tensor(np.asarray(hidden_states, np.float32))]})


def generate_dataset(config, pipe, dataset, batch_size: int = 16) -> list:
  writer = ShardedWriter(config.tfrecords_dir, int(config.no_records_per_shard))
  gen = torch.Generator().manual_seed(int(config.get("seed", 0)))
  res = int(config.resolution)
  for i in range(0, len(dataset), batch_size):
    rows = dataset[i:i + batch_size]
    lat = transform_images({config.image_column: rows[config.image_column]}, config.image_column, res, vae=pipe.vae, generator=gen)["pixel_values"]
    tok = pipe.tokenizers[0]
    ids = tok(list(rows[config.caption_column]), max_length=tok.model_max_length, padding="max_length", truncation=True, return_tensors="pt").input_ids
    with torch.no_grad():
      hs = encode(ids, pipe.text_encoders[0]).float().cpu().numpy()
    for a, b in zip(lat, hs):
      writer.write(create_example(a, b))
  files = writer.close()
  max_logging.log(f"wrote {writer.total} examples to {len(files)} shards")
  return files


def run(config):
  import datasets

  from ..checkpointing.base_stable_diffusion_checkpointer import BaseStableDiffusionCheckpointer
  from ..pipelines.stable_diffusion.pipeline_stable_diffusion import StableDiffusionPipeline

  pipe = BaseStableDiffusionCheckpointer(config).load_pipeline(StableDiffusionPipeline)
  ds = datasets.load_from_disk(config.dataset_name)
  return generate_dataset(config, pipe, ds)


if __name__ == "__main__":
  run(pyconfig.initialize(sys.argv))
