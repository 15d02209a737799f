"""Raw (video, caption) pairs -> Wan VAE latents + umT5 embeddings -> TFRecord shards.

`python -m maxdiffusion_b200.data_preprocessing.wan_txt2vid_data_preprocessing configs/base_wan_14b.yml
dataset_name=<HF dataset saved on disk> tfrecords_dir=… no_records_per_shard=…`. The pipeline is loaded without its
transformer; videos are resized to `height` x `width`, encoded in batches, normalised with the VAE's latent statistics,
and written next to the caption's text-encoder states (reference: wan_txt2vid_data_preprocessing.py:92-144).
"""
from __future__ import annotations

import sys
from typing import Iterable, Tuple

import torch

from .. import max_logging, pyconfig
from ..video_processor import VideoProcessor
from .tfrecord_shards import ShardedWriter, create_example


def vae_encode(video: torch.Tensor, vae, generator=None) -> torch.Tensor:
  """[B,3,F,H,W] in [-1,1] -> normalised latents [B,z,F',H/8,W/8] sampled from the posterior."""
  p = next(vae.parameters())
  # on a GPU bf16 frames select the encoder on this repository's convolution kernels
  dtype = torch.bfloat16 if p.is_cuda and hasattr(vae, "channels_last_decoder") else p.dtype
  with torch.no_grad():
    moments = vae.encode(video.to(p.device, dtype))
    moments.mean, moments.logvar = moments.mean.float(), moments.logvar.float()
    return vae.normalize_latents(moments.sample(generator))


def _batches(ds, caption_column: str, video_column: str, batch_size: int) -> Iterable[Tuple[list, list]]:
  n = len(ds)
  for i in range(0, n, batch_size):
    chunk = ds[i:i + batch_size]
    yield chunk[caption_column], chunk[video_column]


def generate_dataset(config, pipeline, dataset=None, batch_size: int = 10) -> list:
  if dataset is None:
    import datasets

    dataset = datasets.load_from_disk(config.dataset_name) if config.get("dataset_name", "") else datasets.load_dataset(
        "videofolder", data_dir=config.train_data_dir, split="train")
    dataset = dataset.shuffle(seed=int(config.get("seed", 0))).select_columns([config.caption_column, config.image_column])
  writer = ShardedWriter(config.tfrecords_dir, int(config.no_records_per_shard))
  proc = VideoProcessor(vae_scale_factor=8)
  gen = torch.Generator(device=pipeline.device).manual_seed(int(config.get("seed", 0)))
  for text, videos in _batches(dataset, config.caption_column, config.image_column, batch_size):
    video = torch.cat([proc.preprocess_video(v, height=int(config.height), width=int(config.width)) for v in videos])
    latents = vae_encode(video, pipeline.vae, gen).float().cpu().numpy()
    with torch.no_grad():
      states = pipeline.encode_prompt(list(text), int(config.get("max_sequence_length", 512))).float().cpu().numpy()
    for lat, emb in zip(latents, states):
      writer.write(create_example(lat, emb))
  files = writer.close()
  max_logging.log(f"wrote {writer.total} examples to {len(files)} shards under {config.tfrecords_dir}")
  return files


def run(config, dataset=None):
  from ..pipelines.wan.wan_pipeline import WanPipeline

  pipeline = WanPipeline.from_pretrained(config, load_transformer=False)
  return generate_dataset(config, pipeline, dataset)


def main(argv=None):
  return run(pyconfig.initialize(list(argv if argv is not None else sys.argv)))


if __name__ == "__main__":
  main()
