"""python -m maxdiffusion_b200.generate_wan <config.yml> key=value ...

Flow of the reference entry point (src/maxdiffusion/generate_wan.py:146-438): optional tile search -> load the
pipeline (checkpoint step, else the pretrained-weights cache / diffusers directory, else random init when
`random_init=true`) -> optional LoRA merge -> warm-up call -> timed call -> TIMING SUMMARY -> write the videos.
"""
import os
import sys
import time

import torch

from . import max_logging, pyconfig
from .parallel.mesh import create_device_mesh, init_distributed
from .pipelines.wan.wan_pipeline import (WanPipeline2_1, WanPipeline2_2, WanPipelineI2V_2_1, WanPipelineI2V_2_2)
from .utils.export_utils import export_to_video


def pipeline_class(config):
  name, kind = str(config.model_name), str(config.get("model_type", "T2V")).upper()
  table = {("wan2.1", "T2V"): WanPipeline2_1, ("wan2.2", "T2V"): WanPipeline2_2, ("wan2.1", "I2V"): WanPipelineI2V_2_1,
           ("wan2.2", "I2V"): WanPipelineI2V_2_2}
  if (name, kind) not in table:
    raise ValueError(f"no Wan pipeline for model_name={name} model_type={kind}")
  return table[(name, kind)]


def maybe_tune_block_sizes(config):
  if not config.get("enable_tile_search", False):
    return None
  from .utils.wan_block_benchmark import tune_wan_block_sizes

  return tune_wan_block_sizes(config)


def load_pipeline(config):
  from .checkpointing.wan_checkpointer import WanCheckpointer

  cls = pipeline_class(config)
  if config.get("random_init", False):
    return cls.from_config(config)
  ck = WanCheckpointer(config)
  if config.get("checkpoint_dir", "") and ck.manager.latest_step() is not None:
    return cls.from_checkpoint(config)
  return ck.load_pretrained_pipeline_or_diffusers(cls)


def run(config):
  t_load = time.perf_counter()
  maybe_tune_block_sizes(config)
  pipe = load_pipeline(config)
  if config.get("enable_lora", False):
    from .loaders.lora_loader import merge_wan_loras

    merge_wan_loras(pipe, config)
  load_s = time.perf_counter() - t_load
  embeds = {}
  if pipe.text_encoder is None:  # no encoder weights: synthetic conditioning of the right shape
    g = torch.Generator().manual_seed(int(config.seed))
    text_dim = pipe.transformer.cfg.text_dim
    embeds = {"prompt_embeds": torch.randn((1, int(config.max_sequence_length), text_dim), generator=g),
              "negative_prompt_embeds": torch.randn((1, int(config.max_sequence_length), text_dim), generator=g)}
  t0 = time.perf_counter()
  pipe(num_inference_steps=2, output_type="latent", **embeds)  # warm-up: kernels, allocator, autotune caches
  warm_s = time.perf_counter() - t0
  t0 = time.perf_counter()
  videos, trace = pipe(return_trace=True, **embeds)
  gen_s = time.perf_counter() - t0
  max_logging.log("=" * 30 + " TIMING SUMMARY " + "=" * 30)
  max_logging.log(f"load: {load_s:.1f}s  warm-up: {warm_s:.1f}s  generation: {gen_s:.1f}s "
                  f"({gen_s / max(1, videos.shape[0]):.1f}s per video)")
  for k, v in trace.items():
    max_logging.log(f"  {k}: {v:.3f}s")
  if int(os.environ.get("RANK", "0")) == 0:
    out_dir = config.get("output_dir", ".") or "."
    os.makedirs(out_dir, exist_ok=True)
    for i in range(videos.shape[0]):
      path = os.path.join(out_dir, f"wan_output_{config.seed}_{i}.mp4")
      max_logging.log(f"wrote {export_to_video(videos[i].cpu().numpy(), path, fps=int(config.fps))}")
  return videos


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  init_distributed()
  run(pyconfig.initialize(argv))


if __name__ == "__main__":
  main()
