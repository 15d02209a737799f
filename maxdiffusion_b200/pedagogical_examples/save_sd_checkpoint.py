"""Writes a Stable Diffusion (or, with an SDXL config, SDXL) pipeline in the diffusers folder layout, after training or
after merging LoRA weights, so that any diffusers-compatible tool can read it.

  python -m maxdiffusion_b200.pedagogical_examples.save_sd_checkpoint configs/base15.yml output_dir=/tmp/sd15_export
  python -m maxdiffusion_b200.pedagogical_examples.save_sdxl_checkpoint configs/base_xl.yml output_dir=/tmp/sdxl_export
"""
from __future__ import annotations

import os
import sys

from .. import max_logging, pyconfig
from ..checkpointing.base_stable_diffusion_checkpointer import BaseStableDiffusionCheckpointer
from ..pipelines.pipeline_utils import save_pipeline
from ..pipelines.stable_diffusion.pipeline_stable_diffusion import StableDiffusionPipeline, StableDiffusionXLPipeline


def run(config, xl: bool = False) -> str:
  pipe = BaseStableDiffusionCheckpointer(config).load_pipeline(StableDiffusionXLPipeline if xl else StableDiffusionPipeline, device="cpu")
  out = os.path.join(config.output_dir, "checkpoint_final")
  save_pipeline(pipe, out, components=("unet", "vae", "scheduler", "text_encoder", "text_encoder_2", "tokenizer", "tokenizer_2"))
  max_logging.log(f"pipeline written to {out}")
  return out


if __name__ == "__main__":
  run(pyconfig.initialize(sys.argv))
