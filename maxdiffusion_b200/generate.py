"""python -m maxdiffusion_b200.generate <config.yml> key=value ...   (reference: src/maxdiffusion/generate.py)"""
import sys

import torch

from . import pyconfig
from ._generate_common import run_image_pipeline
from .parallel.mesh import init_distributed
from .pipelines.stable_diffusion.pipeline_stable_diffusion import StableDiffusionPipeline


def run(config):
  if config.get("random_init", False):
    pipe = StableDiffusionPipeline.from_config(config)
  else:
    from .loaders.sd_loader import load_sd_pipeline

    pipe = load_sd_pipeline(config, StableDiffusionPipeline)
  if config.get("enable_lora", False):
    from .loaders.lora_loader import apply_unet_loras

    apply_unet_loras(pipe, config)  # reference: `maybe_load_lora` in generate_sdxl.py:60-110
  kw = {}
  if not pipe.text_encoders:
    g = torch.Generator().manual_seed(int(config.seed))
    c = pipe.unet.cfg
    kw = {"prompt_embeds": torch.randn((1, 77, c.cross_attention_dim), generator=g),
          "negative_prompt_embeds": torch.randn((1, 77, c.cross_attention_dim), generator=g)}
    if pipe.is_xl:
      pd = c.projection_class_embeddings_input_dim - 6 * c.addition_time_embed_dim
      kw.update(pooled_prompt_embeds=torch.randn((1, pd), generator=g), negative_pooled_prompt_embeds=torch.randn((1, pd), generator=g))
  return run_image_pipeline(config, pipe, kw, "generate")


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
