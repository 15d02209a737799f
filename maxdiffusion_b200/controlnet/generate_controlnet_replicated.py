"""python -m maxdiffusion_b200.controlnet.generate_controlnet_replicated <config.yml> key=value ...

SD 1.x ControlNet inference, one replica per rank (reference:
src/maxdiffusion/controlnet/generate_controlnet_replicated.py). `controlnet_image` is a local image (an edge map for
the canny ControlNet); without it a synthetic conditioning image is used (benchmarks with `random_init`)."""
import os
import sys

import torch

from .. import pyconfig
from .._generate_common import run_image_pipeline
from ..parallel.mesh import init_distributed
from ..pipelines.stable_diffusion.pipeline_stable_diffusion import (StableDiffusionControlNetPipeline,
                                                                    StableDiffusionXLControlNetPipeline)


def conditioning_image(config, size: int) -> torch.Tensor:
  path = str(config.get("controlnet_image", "") or "")
  if path and os.path.exists(path):
    from ..image_processor import VaeImageProcessor
    from ..utils.loading_utils import load_image

    return (VaeImageProcessor().preprocess(load_image(path), size, size) + 1) / 2  # ControlNet conditioning is in [0, 1]
  g = torch.Generator().manual_seed(int(config.seed))
  return (torch.rand((1, 3, size, size), generator=g) > 0.9).float()


def run(config, xl: bool = False):
  cls = StableDiffusionXLControlNetPipeline if xl else StableDiffusionControlNetPipeline
  if config.get("random_init", False):
    pipe = cls.from_config(config, with_controlnet=True)
  else:
    from ..loaders.sd_loader import load_sd_pipeline

    pipe = load_sd_pipeline(config, cls)
  rank = int(os.environ.get("RANK", "0"))
  config = config.replace(seed=int(config.seed) + rank)
  kw = {"controlnet_image": conditioning_image(config, int(config.resolution))}
  if not pipe.text_encoders:
    g = torch.Generator().manual_seed(int(config.seed))
    c = pipe.unet.cfg
    kw.update(prompt_embeds=torch.randn((1, 77, c.cross_attention_dim), generator=g),
              negative_prompt_embeds=torch.randn((1, 77, c.cross_attention_dim), generator=g))
    if pipe.is_xl:
      pd = c.projection_class_embeddings_input_dim - 6 * c.addition_time_embed_dim
      kw.update(pooled_prompt_embeds=torch.randn((1, pd), generator=g), negative_pooled_prompt_embeds=torch.randn((1, pd), generator=g))
  return run_image_pipeline(config, pipe, kw, "controlnet_sdxl" if xl else "controlnet")


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
