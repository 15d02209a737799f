"""python -m maxdiffusion_b200.generate_flux <config.yml> key=value ...   (reference: src/maxdiffusion/generate_flux.py)"""
import sys

from . import pyconfig
from ._generate_common import run_image_pipeline, synthetic_text_conditioning
from .parallel.mesh import init_distributed
from .pipelines.flux.flux_pipeline import FluxPipeline


def run(config):
  if config.get("random_init", False):
    pipe = FluxPipeline.from_config(config)
  else:
    from .loaders.flux_loader import load_flux_pipeline

    pipe = load_flux_pipeline(config)
  if config.get("enable_lora", False):
    from .loaders.lora_loader import apply_flux_loras

    apply_flux_loras(pipe, config)
  kw = {}
  if pipe.t5 is None:
    cfg = pipe.transformer.cfg
    e, p = synthetic_text_conditioning(int(config.get("batch_size", 1)), int(config.max_sequence_length),
                                       cfg.joint_attention_dim, cfg.pooled_projection_dim, int(config.seed))
    kw = {"prompt_embeds": e, "pooled_prompt_embeds": p}
  return run_image_pipeline(config, pipe, kw, str(config.get("output_name", "flux")))


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
