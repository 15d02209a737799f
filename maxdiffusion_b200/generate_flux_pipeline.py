"""python -m maxdiffusion_b200.generate_flux_pipeline <config.yml> key=value ...

Pipeline-class flavoured Flux inference (reference: src/maxdiffusion/generate_flux_pipeline.py): builds `FluxPipeline`
through the Flux checkpointer (Orbax-layout step if present, else the pretrained folder) and calls it."""
import sys

from . import pyconfig
from ._generate_common import run_image_pipeline, synthetic_text_conditioning
from .checkpointing.flux_checkpointer import FluxCheckpointer
from .parallel.mesh import init_distributed


def run(config):
  pipe = FluxCheckpointer(config).load_pipeline()
  kw = {}
  if pipe.t5 is None:
    cfg = pipe.transformer.cfg
    e, p = synthetic_text_conditioning(int(config.get("batch_size", 1)), int(config.max_sequence_length),
                                       cfg.joint_attention_dim, cfg.pooled_projection_dim, int(config.seed))
    kw = {"prompt_embeds": e, "pooled_prompt_embeds": p}
  return run_image_pipeline(config, pipe, kw, str(config.get("output_name", "flux_pipeline")))


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
