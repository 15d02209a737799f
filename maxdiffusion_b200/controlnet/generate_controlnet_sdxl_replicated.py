"""python -m maxdiffusion_b200.controlnet.generate_controlnet_sdxl_replicated <config.yml> key=value ...

SDXL ControlNet inference (reference: src/maxdiffusion/controlnet/generate_controlnet_sdxl_replicated.py)."""
import sys

from .. import pyconfig
from ..parallel.mesh import init_distributed
from .generate_controlnet_replicated import run as _run


def run(config):
  return _run(config, xl=True)


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
