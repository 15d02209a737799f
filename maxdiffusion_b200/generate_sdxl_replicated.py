"""python -m maxdiffusion_b200.generate_sdxl_replicated <config.yml> key=value ...

Data-parallel SDXL inference: every rank holds a full replica and renders `per_device_batch_size` images with its own
seed (the reference replicates with `jax.pmap`, src/maxdiffusion/generate_sdxl_replicated.py). Launch with torchrun;
rank r writes `generate_sdxl_replicated_<seed + r>_*.png`."""
import os
import sys

from . import pyconfig
from .generate_sdxl import run as run_single
from .parallel.mesh import init_distributed


def run(config):
  rank = int(os.environ.get("RANK", "0"))
  return run_single(config.replace(seed=int(config.seed) + rank, write_all_ranks=True))


def main(argv=None):
  init_distributed()
  run(pyconfig.initialize(list(sys.argv if argv is None else argv)))


if __name__ == "__main__":
  main()
