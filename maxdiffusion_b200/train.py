"""python -m maxdiffusion_b200.train <config.yml> key=value ...   (reference: src/maxdiffusion/train.py)"""
import sys

from . import pyconfig
from .parallel.mesh import create_device_mesh, init_distributed
from .train_utils import validate_train_config
from .trainers.stable_diffusion_trainer import StableDiffusionTrainer


def train(config):
  return StableDiffusionTrainer(config, mesh=create_device_mesh(config)).start_training()


def main(argv=None):
  init_distributed()
  config = pyconfig.initialize(list(sys.argv if argv is None else argv), validate_training=True)
  validate_train_config(config)
  train(config)


if __name__ == "__main__":
  main()
