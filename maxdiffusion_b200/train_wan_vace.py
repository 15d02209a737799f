"""python -m maxdiffusion_b200.train_wan_vace <config.yml> key=value ...   (reference: src/maxdiffusion/train_wan_vace.py)"""
import sys

from . import max_logging, pyconfig
from .parallel.mesh import create_device_mesh, init_distributed
from .train_utils import validate_train_config
from .trainers.wan_vace_trainer import WanVACETrainer


def train(config):
  trainer = WanVACETrainer(config, mesh=create_device_mesh(config))
  trainer.start_training()
  return trainer


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  init_distributed()
  config = pyconfig.initialize(argv, validate_training=True)
  validate_train_config(config)
  max_logging.log(f"Found {config.total_train_batch_size} samples per step over {pyconfig.world_size()} devices")
  train(config)


if __name__ == "__main__":
  main()
