"""SDXL variant of `save_sd_checkpoint` (two text encoders, `text_time` conditioning in the UNet config)."""
from __future__ import annotations

import sys

from .. import pyconfig
from .save_sd_checkpoint import run as _run


def run(config) -> str:
  return _run(config, xl=True)


if __name__ == "__main__":
  run(pyconfig.initialize(sys.argv))
