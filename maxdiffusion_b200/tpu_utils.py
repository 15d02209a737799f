"""The reference's module name for accelerator queries (`src/maxdiffusion/tpu_utils.py`); here they are answered for
the GPU by `gpu_utils`, and this module re-exports it so that `from maxdiffusion import tpu_utils` style imports keep
working after the package name is changed."""
from .gpu_utils import *  # noqa: F401,F403
from . import gpu_utils as _gpu_utils

__all__ = [n for n, v in vars(_gpu_utils).items()
           if not n.startswith("_") and getattr(v, "__module__", None) == _gpu_utils.__name__]
