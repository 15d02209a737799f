"""FLOPs of one training step, counted two ways: tracing a forward pass with PyTorch's FLOP counter, and the analytic
formula the trainers report as TFLOP/s/device.

  python -m maxdiffusion_b200.pedagogical_examples.model_flop_calculation configs/base_wan_14b.yml wan_preset=tiny height=64 width=64 num_frames=9
"""
from __future__ import annotations

import sys

import torch

from .. import pyconfig
from ..max_utils import calculate_model_tflops
from ..maxdiffusion_utils import calculate_wan_tflops, get_dummy_wan_inputs


def run(config) -> dict:
  from ..models.wan.transformer_wan import WanModel
  from ..trainers.wan_trainer import resolve_wan_config

  model = WanModel(resolve_wan_config(config))
  traced = calculate_model_tflops(model, *get_dummy_wan_inputs(config, model), train=True)
  analytic = calculate_wan_tflops(config, model, train=True)
  print(f"traced   : {traced:.6f} TFLOP per step (forward x3)")
  print(f"analytic : {analytic:.6f} TFLOP per step")
  return {"traced": traced, "analytic": analytic}


if __name__ == "__main__":
  run(pyconfig.initialize(sys.argv))
