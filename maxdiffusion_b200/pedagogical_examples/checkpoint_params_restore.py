"""Saves a model's parameters with the checkpoint manager and restores them into a freshly initialised copy.

  python -m maxdiffusion_b200.pedagogical_examples.checkpoint_params_restore /tmp/ckpt_demo
"""
from __future__ import annotations

import sys

import torch

from ..checkpointing.checkpointing_utils import WAN_CHECKPOINT, create_checkpoint_manager
from ..models.wan.transformer_wan import WAN_PRESETS, WanConfig, WanModel


def run(folder: str) -> bool:
  torch.manual_seed(0)
  model = WanModel(WanConfig(**WAN_PRESETS["tiny"]))
  mgr = create_checkpoint_manager(folder, WAN_CHECKPOINT, enable_async=True)
  mgr.save(1, {"wan_state": {k: v.detach() for k, v in model.state_dict().items()}, "wan_config": model.cfg.to_dict()})
  mgr.wait_until_finished()  # the write happened on a background thread
  torch.manual_seed(1)
  other = WanModel(WanConfig.from_dict(mgr.restore_json(mgr.latest_step(), "wan_config")))
  other.load_state_dict(mgr.restore_state(mgr.latest_step(), "wan_state"))
  same = all(torch.equal(a, b) for a, b in zip(model.state_dict().values(), other.state_dict().values()))
  print(f"restored step {mgr.latest_step()} from {folder}: parameters identical = {same}")
  return same


if __name__ == "__main__":
  run(sys.argv[1] if len(sys.argv) > 1 else "/tmp/ckpt_demo")
