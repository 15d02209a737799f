"""Checkpointing of the Wan 2.1 VACE transformer (reference: src/maxdiffusion/checkpointing/wan_vace_checkpointer_2_1.py).

Same items and layout as `WanCheckpointer` (`wan_config`, `wan_state`, optional optimizer shards); the config item
additionally carries `vace_layers` / `vace_in_channels`, and the state holds the `vace_blocks/N/...` and
`vace_patch_embedding` entries (per layer, not stacked: the reference does not scan the control blocks).
"""
from __future__ import annotations

from .wan_checkpointer import WanCheckpointer


class WanVACECheckpointer2_1(WanCheckpointer):

  def load_pipeline(self, device=None):
    from ..pipelines.wan.wan_vace_pipeline import WanVACEPipeline2_1

    return self.load_pretrained_pipeline_or_diffusers(WanVACEPipeline2_1, device=device)
