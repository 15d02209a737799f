"""Rematerialisation policies by the reference's names, mapped onto `ops.functional.checkpoint_block`.

reference: `GradientCheckpointType` (src/maxdiffusion/models/gradient_checkpoint.py:30-126). The reference selects
what XLA may keep by `checkpoint_name` tags; here a transformer block is the unit: its inputs are always kept, its
internals are recomputed, and the policy decides (a) whether the flash-attention outputs (O, LSE) of the first
pass are kept — they are the expensive part of the recomputation — and (b) whether the block input waits in pinned
host memory.

  NONE                          keep everything (no recomputation)
  FULL                          keep block inputs only
  MATMUL_WITHOUT_BATCH          keep block inputs + attention outputs            (alias SAVE_ATTENTION)
  OFFLOAD_MATMUL_WITHOUT_BATCH  as above, block inputs offloaded to the host
  HIDDEN_STATE_WITH_OFFLOAD     keep nothing on the device but attention outputs; inputs offloaded
  FLUX_OPTIMIZED                as MATMUL_WITHOUT_BATCH
  CUSTOM                        from `names_which_can_be_saved` / `names_which_can_be_offloaded`: "self_attn" /
                                "attn_output" in the saved names keeps attention outputs; "hidden_states" in the
                                offloaded names offloads the block input
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Sequence


@dataclass(frozen=True)
class RematPlan:
  checkpoint: bool
  save_attention: bool
  offload_input: bool

  @property
  def policy_name(self) -> str:
    """The name understood by the models' `remat_policy` attribute."""
    if not self.checkpoint:
      return "NONE"
    base = "SAVE_ATTENTION" if self.save_attention else "FULL"
    return base + ("_OFFLOAD" if self.offload_input else "")


class GradientCheckpointType(enum.Enum):
  NONE = "NONE"
  FULL = "FULL"
  MATMUL_WITHOUT_BATCH = "MATMUL_WITHOUT_BATCH"
  OFFLOAD_MATMUL_WITHOUT_BATCH = "OFFLOAD_MATMUL_WITHOUT_BATCH"
  CUSTOM = "CUSTOM"
  HIDDEN_STATE_WITH_OFFLOAD = "HIDDEN_STATE_WITH_OFFLOAD"
  FLUX_OPTIMIZED = "FLUX_OPTIMIZED"
  SAVE_ATTENTION = "SAVE_ATTENTION"

  @classmethod
  def from_str(cls, s: str = "NONE") -> "GradientCheckpointType":
    if s is None:
      s = "NONE"
    key = str(s).upper()
    if key not in cls.__members__:
      raise ValueError(f"unknown remat policy '{s}'; known: {sorted(cls.__members__)}")
    return cls[key]

  def plan(self, names_which_can_be_saved: Sequence[str] = (), names_which_can_be_offloaded: Sequence[str] = ()) -> RematPlan:
    T = GradientCheckpointType
    if self is T.NONE:
      return RematPlan(False, False, False)
    if self is T.FULL:
      return RematPlan(True, False, False)
    if self in (T.MATMUL_WITHOUT_BATCH, T.FLUX_OPTIMIZED, T.SAVE_ATTENTION):
      return RematPlan(True, True, False)
    if self in (T.OFFLOAD_MATMUL_WITHOUT_BATCH, T.HIDDEN_STATE_WITH_OFFLOAD):
      return RematPlan(True, True, True)
    saved, off = set(names_which_can_be_saved), set(names_which_can_be_offloaded)
    return RematPlan(True, bool(saved & {"self_attn", "attn_output", "cross_attn"}), "hidden_states" in off)


def resolve_remat(policy: str, names_which_can_be_saved: Sequence[str] = (), names_which_can_be_offloaded: Sequence[str] = ()) -> str:
  """Config value -> the `remat_policy` string of the models (NONE / FULL / SAVE_ATTENTION [+ _OFFLOAD])."""
  p = str(policy).upper()
  if p.endswith("_OFFLOAD") and p[:-8] in ("FULL", "SAVE_ATTENTION"):
    return p
  return GradientCheckpointType.from_str(policy).plan(names_which_can_be_saved, names_which_can_be_offloaded).policy_name
