"""Checkpointers, imported on first use (reference: src/maxdiffusion/checkpointing/).
"""
_EXPORTS = {
    "WanCheckpointer": (".wan_checkpointer", "WanCheckpointer"),
    "WanCheckpointer2_1": (".wan_checkpointer", "WanCheckpointer2_1"),
    "WanCheckpointer2_2": (".wan_checkpointer", "WanCheckpointer2_2"),
    "WanCheckpointerI2V_2_1": (".wan_checkpointer", "WanCheckpointerI2V_2_1"),
    "WanCheckpointerI2V_2_2": (".wan_checkpointer", "WanCheckpointerI2V_2_2"),
    "WanVaceCheckpointer2_1": (".wan_vace_checkpointer", "WanVACECheckpointer2_1"),
    "WanVACECheckpointer2_1": (".wan_vace_checkpointer", "WanVACECheckpointer2_1"),
    "FluxCheckpointer": (".flux_checkpointer", "FluxCheckpointer"),
    "BaseStableDiffusionCheckpointer": (".base_stable_diffusion_checkpointer", "BaseStableDiffusionCheckpointer"),
    "LTX2Checkpointer": (".ltx2_checkpointer", "LTX2Checkpointer"),
    "ZImageCheckpointer": (".z_image_checkpointer", "ZImageCheckpointer"),
    "CheckpointManager": (".checkpointing_utils", "CheckpointManager"),
    "create_checkpoint_manager": (".checkpointing_utils", "create_checkpoint_manager"),
}

def __getattr__(name):
  if name in _EXPORTS:
    import importlib

    mod, attr = _EXPORTS[name]
    value = getattr(importlib.import_module(mod, __name__), attr)
    globals()[name] = value
    return value
  raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
  return sorted(list(globals()) + list(_EXPORTS))


__all__ = list(_EXPORTS)
