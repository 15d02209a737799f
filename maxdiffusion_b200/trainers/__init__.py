"""Trainers, imported on first use (reference: src/maxdiffusion/trainers/).
"""
_EXPORTS = {
    "WanTrainer": (".wan_trainer", "WanTrainer"),
    "WanVaceTrainer": (".wan_vace_trainer", "WanVACETrainer"),
    "WanVACETrainer": (".wan_vace_trainer", "WanVACETrainer"),
    "FluxTrainer": (".flux_trainer", "FluxTrainer"),
    "StableDiffusionTrainer": (".stable_diffusion_trainer", "StableDiffusionTrainer"),
    "StableDiffusionXLTrainer": (".stable_diffusion_trainer", "StableDiffusionXLTrainer"),
    "DreamboothTrainer": (".stable_diffusion_trainer", "DreamboothTrainer"),
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
