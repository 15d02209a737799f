"""Utilities: exporters, loaders, benchmarks, and the diffusers-style plumbing (optional-dependency probing, logger,
outputs, PIL helpers). Imported on first use (reference: src/maxdiffusion/utils/__init__.py)."""
_EXPORTS = {
    "export_to_video": (".export_utils", "export_to_video"), "export_to_video_with_audio": (".export_utils", "export_to_video_with_audio"),
    "export_to_png": (".export_utils", "export_to_png"), "load_image": (".loading_utils", "load_image"), "load_video": (".loading_utils", "load_video"),
    "BaseOutput": (".outputs", "BaseOutput"), "numpy_to_pil": (".pil_utils", "numpy_to_pil"), "pt_to_pil": (".pil_utils", "pt_to_pil"),
    "make_image_grid": (".pil_utils", "make_image_grid"), "deprecate": (".deprecation_utils", "deprecate"),
    "randn_tensor": (".torch_utils", "randn_tensor"), "get_logger": (".logging", "get_logger"),
    "is_available": (".import_utils", "is_available"), "requires_backends": (".import_utils", "requires_backends"),
    "OptionalDependencyNotAvailable": (".import_utils", "OptionalDependencyNotAvailable"), "DummyObject": (".import_utils", "DummyObject"),
    "is_transformers_available": (".import_utils", "is_transformers_available"), "is_torch_available": (".import_utils", "is_torch_available"),
    "convert_state_dict_to_peft": (".state_dict_utils", "convert_state_dict_to_peft"),
    "convert_state_dict_to_diffusers": (".state_dict_utils", "convert_state_dict_to_diffusers"),
    "convert_state_dict_to_kohya": (".state_dict_utils", "convert_state_dict_to_kohya"),
    "resolve_model_path": (".hub_utils", "resolve_model_path"), "grid_search": (".tile_size_grid_search", "grid_search"),
    "CONFIG_NAME": (".constants", "CONFIG_NAME"), "SAFETENSORS_WEIGHTS_NAME": (".constants", "SAFETENSORS_WEIGHTS_NAME"),
}


def __getattr__(name):
  if name in _EXPORTS:
    import importlib

    mod, attr = _EXPORTS[name]
    value = getattr(importlib.import_module(mod, __name__), attr)
    globals()[name] = value
    return value
  raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = list(_EXPORTS)
