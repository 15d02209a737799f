"""Model classes by the names users import (the reference's `Flax*` names resolve to the same classes), loaded on first
access so that importing the package stays cheap (reference: src/maxdiffusion/models/__init__.py, `_LazyModule`)."""
_EXPORTS = {
    "AutoencoderKL": (".vae", "AutoencoderKL"),
    "FlaxAutoencoderKL": (".vae", "AutoencoderKL"),
    "UNet2DConditionModel": (".unet_2d_condition", "UNet2DConditionModel"),
    "FlaxUNet2DConditionModel": (".unet_2d_condition", "UNet2DConditionModel"),
    "ControlNetModel": (".controlnet", "ControlNetModel"),
    "FlaxControlNetModel": (".controlnet", "ControlNetModel"),
    "ModelMixin": (".modeling_utils", "ModelMixin"),
    "WanModel": (".wan.transformer_wan", "WanModel"),
    "WanVACEModel": (".wan.transformer_wan_vace", "WanVACEModel"),
    "WanAnimateModel": (".wan.transformer_wan_animate", "WanAnimateModel"),
    "AutoencoderKLWan": (".wan.autoencoder_kl_wan", "AutoencoderKLWan"),
    "FluxTransformer2DModel": (".flux.transformer_flux", "FluxTransformer2DModel"),
    "Flux2KleinTransformer2DModel": (".flux.transformer_flux2_klein", "Flux2KleinTransformer2DModel"),
    "LTX2VideoTransformer3DModel": (".ltx2.transformer_ltx2", "LTX2VideoTransformer3DModel"),
    "Transformer3DModel": (".ltx_video.transformer3d", "Transformer3DModel"),
    "ZImageTransformer2DModel": (".z_image.transformer_z_image", "ZImageTransformer2DModel"),
    "Qwen3Model": (".qwen3", "Qwen3Model"),
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
