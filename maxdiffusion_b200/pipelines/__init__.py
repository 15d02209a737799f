"""Pipelines of every model family, imported on first use. The reference's `Flax*` names are kept as aliases
(src/maxdiffusion/pipelines/__init__.py).
"""
_EXPORTS = {
    "WanPipeline": (".wan.wan_pipeline", "WanPipeline"),
    "WanPipeline2_1": (".wan.wan_pipeline", "WanPipeline2_1"),
    "WanPipeline2_2": (".wan.wan_pipeline", "WanPipeline2_2"),
    "WanPipelineI2V_2_1": (".wan.wan_pipeline", "WanPipelineI2V_2_1"),
    "WanPipelineI2V_2_2": (".wan.wan_pipeline", "WanPipelineI2V_2_2"),
    "VaceWanPipeline2_1": (".wan.wan_vace_pipeline", "WanVACEPipeline2_1"),
    "WanVACEPipeline2_1": (".wan.wan_vace_pipeline", "WanVACEPipeline2_1"),
    "WanAnimatePipeline": (".wan.wan_pipeline_animate", "WanAnimatePipeline"),
    "FluxPipeline": (".flux.flux_pipeline", "FluxPipeline"),
    "Flux2KleinPipeline": (".flux.flux2klein_pipeline", "Flux2KleinPipeline"),
    "FlaxFlux2KleinPipeline": (".flux.flux2klein_pipeline", "Flux2KleinPipeline"),
    "LTX2Pipeline": (".ltx2.ltx2_pipeline", "LTX2Pipeline"),
    "LTX2LatentUpsamplePipeline": (".ltx2.pipeline_ltx2_latent_upsample", "LTX2LatentUpsamplePipeline"),
    "LTXVideoPipeline": (".ltx_video.ltx_video_pipeline", "LTXVideoPipeline"),
    "LTXMultiScalePipeline": (".ltx_video.ltx_video_pipeline", "LTXMultiScalePipeline"),
    "ZImagePipeline": (".z_image.z_image_pipeline", "ZImagePipeline"),
    "StableDiffusionPipeline": (".stable_diffusion.pipeline_stable_diffusion", "StableDiffusionPipeline"),
    "StableDiffusionXLPipeline": (".stable_diffusion.pipeline_stable_diffusion", "StableDiffusionXLPipeline"),
    "StableDiffusionControlNetPipeline": (".stable_diffusion.pipeline_stable_diffusion", "StableDiffusionControlNetPipeline"),
    "StableDiffusionXLControlNetPipeline": (".stable_diffusion.pipeline_stable_diffusion", "StableDiffusionXLControlNetPipeline"),
    "FlaxStableDiffusionPipeline": (".stable_diffusion.pipeline_stable_diffusion", "StableDiffusionPipeline"),
    "FlaxStableDiffusionXLPipeline": (".stable_diffusion.pipeline_stable_diffusion", "StableDiffusionXLPipeline"),
    "FlaxStableDiffusionControlNetPipeline": (".stable_diffusion.pipeline_stable_diffusion", "StableDiffusionControlNetPipeline"),
    "FlaxStableDiffusionXLControlNetPipeline": (".stable_diffusion.pipeline_stable_diffusion", "StableDiffusionXLControlNetPipeline"),
    "StableDiffusionSafetyChecker": (".stable_diffusion.safety_checker", "StableDiffusionSafetyChecker"),
    "FlaxStableDiffusionSafetyChecker": (".stable_diffusion.safety_checker", "StableDiffusionSafetyChecker"),
    "save_pipeline": (".pipeline_utils", "save_pipeline"),
    "load_components": (".pipeline_utils", "load_components"),
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
