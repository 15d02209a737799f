"""maxdiffusion_b200: diffusion-model training and inference on NVIDIA B200 (sm_100a).

Public names are imported on first use, so `import maxdiffusion_b200` stays cheap and optional dependencies of one
model family do not block another (reference: the `_LazyModule` structure of src/maxdiffusion/__init__.py).
"""
_EXPORTS = {
    "WanPipeline": (".pipelines.wan.wan_pipeline", "WanPipeline"),
    "WanPipeline2_1": (".pipelines.wan.wan_pipeline", "WanPipeline2_1"),
    "WanPipeline2_2": (".pipelines.wan.wan_pipeline", "WanPipeline2_2"),
    "WanPipelineI2V_2_1": (".pipelines.wan.wan_pipeline", "WanPipelineI2V_2_1"),
    "WanPipelineI2V_2_2": (".pipelines.wan.wan_pipeline", "WanPipelineI2V_2_2"),
    "VaceWanPipeline2_1": (".pipelines.wan.wan_vace_pipeline", "WanVACEPipeline2_1"),
    "WanVACEPipeline2_1": (".pipelines.wan.wan_vace_pipeline", "WanVACEPipeline2_1"),
    "WanAnimatePipeline": (".pipelines.wan.wan_pipeline_animate", "WanAnimatePipeline"),
    "FluxPipeline": (".pipelines.flux.flux_pipeline", "FluxPipeline"),
    "Flux2KleinPipeline": (".pipelines.flux.flux2klein_pipeline", "Flux2KleinPipeline"),
    "FlaxFlux2KleinPipeline": (".pipelines.flux.flux2klein_pipeline", "Flux2KleinPipeline"),
    "LTX2Pipeline": (".pipelines.ltx2.ltx2_pipeline", "LTX2Pipeline"),
    "LTX2LatentUpsamplePipeline": (".pipelines.ltx2.pipeline_ltx2_latent_upsample", "LTX2LatentUpsamplePipeline"),
    "LTXVideoPipeline": (".pipelines.ltx_video.ltx_video_pipeline", "LTXVideoPipeline"),
    "LTXMultiScalePipeline": (".pipelines.ltx_video.ltx_video_pipeline", "LTXMultiScalePipeline"),
    "ZImagePipeline": (".pipelines.z_image.z_image_pipeline", "ZImagePipeline"),
    "StableDiffusionPipeline": (".pipelines.stable_diffusion.pipeline_stable_diffusion", "StableDiffusionPipeline"),
    "StableDiffusionXLPipeline": (".pipelines.stable_diffusion.pipeline_stable_diffusion", "StableDiffusionXLPipeline"),
    "StableDiffusionControlNetPipeline": (".pipelines.stable_diffusion.pipeline_stable_diffusion", "StableDiffusionControlNetPipeline"),
    "StableDiffusionXLControlNetPipeline": (".pipelines.stable_diffusion.pipeline_stable_diffusion", "StableDiffusionXLControlNetPipeline"),
    "FlaxStableDiffusionPipeline": (".pipelines.stable_diffusion.pipeline_stable_diffusion", "StableDiffusionPipeline"),
    "FlaxStableDiffusionXLPipeline": (".pipelines.stable_diffusion.pipeline_stable_diffusion", "StableDiffusionXLPipeline"),
    "FlaxStableDiffusionControlNetPipeline": (".pipelines.stable_diffusion.pipeline_stable_diffusion", "StableDiffusionControlNetPipeline"),
    "FlaxStableDiffusionXLControlNetPipeline": (".pipelines.stable_diffusion.pipeline_stable_diffusion", "StableDiffusionXLControlNetPipeline"),
    "StableDiffusionSafetyChecker": (".pipelines.stable_diffusion.safety_checker", "StableDiffusionSafetyChecker"),
    "FlaxStableDiffusionSafetyChecker": (".pipelines.stable_diffusion.safety_checker", "StableDiffusionSafetyChecker"),
    "save_pipeline": (".pipelines.pipeline_utils", "save_pipeline"),
    "load_components": (".pipelines.pipeline_utils", "load_components"),
    "WanTrainer": (".trainers.wan_trainer", "WanTrainer"),
    "WanVaceTrainer": (".trainers.wan_vace_trainer", "WanVACETrainer"),
    "WanVACETrainer": (".trainers.wan_vace_trainer", "WanVACETrainer"),
    "FluxTrainer": (".trainers.flux_trainer", "FluxTrainer"),
    "StableDiffusionTrainer": (".trainers.stable_diffusion_trainer", "StableDiffusionTrainer"),
    "StableDiffusionXLTrainer": (".trainers.stable_diffusion_trainer", "StableDiffusionXLTrainer"),
    "DreamboothTrainer": (".trainers.stable_diffusion_trainer", "DreamboothTrainer"),
    "WanCheckpointer": (".checkpointing.wan_checkpointer", "WanCheckpointer"),
    "WanCheckpointer2_1": (".checkpointing.wan_checkpointer", "WanCheckpointer2_1"),
    "WanCheckpointer2_2": (".checkpointing.wan_checkpointer", "WanCheckpointer2_2"),
    "WanCheckpointerI2V_2_1": (".checkpointing.wan_checkpointer", "WanCheckpointerI2V_2_1"),
    "WanCheckpointerI2V_2_2": (".checkpointing.wan_checkpointer", "WanCheckpointerI2V_2_2"),
    "WanVaceCheckpointer2_1": (".checkpointing.wan_vace_checkpointer", "WanVACECheckpointer2_1"),
    "WanVACECheckpointer2_1": (".checkpointing.wan_vace_checkpointer", "WanVACECheckpointer2_1"),
    "FluxCheckpointer": (".checkpointing.flux_checkpointer", "FluxCheckpointer"),
    "BaseStableDiffusionCheckpointer": (".checkpointing.base_stable_diffusion_checkpointer", "BaseStableDiffusionCheckpointer"),
    "LTX2Checkpointer": (".checkpointing.ltx2_checkpointer", "LTX2Checkpointer"),
    "ZImageCheckpointer": (".checkpointing.z_image_checkpointer", "ZImageCheckpointer"),
    "CheckpointManager": (".checkpointing.checkpointing_utils", "CheckpointManager"),
    "create_checkpoint_manager": (".checkpointing.checkpointing_utils", "create_checkpoint_manager"),
    "DDIMScheduler": (".schedulers", "DDIMScheduler"),
    "FlaxDDIMScheduler": (".schedulers", "FlaxDDIMScheduler"),
    "DDPMScheduler": (".schedulers", "DDPMScheduler"),
    "FlaxDDPMScheduler": (".schedulers", "FlaxDDPMScheduler"),
    "DPMSolverMultistepScheduler": (".schedulers", "DPMSolverMultistepScheduler"),
    "FlaxDPMSolverMultistepScheduler": (".schedulers", "FlaxDPMSolverMultistepScheduler"),
    "EulerDiscreteScheduler": (".schedulers", "EulerDiscreteScheduler"),
    "FlaxEulerDiscreteScheduler": (".schedulers", "FlaxEulerDiscreteScheduler"),
    "LMSDiscreteScheduler": (".schedulers", "LMSDiscreteScheduler"),
    "FlaxLMSDiscreteScheduler": (".schedulers", "FlaxLMSDiscreteScheduler"),
    "PNDMScheduler": (".schedulers", "PNDMScheduler"),
    "FlaxPNDMScheduler": (".schedulers", "FlaxPNDMScheduler"),
    "UniPCMultistepScheduler": (".schedulers", "UniPCMultistepScheduler"),
    "FlaxUniPCMultistepScheduler": (".schedulers", "FlaxUniPCMultistepScheduler"),
    "FlowMatchScheduler": (".schedulers", "FlowMatchScheduler"),
    "FlaxFlowMatchScheduler": (".schedulers", "FlaxFlowMatchScheduler"),
    "RectifiedFlowMultistepScheduler": (".schedulers", "RectifiedFlowMultistepScheduler"),
    "FlaxRectifiedFlowMultistepScheduler": (".schedulers", "FlaxRectifiedFlowMultistepScheduler"),
    "WanModel": (".models.wan.transformer_wan", "WanModel"),
    "WanVACEModel": (".models.wan.transformer_wan_vace", "WanVACEModel"),
    "WanAnimateModel": (".models.wan.transformer_wan_animate", "WanAnimateModel"),
    "AutoencoderKLWan": (".models.wan.autoencoder_kl_wan", "AutoencoderKLWan"),
    "FluxTransformer2DModel": (".models.flux.transformer_flux", "FluxTransformer2DModel"),
    "UNet2DConditionModel": (".models.unet_2d_condition", "UNet2DConditionModel"),
    "FlaxUNet2DConditionModel": (".models.unet_2d_condition", "UNet2DConditionModel"),
    "AutoencoderKL": (".models.vae", "AutoencoderKL"),
    "FlaxAutoencoderKL": (".models.vae", "AutoencoderKL"),
    "ControlNetModel": (".models.controlnet", "ControlNetModel"),
    "FlaxControlNetModel": (".models.controlnet", "ControlNetModel"),
    "LTX2VideoTransformer3DModel": (".models.ltx2.transformer_ltx2", "LTX2VideoTransformer3DModel"),
    "ZImageTransformer2DModel": (".models.z_image.transformer_z_image", "ZImageTransformer2DModel"),
    "Qwen3Model": (".models.qwen3", "Qwen3Model"),
    "Transformer3DModel": (".models.ltx_video.transformer3d", "Transformer3DModel"),
    "ModelMixin": (".models.modeling_utils", "ModelMixin"),
    "make_splash_mha": (".kernels", "make_splash_mha"),
    "make_ring_attention": (".kernels", "make_ring_attention"),
    "make_custom_ring_attention": (".kernels", "make_custom_ring_attention"),
    "KERNEL_REGISTRY": (".kernels", "KERNEL_REGISTRY"),
    "create_device_mesh": (".parallel.mesh", "create_device_mesh"),
    "ConfigMixin": (".configuration_utils", "ConfigMixin"),
    "FrozenDict": (".configuration_utils", "FrozenDict"),
    "register_to_config": (".configuration_utils", "register_to_config"),
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

__version__ = "0.1.0"

from .dependency_versions_check import check_required as _check_required  # noqa: E402

_check_required()
