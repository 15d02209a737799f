"""Schedulers with explicit state: `create_state`, `set_timesteps`, `step`, `add_noise`.

The reference's `Flax*` class names are kept as aliases (src/maxdiffusion/schedulers/__init__.py).
"""
from .scheduling_ddim import DDIMScheduler
from .scheduling_ddpm import DDPMScheduler
from .scheduling_dpmsolver_multistep import DPMSolverMultistepScheduler
from .scheduling_euler_discrete import EulerDiscreteScheduler
from .scheduling_flow_match import FlowMatchScheduler
from .scheduling_lms_discrete import LMSDiscreteScheduler
from .scheduling_pndm import PNDMScheduler
from .scheduling_rectified_flow import RectifiedFlowMultistepScheduler
from .scheduling_unipc_multistep import UniPCMultistepScheduler

SCHEDULERS = {
    "DDIMScheduler": DDIMScheduler, "DDPMScheduler": DDPMScheduler,
    "DPMSolverMultistepScheduler": DPMSolverMultistepScheduler, "EulerDiscreteScheduler": EulerDiscreteScheduler,
    "FlowMatchScheduler": FlowMatchScheduler, "LMSDiscreteScheduler": LMSDiscreteScheduler, "PNDMScheduler": PNDMScheduler,
    "RectifiedFlowMultistepScheduler": RectifiedFlowMultistepScheduler, "UniPCMultistepScheduler": UniPCMultistepScheduler,
}
FlaxDDIMScheduler, FlaxDDPMScheduler = DDIMScheduler, DDPMScheduler
FlaxDPMSolverMultistepScheduler, FlaxEulerDiscreteScheduler = DPMSolverMultistepScheduler, EulerDiscreteScheduler
FlaxFlowMatchScheduler, FlaxLMSDiscreteScheduler, FlaxPNDMScheduler = FlowMatchScheduler, LMSDiscreteScheduler, PNDMScheduler
FlaxRectifiedFlowMultistepScheduler, FlaxUniPCMultistepScheduler = RectifiedFlowMultistepScheduler, UniPCMultistepScheduler
