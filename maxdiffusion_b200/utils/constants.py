"""File-name and environment constants of the diffusers folder layout (reference: src/maxdiffusion/utils/constants.py)."""
import os

CONFIG_NAME = "config.json"
MODEL_INDEX_NAME = "model_index.json"
WEIGHTS_NAME = "diffusion_pytorch_model.bin"
SAFETENSORS_WEIGHTS_NAME = "diffusion_pytorch_model.safetensors"
SAFETENSORS_INDEX_NAME = SAFETENSORS_WEIGHTS_NAME + ".index.json"
SCHEDULER_CONFIG_NAME = "scheduler_config.json"
LORA_WEIGHT_NAME = "pytorch_lora_weights.bin"
LORA_WEIGHT_NAME_SAFE = "pytorch_lora_weights.safetensors"
TEXT_ENCODER_ATTN_MODULE = ".self_attn"
HF_HOME = os.environ.get("HF_HOME", os.path.join(os.path.expanduser("~"), ".cache", "huggingface"))
HF_HUB_OFFLINE = os.environ.get("HF_HUB_OFFLINE", "1") not in ("0", "false", "False", "")
DEPRECATED_REVISION_ARGS = ("fp16", "non-ema")
