"""YAML + `key=value` configuration.

    python -m maxdiffusion_b200.train_wan maxdiffusion_b200/configs/base_wan_14b.yml run_name=x learning_rate=2e-5

Contract (the reference's, src/maxdiffusion/pyconfig.py:79-153,199-310,335-358):
  * every override must name a key that the YAML (or one of its `base_config` parents) defines;
  * the override is parsed with the type of the YAML default (bool accepts true/false, lists and tuples go
    through `ast.literal_eval`, dicts through JSON);
  * derived keys are added afterwards: `tensorboard_dir`, `checkpoint_dir`, `metrics_dir`,
    `total_train_batch_size`, `global_batch_size_to_load`, `global_batch_size_to_train_on`, `num_slices`,
    `context_strategy` (what the `attention` name means for sequence sharding), torch dtypes;
  * the result is exposed read-only as `pyconfig.config`.

Additions: a YAML may start from another with `base_config: other.yml` (relative to its own folder), which
keeps the per-model files to the keys they change; keys that only steer the TPU runtime are accepted and ignored.
"""
from __future__ import annotations

import ast
import json
import os
import sys
from typing import Any

import torch
import yaml

from . import common_types, max_logging

TPU_ONLY_KEYS = (
    "hardware", "allow_split_physical_axes", "compile_topology_num_slices", "jax_cache_dir",
    "use_experimental_scheduler", "tile_search_vmem_limit_bytes", "enable_ondemand_xprof",
    "enable_ml_diagnostics", "run_text_encoder_on_tpu", "skip_jax_distributed_system", "jit_initializers",
)

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
    "float16": torch.float16, "fp16": torch.float16, "float64": torch.float64,
}
DTYPE_KEYS = ("weights_dtype", "activations_dtype", "text_encoder_dtype", "vae_weights_dtype", "vae_dtype",
              "scheduler_dtype", "opt_state_dtype")


def to_dtype(name: Any) -> torch.dtype:
  if isinstance(name, torch.dtype):
    return name
  try:
    return _DTYPES[str(name)]
  except KeyError:
    raise ValueError(f"unknown dtype '{name}'") from None


def _parse_bool(s: str) -> bool:
  if s.lower() in ("true", "1", "yes"):
    return True
  if s.lower() in ("false", "0", "no"):
    return False
  raise ValueError(f"cannot read '{s}' as a boolean")


def _coerce(key: str, text: str, default: Any) -> Any:
  """Parses the command-line text of `key` with the type of its YAML default."""
  if isinstance(default, bool):
    return _parse_bool(text)
  if isinstance(default, int):
    try:
      return int(text)
    except ValueError:
      return int(float(text))
  if isinstance(default, float):
    return float(text)
  if isinstance(default, dict):
    try:
      return json.loads(text)
    except json.JSONDecodeError as e:
      raise ValueError(f"{key} expects a JSON object: {e}") from None
  if isinstance(default, (list, tuple)):
    value = ast.literal_eval(text)
    if not isinstance(value, (list, tuple)):
      raise ValueError(f"{key} expects a list")
    return list(value)
  if default is None:
    try:
      return ast.literal_eval(text)
    except (ValueError, SyntaxError):
      return text
  return text


def load_yaml(path: str) -> dict:
  """Loads a YAML file, resolving its chain of `base_config` parents (child wins)."""
  with open(path, "r", encoding="utf-8") as f:
    data = yaml.safe_load(f) or {}
  parent = data.pop("base_config", None)
  if parent:
    parent_path = parent if os.path.isabs(parent) else os.path.join(os.path.dirname(os.path.abspath(path)), parent)
    merged = load_yaml(parent_path)
    merged.update(data)
    return merged
  return data


def world_size() -> int:
  return int(os.environ.get("WORLD_SIZE", os.environ.get("NNODES_TIMES_GPUS", "1")))


def global_batch_sizes(per_device_batch_size: float, num_devices: int) -> tuple[int, int]:
  """(to_load, to_train_on); below one sample per device the loader still reads one per device."""
  to_load = num_devices if per_device_batch_size < 1 else int(num_devices * per_device_batch_size)
  return to_load, int(num_devices * per_device_batch_size)


class _HyperParameters:

  def __init__(self, argv: list[str], **kwargs):
    if len(argv) < 2:
      raise ValueError("usage: <entry point> <config.yml> [key=value ...]")
    raw = load_yaml(argv[1])
    overrides: dict[str, Any] = {}
    for item in argv[2:]:
      if "=" not in item:
        raise ValueError(f"override '{item}' is not of the form key=value")
      key, text = item.split("=", 1)
      if key not in raw:
        if key in TPU_ONLY_KEYS:      # steers the TPU runtime only: accepted whether or not the file lists it
          overrides[key] = yaml.safe_load(text)
          continue
        raise ValueError(f"Key {key} was passed at the command line but is not in the config file {argv[1]}")
      overrides[key] = _coerce(key, text, raw[key])
    for key, value in kwargs.items():
      if key in ("unittest", "validate_training"):
        continue
      if key not in raw and key not in TPU_ONLY_KEYS:
        raise ValueError(f"Key {key} was passed as a keyword but is not in the config file {argv[1]}")
      overrides[key] = value
    raw.update(overrides)
    self.unittest = bool(kwargs.get("unittest", False))
    _HyperParameters.user_init(raw)
    if raw.get("model_name") in common_types.WAN_MODELS:
      _HyperParameters.wan_init(raw)
    if kwargs.get("validate_training") and "model_name" in raw:
      if raw["model_name"] in common_types.WAN_MODELS and raw["model_name"] not in common_types.TRAINABLE_WAN_MODELS:
        raise ValueError(f"training is implemented for {common_types.TRAINABLE_WAN_MODELS}, not {raw['model_name']}")
    self.keys = raw
    if not self.unittest and os.environ.get("RANK", "0") == "0" and raw.get("log_config", True):
      for k in sorted(raw):
        max_logging.log(f"Config param {k}: {raw[k]}")
    ignored = [k for k in TPU_ONLY_KEYS if k in overrides]
    if ignored:
      max_logging.log(f"TPU-runtime keys accepted and ignored on this backend: {ignored}")

  @staticmethod
  def wan_init(raw: dict) -> None:
    if raw.get("wan_transformer_pretrained_model_name_or_path", "") == "":
      raw["wan_transformer_pretrained_model_name_or_path"] = raw.get("pretrained_model_name_or_path", "")
    if raw.get("use_qwix_quantization") and raw.get("quantization") not in ("int8", "fp8", "fp8_full"):
      raise ValueError(f"quantization '{raw.get('quantization')}' is not one of int8, fp8, fp8_full")

  @staticmethod
  def user_init(raw: dict) -> None:
    raw.setdefault("remat_policy", "NONE")
    raw.setdefault("names_which_can_be_saved", [])
    raw.setdefault("names_which_can_be_offloaded", [])
    raw.setdefault("offload_encoders", False)
    raw.setdefault("vae_spatial", -1)
    raw.setdefault("opt_state_dtype", raw.get("weights_dtype", "bfloat16"))
    for key in DTYPE_KEYS:
      if key in raw:
        raw[key] = to_dtype(raw[key])

    if raw.get("run_name", "") == "":
      raw["run_name"] = os.environ.get("JOBSET_NAME", "") or ""
    if raw["run_name"]:
      base = raw.get("output_dir", "")
      raw["tensorboard_dir"] = os.path.join(base, raw["run_name"], "tensorboard", "")
      raw["checkpoint_dir"] = os.path.join(base, raw["run_name"], "checkpoints", "")
      raw["metrics_dir"] = os.path.join(base, raw["run_name"], "metrics", "")

    attention = raw.get("attention", "flash")
    strategy = common_types.context_strategy(attention)
    if attention in common_types.USP_KERNELS and int(raw.get("ulysses_shards", -1)) <= 0:
      raise ValueError(f"{attention} requires ulysses_shards to be set from config or command line.")
    raw["context_strategy"] = strategy
    raw["fixed_m_softmax"] = attention in common_types.FIXED_M_KERNELS

    if raw.get("learning_rate_schedule_steps", -1) == -1:
      raw["learning_rate_schedule_steps"] = raw.get("max_train_steps", 0)
    raw["tokenizer_model_name_or_path"] = raw.get("pretrained_model_name_or_path", "")
    for key in ("hf_train_files", "hf_access_token"):
      if key in raw and not raw[key]:
        raw[key] = None

    n = world_size()
    pdb = float(raw.get("per_device_batch_size", 1))
    raw["total_train_batch_size"] = max(1, int(n * pdb)) if pdb >= 1 else max(1, int(round(n * pdb)))
    raw["global_batch_size_to_load"], raw["global_batch_size_to_train_on"] = global_batch_sizes(pdb, n)
    raw["num_slices"] = max(1, int(os.environ.get("NNODES", "1")))
    if int(raw.get("quantization_local_shard_count", -1)) == -1:
      raw["quantization_local_shard_count"] = raw["num_slices"]


class HyperParameters:
  """Read-only facade over the resolved keys."""

  def __init__(self, params: _HyperParameters):
    object.__setattr__(self, "_params", params)

  def __getattr__(self, attr: str) -> Any:
    keys = object.__getattribute__(self, "_params").keys
    if attr not in keys:
      raise AttributeError(f"Requested key {attr}, not in config")
    return keys[attr]

  def __setattr__(self, attr: str, value: Any) -> None:
    raise ValueError("the config is read-only; pass overrides to pyconfig.initialize")

  def get_keys(self) -> dict:
    return object.__getattribute__(self, "_params").keys

  def get(self, attr: str, default: Any = None) -> Any:
    return self.get_keys().get(attr, default)

  def replace(self, **updates) -> "HyperParameters":
    """A copy with some keys changed (entry points use it for the warm-up / profiling passes)."""
    params = object.__getattribute__(self, "_params")
    clone = object.__new__(_HyperParameters)
    clone.keys = dict(params.keys)
    for k, v in updates.items():
      if k not in clone.keys:
        raise ValueError(f"Key {k} is not in the config")
      clone.keys[k] = v
    clone.unittest = params.unittest
    return HyperParameters(clone)


_config: _HyperParameters | None = None
config: HyperParameters | None = None


def initialize(argv, **kwargs) -> HyperParameters:
  """Parses `argv` (program, yaml, overrides...) and publishes the result as `pyconfig.config`."""
  global _config, config
  _config = _HyperParameters(list(argv), **kwargs)
  config = HyperParameters(_config)
  return config


if __name__ == "__main__":
  initialize(sys.argv)
  print(config.get_keys())
