"""`config.json` round trip for models, schedulers and pipelines components (the diffusers convention).

A class lists its constructor arguments once -- `@register_to_config` on `__init__`, or an explicit
`self.register_to_config(**kwargs)` -- and gets `config` (frozen), `save_config` / `load_config` / `from_config`,
`to_json_string` and `to_json_file`. What differs from a plain dict dump: private keys (leading underscore) never reach
`__init__`, `_use_default_values` remembers which arguments were left at their defaults so that a newer default wins on
reload, and run-time objects (`mesh`, `precision`, `weights_dtype`, `quant`, generators) are not serialised.

Reference: src/maxdiffusion/configuration_utils.py:71-101 (FrozenDict), :104-632 (ConfigMixin), :635-678
(`register_to_config`). The schedulers of this package use the lighter `schedulers.configuration_utils`.
"""
from __future__ import annotations

import dataclasses
import functools
import inspect
import json
import os
import warnings
from collections import OrderedDict
from pathlib import PurePath
from typing import Any, Dict, Tuple, Union

import numpy as np

from . import __version__, max_logging

_NOT_SERIALISED = ("_ignore_files", "_use_default_values", "mesh", "precision", "weights_dtype", "quant")


class FrozenDict(OrderedDict):
  """Ordered dict whose items are also attributes and cannot be changed after construction."""

  def __init__(self, *args, **kwargs):
    super().__init__(*args, **kwargs)
    for key, value in self.items():
      object.__setattr__(self, key, value)
    object.__setattr__(self, "_frozen", True)

  def _refuse(self, *args, **kwargs):
    raise TypeError(f"a {type(self).__name__} cannot be modified")

  __delitem__ = setdefault = pop = update = popitem = clear = _refuse

  def __setattr__(self, name, value):
    if getattr(self, "_frozen", False):
      self._refuse()
    object.__setattr__(self, name, value)

  def __setitem__(self, name, value):
    if getattr(self, "_frozen", False):
      self._refuse()
    super().__setitem__(name, value)

  def __reduce__(self):
    return (type(self), (list(self.items()),))


class _Encoder(json.JSONEncoder):

  def default(self, o):
    if isinstance(o, np.ndarray):
      return o.tolist()
    if isinstance(o, (np.integer, np.floating)):
      return o.item()
    if isinstance(o, PurePath):
      return str(o)
    if dataclasses.is_dataclass(o) and not isinstance(o, type):
      return dataclasses.asdict(o)
    try:
      import torch

      if isinstance(o, torch.dtype):
        return str(o)
      if isinstance(o, torch.Tensor):
        return o.tolist()
    except ImportError:
      pass
    return str(o)


class ConfigMixin:
  """Base of every class whose constructor arguments are its configuration.

  Class attributes: `config_name` (file name inside a folder; required), `ignore_for_config` (constructor arguments
  that are not configuration), `has_compatibles` (a scheduler may be built from a compatible scheduler's file)."""

  config_name: str | None = None
  ignore_for_config: list = []
  has_compatibles: bool = False

  # ---- registration ------------------------------------------------------------------------
  def register_to_config(self, **kwargs) -> None:
    if self.config_name is None:
      raise NotImplementedError(f"{type(self).__name__} has to define `config_name`")
    kwargs.pop("kwargs", None)
    merged = {**getattr(self, "_internal_dict", {}), **kwargs}
    object.__setattr__(self, "_internal_dict", FrozenDict(merged))

  @property
  def config(self) -> FrozenDict:
    return self._internal_dict

  def __getattr__(self, name: str) -> Any:
    # only reached when normal lookup failed: fall through to the config, with a nudge towards `obj.config.name`
    internal = self.__dict__.get("_internal_dict")
    if internal is not None and name in internal:
      warnings.warn(f"read `{name}` from `{type(self).__name__}.config.{name}`: direct attribute access to configuration "
                    "values is deprecated", FutureWarning, stacklevel=2)
      return internal[name]
    parent = super()
    if hasattr(parent, "__getattr__"):  # torch.nn.Module resolves parameters and sub-modules this way
      return parent.__getattr__(name)
    raise AttributeError(f"'{type(self).__name__}' object has no attribute '{name}'")

  # ---- serialisation -----------------------------------------------------------------------
  def to_json_string(self) -> str:
    d = dict(getattr(self, "_internal_dict", {}))
    d["_class_name"] = type(self).__name__
    d["_diffusers_version"] = __version__
    for key in _NOT_SERIALISED:
      d.pop(key, None)
    dropped = [k for k, v in d.items() if type(v).__name__ in ("Rngs", "Generator", "ProcessGroup", "DeviceMesh")]
    if dropped:
      max_logging.log(f"Skipping non-serializable config keys: {dropped}")
      for k in dropped:
        d.pop(k)
    return json.dumps(d, indent=2, sort_keys=True, cls=_Encoder) + "\n"

  def to_json_file(self, json_file_path: Union[str, os.PathLike]) -> None:
    with open(json_file_path, "w", encoding="utf-8") as f:
      f.write(self.to_json_string())

  def __repr__(self) -> str:
    return f"{type(self).__name__} {self.to_json_string()}"

  def save_config(self, save_directory: Union[str, os.PathLike], **unused) -> str:
    if os.path.isfile(save_directory):
      raise AssertionError(f"Provided path ({save_directory}) should be a directory, not a file")
    os.makedirs(save_directory, exist_ok=True)
    path = os.path.join(save_directory, self.config_name)
    self.to_json_file(path)
    return path

  # ---- loading -----------------------------------------------------------------------------
  @classmethod
  def load_config(cls, pretrained_model_name_or_path: Union[str, os.PathLike], subfolder: str | None = None,
                  return_unused_kwargs: bool = False, **kwargs):
    """Reads `config_name` from a file, a folder or `<folder>/<subfolder>` (local paths; a hub id has to be downloaded
    into a folder first, `utils.hub_utils`). Returns the dict, and the keyword arguments it did not consume on request."""
    if cls.config_name is None:
      raise ValueError("`config_name` is not defined: `load_config` must be called on a concrete class")
    path = os.fspath(pretrained_model_name_or_path)
    if os.path.isfile(path):
      config_file = path
    elif os.path.isdir(path):
      candidates = ([os.path.join(path, subfolder, cls.config_name)] if subfolder else []) + [os.path.join(path, cls.config_name)]
      config_file = next((c for c in candidates if os.path.isfile(c)), None)
      if config_file is None:
        raise EnvironmentError(f"Error no file named {cls.config_name} found in directory {path}.")
    else:
      raise EnvironmentError(f"{path} is neither a file nor a folder; download the repository first (`utils.hub_utils`)")
    try:
      config = cls._dict_from_json_file(config_file)
    except (json.JSONDecodeError, UnicodeDecodeError) as e:
      raise EnvironmentError(f"It looks like the config file at '{config_file}' is not a valid JSON file.") from e
    return (config, kwargs) if return_unused_kwargs else config

  get_config_dict = load_config  # older name

  @staticmethod
  def _dict_from_json_file(json_file: Union[str, os.PathLike]) -> dict:
    with open(json_file, "r", encoding="utf-8") as f:
      return json.load(f)

  @classmethod
  def _get_init_keys(cls) -> set:
    return set(inspect.signature(cls.__init__).parameters)

  @classmethod
  def extract_init_dict(cls, config_dict: Dict[str, Any], **kwargs) -> Tuple[dict, dict, dict]:
    """Splits a loaded config (+ overrides) into (arguments of `__init__`, keyword arguments nobody consumed, keys of
    the file that `__init__` does not take and that stay in the config as hidden entries)."""
    used_defaults = set(config_dict.get("_use_default_values", []))
    config_dict = {k: v for k, v in config_dict.items() if k not in used_defaults and k != "_use_default_values"}
    original = dict(config_dict)
    expected = cls._get_init_keys() - {"self", "kwargs", "args"} - set(cls.ignore_for_config)
    config_dict = {k: v for k, v in config_dict.items() if not k.startswith("_")}
    init_dict = {}
    for key in expected:
      if key in kwargs:
        init_dict[key] = kwargs.pop(key)      # an override wins over the file
      elif key in config_dict:
        init_dict[key] = config_dict.pop(key)
    if config_dict:
      max_logging.log(f"The config attributes {config_dict} were passed to {cls.__name__}, but are not expected and will "
                      "be ignored.")
    missing = expected - set(init_dict)
    required = {n for n, p in inspect.signature(cls.__init__).parameters.items()
                if p.default is inspect.Parameter.empty and p.kind in (p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)} - {"self"}
    if missing & required:
      raise ValueError(f"{cls.__name__} needs {sorted(missing & required)}, which the config does not provide")
    unused_kwargs = {**config_dict, **kwargs}
    hidden = {k: v for k, v in original.items() if k not in init_dict}
    return init_dict, unused_kwargs, hidden

  @classmethod
  def from_config(cls, config: Union[FrozenDict, Dict[str, Any]], return_unused_kwargs: bool = False, **kwargs):
    if not isinstance(config, dict):
      raise ValueError("`from_config` takes the dictionary returned by `load_config` (or an instance's `.config`)")
    init_dict, unused, hidden = cls.extract_init_dict(dict(config), **kwargs)
    obj = cls(**init_dict)
    keep = {k: v for k, v in hidden.items() if k.startswith("_") and k not in ("_class_name", "_diffusers_version")}
    if keep:
      obj.register_to_config(**keep)
    return (obj, unused) if return_unused_kwargs else obj


def register_to_config(init):
  """Decorator for `__init__`: every argument (positional or keyword, defaults included) is registered before the
  body runs. Arguments in `ignore_for_config` are skipped; private keyword arguments (leading underscore) are recorded
  but not handed to `__init__`; the names left at their defaults are remembered under `_use_default_values`."""

  @functools.wraps(init)
  def inner(self, *args, **kwargs):
    if not isinstance(self, ConfigMixin):
      raise RuntimeError(f"`@register_to_config` was applied to {type(self).__name__}.__init__, which does not inherit "
                         "from `ConfigMixin`")
    public = {k: v for k, v in kwargs.items() if not k.startswith("_")}
    private = {k: v for k, v in kwargs.items() if k.startswith("_")}
    ignore = set(getattr(self, "ignore_for_config", []))
    params = [(n, p.default) for i, (n, p) in enumerate(inspect.signature(init).parameters.items())
              if i > 0 and n not in ignore and p.kind not in (p.VAR_POSITIONAL, p.VAR_KEYWORD)]
    recorded = {name: arg for arg, (name, _) in zip(args, params)}
    for name, default in params:
      if name not in recorded:
        recorded[name] = public.get(name, default)
    defaults_used = sorted(set(recorded) - set(public) - {name for _, (name, _) in zip(args, params)})
    if defaults_used:
      recorded["_use_default_values"] = defaults_used
    self.register_to_config(**{**private, **recorded})
    init(self, *args, **public)

  return inner
