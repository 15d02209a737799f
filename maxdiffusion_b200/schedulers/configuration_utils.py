"""`register_to_config` / `config.json` round trip for schedulers and models (diffusers convention).

Reference: src/maxdiffusion/configuration_utils.py:104-681 (ConfigMixin, register_to_config).
"""
from __future__ import annotations

import json
import os
from types import SimpleNamespace


class FrozenConfig(SimpleNamespace):

  def to_dict(self) -> dict:
    return dict(self.__dict__)

  def get(self, key, default=None):
    return self.__dict__.get(key, default)


class SchedulerConfigMixin:
  config_name = "scheduler_config.json"

  def register_to_config(self, **kwargs) -> None:
    self.config = FrozenConfig(**kwargs)

  @classmethod
  def from_config(cls, config: dict | FrozenConfig, **overrides):
    d = config.to_dict() if isinstance(config, FrozenConfig) else dict(config)
    d.update(overrides)
    import inspect

    accepted = set(inspect.signature(cls.__init__).parameters) - {"self"}
    return cls(**{k: v for k, v in d.items() if k in accepted})

  @classmethod
  def from_pretrained(cls, path: str, subfolder: str | None = None, **overrides):
    folder = os.path.join(path, subfolder) if subfolder else path
    with open(os.path.join(folder, cls.config_name), "r", encoding="utf-8") as f:
      return cls.from_config(json.load(f), **overrides)

  def save_pretrained(self, path: str) -> None:
    os.makedirs(path, exist_ok=True)
    d = {"_class_name": type(self).__name__, **{k: v for k, v in self.config.to_dict().items()}}
    with open(os.path.join(path, self.config_name), "w", encoding="utf-8") as f:
      json.dump(d, f, indent=2, sort_keys=True, default=str)
