"""`BaseOutput`: a dataclass that can also be indexed like a tuple or a dict, as pipeline and model outputs are
(reference: src/maxdiffusion/utils/outputs.py)."""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import fields, is_dataclass
from typing import Any, Tuple


class BaseOutput(OrderedDict):

  def __init_subclass__(cls) -> None:
    super().__init_subclass__()

  def __post_init__(self):
    if not is_dataclass(self):
      raise TypeError(f"{type(self).__name__} must be a dataclass")
    self.clear()  # attribute assignment during __init__ already filled the mapping: rebuild it in field order
    for f in fields(self):
      v = getattr(self, f.name)
      if v is not None:
        super().__setitem__(f.name, v)

  def __getitem__(self, k):
    if isinstance(k, str):
      return dict(self.items())[k]
    return self.to_tuple()[k]

  def __setattr__(self, name, value):
    if value is not None and (name in self.keys() or name in getattr(type(self), "__dataclass_fields__", {})):
      super().__setitem__(name, value)
    super().__setattr__(name, value)

  def __setitem__(self, key, value):
    super().__setitem__(key, value)
    super().__setattr__(key, value)

  def __delitem__(self, *a, **k):
    raise TypeError(f"{type(self).__name__} does not support item deletion")

  def pop(self, *a, **k):
    raise TypeError(f"{type(self).__name__} does not support pop")

  def update(self, *a, **k):
    raise TypeError(f"{type(self).__name__} does not support update")

  def __reduce__(self):
    return (type(self), tuple(getattr(self, f.name) for f in fields(self)))

  def to_tuple(self) -> Tuple[Any, ...]:
    return tuple(self[k] for k in self.keys())
