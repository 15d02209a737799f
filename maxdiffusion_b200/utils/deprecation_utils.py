"""`deprecate(name, removed_in, message, take_from=kwargs)`: warns once per call site, pops the old argument, and raises
once this package's version has reached `removed_in` (reference: src/maxdiffusion/utils/deprecation_utils.py)."""
from __future__ import annotations

import warnings
from typing import Any, Dict, Optional, Tuple, Union


def _ver(v: str) -> Tuple[int, ...]:
  return tuple(int(x) for x in v.split(".")[:3] if x.isdigit())


def deprecate(*args, take_from: Optional[Union[Dict, Any]] = None, standard_warn: bool = True, stacklevel: int = 2):
  from .. import __version__

  if args and not isinstance(args[0], tuple):
    args = (args,)
  values = ()
  for name, removed_in, message in args:
    if _ver(__version__) >= _ver(removed_in):
      raise ValueError(f"`{name}` was scheduled for removal in {removed_in} and this is {__version__}: delete the deprecated path")
    warn = None
    if isinstance(take_from, dict) and name in take_from:
      values += (take_from.pop(name),)
      warn = f"The `{name}` argument is deprecated and will be removed in version {removed_in}."
    elif take_from is not None and hasattr(take_from, name):
      values += (getattr(take_from, name),)
      warn = f"The `{name}` attribute is deprecated and will be removed in version {removed_in}."
    elif take_from is None:
      warn = f"`{name}` is deprecated and will be removed in version {removed_in}."
    if warn is not None:
      warnings.warn((warn + " " if standard_warn else "") + message, FutureWarning, stacklevel=stacklevel)
  if isinstance(take_from, dict) and take_from:
    key = next(iter(take_from))
    raise TypeError(f"got an unexpected keyword argument `{key}`")
  if not values:
    return None
  return values[0] if len(values) == 1 else values
