"""Offload hooks on methods other than `forward`.

A module that keeps its weights in host memory between uses (an offload hook object stored as `_hf_hook`, the
convention of the `accelerate` package) is brought to the device by the hook's `pre_forward`, which PyTorch only
triggers for `forward`. `@apply_forward_hook` gives `encode` / `decode`-style methods the same treatment. Without
a hook on the instance the method runs as it is (reference: src/maxdiffusion/utils/accelerate_utils.py)."""
from __future__ import annotations

import functools


def apply_forward_hook(method):
  @functools.wraps(method)
  def wrapper(self, *args, **kwargs):
    hook = getattr(self, "_hf_hook", None)
    if hook is not None and hasattr(hook, "pre_forward"):
      hook.pre_forward(self)
    return method(self, *args, **kwargs)

  return wrapper
