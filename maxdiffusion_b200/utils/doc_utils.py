"""Docstring helper: one usage example shared by several call signatures.

`@replace_example_docstring(text)` substitutes `text` for the placeholder line `Examples:` (or `Example:`) of the
decorated function's docstring, so that a pipeline's `__call__` documents a runnable example that is kept in one
constant (reference: src/maxdiffusion/utils/doc_utils.py)."""
from __future__ import annotations

import re

_PLACEHOLDER = re.compile(r"^\s*Examples?:\s*$")


def replace_example_docstring(example_docstring: str):
  def decorate(fn):
    lines = (fn.__doc__ or "").split("\n")
    hits = [i for i, line in enumerate(lines) if _PLACEHOLDER.match(line)]
    if not hits:
      raise ValueError(f"{fn.__qualname__} needs an empty 'Examples:' line in its docstring as the placeholder; its "
                       f"docstring is:\n{fn.__doc__}")
    lines[hits[0]] = example_docstring
    fn.__doc__ = "\n".join(lines)
    return fn

  return decorate
