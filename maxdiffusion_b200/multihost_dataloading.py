"""Per-rank batches with retry on transient data errors.

The reference assembles a global `jax.Array` from per-host numpy batches and retries the loader up to 30 times, 10 s
apart, on `FailedPreconditionError` (src/maxdiffusion/multihost_dataloading.py:39-117). With one process per GPU each
rank simply owns its slice; what remains is the retry loop and the agreement check that every context / tensor rank
of a replica sees the same samples.
"""
from __future__ import annotations

import time
from typing import Callable, Iterator

import torch
import torch.distributed as dist

from . import max_logging


class MultiHostDataLoadIterator:

  def __init__(self, iterator: Iterator[dict], max_retries: int = 30, sleep_s: float = 10.0,
               retry_on: tuple = (OSError, RuntimeError), broadcast_group=None, src: int = 0):
    self.iterator, self.max_retries, self.sleep_s, self.retry_on = iterator, max_retries, sleep_s, retry_on
    self.group, self.src = broadcast_group, src

  def __iter__(self):
    return self

  def __next__(self) -> dict:
    last = None
    for attempt in range(self.max_retries):
      try:
        batch = next(self.iterator)
        break
      except StopIteration:
        raise
      except self.retry_on as e:
        last = e
        max_logging.log(f"data loading failed ({e}); retry {attempt + 1}/{self.max_retries}")
        time.sleep(self.sleep_s)
    else:
      raise RuntimeError(f"data loading failed {self.max_retries} times") from last
    if self.group is not None:
      # the ranks that share a sample (context / tensor axes) take it from one source rank
      for k, v in batch.items():
        if torch.is_tensor(v):
          dist.broadcast(v, src=self.src, group=self.group)
    return batch
