"""Forward + backward of a training objective captured once in a CUDA graph and replayed every step.

A UNet training step is thousands of small launches (SDXL at batch 8: about 3300), and issuing them costs the host
about as long as the device needs to run them. The objective is a fixed sequence of kernels on fixed shapes, so it is
captured once (`torch.cuda.graph`: every kernel of this repository launches on the current stream, and their tensor
maps are kernel parameters, copied into the graph) and replayed with one launch. What varies from step to step stays
outside: the batch is copied into the graph's input buffers, the learning rate, step count and RNG seed of the
optimizer are host values of the eager optimizer step that follows.

The reference gets the same effect from `jax.jit`: its train step is one compiled executable
(src/maxdiffusion/trainers/sdxl_trainer.py:178-291, `p_train_step`).

Rules the captured function has to follow (checked where they can be): no host reads of device values, no random
draws from a generator that is not registered with the graph (draw before the call and pass the tensors in), every
tensor it needs is either an argument or a parameter.
"""
from __future__ import annotations

from typing import Callable, Dict, Sequence

import torch


class GraphedObjective:
  """`loss = objective(**inputs)` followed by `loss.backward()`, as one graph per input signature.

  The first `eager_calls` calls run eagerly (they warm up allocator pools, packed weights and tuned variants, which
  must not happen inside a capture); the next call captures; later calls replay. Parameters' `.grad` are the graph's
  own buffers: they are set again before each replay because optimizers may drop them."""

  def __init__(self, objective: Callable[..., torch.Tensor], params: Sequence[torch.nn.Parameter], eager_calls: int = 2):
    self.objective = objective
    self.params = [p for p in params if p.requires_grad]
    self.eager_calls = eager_calls
    self.calls = 0
    self.graphs: Dict[tuple, tuple] = {}
    self.replays = 0

  @staticmethod
  def _signature(inputs: Dict[str, torch.Tensor]) -> tuple:
    return tuple((k, tuple(v.shape), v.dtype) for k, v in sorted(inputs.items()) if torch.is_tensor(v))

  def _eager(self, inputs):
    loss = self.objective(**inputs)
    loss.backward()
    return loss.detach()

  def __call__(self, inputs: Dict[str, torch.Tensor]) -> torch.Tensor:
    self.calls += 1
    if self.calls <= self.eager_calls or not all(v.is_cuda for v in inputs.values() if torch.is_tensor(v)):
      return self._eager(inputs)
    key = self._signature(inputs)
    entry = self.graphs.get(key)
    if entry is None:
      entry = self._capture(inputs)
      self.graphs[key] = entry
    graph, static_in, static_loss, static_grads = entry
    for k, v in inputs.items():
      if torch.is_tensor(v):
        static_in[k].copy_(v, non_blocking=True)
    for p, g in zip(self.params, static_grads):
      p.grad = g
    graph.replay()
    self.replays += 1
    return static_loss.detach().clone()

  def _capture(self, inputs):
    static_in = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in inputs.items()}
    for p in self.params:
      p.grad = None  # the backward inside the capture allocates the gradients from the graph's pool
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
      loss = self.objective(**static_in)
      loss.backward()
    grads = [p.grad for p in self.params]
    missing = [i for i, g in enumerate(grads) if g is None]
    if missing:
      # a parameter the objective does not reach keeps a zero gradient of its own
      for i in missing:
        grads[i] = torch.zeros_like(self.params[i])
    return graph, static_in, loss, grads
