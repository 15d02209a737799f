"""Spawns gloo ranks on CPU for the multi-process tests (rendezvous on 127.0.0.1)."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _entry(rank, world, port, fn, args, queue):
  os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world),
                     "LOCAL_RANK": str(rank)})
  torch.set_num_threads(2)
  try:
    dist.init_process_group("gloo", rank=rank, world_size=world)
    out = fn(rank, world, *args)
    queue.put((rank, "ok", out))
  except Exception:
    queue.put((rank, "error", traceback.format_exc()))
  finally:
    if dist.is_initialized():
      dist.destroy_process_group()


def run_ranks(fn, world: int, *args, timeout: float = 300.0):
  """Runs fn(rank, world, *args) on `world` gloo ranks; returns the per-rank results ordered by rank."""
  ctx = mp.get_context("spawn")
  queue = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, queue)) for r in range(world)]
  for p in procs:
    p.start()
  results = {}
  try:
    for _ in range(world):
      rank, status, payload = queue.get(timeout=timeout)
      if status != "ok":
        raise RuntimeError(f"rank {rank} failed:\n{payload}")
      results[rank] = payload
  finally:
    for p in procs:
      p.join(timeout=10)
      if p.is_alive():
        p.kill()
  return [results[r] for r in range(world)]
