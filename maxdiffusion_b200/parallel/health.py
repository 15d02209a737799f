"""Failure detection between ranks, entirely on the host: heartbeats through the rendezvous store, a watchdog that
turns a silent peer into an exception BEFORE the next kernel or collective is launched, and a bounded barrier.

The reference has no counterpart in its own tree: on GPUs it relies on `jax.distributed` coordination-service
heartbeats (src/maxdiffusion/max_utils.py:925-955) and a bash launcher that waits on the ranks' pids
(gpu_multi_process_run.sh:120-155). Here:

  * every rank publishes `hb/<rank> = (step, wall time)` in the `torch.distributed` TCPStore between steps;
  * `check()` (called by the trainers before a step's first launch) reads the peers' entries and raises
    `RankFailure` naming the ranks whose heartbeat is older than `timeout_s` or that announced an exception;
  * `report_failure(exc)` lets a rank that caught an exception tell the others why it is leaving;
  * `barrier(timeout_s)` is a store-based barrier that raises instead of waiting forever.

On the device side every wait of the kernel library is bounded and records its failure in the status word
(`ops/_lib.raise_on_device_status`), so a peer that stopped signalling surfaces as an exception, not as a hang.
A rank leaves only between steps, with none of its kernels or collectives in flight.
"""
from __future__ import annotations

import json
import os
import threading
import time
from typing import Optional

import torch.distributed as dist


class RankFailure(RuntimeError):

  def __init__(self, ranks, reasons):
    self.ranks, self.reasons = list(ranks), dict(reasons)
    super().__init__("ranks not healthy: " + ", ".join(f"{r} ({self.reasons.get(r, 'no heartbeat')})" for r in self.ranks))


def _default_store():
  if dist.is_available() and dist.is_initialized():
    try:
      return dist.distributed_c10d._get_default_store()
    except Exception:
      return None
  return None


class HealthMonitor:
  """Heartbeats and peer checks over a key-value store (`torch.distributed` store or any object with set/get)."""

  def __init__(self, rank: Optional[int] = None, world_size: Optional[int] = None, store=None, timeout_s: float = 60.0,
               interval_s: float = 5.0, prefix: str = "mdb_health"):
    init = dist.is_available() and dist.is_initialized()
    self.rank = rank if rank is not None else (dist.get_rank() if init else 0)
    self.world = world_size if world_size is not None else (dist.get_world_size() if init else 1)
    self.store = store if store is not None else _default_store()
    self.timeout_s, self.interval_s, self.prefix = timeout_s, interval_s, prefix
    self.step = 0
    self._thread: Optional[threading.Thread] = None
    self._stop = threading.Event()
    self._barrier_round = 0

  # ---- publishing --------------------------------------------------------------------------
  def _key(self, kind: str, rank: int) -> str:
    return f"{self.prefix}/{kind}/{rank}"

  def beat(self, step: Optional[int] = None) -> None:
    if step is not None:
      self.step = step
    if self.store is not None:
      self.store.set(self._key("hb", self.rank), json.dumps({"step": self.step, "time": time.time(), "pid": os.getpid()}))

  def report_failure(self, exc: BaseException) -> None:
    if self.store is not None:
      self.store.set(self._key("fail", self.rank), f"{type(exc).__name__}: {exc}"[:500])

  def start(self) -> "HealthMonitor":
    """Background heartbeat every `interval_s` (covers long steps and checkpoint writes)."""
    self.beat()
    if self._thread is None and self.store is not None and self.world > 1:
      def loop():
        while not self._stop.wait(self.interval_s):
          try:
            self.beat()
          except Exception:
            return
      self._thread = threading.Thread(target=loop, daemon=True, name="mdb-heartbeat")
      self._thread.start()
    return self

  def stop(self) -> None:
    self._stop.set()
    if self._thread is not None:
      self._thread.join(timeout=2 * self.interval_s)
      self._thread = None

  # ---- checking ----------------------------------------------------------------------------
  def _get(self, key: str) -> Optional[str]:
    try:
      if hasattr(self.store, "check") and not self.store.check([key]):
        return None
      v = self.store.get(key)
      return v.decode() if isinstance(v, (bytes, bytearray)) else v
    except Exception:
      return None

  def unhealthy(self) -> dict:
    """{rank: reason} of the peers that announced a failure or whose heartbeat is stale."""
    bad = {}
    if self.store is None:
      return bad
    now = time.time()
    for r in range(self.world):
      if r == self.rank:
        continue
      fail = self._get(self._key("fail", r))
      if fail:
        bad[r] = fail
        continue
      hb = self._get(self._key("hb", r))
      if hb is None:
        continue  # not started yet: start-up is covered by the rendezvous timeout
      age = now - json.loads(hb)["time"]
      if age > self.timeout_s:
        bad[r] = f"last heartbeat {age:.0f}s ago"
    return bad

  def check(self) -> None:
    """Raises `RankFailure` if a peer is unhealthy. Call between steps, before the next launch."""
    bad = self.unhealthy()
    if bad:
      raise RankFailure(sorted(bad), bad)

  def barrier(self, timeout_s: Optional[float] = None, poll_s: float = 0.05) -> None:
    """Store-based barrier; raises `RankFailure` (failed peers) or `TimeoutError` instead of blocking forever."""
    if self.store is None or self.world == 1:
      return
    self._barrier_round += 1
    key = f"{self.prefix}/barrier/{self._barrier_round}"
    self.store.add(key, 1)
    deadline = time.time() + (timeout_s if timeout_s is not None else self.timeout_s)
    nap = 2e-4  # ranks in step arrive within a fraction of a millisecond: poll fast first, back off to poll_s
    while int(self.store.add(key, 0)) < self.world:
      self.check()
      if time.time() > deadline:
        raise TimeoutError(f"barrier {self._barrier_round}: {int(self.store.add(key, 0))}/{self.world} ranks arrived")
      time.sleep(nap)
      nap = min(poll_s, nap * 2)


class guarded_step:
  """Context manager around one training / sampling step: checks the peers first, publishes a heartbeat after, and
  announces this rank's exception to the others before re-raising it."""

  def __init__(self, monitor: Optional[HealthMonitor], step: int):
    self.monitor, self.step = monitor, step

  def __enter__(self):
    if self.monitor is not None:
      self.monitor.check()
    return self

  def __exit__(self, exc_type, exc, tb):
    if self.monitor is None:
      return False
    if exc is not None:
      self.monitor.report_failure(exc)
    else:
      self.monitor.beat(self.step + 1)
    return False
