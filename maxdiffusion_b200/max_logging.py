"""Logging: one flushed line per message, prefixed with the rank when running multi-process.

Same role as the reference's `max_logging.log` (src/maxdiffusion/max_logging.py).
"""
import os
import sys


def log(msg: str) -> None:
  rank = os.environ.get("RANK")
  prefix = f"[rank {rank}] " if rank not in (None, "0") else ""
  print(f"{prefix}{msg}", flush=True)


def warn(msg: str) -> None:
  print(f"WARNING: {msg}", file=sys.stderr, flush=True)
