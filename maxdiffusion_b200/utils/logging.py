"""Library logger with a process-wide verbosity (`MAXDIFFUSION_VERBOSITY` = debug|info|warning|error|critical) and
rank-aware output: only rank 0 logs below WARNING unless `all_ranks=True`
(reference: src/maxdiffusion/utils/logging.py)."""
from __future__ import annotations

import logging as _logging
import os
import sys
import threading
from typing import Optional

DEBUG, INFO, WARNING, ERROR, CRITICAL = _logging.DEBUG, _logging.INFO, _logging.WARNING, _logging.ERROR, _logging.CRITICAL
_LEVELS = {"debug": DEBUG, "info": INFO, "warning": WARNING, "error": ERROR, "critical": CRITICAL}
_lock = threading.Lock()
_handler: Optional[_logging.Handler] = None
_ROOT = "maxdiffusion_b200"


def _default_level() -> int:
  v = os.environ.get("MAXDIFFUSION_VERBOSITY", "").lower()
  if v and v not in _LEVELS:
    _logging.getLogger().warning(f"unknown MAXDIFFUSION_VERBOSITY={v}; one of {', '.join(_LEVELS)}")
  return _LEVELS.get(v, WARNING)


class _RankFilter(_logging.Filter):

  def filter(self, record):
    if record.levelno >= WARNING or getattr(record, "all_ranks", False):
      return True
    return int(os.environ.get("RANK", "0")) == 0


class _StderrHandler(_logging.StreamHandler):
  """Writes to whatever `sys.stderr` is when a record is emitted, so that a redirection installed after the first
  logger was created (a test's capture, a launcher's per-rank log file) still receives the output."""

  def __init__(self):
    _logging.Handler.__init__(self)

  @property
  def stream(self):
    return sys.stderr


def _configure() -> None:
  global _handler
  with _lock:
    if _handler is not None:
      return
    _handler = _StderrHandler()
    _handler.addFilter(_RankFilter())
    root = _logging.getLogger(_ROOT)
    root.addHandler(_handler)
    root.setLevel(_default_level())
    root.propagate = False


def get_logger(name: Optional[str] = None) -> _logging.Logger:
  _configure()
  return _logging.getLogger(name or _ROOT)


def get_verbosity() -> int:
  _configure()
  return _logging.getLogger(_ROOT).getEffectiveLevel()


def set_verbosity(level) -> None:
  _configure()
  _logging.getLogger(_ROOT).setLevel(_LEVELS[level] if isinstance(level, str) else level)


def set_verbosity_info(): set_verbosity(INFO)
def set_verbosity_warning(): set_verbosity(WARNING)
def set_verbosity_debug(): set_verbosity(DEBUG)
def set_verbosity_error(): set_verbosity(ERROR)


def enable_explicit_format() -> None:
  _configure()
  _handler.setFormatter(_logging.Formatter("[%(levelname)s|%(filename)s:%(lineno)s] %(asctime)s >> %(message)s"))


def reset_format() -> None:
  _configure()
  _handler.setFormatter(None)


_seen = set()


def warning_once(logger: _logging.Logger, msg: str) -> None:
  if msg not in _seen:
    _seen.add(msg)
    logger.warning(msg)
