"""Process-wide logging setup (reference: siirl/utils/logger/logging_utils.py:26-62, built on loguru there; the
standard library here).

``set_basic_config()`` is called once per rank by ``main_dag.run_rank``:

* messages of level ``SIIRL_LOG_LEVEL`` (``LOGURU_LEVEL`` is read too, for launch scripts written for the reference;
  default ``INFO``) go to stderr, prefixed with time, level, rank and ``file:line:function``;
* when ``SIIRL_LOG_DIR`` is set, every rank also appends to ``<dir>/<SIIRL_LOGGING_FILENAME>_rank<r>.log``, rotated
  at 500 MB with five files kept.

``log_with_rank`` and ``DecoratorLoggerBase`` are the helpers the reference's workers use to tag messages with a role
and to keep a message to rank 0 (siirl/utils/logger/aggregate_logger.py:43-78).
"""
from __future__ import annotations

import logging
import logging.handlers
import os
import sys
from typing import Optional

_CONFIGURED = False


class _RankFilter(logging.Filter):
    def filter(self, record: logging.LogRecord) -> bool:
        record.rank = os.environ.get("RANK", "0")
        return True


def log_level() -> int:
    name = (os.environ.get("SIIRL_LOG_LEVEL") or os.environ.get("LOGURU_LEVEL") or "INFO").upper()
    return getattr(logging, name, logging.INFO) if isinstance(getattr(logging, name, None), int) else logging.INFO


def set_basic_config(force: bool = False) -> logging.Logger:
    """Configure the ``siirl_b200`` logger tree (idempotent).  Returns the package logger."""
    global _CONFIGURED
    root = logging.getLogger("siirl_b200")
    if _CONFIGURED and not force:
        return root
    for h in list(root.handlers):
        root.removeHandler(h)
        h.close()
    level = log_level()
    root.setLevel(level)
    root.propagate = False
    fmt = logging.Formatter("%(asctime)s.%(msecs)03d | %(levelname)-8s | rank %(rank)s | "
                            "%(filename)s:%(lineno)d:%(funcName)s >> %(message)s", datefmt="%Y-%m-%d %H:%M:%S")
    err = logging.StreamHandler(sys.stderr)
    err.setLevel(level)
    err.setFormatter(fmt)
    err.addFilter(_RankFilter())
    root.addHandler(err)
    log_dir = os.environ.get("SIIRL_LOG_DIR")
    if log_dir:
        try:
            os.makedirs(log_dir, exist_ok=True)
            stem = os.environ.get("SIIRL_LOGGING_FILENAME", "siirl") or "siirl"
            path = os.path.join(log_dir, f"{stem}_rank{os.environ.get('RANK', '0')}.log")
            fh = logging.handlers.RotatingFileHandler(path, maxBytes=500 * 2 ** 20, backupCount=5, encoding="utf-8")
            fh.setLevel(level)
            fh.setFormatter(fmt)
            fh.addFilter(_RankFilter())
            root.addHandler(fh)
        except OSError as e:
            root.warning("no log file under %s: %s", log_dir, e)
    _CONFIGURED = True
    return root


def log_with_rank(message: str, rank: int, logger: Optional[logging.Logger] = None, level: int = logging.INFO,
                  log_only_rank_0: bool = False) -> None:
    if log_only_rank_0 and rank != 0:
        return
    (logger or logging.getLogger("siirl_b200")).log(level, f"[Rank {rank}] {message}")


class DecoratorLoggerBase:
    """Role-tagged messages, through a logger or plain ``print``; optionally rank 0 only."""

    def __init__(self, role: str, logger: Optional[logging.Logger] = None, level: int = logging.DEBUG, rank: int = 0,
                 log_only_rank_0: bool = True):
        self.role, self.logger, self.level, self.rank, self.log_only_rank_0 = role, logger, level, rank, log_only_rank_0

    def log(self, text: str) -> None:
        if self.log_only_rank_0 and self.rank != 0:
            return
        if self.logger is None:
            print(f"{self.role} {text}", flush=True)
        else:
            self.logger.log(self.level, f"{self.role} {text}")
