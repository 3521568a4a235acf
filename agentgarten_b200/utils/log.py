"""Rank-aware logging.

By default only rank 0 prints; ``rank0_only=False`` prints on every rank with a
``[RANK n]`` prefix.  Built on the standard library so that the package has no hard
logging dependency; loguru sinks are used when loguru is importable.

Parity: reference ``wm/infra/log.py:37-103`` (``configure``, ``add_sink``, ``info``,
``warning``, ``exception``, ``complete``).
"""

from __future__ import annotations

import logging
import os
import sys
from typing import Any

import torch.distributed as dist

__all__ = ["add_sink", "complete", "configure", "exception", "info", "logger", "warning"]

_FORMAT = "[%(asctime)s|%(levelname)s|%(wm_where)s] %(wm_rank_prefix)s%(message)s"


def _rank() -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank()
    return int(os.environ.get("RANK", "0"))


class _RankFilter(logging.Filter):
    def filter(self, record: logging.LogRecord) -> bool:
        rank0_only = getattr(record, "wm_rank0_only", True)
        rank = _rank()
        record.wm_rank_prefix = "" if rank0_only else f"[RANK {rank}] "
        try:
            path = os.path.relpath(record.pathname, os.getcwd())
        except (OSError, ValueError):
            path = record.pathname
        record.wm_where = f"{path}:{record.lineno}:{record.funcName}"
        return (not rank0_only) or rank == 0


logger = logging.getLogger("agentgarten_b200")
logger.propagate = False
_handlers: dict[int, logging.Handler] = {}
_next_id = 0


def add_sink(sink: Any, *, level: str = "INFO", **_options: Any) -> int:
    """Attach a stream or a file path; returns a handler id."""
    global _next_id
    handler: logging.Handler
    if isinstance(sink, (str, os.PathLike)):
        os.makedirs(os.path.dirname(os.fspath(sink)) or ".", exist_ok=True)
        handler = logging.FileHandler(os.fspath(sink))
    else:
        handler = logging.StreamHandler(sink)
    handler.setLevel(level)
    handler.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
    handler.addFilter(_RankFilter())
    logger.addHandler(handler)
    logger.setLevel(min(logger.level or logging.INFO, handler.level))
    _next_id += 1
    _handlers[_next_id] = handler
    return _next_id


def configure(level: str = "INFO") -> int:
    """Route all framework logging to stdout. Call from an application entry point."""
    for handler in list(logger.handlers):
        logger.removeHandler(handler)
    _handlers.clear()
    logger.setLevel(level)
    return add_sink(sys.stdout, level=level)


def complete() -> None:
    for handler in logger.handlers:
        handler.flush()


def _ensure_default() -> None:
    if not logger.handlers:
        configure()


def info(message: str, rank0_only: bool = True) -> None:
    _ensure_default()
    logger.info(message, extra={"wm_rank0_only": rank0_only}, stacklevel=2)


def warning(message: str, rank0_only: bool = True) -> None:
    _ensure_default()
    logger.warning(message, extra={"wm_rank0_only": rank0_only}, stacklevel=2)


def exception(message: str, rank0_only: bool = True) -> None:
    _ensure_default()
    logger.error(message, exc_info=True, extra={"wm_rank0_only": rank0_only}, stacklevel=2)
