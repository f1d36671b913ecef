"""Logging facade with the reference's bracketed decision tags.

The reference logs placement and fallback decisions as tagged lines (``[TensorParallel]``,
``[CfgParallel]``, ``[Collective] transport=...``, ``[ParallelPlan]``, ``[Placement]``;
src/HartsyInference.Core/Logging/Logs.cs, src/HartsyInference.Cuda/CollectiveComm.cs:47,55).
``decision(tag, msg)`` keeps that convention on top of :mod:`logging`, and ``set_logger`` lets a
host application (or the C ABI callback) replace the sink.
"""
from __future__ import annotations

import logging
from typing import Callable, Optional

from . import config

_LEVELS = {"trace": 5, "debug": logging.DEBUG, "info": logging.INFO, "warn": logging.WARNING,
           "warning": logging.WARNING, "error": logging.ERROR}

logger = logging.getLogger("hartsyinference_b200")
_sink: Optional[Callable[[int, str], None]] = None
_decisions: list[tuple[str, str]] = []


def _ensure_handler() -> None:
    if not logger.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(message)s"))
        logger.addHandler(h)
    logger.setLevel(_LEVELS.get(str(config.get("log_level")).lower(), logging.INFO))


def set_logger(sink: Optional[Callable[[int, str], None]]) -> None:
    """Route every record to ``sink(level, message)``; ``None`` restores the default handler."""
    global _sink
    _sink = sink


def log(level: int, msg: str) -> None:
    if _sink is not None:
        _sink(level, msg)
        return
    _ensure_handler()
    logger.log(level, msg)


def info(msg: str) -> None:
    log(logging.INFO, msg)


def warn(msg: str) -> None:
    log(logging.WARNING, msg)


def debug(msg: str) -> None:
    log(logging.DEBUG, msg)


def decision(tag: str, msg: str) -> None:
    """Record a placement / fallback decision, e.g. ``decision("Collective", "transport=nccl")``."""
    _decisions.append((tag, msg))
    if len(_decisions) > 1000:
        del _decisions[:500]
    log(logging.INFO, f"[{tag}] {msg}")


def recent_decisions(tag: Optional[str] = None) -> list[tuple[str, str]]:
    return [d for d in _decisions if tag is None or d[0] == tag]
