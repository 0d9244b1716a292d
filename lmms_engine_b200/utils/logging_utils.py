"""Rank-aware logging (reference: src/lmms_engine/utils/logging_utils.py:19-49 uses loguru +
Rich with a rank-0 filter; this uses loguru when importable and ``logging`` otherwise)."""
from __future__ import annotations

import logging
import os
import sys

try:  # pragma: no cover - exercised implicitly
    from loguru import logger as _loguru

    HAVE_LOGURU = True
except Exception:  # pragma: no cover
    _loguru = None
    HAVE_LOGURU = False


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


class _StdLogger:
    def __init__(self):
        self._l = logging.getLogger("lmms_engine_b200")
        if not self._l.handlers:
            h = logging.StreamHandler(sys.stderr)
            h.setFormatter(logging.Formatter("%(asctime)s | %(levelname)s | %(message)s"))
            self._l.addHandler(h)
            self._l.setLevel(logging.INFO)

    def info(self, m, *a):
        self._l.info(m, *a)

    def warning(self, m, *a):
        self._l.warning(m, *a)

    def error(self, m, *a):
        self._l.error(m, *a)

    def debug(self, m, *a):
        self._l.debug(m, *a)

    def exception(self, m, *a):
        self._l.exception(m, *a)


logger = _loguru if HAVE_LOGURU else _StdLogger()


def setup_distributed_logging(all_ranks: bool = False) -> None:
    """Keep INFO output on rank 0 only; warnings and errors from every rank."""
    if HAVE_LOGURU:
        _loguru.remove()
        rank = _rank()
        _loguru.add(sys.stderr, level="INFO", filter=lambda rec: all_ranks or rank == 0 or rec["level"].no >= 30,
                    format="<green>{time:HH:mm:ss}</green> | <level>{level: <7}</level> | r" + str(rank) + " | {message}")
    elif _rank() != 0 and not all_ranks:
        logging.getLogger("lmms_engine_b200").setLevel(logging.WARNING)


def rank0_print(*args) -> None:
    if _rank() == 0:
        print(*args, flush=True)


class Logging:
    """The reference's older logging surface (src/lmms_engine/utils/logging_utils.py:52-95): static methods that print
    on rank 0 only.  Kept for code written against it; new code uses ``logger``."""

    @staticmethod
    def _emit(level: str, msg: str) -> None:
        if _rank() == 0:
            getattr(logger, level)(msg)

    @staticmethod
    def info(msg: str) -> None:
        Logging._emit("info", msg)

    @staticmethod
    def warning(msg: str) -> None:
        Logging._emit("warning", msg)

    @staticmethod
    def error(msg: str) -> None:
        Logging._emit("error", msg)

    @staticmethod
    def debug(msg: str) -> None:
        Logging._emit("debug", msg)

    @staticmethod
    def null_logging(msg: str) -> None:
        return None
