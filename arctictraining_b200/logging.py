# SPDX-License-Identifier: Apache-2.0
"""Per-rank logging on top of loguru.

Behaviour parity: arctic_training/logging.py:37-156 (rank-tagged format, optional per-rank file sink
``<output_dir>/logs/rank_<local_rank>.log``, rank filters for console and file output, standard
``logging`` records routed into loguru, silent stdout and tqdm on non-printing ranks, level from
``AT_LOG_LEVEL``).
"""

from __future__ import annotations

import logging as _pylogging
import os
import sys
from typing import TYPE_CHECKING

from loguru import logger

if TYPE_CHECKING:
    from .config.logger import LoggerConfig

_FORMAT = (
    "<green>{time:YYYY-MM-DD HH:mm:ss.SSS}</green> | <level>{level: <8}</level> | "
    "<cyan>rank {extra[rank]}</cyan> | <cyan>{name}</cyan>:<cyan>{line}</cyan> - <level>{message}</level>"
)
_configured = False


class _LoguruBridge(_pylogging.Handler):
    """Forward records of the standard logging module to loguru, keeping the level name."""

    def emit(self, record: _pylogging.LogRecord) -> None:
        try:
            level = logger.level(record.levelname).name
        except ValueError:
            level = record.levelno
        logger.opt(depth=6, exception=record.exc_info).log(level, record.getMessage())


def _rank() -> int:
    return int(os.getenv("RANK", 0))


def _local_rank() -> int:
    return int(os.getenv("LOCAL_RANK", 0))


def _default_setup() -> None:
    logger.remove()
    logger.configure(extra={"rank": _rank()})
    level = os.getenv("AT_LOG_LEVEL", "WARNING" if _rank() != 0 else "INFO")
    logger.add(sys.stderr, colorize=False, format=_FORMAT, level=level)


_default_setup()


def setup_init_logger() -> None:
    """(Re-)install the sink that is active before a recipe's ``logger:`` section has been read: standard error, level
    from ``AT_LOG_LEVEL`` (INFO on rank 0, WARNING elsewhere)."""
    _default_setup()


def setup_logger(config: "LoggerConfig") -> None:
    """Install console and file sinks as the ``logger:`` section of a recipe asks.  Idempotent."""
    global _configured
    if _configured:
        return
    _configured = True
    logger.remove()
    logger.configure(extra={"rank": _rank()})
    level = os.getenv("AT_LOG_LEVEL", config.level)
    local_rank = _local_rank()

    if config.file_enabled and local_rank in config.file_output_ranks:
        log_dir = config.output_dir / "logs" if config.output_dir.name != "logs" else config.output_dir
        log_dir.mkdir(parents=True, exist_ok=True)
        logger.add(log_dir / f"rank_{local_rank}.log", colorize=False, format=_FORMAT, level=level)

    if local_rank in config.print_output_ranks:
        logger.add(sys.stderr, colorize=True, format=_FORMAT, level=level)
    else:
        # ranks that should stay quiet neither print nor draw progress bars
        sys.stdout = open(os.devnull, "w")
        try:
            from functools import partialmethod

            from tqdm import tqdm

            tqdm.__init__ = partialmethod(tqdm.__init__, disable=True)  # type: ignore[method-assign]
        except Exception:
            pass

    _pylogging.basicConfig(handlers=[_LoguruBridge()], level=_pylogging.WARNING, force=True)
    logger.info("logger initialised")


def reset_logger_for_tests() -> None:
    global _configured
    _configured = False
    _default_setup()


__all__ = ["logger", "setup_logger"]
