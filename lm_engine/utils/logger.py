"""Rank-aware logging helpers (parity: lm_engine/utils/logger.py:14-74)."""

from __future__ import annotations

import logging
import warnings

from .packages import is_colorlog_available
from .parallel import ProcessGroupManager, is_tracking_rank, run_rank_n

_LOGGER: logging.Logger | None = None


def set_logger(level: int | str = logging.INFO, colored_log: bool = False) -> None:
    global _LOGGER
    if isinstance(level, str):
        level = getattr(logging, level.upper())
    fmt = "%(asctime)s - [%(levelname)-8s] ▶ %(message)s"
    handler = logging.StreamHandler()
    if colored_log and is_colorlog_available():
        from colorlog import ColoredFormatter

        handler.setFormatter(ColoredFormatter("%(asctime)s - %(log_color)s[%(levelname)-8s] ▶%(reset)s %(message)s"))
    else:
        handler.setFormatter(logging.Formatter(fmt))
    logger = logging.getLogger("lm_engine")
    logger.handlers = [handler]
    logger.setLevel(level)
    logger.propagate = False
    _LOGGER = logger


def get_logger() -> logging.Logger:
    if _LOGGER is None:
        set_logger()
    return _LOGGER


def log_rank_0(level: int, msg: str) -> None:
    if ProcessGroupManager.get_global_rank() == 0:
        get_logger().log(level, msg, stacklevel=3)


def log_metrics(level: int, msg: str) -> None:
    if is_tracking_rank():
        get_logger().log(level, msg, stacklevel=3)


def print_rank_0(*args, **kwargs) -> None:
    if ProcessGroupManager.get_global_rank() == 0:
        print(*args, **kwargs)


def print_ranks_all(*args, **kwargs) -> None:
    """Every rank prints in rank order (a barrier separates consecutive ranks)."""
    import torch.distributed as dist

    world = ProcessGroupManager.get_world_size()
    for rank in range(world):
        if rank == ProcessGroupManager.get_global_rank():
            print(f"rank {rank}:", *args, **kwargs)
        if dist.is_initialized():
            dist.barrier()


def warn_rank_0(*args, **kwargs) -> None:
    if ProcessGroupManager.get_global_rank() == 0:
        warnings.warn(*args, **kwargs, stacklevel=3)
