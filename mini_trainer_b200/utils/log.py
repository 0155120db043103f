"""Console logging helpers (reference utils.py:12-34)."""
from __future__ import annotations

import inspect
import logging

import torch.distributed as dist


def get_caller(num_frames: int = 1) -> str:
    frame = inspect.currentframe().f_back
    for _ in range(num_frames - 1):
        frame = frame.f_back
    return f"In {frame.f_code.co_filename}, line {frame.f_lineno}"


def log_rank_0(msg, include_caller: bool = False, rank=None, to_print: bool = True) -> None:
    """Prints (or logs at INFO) only on rank 0, or when no process group exists."""
    if rank is None:
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    if rank <= 0:
        if include_caller:
            msg = f"{get_caller(num_frames=2)}: {msg}"
        if to_print:
            print(msg)
        else:
            logging.info(msg)


def setup_logger(level: str = "DEBUG") -> None:
    try:
        from rich.logging import RichHandler
        handlers = [RichHandler()]
    except Exception:  # rich is optional
        handlers = None
    logging.basicConfig(level=level, format="%(message)s", datefmt="[%X]", handlers=handlers, force=True)
