"""NVTX ranges around the phases of a training step and around every kernel family.

Off by default (a range push/pop per kernel launch is measurable on a launch-bound model); set
``MTB200_NVTX=1`` to emit them. A timeline tool attached to the process then shows
``forward/block12``, ``backward/block12``, ``reduce/block12``, ``head``, ``optimizer`` and, nested
inside, one range per native op (``gemm_nt``, ``mtb200_attn_fwd`` ...). The reference has no such
ranges of its own; FSDP2 emits ``record_function("FSDP::...")`` scopes
(torch/distributed/fsdp/_fully_shard/_fsdp_param_group.py:338-533), which these replace.
"""
from __future__ import annotations

import contextlib
import os

ENABLED = os.environ.get("MTB200_NVTX", "0") == "1"
_pushed = []   # names pushed through this module (inspected by tests; NVTX itself cannot be read back)


def enable(on: bool = True) -> None:
    global ENABLED
    ENABLED = bool(on)


def push(name: str) -> None:
    if not ENABLED:
        return
    _pushed.append(name)
    try:
        import torch
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)
    except Exception:
        pass


def pop() -> None:
    if not ENABLED:
        return
    try:
        import torch
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
    except Exception:
        pass


@contextlib.contextmanager
def range(name: str):   # noqa: A001  (mirrors torch.cuda.nvtx.range)
    if not ENABLED:
        yield
        return
    push(name)
    try:
        yield
    finally:
        pop()
