"""Process-group bootstrap (reference utils.py:48-53).

One process per GPU, launched by ``torchrun``: ``LOCAL_RANK`` selects the device, the NCCL group
is created with a long timeout and warmed up with a 1-byte all-reduce and a barrier. Without a
GPU the same call creates a ``gloo`` group, which is what the CPU tests use. A single process
started without torchrun gets a group of size one so the rest of the code has one code path.
"""
from __future__ import annotations

import os
from datetime import timedelta

import torch
import torch.distributed as dist


def init_distributed_environment(backend: str | None = None, timeout_minutes: float = 180.0) -> torch.device:
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    if use_cuda:
        # Training targets ~90 % of device memory with a different token count and a different mix of
        # kept activations every minibatch; fixed-size allocator segments fragment under that pattern.
        # Expandable segments grow and shrink in place. An explicit PYTORCH_CUDA_ALLOC_CONF wins.
        if "PYTORCH_CUDA_ALLOC_CONF" not in os.environ:
            try:
                torch.cuda.memory._set_allocator_settings("expandable_segments:True")
            except Exception:
                pass
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        device = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    else:
        device = torch.device("cpu")
    if not dist.is_initialized():
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = device
        dist.init_process_group(backend, timeout=timedelta(minutes=timeout_minutes), **kwargs)
    flag = torch.zeros(1, dtype=torch.uint8, device=device)
    dist.all_reduce(flag)
    dist.barrier()
    return device


def world_info() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
