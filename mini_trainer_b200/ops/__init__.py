"""Op backends. ``get_ops(device)`` returns the sm_100a kernel backend on CUDA devices and the
PyTorch reference backend on CPU. On a CUDA device a missing native library is an error, never a
silent fallback."""
from __future__ import annotations

import torch

from .torch_ref import TorchOps


def get_ops(device, kind: str = "auto"):
    device = torch.device(device)
    if kind == "torch" or (kind == "auto" and device.type != "cuda"):
        return TorchOps()
    from .native import NativeOps
    return NativeOps(device)
