"""Per-step metric accumulation with a single cross-rank reduction.

Same contract as the reference ``BatchMetrics`` (batch_metrics.py:4-35): minibatch values are
summed locally under arbitrary keys; ``reduce_batch_metrics`` packs them into one fp32 vector
in key order, sums it across ranks with ONE all-reduce and publishes ``totals``.
"""
from __future__ import annotations

from collections import defaultdict

import torch
import torch.distributed as dist


class BatchMetrics:
    def __init__(self):
        self.totals = defaultdict(float)
        self.minibatch_metrics = defaultdict(float)

    def accumulate_minibatch_metrics(self, **kwargs) -> None:
        for key, value in kwargs.items():
            self.minibatch_metrics[key] += value

    def reduce_batch_metrics(self, device) -> None:
        keys = list(self.minibatch_metrics.keys())
        vec = torch.tensor([float(self.minibatch_metrics[k]) for k in keys], dtype=torch.float32, device=device)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(vec, op=dist.ReduceOp.SUM)
        self.totals = dict(zip(keys, vec.tolist()))
        self.minibatch_metrics.clear()

    def reset_batch(self) -> None:
        self.totals.clear()
        self.minibatch_metrics.clear()
