"""Learning-rate schedules that need no total step count.

The reference builds ``transformers.get_scheduler(name, optimizer, num_warmup_steps)`` without
``num_training_steps`` and then calls ``step()`` once so that the first update does not run at
zero learning rate (setup_model_for_training.py:145-151). Net effect, reproduced here in closed
form: optimizer step ``n`` (1-based) uses ``lr * factor(n)``, and the value logged after step
``n`` is the one step ``n + 1`` will use.

    constant               factor = 1
    constant_with_warmup   factor = min(1, n / W)
    inverse_sqrt           factor = n / W during warm-up, then sqrt(W' / (n + shift))
                           with W' = max(W, 1) timescale and shift = W' - W (HF definition)
"""
from __future__ import annotations

import math

SCHEDULES = ("constant", "constant_with_warmup", "inverse_sqrt")


def lr_factor(name: str, step: int, num_warmup_steps: int) -> float:
    """Multiplier applied at 0-based scheduler step ``step`` (HF ``LambdaLR`` convention)."""
    w = int(num_warmup_steps)
    if name == "constant":
        return 1.0
    if name == "constant_with_warmup":
        return float(step) / float(max(1, w)) if step < w else 1.0
    if name == "inverse_sqrt":
        if step < w:
            return float(step) / float(max(1, w))
        timescale = w or 10_000
        shift = timescale - w
        return 1.0 / math.sqrt((step + shift) / timescale)
    raise ValueError(f"scheduler {name!r} needs a total step count or is unknown; choose one of {SCHEDULES}")


class LRSchedule:
    """Primed schedule: ``current()`` is the rate of the NEXT optimizer step."""

    def __init__(self, base_lr: float, name: str = "constant_with_warmup", num_warmup_steps: int = 10):
        lr_factor(name, 0, num_warmup_steps)  # validates the name early
        self.base_lr, self.name, self.num_warmup_steps = float(base_lr), name, int(num_warmup_steps)
        self._step = 1  # the priming step

    def current(self) -> float:
        return self.base_lr * lr_factor(self.name, self._step, self.num_warmup_steps)

    def step(self) -> None:
        self._step += 1

    def get_last_lr(self):
        return [self.current()]

    def state_dict(self) -> dict:
        return {"step": self._step}

    def load_state_dict(self, sd: dict) -> None:
        self._step = int(sd["step"])
