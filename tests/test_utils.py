import json

import torch

from mini_trainer_b200.utils.async_logger import AsyncStructuredLogger
from mini_trainer_b200.utils.lr import LRSchedule, lr_factor
from mini_trainer_b200.utils.metrics import BatchMetrics


def test_batch_metrics_sum_and_reset():
    bm = BatchMetrics()
    bm.accumulate_minibatch_metrics(a=1.0, b=2)
    bm.accumulate_minibatch_metrics(a=0.5, b=3)
    bm.reduce_batch_metrics("cpu")
    assert bm.totals == {"a": 1.5, "b": 5.0}
    assert not bm.minibatch_metrics
    bm.reset_batch()
    assert not bm.totals


def test_logger_appends_jsonl_and_reloads(tmp_path):
    p = str(tmp_path / "m.jsonl")
    lg = AsyncStructuredLogger(p, echo=False)
    lg.log_sync({"step": 1, "loss": 2.5})
    lg.log_sync({"step": 2, "loss": 2.0})
    lg.close()
    rows = [json.loads(l) for l in open(p)]
    assert [r["step"] for r in rows] == [1, 2] and all("timestamp" in r for r in rows)
    lg2 = AsyncStructuredLogger(p, echo=False)
    assert len(lg2.logs) == 2
    lg2.log_sync({"step": 3})
    lg2.close()
    assert len(open(p).readlines()) == 3


def test_lr_schedule_matches_transformers_primed():
    from transformers import get_scheduler
    for name in ("constant", "constant_with_warmup", "inverse_sqrt"):
        p = torch.nn.Parameter(torch.zeros(1))
        opt = torch.optim.AdamW([p], lr=3e-4)
        hf = get_scheduler(name=name, optimizer=opt, num_warmup_steps=4)
        hf.step()
        mine = LRSchedule(3e-4, name, 4)
        for _ in range(12):
            assert abs(hf.get_last_lr()[0] - mine.current()) < 1e-12
            opt.step(); hf.step(); mine.step()
    s = LRSchedule(1.0, "constant_with_warmup", 10)
    assert abs(s.current() - 0.1) < 1e-12  # first update never runs at zero
    assert lr_factor("constant_with_warmup", 20, 10) == 1.0
