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


def test_nvtx_ranges_cover_the_step_phases(monkeypatch):
    """With ranges switched on, one training step opens a range per phase (and nothing when off)."""
    import torch
    from mini_trainer_b200.data.sampler import mb_collate_fn
    from mini_trainer_b200.models.config import get_preset
    from mini_trainer_b200.ops import get_ops
    from mini_trainer_b200.parallel.engine import ShardedEngine
    from mini_trainer_b200.utils import nvtx
    cfg = get_preset("tiny-qwen2")
    eng = ShardedEngine(cfg, "cpu", get_ops("cpu"), activation_budget_bytes=0)
    eng.init_random(seed=0)
    ids = torch.randint(0, cfg.vocab_size, (17,))
    mb = mb_collate_fn([{"input_ids": ids, "labels": ids, "len": 17, "num_loss_counted_tokens": 17}], 17)
    del nvtx._pushed[:]
    eng.train_step([mb], 1e-4)
    assert nvtx._pushed == []
    nvtx.enable(True)
    try:
        eng.train_step([mb], 1e-4)
    finally:
        nvtx.enable(False)
    names = list(nvtx._pushed)
    for want in ("forward/block0", "forward/block1", "head", "recompute/block1", "backward/block1", "reduce/block0", "optimizer"):
        assert want in names, (want, names)
    assert names.index("forward/block1") < names.index("head") < names.index("backward/block1") < names.index("optimizer")


def test_static_memory_plan():
    """The planning tool reproduces the decisions recorded for the benchmark configurations: a 70B model on eight 183 GiB
    GPUs needs bf16 moments and keeps a few attention outputs at 16 000 tokens; a 1.5B model keeps everything in fp32; a
    70B model on ONE GPU does not fit."""
    from mini_trainer_b200.cli.plan import memory_plan
    from mini_trainer_b200.models.config import get_preset
    big = memory_plan(get_preset("llama-3.1-70b"), 8, 16000)
    assert big["moment_dtype"] == "bf16" and big["fits"] and 100 < big["per_gpu_gb"]["optimizer_and_parameter_state"] < 130
    assert big["blocks"]["keeping_every_gemm_output"] == 0
    small = memory_plan(get_preset("qwen2.5-1.5b"), 8, 128000)
    assert small["moment_dtype"] == "fp32" and small["fits"] and small["blocks"]["keeping_attention_output"] == 28
    assert not memory_plan(get_preset("llama-3.1-70b"), 1, 16000)["fits"]
    moe = memory_plan(get_preset("mixtral-8x7b"), 8, 32000)
    assert 46 < moe["model_parameters_billion"] < 47.5 and moe["fits"]
