"""Two gloo ranks on CPU: the sharded engine must reproduce the single-process run.

This is the tiny Qwen2 configuration (2 layers, hidden 256, 4/2 heads, FFN 688, vocab 32000, tied
embeddings, fp32, lognormal lengths, LPT packing to 4096 tokens per rank, batch 32, AdamW 1e-4,
seed 893) followed by a bf16 safetensors save / load round trip.
"""
import json
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mini_trainer_b200.ckpt.hf_checkpoint import load_hf_checkpoint
from mini_trainer_b200.data.sampler import get_data_loader
from mini_trainer_b200.data.synthetic import CONFIG_DATA, synthetic_dataset
from mini_trainer_b200.models.config import ModelConfig, get_preset
from mini_trainer_b200.ops import get_ops
from mini_trainer_b200.parallel.comm import make_comm
from mini_trainer_b200.parallel.engine import OptimConfig, ShardedEngine
from mini_trainer_b200.trainer import setup_training_components, train

STEPS = int(os.environ.get("MTB200_TINY_STEPS", "2"))


def free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def run_training(rank, world, port, out_dir, steps, preset="tiny-qwen2"):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    spec, vocab, max_tokens, batch_size = CONFIG_DATA["tiny-qwen2"]
    cfg = get_preset(preset)
    ds = synthetic_dataset(512, spec, min(vocab, cfg.vocab_size), seed=893)
    eng = ShardedEngine(cfg, "cpu", get_ops("cpu"), comm=make_comm("auto"), optim=OptimConfig())
    eng.init_random(seed=893)
    model, opt, sched = setup_training_components(eng, learning_rate=1e-4, num_warmup_steps=2)
    loader = get_data_loader(dataset=ds, batch_size=batch_size, max_tokens_per_gpu=max_tokens, seed=893,
                             rank=rank, world_size=world, prefetch=0)
    train(model, opt, sched, loader, out_dir, min_samples_per_checkpoint=batch_size * steps, max_steps=steps,
          log_echo=False)
    if world > 1:
        dist.destroy_process_group()


def _spawn_entry(rank, world, port, out_dir, steps, preset="tiny-qwen2"):
    run_training(rank, world, port, out_dir, steps, preset)


@pytest.mark.timeout(900)
def test_two_ranks_match_one_rank_and_checkpoint_roundtrip(tmp_path):
    one, two = str(tmp_path / "w1"), str(tmp_path / "w2")
    os.makedirs(one); os.makedirs(two)
    run_training(0, 1, free_port(), one, STEPS)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    mp.spawn(_spawn_entry, args=(2, free_port(), two, STEPS), nprocs=2, join=True)

    r1 = [json.loads(l) for l in open(os.path.join(one, "training_metrics_0.jsonl"))]
    r2 = [json.loads(l) for l in open(os.path.join(two, "training_metrics_0.jsonl"))]
    assert len(r1) == len(r2) == STEPS
    for a, b in zip(r1, r2):
        assert abs(a["loss"] - b["loss"]) < 2e-4 * abs(a["loss"]), (a["loss"], b["loss"])
        assert abs(a["grad_norm"] - b["grad_norm"]) < 2e-3 * a["grad_norm"]
        assert a["num_samples"] == b["num_samples"] == 32
        assert a["num_loss_counted_tokens"] == b["num_loss_counted_tokens"]
        assert a["lr"] == b["lr"]
    assert r1[-1]["loss"] < r1[0]["loss"] + 0.5
    assert set(r1[0]) >= {"step", "lr", "grad_norm", "loss", "avg_loss_backward", "num_samples",
                          "num_loss_counted_tokens", "batch_num_loss_counted_tokens", "num_total_tokens",
                          "grad_accum", "avg_time_per_minibatch", "time_per_batch", "tokens_per_second",
                          "total_samples_accumulated", "samples_per_second", "peak_memory_usage_GB", "timestamp"}

    # export written by both runs; weights agree within bf16 rounding of nearly equal fp32 values
    n = float(32 * STEPS)
    d1 = os.path.join(one, "hf_format", f"samples_{n}")
    d2 = os.path.join(two, "hf_format", f"samples_{n}")
    assert os.path.exists(os.path.join(d1, "model.safetensors")) and os.path.exists(os.path.join(d2, "config.json"))
    e1 = ShardedEngine(ModelConfig.from_pretrained(d1), "cpu", get_ops("cpu")); load_hf_checkpoint(e1, d1)
    e2 = ShardedEngine(ModelConfig.from_pretrained(d2), "cpu", get_ops("cpu")); load_hf_checkpoint(e2, d2)
    for a, b in zip(e1.groups, e2.groups):
        assert torch.allclose(a.master, b.master, atol=1e-2, rtol=2e-2)
    assert e1.cfg.tie_word_embeddings and e1.cfg.vocab_size == 32000


@pytest.mark.timeout(900)
def test_three_ranks_match_one_rank(tmp_path):
    """An odd world size: group sizes do not divide evenly, so the shard padding and an idle rank's dummy
    minibatches are exercised; one step is enough."""
    one, three = str(tmp_path / "w1"), str(tmp_path / "w3")
    os.makedirs(one); os.makedirs(three)
    run_training(0, 1, free_port(), one, 1)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    mp.spawn(_spawn_entry, args=(3, free_port(), three, 1), nprocs=3, join=True)
    a = json.loads(open(os.path.join(one, "training_metrics_0.jsonl")).readline())
    b = json.loads(open(os.path.join(three, "training_metrics_0.jsonl")).readline())
    assert abs(a["loss"] - b["loss"]) < 2e-4 * abs(a["loss"]), (a["loss"], b["loss"])
    assert abs(a["grad_norm"] - b["grad_norm"]) < 2e-3 * a["grad_norm"]
    assert a["num_loss_counted_tokens"] == b["num_loss_counted_tokens"] and b["num_samples"] == 32


@pytest.mark.timeout(900)
def test_two_ranks_match_one_rank_mixture_of_experts(tmp_path):
    """A small Mixtral (4 experts, 2 per token): expert and router parameters are sharded, gathered and reduced like any
    other tensor of the block's flat buffer, and the export carries the published checkpoint names."""
    one, two = str(tmp_path / "w1"), str(tmp_path / "w2")
    os.makedirs(one); os.makedirs(two)
    run_training(0, 1, free_port(), one, 2, "tiny-mixtral")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    mp.spawn(_spawn_entry, args=(2, free_port(), two, 2, "tiny-mixtral"), nprocs=2, join=True)
    r1 = [json.loads(l) for l in open(os.path.join(one, "training_metrics_0.jsonl"))]
    r2 = [json.loads(l) for l in open(os.path.join(two, "training_metrics_0.jsonl"))]
    for a, b in zip(r1, r2):
        assert abs(a["loss"] - b["loss"]) < 2e-4 * abs(a["loss"]), (a["loss"], b["loss"])
        assert abs(a["grad_norm"] - b["grad_norm"]) < 2e-3 * a["grad_norm"]
    d2 = os.path.join(two, "hf_format", "samples_64.0")
    from mini_trainer_b200.ckpt import safetensors_io as st
    names = set(st.load_file(os.path.join(d2, "model.safetensors")))
    assert {"model.layers.1.block_sparse_moe.gate.weight", "model.layers.0.block_sparse_moe.experts.3.w2.weight"} <= names
    cfg = ModelConfig.from_pretrained(d2)
    assert cfg.is_moe and cfg.num_local_experts == 4 and cfg.architectures == ["MixtralForCausalLM"]
