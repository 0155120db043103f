"""Sequence-length / token-budget sweep (reference research_scratch/sequence_length_experiment.py).

At a fixed token budget the sweep starts from many short sequences and doubles the sequence
length (halving the count) until one sequence fills the budget; then the budget grows by
``--budget-increase`` and the pass repeats, until the first configuration of a pass runs out of
memory or ``--max-tokens`` is reached. Every configuration runs ``--num-iterations`` full training
steps (forward, backward, optimizer) on a uniform packed batch and records tokens/s (device-timed,
max over ranks) and peak memory. Rank 0 writes a JSON file and prints a summary table.

    torchrun --nproc-per-node 8 -m mini_trainer_b200.cli.seq_sweep --model-name-or-path random:llama-3.1-8b \
        --start-tokens 30000 --budget-increase 10000 --output-file sweep.json
"""
from __future__ import annotations

import json
import os

import typer

app = typer.Typer()


def create_uniform_batch(num_sequences: int, sequence_length: int, vocab_size: int = 32000, seed: int = 0) -> dict:
    """One padding-free minibatch of ``num_sequences`` equal-length samples (all tokens count)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    total = num_sequences * sequence_length
    ids = torch.randint(0, vocab_size, (total,), generator=g)
    labels = torch.randint(0, vocab_size, (total,), generator=g)
    pos = torch.arange(sequence_length).repeat(num_sequences)
    cu = torch.arange(0, total + 1, sequence_length, dtype=torch.int32)
    return {"input_ids": ids[None], "labels": labels[None], "position_ids": pos[None], "cu_seqlens": cu,
            "max_seqlen": sequence_length, "num_loss_counted_tokens": total, "num_samples": num_sequences,
            "batch_num_loss_counted_tokens": total}


def measure_iteration(engine, batch: dict, num_iterations: int = 5, lr: float = 1e-6) -> dict:
    import torch
    import torch.distributed as dist
    dev = engine.device
    cuda = dev.type == "cuda"
    if cuda:
        torch.cuda.reset_peak_memory_stats(dev)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    import time
    t0 = time.time()
    for _ in range(num_iterations):
        engine.train_step([batch], lr)
    if cuda:
        e1.record()
        torch.cuda.synchronize(dev)
        sec = e0.elapsed_time(e1) / 1e3
    else:
        sec = time.time() - t0
    t = torch.tensor([sec], device=dev)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    tokens = batch["input_ids"].shape[1] * num_iterations * engine.world
    return {"seconds": t.item(), "tokens_per_second": tokens / t.item(),
            "peak_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9 if cuda else 0.0}


def sweep_configs(token_budget: int, min_seq_len: int):
    """(num_sequences, sequence_length) pairs at a constant budget, doubling the length."""
    out, length = [], min_seq_len
    while length <= token_budget:
        n = max(1, token_budget // length)
        out.append((n, length))
        if n == 1:
            break
        length *= 2
    return out


@app.command()
def main(
    model_name_or_path: str = typer.Option("random:smoke-llama"),
    start_tokens: int = typer.Option(30000, help="token budget per GPU of the first pass"),
    budget_increase: int = typer.Option(10000),
    max_tokens: int = typer.Option(1_000_000),
    min_seq_len: int = typer.Option(1024),
    num_iterations: int = typer.Option(3),
    output_file: str = typer.Option("sequence_length_results.json"),
    comm_backend: str = typer.Option("auto"),
):
    import torch

    from ..trainer import setup_model
    from ..utils.dist import init_distributed_environment
    from ..utils.log import log_rank_0

    device = init_distributed_environment()
    engine = setup_model(model_name_or_path, device=device, comm_backend=comm_backend, max_tokens_per_gpu=start_tokens)
    results, budget = [], start_tokens
    while budget <= max_tokens:
        first_failed = False
        for k, (n, length) in enumerate(sweep_configs(budget, min_seq_len)):
            batch = create_uniform_batch(n, length, engine.cfg.vocab_size)
            try:
                measure_iteration(engine, batch, 1)            # warm-up
                r = measure_iteration(engine, batch, num_iterations)
                r.update(token_budget=budget, num_sequences=n, sequence_length=length, status="ok")
            except torch.OutOfMemoryError:
                engine.zero_grad()
                torch.cuda.empty_cache()
                r = dict(token_budget=budget, num_sequences=n, sequence_length=length, status="oom")
                first_failed = first_failed or k == 0
            results.append(r)
            log_rank_0(json.dumps(r))
            if r["status"] == "oom":
                break
        if first_failed:
            break
        budget += budget_increase
    if int(os.environ.get("RANK", 0)) == 0:
        with open(output_file, "w") as f:
            json.dump(results, f, indent=2)
        print(f"{'budget':>9} {'seqs':>6} {'len':>8} {'tok/s':>12} {'peak GB':>8}  status")
        for r in results:
            print(f"{r['token_budget']:>9} {r['num_sequences']:>6} {r['sequence_length']:>8} "
                  f"{r.get('tokens_per_second', 0):>12.0f} {r.get('peak_memory_gb', 0):>8.1f}  {r['status']}")
    import torch.distributed as dist
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    app()
