"""Sharding smoke run over the plain-collectives backend.

Counterpart of the reference's research smoke script (research_scratch/fsdp1_dummy_script.py:79-180,
wrapper in research_scratch/fsdp1_wrapper.py:17-73): build the model, shard it with the backend
that uses library collectives only (``torchdist``: NCCL on GPUs, gloo on CPUs — the role FSDP1
plays next to FSDP2 in the reference), run a few forward / backward / optimizer steps on a dummy
uniform batch and report loss, gradient norm and peak memory. ``--comm-backend symmetric`` runs
the same steps over the in-kernel NVLink backend, so the two sharding paths can be compared.

    torchrun --nnodes=1 --nproc-per-node=8 -m mini_trainer_b200.cli.smoke_run --model-name-or-path random:llama-3.1-8b
"""
from __future__ import annotations

import json

import typer

app = typer.Typer()


@app.command()
def main(
    model_name_or_path: str = typer.Option("random:tiny-qwen2", help="HF checkpoint directory, or random:<preset>"),
    comm_backend: str = typer.Option("torchdist", help="torchdist | symmetric | auto"),
    num_sequences: int = typer.Option(4, help="Samples in the dummy minibatch"),
    sequence_length: int = typer.Option(128, help="Tokens per sample"),
    num_steps: int = typer.Option(2, help="Optimizer steps to run"),
    learning_rate: float = typer.Option(1e-5),
    seed: int = typer.Option(0),
):
    import torch
    import torch.distributed as dist

    from ..trainer import setup_model
    from ..utils.dist import init_distributed_environment
    from ..utils.log import log_rank_0
    from .seq_sweep import create_uniform_batch

    device = init_distributed_environment()
    world = dist.get_world_size()
    log_rank_0(f"sharding {model_name_or_path} over {world} rank(s), backend {comm_backend}")
    engine = setup_model(model_name_or_path=model_name_or_path, device=device, comm_backend=comm_backend, seed=seed,
                         max_tokens_per_gpu=num_sequences * sequence_length)
    batch = create_uniform_batch(num_sequences, sequence_length, engine.cfg.vocab_size, seed=seed + dist.get_rank())
    denom = float(batch["batch_num_loss_counted_tokens"] * world)
    batch["batch_num_loss_counted_tokens"] = denom
    records = []
    for step in range(num_steps):
        if device.type == "cuda":
            torch.cuda.reset_peak_memory_stats(device)
        out = engine.train_step([batch], learning_rate)
        stats = torch.stack([out["loss_sum"].float(), out["grad_norm"].float().reshape(())])
        loss_sum = stats[:1].clone()
        if world > 1:
            dist.all_reduce(loss_sum)
        peak = torch.cuda.max_memory_allocated(device) / 1e9 if device.type == "cuda" else 0.0
        rec = {"step": step + 1, "loss": float(loss_sum) / denom, "grad_norm": float(stats[1]), "peak_memory_GB": round(peak, 3)}
        if not all(map(lambda v: v == v and abs(v) != float("inf"), (rec["loss"], rec["grad_norm"]))):
            raise RuntimeError(f"non-finite result in smoke run: {rec}")
        records.append(rec)
        log_rank_0(json.dumps(rec))
    log_rank_0("smoke run ok")
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return records


if __name__ == "__main__":
    app()
