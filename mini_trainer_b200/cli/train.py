"""``train`` command line: the reference's twelve options with the same names and defaults
(train.py:160-178), plus opt-in extras that default to the reference's behaviour."""
from __future__ import annotations

import json
import os
from enum import Enum
from pathlib import Path
from typing import Optional

from typer import Option, Typer

app = Typer(pretty_exceptions_show_locals=False, pretty_exceptions_short=True)


class LogLevelEnum(str, Enum):
    DEBUG = "DEBUG"
    INFO = "INFO"
    WARNING = "WARNING"
    ERROR = "ERROR"
    CRITICAL = "CRITICAL"


@app.command()
def main(
    model_name_or_path: str = Option("Qwen/Qwen2.5-1.5B-Instruct", help="HF checkpoint directory, or random:<preset>"),
    data_path: str = Option("test.jsonl", help="Path to the training data JSONL file, or synthetic:<preset>[:num_samples[:longest_sample]]"),
    batch_size: int = Option(1024, help="Initial batch size before dynamic splitting"),
    max_tokens_per_gpu: int = Option(10000, help="Maximum tokens per GPU per minibatch"),
    learning_rate: float = Option(5e-6, help="Peak learning rate"),
    num_warmup_steps: int = Option(10, help="Number of warmup steps for the LR scheduler"),
    lr_scheduler: str = Option("constant_with_warmup", help="Learning rate scheduler type"),
    seed: int = Option(42, help="Random seed for reproducibility"),
    use_liger_kernels: bool = Option(False, help="Accepted for parity; the fused linear+CE kernel is always used on GPUs"),
    output_dir: str = Option(..., help="Directory to save checkpoints and logs (required)"),
    logging_level: LogLevelEnum = Option(LogLevelEnum.INFO, help="Logging level", case_sensitive=False),
    min_samples_per_checkpoint: int = Option(..., help="Minimum number of samples processed before saving a checkpoint (required)"),
    # ---- extras (not in the reference) ----
    max_steps: Optional[int] = Option(None, help="Stop after this many optimizer steps (the reference runs forever)"),
    comm_backend: str = Option("auto", help="auto | torchdist | symmetric"),
    num_workers: int = Option(0, help="DataLoader worker processes (0 = packing thread)"),
    max_grad_norm: float = Option(1.0, help="Global gradient-norm clip"),
    weight_decay: float = Option(0.0, help="AdamW weight decay"),
    adam_beta1: float = Option(0.9, help="AdamW beta1"),
    adam_beta2: float = Option(0.95, help="AdamW beta2"),
    adam_eps: float = Option(1e-8, help="AdamW epsilon"),
    max_shard_gb: float = Option(5.0, help="Largest safetensors shard of an exported checkpoint, in GB"),
    dist_timeout_minutes: float = Option(180.0, help="Process-group timeout"),
    optimizer_state_dtype: str = Option("auto", help="auto | fp32 | bf16 (AdamW moments)"),
    balance_by: str = Option("cost", help="cost | tokens: what the LPT packer balances across ranks (same global batch either way)"),
    osft: bool = Option(False, help="Orthogonal-subspace fine-tuning of the attention/MLP projections"),
    osft_rank_ratio: float = Option(0.5, help="Fraction of each projection's singular directions that is frozen"),
    engine: str = Option("auto", help="auto | native | torch: the sm_100a kernels (default on a GPU) or the plain PyTorch ops "
                                      "(the CPU oracle; on a GPU a slow cross-check of the kernels)"),
    no_dropout: bool = Option(False, help="Train a model whose config sets a dropout probability without dropout "
                                          "(dropout is not implemented; such a model is refused otherwise)"),
    save_train_state: bool = Option(False, help="With every exported checkpoint also write the sharded training state "
                                                "(fp32 master weights, AdamW moments, scheduler, data position) under "
                                                "<output-dir>/train_state/samples_<N>"),
    resume_from: Optional[str] = Option(None, help="A train_state/samples_<N> directory written by --save-train-state: "
                                                   "weights, optimizer, scheduler, counters and the data stream continue from it "
                                                   "(on the same or on another number of GPUs)"),
):
    import torch

    from ..data.sampler import get_data_loader
    from ..data.synthetic import CONFIG_DATA, synthetic_dataset
    from ..parallel.engine import OptimConfig
    from ..trainer import setup_model, setup_training_components, train
    from ..utils.dist import init_distributed_environment
    from ..utils.log import setup_logger

    device = init_distributed_environment(timeout_minutes=dist_timeout_minutes)
    output_path = Path(output_dir)
    output_path.mkdir(parents=True, exist_ok=True)
    rank = int(os.environ.get("RANK", 0))
    if rank == 0:
        params = {
            "model_name_or_path": model_name_or_path, "data_path": data_path, "batch_size": batch_size,
            "max_tokens_per_gpu": max_tokens_per_gpu, "learning_rate": learning_rate,
            "num_warmup_steps": num_warmup_steps, "lr_scheduler": lr_scheduler, "seed": seed,
            "use_liger_kernels": use_liger_kernels, "output_dir": output_dir, "logging_level": logging_level.value,
            "min_samples_per_checkpoint": min_samples_per_checkpoint, "RANK": rank,
            "WORLD_SIZE": int(os.environ.get("WORLD_SIZE", 1)),
        }
        params_path = output_path / "training_params.json"
        with open(params_path, "w") as f:
            json.dump(params, f, indent=4)
        print(f"Training with parameters: {json.dumps(params, separators=(',', ':'), indent=4)}")
        print(f"Training parameters saved to {params_path}")
    setup_logger(level=logging_level.value)
    sd = {"auto": None, "fp32": torch.float32, "bf16": torch.bfloat16}[optimizer_state_dtype]
    model = setup_model(model_name_or_path=model_name_or_path, use_liger_kernels=use_liger_kernels, device=device,
                        comm_backend=comm_backend, state_dtype=sd, seed=seed, max_tokens_per_gpu=max_tokens_per_gpu,
                        optim=OptimConfig(max_grad_norm=max_grad_norm, weight_decay=weight_decay, beta1=adam_beta1,
                                          beta2=adam_beta2, eps=adam_eps), no_dropout=no_dropout,
                        ops_kind=engine)
    if osft:
        from ..parallel.osft import enable_osft
        enable_osft(model, rank_ratio=osft_rank_ratio)
    model, optimizer, sched = setup_training_components(model, learning_rate=learning_rate,
                                                        num_warmup_steps=num_warmup_steps, lr_scheduler=lr_scheduler)
    resume_state = None
    if resume_from:
        from ..ckpt.train_state import load_train_state
        resume_state = load_train_state(model, resume_from)
        if "scheduler" in resume_state:
            sched.load_state_dict(resume_state["scheduler"])
    skip_batches = int((resume_state or {}).get("batches_consumed", 0))
    cost_len = model.cfg.attention_cost_length() if balance_by == "cost" else None
    if data_path.startswith("synthetic:"):
        parts = data_path.split(":")
        spec, vocab, _, _ = CONFIG_DATA[parts[1]]
        n = int(parts[2]) if len(parts) > 2 else 4096
        if len(parts) > 3:   # synthetic:<preset>:<num_samples>:<longest sample>
            import dataclasses
            spec = dataclasses.replace(spec, hi=int(parts[3]))
        dataset = synthetic_dataset(n, spec, min(vocab, model.cfg.vocab_size), seed=seed)
        loader = get_data_loader(dataset=dataset, batch_size=batch_size, max_tokens_per_gpu=max_tokens_per_gpu,
                                 seed=seed, pin_memory=device.type == "cuda", cost_len=cost_len, skip_batches=skip_batches)
    else:
        loader = get_data_loader(data_path=data_path, batch_size=batch_size, max_tokens_per_gpu=max_tokens_per_gpu,
                                 seed=seed, num_workers=num_workers, pin_memory=device.type == "cuda", cost_len=cost_len,
                                 skip_batches=skip_batches)
    ds = getattr(loader, "dataset", None)
    if ds is not None and hasattr(ds, "lengths") and len(ds):
        win = model.cfg.attention_window
        if win is not None and int(ds.lengths.max()) > win:   # refused here, before any rank has started a step
            raise ValueError(f"the longest sample has {int(ds.lengths.max())} tokens but the model attends through a sliding "
                             f"window of {win}; only full causal attention is implemented, which is the same function up to "
                             "that length. Filter the data (process_data --max-sample-num-tokens) or use a model without a window")
        model.reserve_host_offload(max(max_tokens_per_gpu, int(ds.lengths.max())))
    train(model, optimizer, sched, loader, output_dir, min_samples_per_checkpoint, model_name_or_path,
          max_steps=max_steps, max_shard_bytes=int(max_shard_gb * 1e9), save_train_state=save_train_state,
          resume_state=resume_state)
    # Leave together: a rank that exits while a peer is still inside its last collective (or tearing down its
    # connections) makes that peer abort, and the launcher then reports a finished run as failed.
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        if device.type == "cuda":
            import torch
            torch.cuda.synchronize(device)
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    app()
