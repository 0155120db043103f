"""Model setup, the training loop and checkpoint cadence.

Public API, named after the reference's functions so that scripts written against it port over:

* ``setup_model(model_name_or_path, ...)``            (setup_model_for_training.py:86-130)
* ``setup_training_components(model, ...)``           (setup_model_for_training.py:132-152)
* ``take_gradient_step(model, optimizer, scheduler)`` (train.py:22-28)
* ``save_model(...)``                                 (train.py:30-70, in ``ckpt.hf_checkpoint``)
* ``train(model, optimizer, scheduler, loader, ...)`` (train.py:72-151)

``model`` here is a ``ShardedEngine``; it is its own optimizer (``optimizer`` is the same object,
kept as a separate return value for signature parity).

Loop semantics kept: every minibatch of the rank's list is one gradient-accumulation pass; the
loss is the sum of token losses divided by the loss-token count of the WHOLE global batch;
metrics are summed over ranks with one all-reduce per step; rank 0 appends one JSONL record per
step with the reference's sixteen keys; a checkpoint is written whenever at least
``min_samples_per_checkpoint`` samples were consumed since the last one.

Loop semantics changed on purpose: no ``.item()`` per minibatch, no ``empty_cache()`` per
minibatch and no per-step barrier — the device queue is only drained once per step, when rank 0
reads the loss and the gradient norm for logging. ``max_steps`` (absent in the reference, whose
loop never ends) bounds the run for benchmarks and tests.
"""
from __future__ import annotations

import math
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from .ckpt.hf_checkpoint import load_hf_checkpoint, save_model
from .models import decoder as D
from .models.config import ModelConfig, get_preset, PRESETS
from .ops import get_ops
from .parallel.comm import make_comm
from .parallel.engine import OptimConfig, ShardedEngine, plan_state_dtype
from .utils.async_logger import AsyncStructuredLogger
from .utils.log import log_rank_0
from .utils.lr import LRSchedule
from .utils.metrics import BatchMetrics

from .models.config import SUPPORTED_ARCHITECTURES  # noqa: E402  (re-exported)


def align_model_and_tokenizer(cfg: ModelConfig, tokenizer) -> ModelConfig:
    """Vocabulary / special-token alignment (reference setup_model_for_training.py:50-84).

    A tokenizer larger than the embedding grows the vocabulary to the next multiple of 8; pad,
    bos and eos ids of the config are set to the tokenizer's when both exist and differ.
    """
    if len(tokenizer) > cfg.vocab_size:
        print(f"WARNING: tokenizer has {len(tokenizer)} tokens but model has {cfg.vocab_size} vocab size")
        cfg.vocab_size = int(8 * math.ceil(len(tokenizer) / 8.0))
    for kind in ("pad", "bos", "eos"):
        attr = f"{kind}_token_id"
        mt, tt = getattr(cfg, attr), getattr(tokenizer, attr, None)
        if mt is not None and tt is not None and mt != tt:
            log_rank_0(f"\033[38;5;226mWARNING: There is a mismatch between {kind} token id of model({mt}) and "
                       f"tokenizer({tt}). Fixing model {kind} token id to be same as tokenizer's {kind} token id\033[0m")
            setattr(cfg, attr, tt)
    return cfg


def resolve_model_path(model_name_or_path: str) -> str:
    """A local directory is returned as is; anything else is taken for a hub id (the reference's
    default is ``Qwen/Qwen2.5-1.5B-Instruct``, train.py:162) and resolved to its snapshot directory
    in the local Hugging Face cache. There is no download here: a model that is not cached is an error."""
    if os.path.isdir(model_name_or_path):
        return model_name_or_path
    try:
        from huggingface_hub import snapshot_download
        return snapshot_download(model_name_or_path, local_files_only=True)
    except Exception as e:
        raise FileNotFoundError(f"{model_name_or_path!r} is neither a directory nor a model in the local Hugging Face "
                                f"cache ({type(e).__name__}); download it first or pass a checkpoint directory") from e


def setup_model(model_name_or_path: str, use_liger_kernels: bool = True, device=None, comm_backend: str = "auto",
                state_dtype: Optional[torch.dtype] = None, seed: int = 0, max_tokens_per_gpu: int = 65536,
                ops_kind: str = "auto", optim: Optional[OptimConfig] = None, no_dropout: bool = False) -> ShardedEngine:
    """Builds the sharded model.

    ``model_name_or_path`` is an HF checkpoint directory (``config.json`` + safetensors), or
    ``random:<preset>`` / ``random:<config.json path>`` for a random-initialised architecture.
    ``use_liger_kernels`` is accepted for CLI parity: the fused linear + cross-entropy is always
    used on GPUs (the unfused logits path exists only as the CPU oracle). ``no_dropout`` accepts a model whose
    config sets a dropout probability and trains it without (the exported config keeps the model's own values).
    """
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    device = torch.device(device)
    random_init = model_name_or_path.startswith("random:")
    if random_init:
        spec = model_name_or_path.split(":", 1)[1]
        cfg = get_preset(spec) if spec in PRESETS else ModelConfig.from_pretrained(os.path.dirname(spec) if spec.endswith(".json") else spec)
    else:
        model_name_or_path = resolve_model_path(model_name_or_path)
        cfg = ModelConfig.from_pretrained(model_name_or_path)
        try:
            from transformers import AutoTokenizer
            cfg = align_model_and_tokenizer(cfg, AutoTokenizer.from_pretrained(model_name_or_path))
        except Exception as e:  # a weights-only directory is fine
            log_rank_0(f"tokenizer not loaded ({type(e).__name__}); skipping vocabulary alignment")
    # The reference only warns about unknown classes because AutoModelForCausalLM brings each model's
    # own forward (setup_model_for_training.py:111-123). The forward and backward here are written
    # for one block structure, so a model whose math differs is refused, not trained wrongly.
    cfg.ignore_dropout = bool(no_dropout)
    cfg.validate_supported()
    if no_dropout:
        set_ = {k: v for k, v in cfg.extra.items() if "drop" in k and v}
        if set_:
            log_rank_0(f"\033[38;5;226mWARNING: training without the model's dropout {set_}\033[0m")
    comm = make_comm(comm_backend, device)
    if state_dtype is None:
        hbm = torch.cuda.get_device_properties(device).total_memory if device.type == "cuda" else 1e15
        state_dtype = plan_state_dtype(cfg, comm.world, hbm, max_tokens_per_gpu)
    engine = ShardedEngine(cfg, device, get_ops(device, ops_kind), comm=comm, state_dtype=state_dtype, optim=optim)
    if random_init:
        engine.init_random(seed=seed, on_device=device.type == "cuda")
    else:
        load_hf_checkpoint(engine, model_name_or_path)
    return engine


def setup_training_components(model: ShardedEngine, learning_rate: float = 5e-6, num_warmup_steps: int = 10,
                              lr_scheduler: str = "constant_with_warmup"):
    """Returns ``(model, optimizer, lr_scheduler)``; AdamW(0.9, 0.95), no weight decay."""
    model.optim.lr = learning_rate
    sched = LRSchedule(learning_rate, lr_scheduler, num_warmup_steps)
    return model, model, sched


def take_gradient_step(model: ShardedEngine, optimizer, lr_scheduler: LRSchedule) -> torch.Tensor:
    """Clip to global norm 1.0, AdamW step, scheduler step, clear gradients; returns the norm."""
    grad_norm = model.optimizer_step(lr_scheduler.current())
    lr_scheduler.step()
    return grad_norm


def train(model: ShardedEngine, optimizer, lr_scheduler: LRSchedule, data_loader, output_dir: str,
          min_samples_per_checkpoint: int, model_name_or_path: Optional[str] = None,
          max_steps: Optional[int] = None, log_echo: bool = True,
          max_shard_bytes: Optional[int] = None, save_train_state: bool = False,
          resume_state: Optional[dict] = None) -> dict:
    """The training loop. ``save_train_state`` also writes a sharded training-state checkpoint
    (``<output_dir>/train_state/samples_<N>``) with every export; ``resume_state`` is the metadata
    ``load_train_state`` returned for such a directory: step, sample counters and checkpoint cadence
    continue from it (the caller builds ``data_loader`` with ``skip_batches=resume_state["batches_consumed"]``).
    ``max_steps`` counts optimizer steps of the whole run, resumed ones included."""
    rank = int(os.environ.get("RANK", 0))
    world_size = model.world
    is_main = rank == 0
    metric_logger = AsyncStructuredLogger(os.path.join(output_dir, f"training_metrics_{rank}.jsonl"), echo=log_echo)
    batch_totals = BatchMetrics()
    device = model.device
    rs = resume_state or {}
    step = int(rs.get("train_step", 0))
    total_samples_accumulated = float(rs.get("total_samples_accumulated", 0.0))
    last_saved_samples = float(rs.get("last_saved_samples", 0.0))
    batches_consumed = int(rs.get("batches_consumed", 0))
    last = {}
    if max_steps is not None and step >= max_steps:
        metric_logger.close()
        return last
    batches = iter(data_loader)
    for batch in batches:
        batch_start = time.time()
        batch_totals.reset_batch()
        if device.type == "cuda":
            torch.cuda.reset_peak_memory_stats(device)
        loss_sum = torch.zeros((), dtype=torch.float32, device=device)
        grad_accum = 0
        batch_num_loss_counted_tokens = 1
        for grad_accum, mb in enumerate(batch):
            mb_start = time.time()
            batch_num_loss_counted_tokens = mb["batch_num_loss_counted_tokens"]
            pb = D.make_packed_batch(mb, device)
            scale = 1.0 / max(1, batch_num_loss_counted_tokens)
            loss = model.forward_backward(pb, scale, last=grad_accum == len(batch) - 1)
            loss_sum += loss.sum()
            batch_totals.accumulate_minibatch_metrics(
                num_loss_counted_tokens=mb["num_loss_counted_tokens"],
                num_total_tokens=pb.num_tokens,
                num_samples=mb["num_samples"],
                time_per_minibatch=time.time() - mb_start,
            )
        step += 1
        batches_consumed += 1
        grad_norm = take_gradient_step(model, optimizer, lr_scheduler)
        # the single device->host read of the step
        local_loss = float(loss_sum.item())
        batch_totals.accumulate_minibatch_metrics(loss=local_loss,
                                                  loss_backward=local_loss / max(1, batch_num_loss_counted_tokens))
        batch_totals.reduce_batch_metrics(device)
        bm = batch_totals.totals
        total_samples_accumulated += bm["num_samples"]
        if is_main:
            batch_time = time.time() - batch_start
            last = {
                "step": step,
                "lr": lr_scheduler.get_last_lr()[0],
                "grad_norm": float(grad_norm.item()),
                "loss": bm["loss"] / batch_num_loss_counted_tokens,
                "avg_loss_backward": bm["loss_backward"] / (grad_accum + 1),
                "num_samples": bm["num_samples"],
                "num_loss_counted_tokens": bm["num_loss_counted_tokens"],
                "batch_num_loss_counted_tokens": batch_num_loss_counted_tokens,
                "num_total_tokens": bm["num_total_tokens"],
                "grad_accum": grad_accum + 1,
                "avg_time_per_minibatch": bm["time_per_minibatch"] / (grad_accum + 1) / world_size,
                "time_per_batch": batch_time,
                "tokens_per_second": bm["num_total_tokens"] / batch_time,
                "total_samples_accumulated": total_samples_accumulated,
                "samples_per_second": bm["num_samples"] / batch_time,
                "peak_memory_usage_GB": float(torch.cuda.max_memory_allocated(device) / 1e9) if device.type == "cuda" else 0.0,
            }
            metric_logger.log_sync(dict(last))
        if total_samples_accumulated - last_saved_samples >= min_samples_per_checkpoint:
            save_model(model, total_samples_accumulated, output_dir, model_name_or_path,
                       **({} if max_shard_bytes is None else {"max_shard_bytes": max_shard_bytes}))
            last_saved_samples = total_samples_accumulated
            if save_train_state:
                from .ckpt.train_state import save_train_state as _save_state
                _save_state(model, os.path.join(output_dir, "train_state", f"samples_{total_samples_accumulated}"),
                            extra={"scheduler": lr_scheduler.state_dict(), "train_step": step,
                                   "batches_consumed": batches_consumed,
                                   "total_samples_accumulated": total_samples_accumulated,
                                   "last_saved_samples": last_saved_samples})
        if max_steps is not None and step >= max_steps:
            break
    if hasattr(batches, "close"):   # stops and joins the packing thread: it must not be mid-batch when the process exits
        batches.close()
    metric_logger.close()
    return last
