"""Static memory plan of a training run, printed before any GPU is touched.

``python -m mini_trainer_b200.cli.plan --model llama-3.1-70b --gpus 8 --max-tokens-per-gpu 16000``
answers the questions the reference leaves to trial and error (its README only says "up to 70B on
one node"): how many bytes of parameters, master weights, moments and gradient accumulators a rank
holds, which moment precision ``--optimizer-state-dtype auto`` will pick, how large the gathered
block buffers are, what a minibatch of the given token budget costs per checkpoint level, and how
many blocks can keep their activations. It uses the same formulas as the engine
(``parallel.engine.plan_state_dtype``, ``ShardedEngine.plan_checkpointing``); nothing is allocated.
"""
from __future__ import annotations

import json
import os

import typer

app = typer.Typer(add_completion=False)


def memory_plan(cfg, gpus: int, max_tokens_per_gpu: int, hbm_gb: float = 183.0, state_dtype: str = "auto") -> dict:
    import torch

    from ..models import layout as L
    from ..parallel.engine import plan_state_dtype
    hbm = hbm_gb * 2 ** 30
    if state_dtype == "auto":
        moments = plan_state_dtype(cfg, gpus, hbm, max_tokens_per_gpu)
    else:
        moments = {"fp32": torch.float32, "bf16": torch.bfloat16}[state_dtype]
    mb = 4 if moments == torch.float32 else 2
    layouts = ([L.GroupLayout("embed", L.embed_entries(cfg), gpus)]
               + [L.GroupLayout(f"block{i}", L.block_entries(cfg), gpus) for i in range(cfg.num_hidden_layers)]
               + [L.GroupLayout("head", L.head_entries(cfg), gpus)])
    shard = sum(l.shard_numel for l in layouts)
    block = layouts[1].padded_numel
    state = shard * (2 + 4 + 4 + 2 * mb)          # working copy, master, gradient accumulator, two moments
    buffers = (2 * block * 2 * (gpus > 1)         # two gathered-parameter buffers
               + 2 * block * 2                    # two block gradient buffers
               + (layouts[0].padded_numel + layouts[-1].padded_numel) * 2 * 2)   # embed / head: gathered and gradient
    t, h, es = max_tokens_per_gpu, cfg.hidden_size, 2
    f = (cfg.expert_intermediate_size if cfg.is_moe else cfg.intermediate_size) * cfg.mlp_rows_factor
    inputs = t * h * es * cfg.num_hidden_layers
    lvl1 = t * (cfg.q_size * es + cfg.num_attention_heads * 4)
    lvl0 = lvl1 + t * ((h + cfg.qkv_size + 2 * f) * es + 8)
    work = t * es * (7 * h + cfg.qkv_size + 6 * f)
    ce = 8192 * cfg.vocab_size * 2 + cfg.vocab_size * h * 4
    free = 0.93 * hbm - state - buffers - inputs - work - ce - 4 * 2 ** 30
    keep_attn = max(0, min(cfg.num_hidden_layers, int(free // lvl1))) if free > 0 else 0
    keep_all = max(0, min(keep_attn, int((free - keep_attn * lvl1) // max(1, lvl0 - lvl1)))) if free > 0 else 0
    gb = lambda x: round(x / 2 ** 30, 2)
    return {
        "model_parameters_billion": round(cfg.param_count() / 1e9, 3),
        "gpus": gpus, "max_tokens_per_gpu": t, "hbm_gb_per_gpu": hbm_gb,
        "moment_dtype": "fp32" if moments == torch.float32 else "bf16",
        "per_gpu_gb": {"optimizer_and_parameter_state": gb(state), "gather_and_gradient_buffers": gb(buffers),
                       "block_inputs_of_one_minibatch": gb(inputs), "working_set_of_one_block": gb(work),
                       "linear_ce_workspace": gb(ce), "left_for_kept_activations": gb(max(free, 0.0))},
        "per_block_gb": {"keep_attention_output": gb(lvl1), "keep_every_gemm_output": gb(lvl0)},
        "blocks": {"total": cfg.num_hidden_layers, "keeping_attention_output": keep_attn, "keeping_every_gemm_output": keep_all,
                   "inputs_parked_in_host_memory": 0 if free > 0 else int(-free // max(1, t * h * es)) + 1},
        "fits": bool(free > 0 or cfg.num_hidden_layers * t * h * es > -free),
    }


@app.command()
def main(
    model: str = typer.Option(..., help="A preset (e.g. llama-3.1-70b), a checkpoint directory or a config.json"),
    gpus: int = typer.Option(8, help="GPUs of the node"),
    max_tokens_per_gpu: int = typer.Option(16000, help="Token budget of a minibatch on one GPU"),
    hbm_gb: float = typer.Option(183.0, help="Device memory per GPU in GiB (B200: 183)"),
    optimizer_state_dtype: str = typer.Option("auto", help="auto | fp32 | bf16"),
):
    from ..models.config import PRESETS, ModelConfig, get_preset
    cfg = get_preset(model) if model in PRESETS else ModelConfig.from_pretrained(os.path.dirname(model) if model.endswith(".json") else model)
    print(json.dumps(memory_plan(cfg, gpus, max_tokens_per_gpu, hbm_gb, optimizer_state_dtype), indent=2))


if __name__ == "__main__":
    app()
