"""Sharded training-state checkpoints for true resume (a superset of the reference, which only
exports weights and restarts the optimizer from zero when a run continues from an export).

Each rank writes ``rank<r>-of-<w>.safetensors`` with its slices of the fp32 master weights, both
AdamW moments for every group (plus the OSFT factors it owns, when that mode is on); rank 0 adds
``state.json``: optimizer step, world size and whatever the training loop passes in ``extra``
(scheduler state, optimizer steps taken, global batches consumed, samples seen, samples at the
last export). Resume requires the same world size. ``trainer.train`` writes one next to every
exported checkpoint when ``save_train_state`` is on, and ``train.py --resume-from`` restores it
and continues the data stream where it stopped.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from . import safetensors_io as st


def save_train_state(engine, directory: str, extra: dict | None = None) -> None:
    os.makedirs(directory, exist_ok=True)
    tensors = {}
    for g in engine.groups:
        n = g.layout.name
        tensors[f"{n}.master"] = g.master
        tensors[f"{n}.m"] = g.m
        tensors[f"{n}.v"] = g.v
    osft = getattr(engine, "osft", None)
    if osft is not None:
        tensors.update(osft.state_tensors())
    st.save_file({k: v.cpu() for k, v in tensors.items()},
                 os.path.join(directory, f"rank{engine.rank}-of-{engine.world}.safetensors"))
    if engine.rank == 0:
        meta = {"step_count": engine.step_count, "world": engine.world}
        meta.update(extra or {})
        with open(os.path.join(directory, "state.json"), "w") as f:
            json.dump(meta, f, indent=2)
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def load_train_state(engine, directory: str) -> dict:
    with open(os.path.join(directory, "state.json")) as f:
        meta = json.load(f)
    if int(meta["world"]) != engine.world:
        raise ValueError(f"training state was saved with world size {meta['world']}, now {engine.world}")
    path = os.path.join(directory, f"rank{engine.rank}-of-{engine.world}.safetensors")
    try:
        tensors = st.load_file(path)
    except Exception as e:
        raise RuntimeError(f"cannot read training state shard {path}: {e}") from e
    for g in engine.groups:
        n = g.layout.name
        for key, dst in ((f"{n}.master", g.master), (f"{n}.m", g.m), (f"{n}.v", g.v)):
            src = tensors[key]
            if src.shape != dst.shape:
                raise RuntimeError(f"{key}: shard shape {tuple(src.shape)} does not match {tuple(dst.shape)}")
            dst.copy_(src.to(dst.dtype))
        g.shard.copy_(g.master.to(g.shard.dtype))
        g.has_grad = False
    osft = getattr(engine, "osft", None)
    if osft is not None:
        osft.load_state_tensors(tensors)
    engine.step_count = int(meta["step_count"])
    return meta
