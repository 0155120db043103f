"""Sharded training-state checkpoints for true resume (a superset of the reference, which only
exports weights and restarts the optimizer from zero when a run continues from an export).

Each rank writes ``rank<r>-of-<w>.safetensors`` with its slices of the fp32 master weights, both
AdamW moments for every group (plus the OSFT factors it owns, when that mode is on); rank 0 adds
``state.json``: optimizer step, world size and whatever the training loop passes in ``extra``
(scheduler state, optimizer steps taken, global batches consumed, samples seen, samples at the
last export). A state written by another number of ranks is re-sliced on load (every group is one flat
buffer cut into equal slices, so a rank reads the parts of the old slices that overlap its new one;
OSFT factors are owned by matrix, so a rank fetches each matrix it owns now from the rank that owned it then).
``trainer.train`` writes one next to every
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


def _flat_slice(files: list, key: str, lo: int, hi: int) -> torch.Tensor:
    """Elements [lo, hi) of the flat tensor whose equal slices ``files`` (one reader per old rank) hold under ``key``;
    elements past the end of the old buffer (padding of the new layout) are zero."""
    s_old = int(files[0].header[key]["shape"][0])
    out = None
    for r, f in enumerate(files):
        a, b = max(lo, r * s_old), min(hi, (r + 1) * s_old)
        if a >= b:
            continue
        part = f.get_slice(key, a - r * s_old, b - r * s_old)
        if out is None:
            out = torch.zeros(hi - lo, dtype=part.dtype)
        out[a - lo: b - lo] = part
    return out if out is not None else torch.zeros(hi - lo, dtype=st._FROM[files[0].header[key]["dtype"]])


def load_train_state(engine, directory: str) -> dict:
    with open(os.path.join(directory, "state.json")) as f:
        meta = json.load(f)
    old_world = int(meta["world"])
    osft = getattr(engine, "osft", None)
    ranks = [engine.rank] if old_world == engine.world else list(range(old_world))
    files = []
    try:
        for r in ranks:
            path = os.path.join(directory, f"rank{r}-of-{old_world}.safetensors")
            try:
                files.append(st.SafeTensorsFile(path))
            except Exception as e:
                raise RuntimeError(f"cannot read training state shard {path}: {e}") from e
        for g in engine.groups:
            n = g.layout.name
            s_new = g.layout.shard_numel
            for key, dst in ((f"{n}.master", g.master), (f"{n}.m", g.m), (f"{n}.v", g.v)):
                try:
                    if old_world == engine.world:
                        src = files[0].get_tensor(key)
                    else:
                        src = _flat_slice(files, key, engine.rank * s_new, (engine.rank + 1) * s_new)
                except KeyError:
                    raise
                except Exception as e:
                    raise RuntimeError(f"cannot read {key} from the training state in {directory}: {e}") from e
                if src.shape != dst.shape:
                    raise RuntimeError(f"{key}: shard shape {tuple(src.shape)} does not match {tuple(dst.shape)}")
                dst.copy_(src.to(dst.dtype))
            g.shard.copy_(g.master.to(g.shard.dtype))
            g.has_grad = False
        if osft is not None and old_world == engine.world:
            osft.load_state_tensors({k: files[0].get_tensor(k) for k in files[0].keys() if k.startswith("osft.")})
        elif osft is not None:   # every matrix this rank owns now is fetched from the rank that owned it then
            osft.load_state_from(files, old_world)
    finally:
        for f in files:
            f.close()
    engine.step_count = int(meta["step_count"])
    return meta
