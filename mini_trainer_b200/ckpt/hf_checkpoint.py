"""Hugging Face-format checkpoints: bf16 safetensors shards + index + config + tokenizer.

Layout written (same as the reference's ``save_model``, train.py:30-70):
``<output_dir>/hf_format/samples_<N>/`` holding ``model.safetensors`` when everything fits in one
5 GB shard, else ``model-0000i-of-0000N.safetensors`` plus ``model.safetensors.index.json``
(``{"metadata": {"total_size"}, "weight_map"}``, indent 2, sorted keys), ``config.json`` and the
tokenizer files copied from ``model_name_or_path``. ``N`` is printed the way the reference prints
its float sample counter (``samples_8192.0``).

Unlike the reference, no rank ever holds the full model on its GPU: the engine yields one
gathered group at a time and rank 0 streams it to the current shard file, so a 70B export needs
one block of device memory. With tied embeddings ``lm_head.weight`` is omitted (HF convention).
"""
from __future__ import annotations

import json
import os
import shutil
import time
from pathlib import Path

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..utils.log import log_rank_0
from . import safetensors_io as st

MAX_SHARD_BYTES = 5 * 10 ** 9  # "5GB" in huggingface_hub means 5e9 bytes
TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "vocab.json",
                   "merges.txt", "tokenizer.model", "added_tokens.json", "chat_template.jinja",
                   "generation_config.json")


def plan_shards(sizes: list, max_shard_bytes: int = MAX_SHARD_BYTES) -> list:
    """Greedy in-order split: ``sizes`` = [(name, nbytes)], returns list of lists of names."""
    shards, cur, cur_bytes = [], [], 0
    for name, n in sizes:
        if cur and cur_bytes + n > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = [], 0
        cur.append(name)
        cur_bytes += n
    if cur:
        shards.append(cur)
    return shards


def _is_rank0() -> bool:
    return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0


def save_hf_checkpoint(engine, save_directory: str, model_name_or_path: str | None = None,
                       max_shard_bytes: int = MAX_SHARD_BYTES) -> None:
    """Collective: every rank takes part in the group gathers, rank 0 writes the files."""
    cfg: ModelConfig = engine.cfg
    rank0 = _is_rank0()
    if rank0:
        os.makedirs(save_directory, exist_ok=True)
    pending, pending_bytes, files, weight_map, total = {}, 0, [], {}, 0

    def flush():
        nonlocal pending, pending_bytes
        if pending:
            tmp = os.path.join(save_directory, f".shard{len(files)}.tmp")
            st.save_file(pending, tmp, metadata={"format": "pt"})
            files.append((tmp, list(pending.keys())))
        pending, pending_bytes = {}, 0

    for name, tensor in engine.iter_hf_tensors(dtype=torch.bfloat16, host_ranks=(0,)):
        if not rank0:
            continue
        n = tensor.numel() * tensor.element_size()
        if pending and pending_bytes + n > max_shard_bytes:
            flush()
        pending[name] = tensor
        pending_bytes += n
        total += n
    if rank0:
        flush()
        nshard = len(files)
        for i, (tmp, names) in enumerate(files):
            fname = "model.safetensors" if nshard == 1 else f"model-{i + 1:05d}-of-{nshard:05d}.safetensors"
            os.replace(tmp, os.path.join(save_directory, fname))
            for k in names:
                weight_map[k] = fname
        if nshard > 1:
            index = {"metadata": {"total_size": total}, "weight_map": weight_map}
            with open(os.path.join(save_directory, "model.safetensors.index.json"), "w") as f:
                json.dump(index, f, indent=2, sort_keys=True)
        cfg.to_json_file(os.path.join(save_directory, "config.json"))
        if model_name_or_path and os.path.isdir(model_name_or_path):
            for fn in TOKENIZER_FILES:
                src = os.path.join(model_name_or_path, fn)
                if os.path.exists(src):
                    shutil.copy(src, os.path.join(save_directory, fn))
        elif model_name_or_path and not model_name_or_path.startswith("random:"):
            try:  # hub id: let transformers resolve it from the local cache
                from transformers import AutoTokenizer
                AutoTokenizer.from_pretrained(model_name_or_path).save_pretrained(save_directory)
            except Exception as e:
                log_rank_0(f"tokenizer not saved: {e}")


def save_model(engine, samples_seen, output_dir: str, model_name_or_path: str | None = None,
               max_shard_bytes: int = MAX_SHARD_BYTES) -> str:
    """Reference-compatible wrapper: path naming, timing message, trailing barrier."""
    log_rank_0(f"Saving model at {samples_seen} samples")
    start = time.time()
    save_directory = str(Path(output_dir) / "hf_format" / f"samples_{samples_seen}")
    save_hf_checkpoint(engine, save_directory, model_name_or_path, max_shard_bytes=max_shard_bytes)
    log_rank_0(f"\033[1;38;2;0;255;255mSaved model at\033[0m {samples_seen} samples in {time.time() - start:.2f} seconds")
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    return save_directory


class HFCheckpointReader:
    """Name -> tensor lookup over a single-file or sharded HF safetensors directory."""

    def __init__(self, path: str):
        self.path = path
        idx = os.path.join(path, "model.safetensors.index.json")
        self._files = {}
        if os.path.exists(idx):
            with open(idx) as f:
                self.weight_map = json.load(f)["weight_map"]
        else:
            f = self._open("model.safetensors")
            self.weight_map = {k: "model.safetensors" for k in f.keys()}

    def _open(self, fname: str) -> st.SafeTensorsFile:
        if fname not in self._files:
            self._files[fname] = st.SafeTensorsFile(os.path.join(self.path, fname))
        return self._files[fname]

    def keys(self):
        return self.weight_map.keys()

    def get_tensor(self, name: str) -> torch.Tensor:
        if name == "lm_head.weight" and name not in self.weight_map:
            name = "model.embed_tokens.weight"  # tied checkpoint
        return self._open(self.weight_map[name]).get_tensor(name)

    def close(self):
        for f in self._files.values():
            f.close()


def load_hf_checkpoint(engine, path: str) -> None:
    r = HFCheckpointReader(path)
    try:
        engine.load_hf_tensors(r.get_tensor)
    finally:
        r.close()
