"""Synthetic tokenised datasets with the length distributions of the benchmark configs.

Each sample has a lognormal length clipped to ``[lo, hi]``, uniformly random token ids and a
``-100`` label mask over a uniform(10%, 60%) prefix — the shape of data ``process_data`` emits
for single-turn chat samples (reference process_data.py:29,70-72; consumed at
sampler.py:108-113).
"""
from __future__ import annotations

import json
from dataclasses import dataclass

import numpy as np

from .sampler import JsonlDataset


@dataclass(frozen=True)
class LengthSpec:
    mu: float
    sigma: float
    lo: int
    hi: int


# name -> (length distribution, vocab, max_tokens_per_gpu, batch_size)
CONFIG_DATA = {
    "tiny-qwen2": (LengthSpec(5.5, 0.8, 16, 2048), 32000, 4096, 32),
    "qwen2.5-1.5b": (LengthSpec(7.0, 1.0, 32, 32768), 151936, 128000, 128),
    "llama-3.1-8b": (LengthSpec(7.5, 1.0, 64, 65536), 128256, 64000, 128),
    "qwen2.5-7b": (LengthSpec(7.5, 1.0, 64, 65536), 152064, 48000, 128),
    "llama-3.1-70b": (LengthSpec(7.5, 1.0, 64, 32768), 128256, 16000, 64),
    "tiny-mixtral": (LengthSpec(5.5, 0.8, 16, 2048), 4096, 4096, 32),
    "mixtral-8x7b": (LengthSpec(7.5, 1.0, 64, 32768), 32000, 32000, 128),
}


def synthetic_samples(num_samples: int, spec: LengthSpec, vocab_size: int, seed: int = 0):
    rng = np.random.default_rng(seed)
    lens = np.clip(np.rint(rng.lognormal(spec.mu, spec.sigma, num_samples)), spec.lo, spec.hi).astype(np.int64)
    for n in lens:
        n = int(n)
        ids = rng.integers(0, vocab_size, n, dtype=np.int64)
        masked = int(np.clip(round(n * rng.uniform(0.1, 0.6)), 1, n - 1))
        labels = ids.copy()
        labels[:masked] = -100
        yield {"input_ids": ids, "labels": labels, "len": n,
               "num_loss_counted_tokens": int(n - masked)}


def synthetic_dataset(num_samples: int, spec: LengthSpec, vocab_size: int, seed: int = 0) -> JsonlDataset:
    return JsonlDataset(samples=list(synthetic_samples(num_samples, spec, vocab_size, seed)))


def write_synthetic_jsonl(path: str, num_samples: int, spec: LengthSpec, vocab_size: int, seed: int = 0) -> None:
    with open(path, "w") as f:
        for s in synthetic_samples(num_samples, spec, vocab_size, seed):
            f.write(json.dumps({"input_ids": s["input_ids"].tolist(), "labels": s["labels"].tolist(),
                                "len": s["len"], "num_loss_counted_tokens": s["num_loss_counted_tokens"]}) + "\n")
