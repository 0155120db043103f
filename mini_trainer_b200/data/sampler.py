"""Dataset, infinite sampler, packing collator and the prefetching loader.

Capabilities mirror the reference data path (sampler.py:97-285):

* ``JsonlDataset`` reads a tokenised JSONL file with the columns ``input_ids``, ``labels``,
  ``len`` and ``num_loss_counted_tokens`` (the output of ``process_data``).
* ``InfiniteSampler`` yields an endless stream of shuffled indices, identical on every rank,
  reshuffled with ``seed + epoch`` each pass.
* ``MaxTokensPerRankCollator`` turns one global batch into THIS rank's list of padding-free
  minibatches: one ``[1, T]`` row per minibatch, ``position_ids`` restarting at 0 for every
  sample, labels ``-100`` where the loss is masked, a 5-token all-masked dummy sample where the
  rank idles, and the whole batch's loss-token count attached to every minibatch.
* ``get_data_loader`` wires them together.

What is different from the reference, on purpose:

* token storage is one flat ``int32`` array per column plus an offset table, so a sample is a
  slice, the lengths of a batch are one fancy-index, and only the samples this rank owns are
  ever turned into tensors (the reference materialises the full global batch on every rank);
* the collator also emits ``cu_seqlens`` (int32 prefix sums) and ``max_seqlen``, computed on the
  host where the sample boundaries are known, so the attention kernel never has to recover
  them from ``position_ids`` with device-side ``nonzero`` calls and host syncs;
* prefetching is a background thread that packs ahead and (on CUDA machines) stages the
  minibatch in pinned memory; ``num_workers`` > 0 switches to ``torch.utils.data.DataLoader``
  worker processes like the reference's ``num_workers=4``.
"""
from __future__ import annotations

import json
import queue
import threading
from typing import Iterator, Optional

import numpy as np
import torch

from .packer import batch_lengths_to_minibatches_lpt

DUMMY_INPUT_IDS = (15, 14, 13, 12, 11)


class JsonlDataset(torch.utils.data.Dataset):
    """Tokenised samples held as flat int32 arrays (reference: sampler.py:97-113)."""

    def __init__(self, path: Optional[str] = None, samples: Optional[list] = None):
        ids, labs, offs, nloss = [], [], [0], []
        if samples is None:
            if path is None:
                raise ValueError("either path or samples is required")
            samples = self._read(path)
        for s in samples:
            a = np.asarray(s["input_ids"], dtype=np.int32)
            b = np.asarray(s["labels"], dtype=np.int32)
            if a.shape != b.shape:
                raise ValueError("input_ids and labels differ in length")
            ids.append(a)
            labs.append(b)
            offs.append(offs[-1] + a.shape[0])
            nloss.append(int(s.get("num_loss_counted_tokens", int((b != -100).sum()))))
        self.input_ids = np.concatenate(ids) if ids else np.zeros(0, np.int32)
        self.labels = np.concatenate(labs) if labs else np.zeros(0, np.int32)
        self.offsets = np.asarray(offs, dtype=np.int64)
        self.lengths = np.diff(self.offsets)
        self.num_loss_counted_tokens = np.asarray(nloss, dtype=np.int64)

    @staticmethod
    def _read(path: str):
        with open(path, "r") as f:
            for line in f:
                line = line.strip()
                if line:
                    yield json.loads(line)

    def __len__(self) -> int:
        return int(self.lengths.shape[0])

    def raw(self, index: int):
        lo, hi = int(self.offsets[index]), int(self.offsets[index + 1])
        return self.input_ids[lo:hi], self.labels[lo:hi]

    def __getitem__(self, index: int):
        a, b = self.raw(int(index))
        return {
            "input_ids": torch.from_numpy(a.astype(np.int64)),
            "labels": torch.from_numpy(b.astype(np.int64)),
            "len": int(self.lengths[index]),
            "num_loss_counted_tokens": int(self.num_loss_counted_tokens[index]),
        }


class InfiniteSampler(torch.utils.data.Sampler):
    """Endless shuffled index stream, the same on all ranks (reference: sampler.py:116-142)."""

    def __init__(self, len_data: int, seed: int = 37, start_index: int = 0):
        self.len_data = len_data
        self.seed = seed
        # indices already consumed by an earlier run (resume): the stream continues where it stopped
        self.start_index = int(start_index)

    def __iter__(self) -> Iterator[int]:
        epoch, skip = divmod(self.start_index, max(1, self.len_data))
        while True:
            g = torch.Generator()
            g.manual_seed(self.seed + epoch)
            perm = torch.randperm(self.len_data, generator=g).tolist()
            yield from perm[skip:]
            skip = 0
            epoch += 1

    def __len__(self) -> int:
        return self.len_data


def default_dummy_sample() -> dict:
    """The filler a rank processes when a minibatch has no real sample for it."""
    return {
        "input_ids": torch.tensor(DUMMY_INPUT_IDS, dtype=torch.long),
        "labels": torch.full((len(DUMMY_INPUT_IDS),), -100, dtype=torch.long),
        "len": len(DUMMY_INPUT_IDS),
        "num_loss_counted_tokens": 0,
    }


def mb_collate_fn(minibatch: list, batch_num_loss_counted_tokens: int) -> dict:
    """Concatenates samples into one padding-free row (reference: sampler.py:144-208)."""
    ids = torch.cat([torch.as_tensor(s["input_ids"], dtype=torch.long) for s in minibatch])
    labels = torch.cat([torch.as_tensor(s["labels"], dtype=torch.long) for s in minibatch])
    lens = [int(s["input_ids"].shape[0]) if hasattr(s["input_ids"], "shape") else len(s["input_ids"])
            for s in minibatch]
    pos = torch.cat([torch.arange(n, dtype=torch.long) for n in lens])
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens, dtype=torch.int64), 0).to(torch.int32)
    return {
        "input_ids": ids.unsqueeze(0),
        "labels": labels.unsqueeze(0),
        "position_ids": pos.unsqueeze(0),
        "cu_seqlens": cu,
        "max_seqlen": max(lens),
        "num_loss_counted_tokens": int(sum(int(s["num_loss_counted_tokens"]) for s in minibatch)),
        # dummy samples carry no loss tokens and are not counted as samples
        "num_samples": int(sum(1 for s in minibatch if int(s["num_loss_counted_tokens"]) > 0)),
        "batch_num_loss_counted_tokens": int(batch_num_loss_counted_tokens),
    }


class MaxTokensPerRankCollator:
    """Global batch -> this rank's packed minibatches (reference: sampler.py:210-267).

    Works on either a list of sample dicts (``torch.utils.data.DataLoader`` style) or, through
    ``collate_indices``, directly on dataset indices so that only owned samples are copied.
    Samples longer than the budget are reported but kept, as in the reference: the LPT packer
    schedules each of them alone.
    """

    def __init__(self, max_tokens_per_rank: int, rank: Optional[int] = None,
                 world_size: Optional[int] = None, dummy_sample: Optional[dict] = None,
                 packer=batch_lengths_to_minibatches_lpt, cost_len: Optional[float] = None):
        import torch.distributed as dist
        self.max_tokens_per_rank = int(max_tokens_per_rank)
        self.rank = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
        self.world_size = world_size if world_size is not None else (
            dist.get_world_size() if dist.is_initialized() else 1)
        self.dummy_sample = dummy_sample if dummy_sample is not None else default_dummy_sample()
        self.packer = packer
        self.cost_len = cost_len   # None: balance tokens like the reference; else balance estimated compute cost
        self._warned = False

    def _plan(self, lengths):
        n_long = int(sum(1 for x in lengths if x > self.max_tokens_per_rank))
        if n_long and not self._warned:
            print(f"\033[38;5;196m{n_long} samples exceed max tokens per gpu; each is scheduled alone\033[0m")
            self._warned = True
        if self.cost_len:
            return self.packer([int(x) for x in lengths], self.max_tokens_per_rank, self.world_size, self.rank,
                               cost_len=self.cost_len)
        return self.packer([int(x) for x in lengths], self.max_tokens_per_rank, self.world_size, self.rank)

    def __call__(self, batch: list) -> list:
        lengths = [int(s["len"]) for s in batch]
        total_loss_tokens = int(sum(int(s["num_loss_counted_tokens"]) for s in batch))
        out = []
        for mb_idx in self._plan(lengths):
            mb = [batch[i] if i != -1 else self.dummy_sample for i in mb_idx]
            out.append(mb_collate_fn(mb, total_loss_tokens))
        return out

    def collate_indices(self, dataset: JsonlDataset, indices: list) -> list:
        idx = np.asarray(indices, dtype=np.int64)
        lengths = dataset.lengths[idx]
        total_loss_tokens = int(dataset.num_loss_counted_tokens[idx].sum())
        out = []
        for mb_idx in self._plan(lengths.tolist()):
            mb = [dataset[int(idx[i])] if i != -1 else self.dummy_sample for i in mb_idx]
            out.append(mb_collate_fn(mb, total_loss_tokens))
        return out


class PackedBatchLoader:
    """Iterable of per-rank minibatch lists with a background packing thread.

    ``prefetch`` global batches are packed ahead of the training loop. With ``pin_memory`` the
    tensors of each minibatch are staged in page-locked memory so the trainer's host-to-device
    copies are asynchronous.
    """

    def __init__(self, dataset: JsonlDataset, batch_size: int, sampler: InfiniteSampler,
                 collator: MaxTokensPerRankCollator, prefetch: int = 2, pin_memory: bool = False):
        self.dataset, self.batch_size = dataset, int(batch_size)
        self.sampler, self.collator = sampler, collator
        self.prefetch, self.pin_memory = int(prefetch), bool(pin_memory)

    def _batches(self):
        buf = []
        for i in self.sampler:
            buf.append(i)
            if len(buf) == self.batch_size:
                yield buf
                buf = []

    def _make(self, indices):
        mbs = self.collator.collate_indices(self.dataset, indices)
        if self.pin_memory:
            for mb in mbs:
                for k, v in mb.items():
                    if isinstance(v, torch.Tensor):
                        mb[k] = v.pin_memory()
        return mbs

    def __iter__(self):
        if self.prefetch <= 0:
            for idx in self._batches():
                yield self._make(idx)
            return
        q: queue.Queue = queue.Queue(maxsize=self.prefetch)
        stop = threading.Event()

        def work():
            try:
                for idx in self._batches():
                    if stop.is_set():
                        return
                    item = self._make(idx)
                    while not stop.is_set():
                        try:
                            q.put(item, timeout=0.1)
                            break
                        except queue.Full:
                            continue
            except BaseException as e:  # surfaced in the consumer
                q.put(e)

        t = threading.Thread(target=work, daemon=True, name="mtb200-packer")
        t.start()
        try:
            while True:
                item = q.get()
                if isinstance(item, BaseException):
                    raise item
                yield item
        finally:
            # the thread is joined, not left to the interpreter's shutdown: a daemon thread that is still inside a
            # tensor operation when the runtime is torn down aborts the process after a finished run
            stop.set()
            t.join(timeout=10)


def get_data_loader(**kwargs):
    """Builds the training loader (reference: sampler.py:269-285).

    Keyword arguments: ``data_path`` (or ``dataset``), ``batch_size``, ``max_tokens_per_gpu``,
    ``seed``; optional ``rank``, ``world_size``, ``dummy_sample`` (bypass ``torch.distributed``,
    which is how tests simulate several ranks in one process), ``cost_len`` (balance ranks on estimated
    compute cost instead of tokens, see ``data.packer.lpt_pack_all``), ``num_workers`` (0 = packing
    thread, >0 = DataLoader worker processes), ``prefetch``, ``pin_memory`` and ``skip_batches``
    (global batches an earlier run already consumed; a resumed run continues the same stream).
    """
    dataset = kwargs.get("dataset") or JsonlDataset(kwargs["data_path"])
    collator = MaxTokensPerRankCollator(kwargs["max_tokens_per_gpu"], rank=kwargs.get("rank"),
                                        world_size=kwargs.get("world_size"),
                                        dummy_sample=kwargs.get("dummy_sample"), cost_len=kwargs.get("cost_len"))
    sampler = InfiniteSampler(len(dataset), seed=kwargs["seed"],
                              start_index=int(kwargs.get("skip_batches", 0)) * int(kwargs["batch_size"]))
    num_workers = int(kwargs.get("num_workers", 0))
    if num_workers > 0:
        return torch.utils.data.DataLoader(dataset, kwargs["batch_size"], sampler=sampler,
                                           collate_fn=collator, num_workers=num_workers)
    return PackedBatchLoader(dataset, kwargs["batch_size"], sampler, collator,
                             prefetch=int(kwargs.get("prefetch", 2)),
                             pin_memory=bool(kwargs.get("pin_memory", False)))
