"""Minibatch packers: split one global batch into per-rank, token-budgeted minibatches.

Public contract (same as the reference's ``batch_lengths_to_minibatches_lpt``,
batch_packer.py:190-230, and the deprecated greedy ``batch_lengths_to_minibatches``,
sampler.py:41-95): given the sequence lengths of a global batch, a per-rank token budget, the
number of ranks and this rank's id, return ``list[list[int]]`` — one inner list per minibatch
holding the batch indices this rank processes, ``[-1]`` meaning "this rank idles in that
minibatch" (the collator substitutes a dummy sample). Every rank returns the same number of
minibatches, so the gradient-accumulation loops stay in lock step.

Three implementations share that contract:

* ``lpt_pack_all`` / ``batch_lengths_to_minibatches_lpt`` — compiled C++ (``csrc/packer.cpp``),
  the production path; one call schedules all ranks.
* ``lpt_pack_all_py`` — pure-Python oracle of the same algorithm, used by tests and as the
  fallback when the shared library has not been built.
* ``batch_lengths_to_minibatches`` — greedy first-come packer, kept for comparison tests.

Ties between equal lengths are broken by ascending batch index (stable sort), which makes the
result deterministic across platforms; the reference leaves tie order to numpy's introsort.
A sequence longer than the budget is never dropped: it is scheduled alone on one rank (the
reference behaves the same way, batch_packer.py:149-155 starts its search at one sequence
without a feasibility check).
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import numpy as np

from .. import build as _build

_LIB = None
_LIB_TRIED = False


def _load_lib():
    global _LIB, _LIB_TRIED
    if _LIB_TRIED:
        return _LIB
    _LIB_TRIED = True
    try:
        path = _build.build_host()
        lib = ctypes.CDLL(str(path))
        i64p = ctypes.POINTER(ctypes.c_int64)
        for name in ("mtb200_lpt_pack", "mtb200_greedy_pack"):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int64
            fn.argtypes = [i64p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, i64p, i64p]
        lib.mtb200_lpt_pack_cost.restype = ctypes.c_int64
        lib.mtb200_lpt_pack_cost.argtypes = [i64p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_double, i64p, i64p]
        _LIB = lib
    except Exception:  # compiler missing: the Python oracle takes over
        _LIB = None
    return _LIB


def native_available() -> bool:
    return _load_lib() is not None


# ----------------------------------------------------------------------------------------
# Pure-Python oracle
# ----------------------------------------------------------------------------------------
class _Heap:
    """1-indexed binary min-heap of per-rank loads; ``ids[slot]`` is the rank in that slot."""

    def __init__(self, ranks: int):
        self.n = ranks
        self.load = [0] * (ranks + 1)
        self.ids = list(range(-1, ranks))

    def reset(self):
        for i in range(self.n + 1):
            self.load[i] = 0
            self.ids[i] = i - 1

    def sift_root(self):
        load, ids, n = self.load, self.ids, self.n
        u = 1
        while (u << 1) <= n:
            v = u << 1
            r = v | 1
            if r <= n and load[r] < load[v]:
                v = r
            if load[u] <= load[v]:
                break
            load[u], load[v] = load[v], load[u]
            ids[u], ids[v] = ids[v], ids[u]
            u = v


def _fits(heap: _Heap, lens, count: int, max_tokens: int) -> bool:
    heap.reset()
    for i in range(count):
        heap.load[1] += lens[i]
        if heap.load[1] > max_tokens:
            return False
        heap.sift_root()
    return True


def _assign_py(lengths: Sequence[int], max_tokens: int, num_ranks: int):
    n = len(lengths)
    rank_of = [0] * n
    mb_of = [0] * n
    if n == 0:
        return rank_of, mb_of, 0
    order = sorted(range(n), key=lambda i: -int(lengths[i]))  # stable: ties by ascending index
    srt = [int(lengths[i]) for i in order]
    csum = np.cumsum(np.asarray(srt, dtype=np.int64))
    heap = _Heap(num_ranks)
    start = n_mb = 0
    while start < n:
        remaining = n - start
        base = int(csum[start - 1]) if start > 0 else 0
        ub = int(np.searchsorted(csum[start:], base + max_tokens * num_ranks, side="right"))
        left, right = 1, min(remaining + 1, ub + 1)
        window = srt[start:]
        while right - left > 1:
            mid = (left + right) // 2
            if _fits(heap, window, mid, max_tokens):
                left = mid
            else:
                right = mid
        take = left
        if take < num_ranks and take < remaining:
            want = min(num_ranks, remaining)
            if _fits(heap, window, want, max_tokens):
                take = want
        heap.reset()
        for i in range(take):
            heap.load[1] += window[i]
            rank_of[order[start + i]] = heap.ids[1]
            mb_of[order[start + i]] = n_mb
            heap.sift_root()
        n_mb += 1
        start += take
    return rank_of, mb_of, n_mb


def _greedy_assign_py(lengths: Sequence[int], max_tokens: int, num_ranks: int):
    n = len(lengths)
    rank_of, mb_of = [0] * n, [0] * n
    loads = [0] * num_ranks
    mb = 0
    for i, ln in enumerate(lengths):
        best = min(range(num_ranks), key=lambda r: loads[r])
        if loads[best] + ln > max_tokens:
            if max(loads) > 0:
                mb += 1
            loads = [0] * num_ranks
            best = 0
        loads[best] += ln
        rank_of[i], mb_of[i] = best, mb
    return rank_of, mb_of, (mb + 1 if n else 0)


# ----------------------------------------------------------------------------------------
# Assembly of the list-of-lists view
# ----------------------------------------------------------------------------------------
def _to_lists(lengths, rank_of, mb_of, n_mb: int, num_ranks: int, longest_first: bool):
    """``out[rank][minibatch]`` = indices, ``[-1]`` where the rank idles."""
    out = [[[] for _ in range(n_mb)] for _ in range(num_ranks)]
    idx = range(len(lengths))
    if longest_first:
        idx = sorted(idx, key=lambda i: -int(lengths[i]))
    for i in idx:
        out[int(rank_of[i])][int(mb_of[i])].append(int(i))
    for r in range(num_ranks):
        for m in range(n_mb):
            if not out[r][m]:
                out[r][m] = [-1]
    return out


def _native_assign(fn_name: str, lengths, max_tokens: int, num_ranks: int):
    lib = _load_lib()
    arr = np.ascontiguousarray(np.asarray(lengths, dtype=np.int64))
    n = arr.shape[0]
    rank_of = np.zeros(max(n, 1), dtype=np.int64)
    mb_of = np.zeros(max(n, 1), dtype=np.int64)
    i64p = ctypes.POINTER(ctypes.c_int64)
    n_mb = getattr(lib, fn_name)(arr.ctypes.data_as(i64p), n, int(max_tokens), int(num_ranks),
                                 rank_of.ctypes.data_as(i64p), mb_of.ctypes.data_as(i64p))
    if n_mb < 0:
        raise ValueError("invalid packer arguments")
    return rank_of[:n], mb_of[:n], int(n_mb)


def lpt_pack_all_py(batch_lengths: Sequence[int], max_tokens_per_rank: int, num_ranks: int):
    """Python oracle: minibatch lists for all ranks, ``result[rank][minibatch]``."""
    if num_ranks <= 0:
        raise ValueError("num_ranks must be positive")
    r, m, n_mb = _assign_py(batch_lengths, max_tokens_per_rank, num_ranks)
    return _to_lists(batch_lengths, r, m, n_mb, num_ranks, longest_first=True)


def _assign_cost_py(lengths: Sequence[int], max_tokens: int, num_ranks: int, cost_len: float):
    """Python oracle of the cost-aware packer (``csrc/packer.cpp: mtb200_lpt_pack_cost``)."""
    import heapq
    n = len(lengths)
    rank_of, mb_of = [0] * n, [0] * n
    order = sorted(range(n), key=lambda i: -int(lengths[i]))
    srt = [int(lengths[i]) for i in order]
    csum = np.cumsum(np.asarray(srt, dtype=np.int64)) if n else np.zeros(0, np.int64)
    cost = lambda ln: float(ln) * (1.0 + float(ln) / cost_len)

    class H(_Heap):
        def __init__(self, ranks):
            super().__init__(ranks)
            self.tok = [0] * (ranks + 1)
            self.load = [0.0] * (ranks + 1)

        def reset(self):
            for i in range(self.n + 1):
                self.load[i], self.tok[i], self.ids[i] = 0.0, 0, i - 1

        def sift_root(self):
            load, ids, tok, nn = self.load, self.ids, self.tok, self.n
            u = 1
            while (u << 1) <= nn:
                v = u << 1
                r = v | 1
                if r <= nn and load[r] < load[v]:
                    v = r
                if load[u] <= load[v]:
                    break
                load[u], load[v] = load[v], load[u]
                ids[u], ids[v] = ids[v], ids[u]
                tok[u], tok[v] = tok[v], tok[u]
                u = v

    heap = H(num_ranks)

    def place(first, count, record, mb):
        heap.reset()
        for i in range(count):
            ln = srt[first + i]
            if heap.tok[1] > 0 and heap.tok[1] + ln > max_tokens:
                return False
            if record:
                rank_of[order[first + i]], mb_of[order[first + i]] = heap.ids[1], mb
            heap.tok[1] += ln
            heap.load[1] += cost(ln)
            heap.sift_root()
        return True

    start = n_mb = 0
    while start < n:
        remaining = n - start
        base = int(csum[start - 1]) if start > 0 else 0
        ub = int(np.searchsorted(csum[start:], base + max_tokens * num_ranks, side="right"))
        left, right = 1, min(remaining + 1, ub + 1)
        while right - left > 1:
            mid = (left + right) // 2
            if place(start, mid, False, 0):
                left = mid
            else:
                right = mid
        take = left
        if take < num_ranks and take < remaining:
            want = min(num_ranks, remaining)
            if place(start, want, False, 0):
                take = want
        place(start, take, True, n_mb)
        n_mb += 1
        start += take
    return rank_of, mb_of, n_mb


def lpt_pack_all(batch_lengths: Sequence[int], max_tokens_per_rank: int, num_ranks: int, cost_len: float | None = None,
                 use_native: bool = True):
    """LPT schedule of every rank in one call (compiled when available).

    ``cost_len`` switches from balancing tokens (the reference's criterion) to balancing an estimated
    compute cost ``len * (1 + len / cost_len)`` — ``cost_len`` is the sequence length at which causal
    attention costs as much as the GEMMs of a token (see ``ModelConfig.attention_cost_length``). The
    token budget stays a hard limit per rank; the global batch and therefore the gradient are the
    same either way, only the slowest rank of each step gets faster.
    """
    if num_ranks <= 0:
        raise ValueError("num_ranks must be positive")
    if len(batch_lengths) == 0:
        return [[] for _ in range(num_ranks)]
    native = use_native and _load_lib() is not None
    if cost_len:
        if native:
            lib = _load_lib()
            arr = np.ascontiguousarray(np.asarray(batch_lengths, dtype=np.int64))
            r, m = np.zeros(arr.shape[0], np.int64), np.zeros(arr.shape[0], np.int64)
            i64p = ctypes.POINTER(ctypes.c_int64)
            n_mb = lib.mtb200_lpt_pack_cost(arr.ctypes.data_as(i64p), arr.shape[0], int(max_tokens_per_rank), int(num_ranks),
                                            float(cost_len), r.ctypes.data_as(i64p), m.ctypes.data_as(i64p))
            if n_mb < 0:
                raise ValueError("invalid packer arguments")
        else:
            r, m, n_mb = _assign_cost_py(batch_lengths, max_tokens_per_rank, num_ranks, float(cost_len))
        return _to_lists(batch_lengths, r, m, int(n_mb), num_ranks, longest_first=True)
    if not native:
        return lpt_pack_all_py(batch_lengths, max_tokens_per_rank, num_ranks)
    r, m, n_mb = _native_assign("mtb200_lpt_pack", batch_lengths, max_tokens_per_rank, num_ranks)
    return _to_lists(batch_lengths, r, m, n_mb, num_ranks, longest_first=True)


def batch_lengths_to_minibatches_lpt(batch_lengths: Sequence[int], max_tokens_per_rank: int,
                                     num_ranks: int, rank: int, cost_len: float | None = None):
    """Reference-compatible entry point (batch_packer.py:190): this rank's minibatches."""
    if len(batch_lengths) == 0:
        return []
    return lpt_pack_all(batch_lengths, max_tokens_per_rank, num_ranks, cost_len=cost_len)[rank]


def batch_lengths_to_minibatches(batch_lengths: Sequence[int], max_tokens_per_rank: int,
                                 num_ranks: int, rank: int, use_native: bool = True):
    """Greedy first-come packer (reference sampler.py:41-95); kept for comparisons."""
    if len(batch_lengths) == 0:
        return []
    if use_native and _load_lib() is not None:
        r, m, n_mb = _native_assign("mtb200_greedy_pack", batch_lengths, max_tokens_per_rank, num_ranks)
    else:
        r, m, n_mb = _greedy_assign_py(batch_lengths, max_tokens_per_rank, num_ranks)
    return _to_lists(batch_lengths, r, m, n_mb, num_ranks, longest_first=False)[rank]


def packing_stats(batch_lengths: Sequence[int], per_rank: list, max_tokens_per_rank: int) -> dict:
    """Load-balance figures used by the comparison tests and the README numbers.

    ``per_rank[rank][minibatch]`` as returned by ``lpt_pack_all``.
    """
    num_ranks = len(per_rank)
    n_mb = len(per_rank[0]) if num_ranks else 0
    balances, effs = [], []
    for m in range(n_mb):
        loads = [sum(batch_lengths[i] for i in per_rank[r][m] if i >= 0) for r in range(num_ranks)]
        nz = [x for x in loads if x > 0]
        balances.append(min(nz) / max(nz) if nz else 1.0)
        effs.append(sum(loads) / (max(loads) * num_ranks) if max(loads) > 0 else 0.0)
    total = float(sum(batch_lengths))
    cap = float(n_mb * num_ranks * max_tokens_per_rank) or 1.0
    return {
        "num_minibatches": n_mb,
        "avg_balance": float(np.mean(balances)) if balances else 1.0,
        "worst_balance": float(min(balances)) if balances else 1.0,
        "row_efficiency": float(np.mean(effs)) if effs else 0.0,
        "capacity_efficiency": total / cap,
    }
