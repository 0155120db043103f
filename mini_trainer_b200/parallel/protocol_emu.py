"""Host-side emulation of the epoch-flag protocol used by the symmetric-memory kernels.

Ranks are threads, each with its own "arena" of flag words; ``signal`` writes an epoch into every
peer's row and ``wait`` polls the local row with a bound, exactly like ``csrc/symm_comm.cu``
(``ready`` / ``consumed`` rows per channel, wrap-safe ``>=`` comparison, error status instead of
an endless spin). It exists so that the protocol — ordering, buffer reuse, behaviour when a peer
never shows up — can be tested on a CPU-only machine, with faults injected on the host.
"""
from __future__ import annotations

import threading
import time


class EmuFabric:
    """Flag storage of ``world`` ranks: ``flags[owner][row][writer]``."""

    def __init__(self, world: int, rows: int = 8):
        self.world = world
        self.flags = [[[0] * world for _ in range(rows)] for _ in range(world)]
        self.buffers = [dict() for _ in range(world)]
        self.lock = threading.Lock()

    def signal(self, rank: int, row: int, epoch: int, drop_to: set | None = None) -> None:
        """``drop_to``: peers for which the message is lost (fault injection)."""
        for p in range(self.world):
            if drop_to and p in drop_to:
                continue
            self.flags[p][row][rank] = epoch

    def wait(self, rank: int, row: int, epoch: int, timeout_s: float = 1.0):
        """Returns ``(ok, first_missing_peer)``; bounded like the device loop."""
        deadline = time.monotonic() + timeout_s
        while True:
            missing = [p for p in range(self.world) if self.flags[rank][row][p] - epoch < 0]
            if not missing:
                return True, None
            if time.monotonic() > deadline:
                return False, missing[0]
            time.sleep(0.0005)


class EmuRank:
    """One rank's view: reduce-scatter over a double-buffered gradient slot with the same
    ready / consumed handshake as the GPU kernels."""
    READY, CONSUMED = 0, 1

    def __init__(self, fabric: EmuFabric, rank: int, timeout_s: float = 1.0):
        self.f, self.rank, self.timeout = fabric, rank, timeout_s
        self.epoch = {}
        self.status = 0

    def publish(self, slot: int, values: list, drop_to: set | None = None) -> None:
        """Write my gradient buffer for this slot, then tell the peers it is complete."""
        e = self.epoch.get(slot, 0)
        if e:   # the previous contents must have been consumed by everybody
            ok, peer = self.f.wait(self.rank, 2 * slot + self.CONSUMED, e, self.timeout)
            if not ok:
                self.status = 42 | (peer << 8)
                return
        self.f.buffers[self.rank][slot] = list(values)
        self.epoch[slot] = e + 1
        self.f.signal(self.rank, 2 * slot + self.READY, e + 1, drop_to)

    def reduce_scatter(self, slot: int):
        """Sum of my slice over all ranks, or ``None`` with ``status`` set when a peer is missing."""
        e = self.epoch[slot]
        ok, peer = self.f.wait(self.rank, 2 * slot + self.READY, e, self.timeout)
        if not ok:
            self.status = 41 | (peer << 8)
            return None
        w = self.f.world
        n = len(self.f.buffers[self.rank][slot]) // w
        out = [sum(self.f.buffers[p][slot][self.rank * n + i] for p in range(w)) for i in range(n)]
        self.f.signal(self.rank, 2 * slot + self.CONSUMED, e)
        return out


class EmuRegionRank(EmuRank):
    """Reduction by tensor region (``ShardedEngine._region_reducer``): a buffer is published region by
    region, back to front, each region with its own ready / consumed rows; before the buffer is
    rewritten only the consumed row of the region that is reduced LAST is awaited, because every peer
    reduces the regions in the same order on one stream. ``overwritten_early`` records whether that shortcut
    ever let a buffer be rewritten while a peer still owed a read of an earlier region."""

    def __init__(self, fabric: EmuFabric, rank: int, regions: list, timeout_s: float = 1.0):
        super().__init__(fabric, rank, timeout_s)
        self.regions = regions          # [(lo, hi)] in the order backward completes them
        self.overwritten_early = False  # set when a buffer is rewritten while a peer still had a region of it to read

    def _row(self, slot: int, k: int, kind: int) -> int:
        return (slot * len(self.regions) + k) * 2 + kind

    def publish_region(self, slot: int, k: int, values: list) -> None:
        lo, hi = self.regions[k]
        e = self.epoch.get((slot, k), 0)
        if k == 0 and e:   # first region of a reuse: the whole previous contents must have been consumed
            last = len(self.regions) - 1
            ok, peer = self.f.wait(self.rank, self._row(slot, last, self.CONSUMED), self.epoch[(slot, last)], self.timeout)
            if not ok:
                self.status = 42 | (peer << 8)
                return
            with self.f.lock:   # bookkeeping for the test: did any peer still owe a read of an earlier region?
                for kk in range(len(self.regions)):
                    row = self._row(slot, kk, self.CONSUMED)
                    if any(self.f.flags[self.rank][row][p] < self.epoch[(slot, kk)] for p in range(self.f.world)):
                        self.overwritten_early = True
        buf = self.f.buffers[self.rank].setdefault(slot, [0.0] * max(h for _, h in self.regions))
        buf[lo:hi] = values
        self.epoch[(slot, k)] = e + 1
        self.f.signal(self.rank, self._row(slot, k, self.READY), e + 1)

    def reduce_region(self, slot: int, k: int):
        """Sum over ranks of the part of region ``k`` that lies in my flat slice (possibly empty)."""
        e = self.epoch[(slot, k)]
        ok, peer = self.f.wait(self.rank, self._row(slot, k, self.READY), e, self.timeout)
        if not ok:
            self.status = 41 | (peer << 8)
            return None
        w = self.f.world
        total = max(h for _, h in self.regions)
        s = total // w
        lo, hi = max(self.regions[k][0], self.rank * s), min(self.regions[k][1], (self.rank + 1) * s)
        out = [sum(self.f.buffers[p][slot][i] for p in range(w)) for i in range(lo, max(lo, hi))]
        self.f.signal(self.rank, self._row(slot, k, self.CONSUMED), e)
        return lo, out


def ticket_gather(n_chunks: int, n_workers: int, resident: list, chunk_first: int = 0):
    """Emulates chunk ownership by ticket (``csrc/gather.cuh``): workers (CTAs) draw tickets from one counter
    until it runs past ``n_chunks``; ``resident[w]`` says whether worker ``w`` ever gets to run. Returns the
    chunks gathered and how many tickets each worker drew. With static ownership (chunk ``k`` belongs to worker
    ``k % n_workers``) a non-resident worker's chunks would never arrive; with tickets every chunk is gathered as
    long as ONE worker runs."""
    counter = [0]
    lock = threading.Lock()
    done, drawn = set(), [0] * n_workers

    def worker(w):
        while True:
            with lock:
                k = counter[0]
                counter[0] += 1
            drawn[w] += 1
            if k >= n_chunks:
                return
            c = chunk_first + k
            if c >= n_chunks:
                c -= n_chunks
            done.add(c)

    threads = [threading.Thread(target=worker, args=(w,)) for w in range(n_workers) if resident[w]]
    for t in threads:
        t.start()
    for t in threads:
        t.join(10)
    return done, drawn
