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
