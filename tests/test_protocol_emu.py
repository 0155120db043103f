"""Flag protocol of the symmetric-memory kernels, emulated on the host with injected faults."""
import threading

from mini_trainer_b200.parallel.protocol_emu import EmuFabric, EmuRank


def run_ranks(world, body):
    out, threads = [None] * world, []
    for r in range(world):
        t = threading.Thread(target=lambda r=r: out.__setitem__(r, body(r)))
        t.start(); threads.append(t)
    for t in threads:
        t.join(20)
    return out


def test_reduce_scatter_with_buffer_reuse():
    world, steps, n = 4, 6, 8
    fab = EmuFabric(world)

    def body(r):
        me, res = EmuRank(fab, r), []
        for s in range(steps):
            slot = s % 2
            me.publish(slot, [(r + 1) * (s + 1)] * (world * n))
            res.append(me.reduce_scatter(slot))
        return me.status, res

    for status, res in run_ranks(world, body):
        assert status == 0
        for s, vals in enumerate(res):
            assert vals == [sum((p + 1) * (s + 1) for p in range(world))] * n


def test_missing_peer_times_out_with_status_instead_of_hanging():
    world = 3
    fab = EmuFabric(world)

    def body(r):
        me = EmuRank(fab, r, timeout_s=0.2)
        if r == 2:
            return "absent", None            # this rank raised / never joined: it publishes nothing
        me.publish(0, [1.0] * (world * 2))
        return me.status, me.reduce_scatter(0) if me.status == 0 else None, me.status

    res = run_ranks(world, body)
    for r in (0, 1):
        out = res[r]
        assert out[1] is None and (out[2] & 0xff) == 41 and (out[2] >> 8) == 2   # waited for rank 2's "ready"


def test_dropped_message_is_detected_by_the_receiver_only():
    world = 2
    fab = EmuFabric(world)

    def body(r):
        me = EmuRank(fab, r, timeout_s=0.2)
        me.publish(0, [float(r)] * 4, drop_to={1} if r == 0 else None)   # rank 0's signal to rank 1 is lost
        return me.reduce_scatter(0), me.status

    res = run_ranks(world, body)
    assert res[0][0] == [1.0, 1.0] and res[0][1] == 0
    assert res[1][0] is None and (res[1][1] & 0xff) == 41 and (res[1][1] >> 8) == 0


def test_reduction_by_region_with_buffer_reuse_waits_only_for_the_last_region():
    """Four regions published back to front and reduced in that order; the buffer is reused every second step.
    Sums are right, the regions that do not touch a rank's slice come back empty, and no buffer is rewritten
    while a peer still owes a read of any region, although only the last region's consumed row is awaited."""
    import random
    from mini_trainer_b200.parallel.protocol_emu import EmuRegionRank
    world, steps, total = 4, 8, 32
    regions = [(24, 32), (12, 24), (4, 12), (0, 4)]          # back to front, like wd | wgu | wo+ln2 | ln1+wqkv
    fab = EmuFabric(world, rows=2 * len(regions) * 2)

    def body(r):
        rng = random.Random(r)
        me, res = EmuRegionRank(fab, r, regions), []
        for s in range(steps):
            slot, got = s % 2, {}
            for k, (lo, hi) in enumerate(regions):
                me.publish_region(slot, k, [float((r + 1) * (s + 1) + i) for i in range(lo, hi)])
                if rng.random() < 0.5:
                    threading.Event().wait(0.001)             # skew between ranks
                lo_i, vals = me.reduce_region(slot, k)
                for j, v in enumerate(vals):
                    got[lo_i + j] = v
            res.append(got)
        return me.status, me.overwritten_early, res

    for r, (status, early, res) in enumerate(run_ranks(world, body)):
        assert status == 0 and not early
        for s, got in enumerate(res):
            assert sorted(got) == list(range(r * 8, r * 8 + 8))              # exactly my slice, every element once
            for i, v in got.items():
                assert v == sum((p + 1) * (s + 1) + i for p in range(world))


def test_chunks_by_ticket_arrive_even_when_most_workers_never_run():
    from mini_trainer_b200.parallel.protocol_emu import ticket_gather
    n_chunks, n_workers = 53, 16
    done, drawn = ticket_gather(n_chunks, n_workers, [True] * n_workers, chunk_first=20)
    assert done == set(range(n_chunks)) and sum(drawn) == n_chunks + n_workers    # every worker overshoots exactly once
    resident = [w in (3, 11) for w in range(n_workers)]                            # 14 of 16 CTAs are still waiting for an SM
    done, drawn = ticket_gather(n_chunks, n_workers, resident)
    assert done == set(range(n_chunks))
    static = {k for k in range(n_chunks) if resident[k % n_workers]}                # what ownership by index would have gathered
    assert len(static) < n_chunks
