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
