"""Packer correctness, invariants, oracle agreement and the greedy-vs-LPT comparison
(test model: the reference's tests/test_batch_lengths_to_minibatches.py)."""
import os
import sys
import time

import numpy as np
import pytest

from mini_trainer_b200.data import packer as P


def all_ranks(fn, lengths, max_tokens, num_ranks):
    return [fn(lengths, max_tokens, num_ranks, r) for r in range(num_ranks)]


def check_invariants(lengths, max_tokens, num_ranks, per_rank):
    n_mb = {len(x) for x in per_rank}
    assert len(n_mb) == 1, "all ranks must have the same number of minibatches"
    seen = []
    for r in range(num_ranks):
        for mb in per_rank[r]:
            real = [i for i in mb if i != -1]
            assert mb == [-1] or (-1 not in mb and len(mb) > 0)
            load = sum(lengths[i] for i in real)
            assert load <= max_tokens or len(real) == 1, "budget exceeded by a multi-sample minibatch"
            seen += real
    assert sorted(seen) == list(range(len(lengths))), "every sample exactly once"


PACKERS = [P.batch_lengths_to_minibatches_lpt, P.batch_lengths_to_minibatches]


@pytest.mark.parametrize("fn", PACKERS)
def test_empty_batch(fn):
    assert fn([], 100, 4, 0) == []


@pytest.mark.parametrize("fn", PACKERS)
def test_single_sequence(fn):
    res = all_ranks(fn, [50], 100, 4)
    assert res[0] == [[0]]
    assert all(r == [[-1]] for r in res[1:])


@pytest.mark.parametrize("fn", PACKERS)
def test_invariants_random(fn):
    rng = np.random.default_rng(42)
    for trial in range(20):
        n = int(rng.integers(1, 200))
        lengths = rng.integers(1, 5000, n).tolist()
        ranks = int(rng.integers(1, 9))
        res = all_ranks(fn, lengths, 8000, ranks)
        check_invariants(lengths, 8000, ranks, res)


def test_oversize_sample_is_kept_alone():
    lengths = [50000, 25000, 140000, 30000, 150000, 20000]
    res = P.lpt_pack_all(lengths, 130000, 4)
    check_invariants(lengths, 130000, 4, res)
    flat = [mb for r in res for mb in r]
    assert [4] in flat and [2] in flat


def test_native_matches_python_oracle():
    assert P.native_available(), "host library must build here"
    rng = np.random.default_rng(0)
    for trial in range(50):
        n = int(rng.integers(1, 300))
        lengths = rng.integers(1, 3000, n).tolist()  # many ties on purpose
        ranks = int(rng.integers(1, 9))
        assert P.lpt_pack_all(lengths, 6000, ranks) == P.lpt_pack_all_py(lengths, 6000, ranks)
        for r in range(ranks):
            assert (P.batch_lengths_to_minibatches(lengths, 6000, ranks, r, use_native=True)
                    == P.batch_lengths_to_minibatches(lengths, 6000, ranks, r, use_native=False))


def _reference_lpt():
    ref = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.exists(os.path.join(ref, "batch_packer.py")):
        return None
    sys.path.insert(0, ref)
    try:
        from batch_packer import batch_lengths_to_minibatches_lpt
        return batch_lengths_to_minibatches_lpt
    except Exception:
        return None
    finally:
        sys.path.remove(ref)


def test_same_schedule_as_reference_without_ties():
    ref = _reference_lpt()
    if ref is None:
        pytest.skip("reference packer not installed")
    rng = np.random.default_rng(7)
    for trial in range(5):
        lengths = rng.permutation(np.arange(100, 100 + 150) * 37).tolist()  # unique lengths
        for ranks in (2, 8):
            mine = P.lpt_pack_all(lengths, 130000 // 8, ranks)
            for r in range(ranks):
                assert mine[r] == ref(lengths, 130000 // 8, ranks, r)


def realistic(rng, n):
    kinds = rng.choice(4, n, p=[0.5, 0.3, 0.15, 0.05])
    lo = np.array([100, 2000, 20000, 60000])[kinds]
    hi = np.array([2000, 20000, 60000, 100000])[kinds]
    return rng.integers(lo, hi).tolist()


def test_lpt_beats_greedy_on_balance():
    rng = np.random.default_rng(42)
    lengths = realistic(rng, 500)
    lpt = P.packing_stats(lengths, P.lpt_pack_all(lengths, 130000, 8), 130000)
    greedy_lists = [P.batch_lengths_to_minibatches(lengths, 130000, 8, r) for r in range(8)]
    greedy = P.packing_stats(lengths, greedy_lists, 130000)
    assert lpt["num_minibatches"] <= greedy["num_minibatches"]
    assert lpt["avg_balance"] > greedy["avg_balance"]
    assert lpt["row_efficiency"] > greedy["row_efficiency"]


def test_speed_1000_sequences_8_ranks():
    rng = np.random.default_rng(1)
    lengths = realistic(rng, 1000)
    P.lpt_pack_all(lengths, 130000, 8)
    t0 = time.perf_counter()
    for _ in range(10):
        P.lpt_pack_all(lengths, 130000, 8)
    ms = (time.perf_counter() - t0) / 10 * 1e3
    print(f"LPT all-ranks 1000 seqs x 8 ranks: {ms:.2f} ms")
    assert ms < 50


def test_cost_aware_packing_balances_compute_not_tokens():
    """Same samples, same budget: balancing len*(1+len/L0) lowers the slowest rank's cost."""
    rng = np.random.default_rng(5)
    lengths = np.clip(np.rint(rng.lognormal(7.5, 1.0, 128)), 64, 65536).astype(int).tolist()
    L0 = 38574.0
    cost = lambda l: l * (1 + l / L0)

    def step_cost(per_rank):
        n_mb = len(per_rank[0])
        return sum(max(sum(cost(lengths[i]) for i in per_rank[r][m] if i >= 0) for r in range(8)) for m in range(n_mb))

    tok = P.lpt_pack_all(lengths, 64000, 8)
    cst = P.lpt_pack_all(lengths, 64000, 8, cost_len=L0)
    check_invariants(lengths, 64000, 8, cst)
    assert cst == P.lpt_pack_all(lengths, 64000, 8, cost_len=L0, use_native=False)
    assert step_cost(cst) <= step_cost(tok)
    ideal = sum(cost(l) for l in lengths) / 8
    assert step_cost(cst) < 1.05 * ideal or step_cost(cst) < 0.97 * step_cost(tok)


# ---------------------------------------------------------------------------------------------
# property-based: any batch, any budget, any world size
# ---------------------------------------------------------------------------------------------
hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st   # noqa: E402

_batches = st.lists(st.integers(min_value=1, max_value=70000), min_size=1, max_size=120)


@settings(max_examples=120, deadline=None)
@given(lengths=_batches, max_tokens=st.integers(min_value=1, max_value=70000), ranks=st.integers(min_value=1, max_value=9),
       cost_len=st.sampled_from([None, 500.0, 8000.0, 1e9]))
def test_property_every_schedule_is_a_partition_within_budget(lengths, max_tokens, ranks, cost_len):
    """Every sample exactly once, every rank the same number of minibatches, the token budget only exceeded by a sample
    that is alone, padding minibatches are exactly ``[-1]``: for the token-balancing and the cost-balancing LPT packer
    and the greedy one, whatever the input (ties, samples above the budget, more ranks than samples)."""
    check_invariants(lengths, max_tokens, ranks, P.lpt_pack_all(lengths, max_tokens, ranks, cost_len=cost_len))
    if cost_len is None:
        check_invariants(lengths, max_tokens, ranks, all_ranks(P.batch_lengths_to_minibatches, lengths, max_tokens, ranks))


@settings(max_examples=80, deadline=None)
@given(lengths=_batches, max_tokens=st.integers(min_value=1, max_value=70000), ranks=st.integers(min_value=1, max_value=9),
       cost_len=st.sampled_from([None, 2000.0]))
def test_property_compiled_packer_equals_python_oracle(lengths, max_tokens, ranks, cost_len):
    if not P.native_available():
        pytest.skip("host library not built")
    assert P.lpt_pack_all(lengths, max_tokens, ranks, cost_len=cost_len, use_native=True) == \
        P.lpt_pack_all(lengths, max_tokens, ranks, cost_len=cost_len, use_native=False)
    for r in range(ranks):
        assert P.batch_lengths_to_minibatches(lengths, max_tokens, ranks, r, use_native=True) == \
            P.batch_lengths_to_minibatches(lengths, max_tokens, ranks, r, use_native=False)


@settings(max_examples=60, deadline=None)
@given(lengths=_batches, ranks=st.integers(min_value=1, max_value=8))
def test_property_lpt_never_needs_more_minibatches_than_samples_and_is_order_invariant(lengths, ranks):
    """The schedule depends on the multiset of lengths, not on the order of the batch (stable ties aside: compare loads)."""
    budget = max(lengths)
    a = P.lpt_pack_all(lengths, budget, ranks)
    b = P.lpt_pack_all(list(reversed(lengths)), budget, ranks)
    assert len(a[0]) == len(b[0]) <= len(lengths)
    rev = list(reversed(lengths))
    loads_a = sorted(sum(lengths[i] for i in mb if i != -1) for r in a for mb in r)
    loads_b = sorted(sum(rev[i] for i in mb if i != -1) for r in b for mb in r)
    assert loads_a == loads_b
