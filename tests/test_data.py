import json

import torch

from mini_trainer_b200.data.sampler import (InfiniteSampler, JsonlDataset, MaxTokensPerRankCollator,
                                            get_data_loader, mb_collate_fn)
from mini_trainer_b200.data.synthetic import CONFIG_DATA, synthetic_dataset, write_synthetic_jsonl
from mini_trainer_b200.models.decoder import make_packed_batch


def test_sampler_same_on_all_ranks_and_reseeds():
    a, b = iter(InfiniteSampler(10, seed=5)), iter(InfiniteSampler(10, seed=5))
    first = [next(a) for _ in range(10)]
    assert first == [next(b) for _ in range(10)]
    second = [next(a) for _ in range(10)]
    assert sorted(first) == sorted(second) == list(range(10))
    assert first != second
    g = torch.Generator(); g.manual_seed(5)
    assert first == torch.randperm(10, generator=g).tolist()


def test_jsonl_roundtrip(tmp_path):
    spec, vocab, _, _ = CONFIG_DATA["tiny-qwen2"]
    p = tmp_path / "d.jsonl"
    write_synthetic_jsonl(str(p), 20, spec, vocab, seed=1)
    ds = JsonlDataset(str(p))
    assert len(ds) == 20
    rows = [json.loads(l) for l in open(p)]
    s = ds[3]
    assert s["input_ids"].tolist() == rows[3]["input_ids"]
    assert s["labels"].tolist() == rows[3]["labels"]
    assert s["len"] == rows[3]["len"] and s["num_loss_counted_tokens"] == rows[3]["num_loss_counted_tokens"]
    assert s["labels"][0].item() == -100


def test_collate_packs_without_padding():
    samples = [{"input_ids": torch.arange(4), "labels": torch.tensor([-100, 1, 2, 3]), "len": 4, "num_loss_counted_tokens": 3},
               {"input_ids": torch.arange(3), "labels": torch.tensor([-100, -100, 2]), "len": 3, "num_loss_counted_tokens": 1}]
    mb = mb_collate_fn(samples, 99)
    assert mb["input_ids"].shape == (1, 7)
    assert mb["position_ids"].tolist() == [[0, 1, 2, 3, 0, 1, 2]]
    assert mb["cu_seqlens"].tolist() == [0, 4, 7] and mb["max_seqlen"] == 4
    assert mb["num_loss_counted_tokens"] == 4 and mb["num_samples"] == 2 and mb["batch_num_loss_counted_tokens"] == 99
    pb = make_packed_batch(mb, "cpu")
    assert pb.targets.tolist() == [1, 2, 3, -100, -100, 2, -100]


def test_collator_ranks_partition_batch_and_pad_with_dummy():
    spec, vocab, _, _ = CONFIG_DATA["tiny-qwen2"]
    ds = synthetic_dataset(64, spec, vocab, seed=3)
    world = 4
    batch = [ds[i] for i in range(9)]
    outs = [MaxTokensPerRankCollator(100000, rank=r, world_size=world)(batch) for r in range(world)]
    assert len({len(o) for o in outs}) == 1
    total = sum(s["num_loss_counted_tokens"] for s in batch)
    assert sum(mb["num_samples"] for o in outs for mb in o) == 9
    assert sum(mb["num_loss_counted_tokens"] for o in outs for mb in o) == total
    assert all(mb["batch_num_loss_counted_tokens"] == total for o in outs for mb in o)
    # one sample on four ranks: three ranks get the dummy
    outs = [MaxTokensPerRankCollator(100000, rank=r, world_size=world)(batch[:1]) for r in range(world)]
    dummies = [o[0] for o in outs if o[0]["num_samples"] == 0]
    assert len(dummies) == 3
    assert dummies[0]["input_ids"].tolist() == [[15, 14, 13, 12, 11]] and (dummies[0]["labels"] == -100).all()


def test_loader_two_ranks_see_same_batches():
    spec, vocab, mt, bs = CONFIG_DATA["tiny-qwen2"]
    ds = synthetic_dataset(128, spec, vocab, seed=0)
    l0 = iter(get_data_loader(dataset=ds, batch_size=bs, max_tokens_per_gpu=mt, seed=893, rank=0, world_size=2))
    l1 = iter(get_data_loader(dataset=ds, batch_size=bs, max_tokens_per_gpu=mt, seed=893, rank=1, world_size=2, prefetch=0))
    for _ in range(3):
        b0, b1 = next(l0), next(l1)
        assert len(b0) == len(b1)
        assert b0[0]["batch_num_loss_counted_tokens"] == b1[0]["batch_num_loss_counted_tokens"]
        assert sum(m["num_samples"] for m in b0 + b1) == bs
        for m in b0 + b1:
            assert m["input_ids"].shape[1] <= mt


def test_worker_process_loader_yields_the_same_stream_as_the_packing_thread(tmp_path):
    """``num_workers > 0`` (the reference's DataLoader worker processes, sampler.py:285) and the in-process packing thread
    draw the same batches and cut them into the same minibatches; a resumed stream (``skip_batches``) continues both."""
    import json
    spec, vocab, mt, bs = CONFIG_DATA["tiny-qwen2"]
    ds = synthetic_dataset(96, spec, vocab, seed=1)
    path = str(tmp_path / "data.jsonl")
    with open(path, "w") as f:
        for i in range(len(ds)):
            s = ds[i]
            f.write(json.dumps({"input_ids": s["input_ids"].tolist(), "labels": s["labels"].tolist(), "len": s["len"],
                                "num_loss_counted_tokens": s["num_loss_counted_tokens"]}) + "\n")
    kw = dict(data_path=path, batch_size=8, max_tokens_per_gpu=mt, seed=5, rank=1, world_size=2)
    thread = iter(get_data_loader(**kw))
    procs = iter(get_data_loader(**kw, num_workers=2))
    seen = []
    for _ in range(4):
        a, b = next(thread), next(procs)
        assert len(a) == len(b)
        for x, y in zip(a, b):
            assert torch.equal(x["input_ids"], y["input_ids"]) and torch.equal(x["labels"], y["labels"])
            assert torch.equal(x["position_ids"], y["position_ids"]) and x["num_samples"] == y["num_samples"]
        seen.append(a)
    resumed = iter(get_data_loader(**kw, skip_batches=2, num_workers=2))
    for want in seen[2:]:
        got = next(resumed)
        assert all(torch.equal(x["input_ids"], y["input_ids"]) for x, y in zip(want, got))
    if hasattr(thread, "close"):
        thread.close()


# ---------------------------------------------------------------------------------------------
# property-based: the collator over any batch and any world size
# ---------------------------------------------------------------------------------------------
import pytest  # noqa: E402

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st   # noqa: E402


def _sample(n, masked, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 1000, (n,), generator=g)
    labels = ids.clone()
    labels[:masked] = -100
    return {"input_ids": ids, "labels": labels, "len": n, "num_loss_counted_tokens": n - masked}


@settings(max_examples=60, deadline=None)
@given(lens=st.lists(st.integers(min_value=2, max_value=600), min_size=1, max_size=40), world=st.integers(min_value=1, max_value=6),
       budget=st.integers(min_value=50, max_value=2000), frac=st.floats(min_value=0.0, max_value=0.95))
def test_property_collator_partitions_the_batch_and_builds_consistent_minibatches(lens, world, budget, frac):
    """Over all ranks every sample appears once with its tokens and labels intact; every minibatch is one padding-free
    row whose position ids restart per sample and whose cu_seqlens, max_seqlen and token counts agree with it; every
    rank has the same number of minibatches; idle slots hold the dummy sample; the batch-wide loss-token count is the
    same everywhere; the targets are the labels shifted over the whole packed row, as the reference's models compute
    them (the last position of a sample gets the next sample's first label, which tokenised chat data always masks)."""
    batch = [_sample(n, min(n - 1, int(n * frac)), i) for i, n in enumerate(lens)]
    outs = [MaxTokensPerRankCollator(budget, rank=r, world_size=world)(batch) for r in range(world)]
    assert len({len(o) for o in outs}) == 1
    total = sum(s["num_loss_counted_tokens"] for s in batch)
    seen = []
    for o in outs:
        for mb in o:
            ids, labels, pos = mb["input_ids"][0], mb["labels"][0], mb["position_ids"][0]
            cu = mb["cu_seqlens"].tolist()
            assert mb["batch_num_loss_counted_tokens"] == total and cu[0] == 0 and cu[-1] == ids.numel()
            assert mb["max_seqlen"] == max(b - a for a, b in zip(cu[:-1], cu[1:]))
            if mb["num_samples"] == 0:   # the dummy sample of an idle rank
                assert (labels == -100).all() and mb["num_loss_counted_tokens"] == 0
                continue
            assert mb["num_samples"] == len(cu) - 1
            assert ids.numel() <= budget or mb["num_samples"] == 1
            assert mb["num_loss_counted_tokens"] == int((labels != -100).sum())
            targets = make_packed_batch(mb, "cpu").targets
            for a, b in zip(cu[:-1], cu[1:]):
                assert pos[a:b].tolist() == list(range(b - a))
                assert targets[a:b - 1].tolist() == labels[a + 1:b].tolist()
                assert targets[b - 1] == (labels[b] if b < ids.numel() else -100)
                seen.append((tuple(ids[a:b].tolist()), tuple(labels[a:b].tolist())))
            assert targets[-1] == -100
    want = sorted((tuple(s["input_ids"].tolist()), tuple(s["labels"].tolist())) for s in batch)
    assert sorted(seen) == want
