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
