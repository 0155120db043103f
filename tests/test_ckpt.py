import json
import os

import torch

from mini_trainer_b200.ckpt import safetensors_io as st
from mini_trainer_b200.ckpt.hf_checkpoint import load_hf_checkpoint, plan_shards, save_hf_checkpoint, save_model
from mini_trainer_b200.ckpt.train_state import load_train_state, save_train_state
from mini_trainer_b200.models.config import ModelConfig, get_preset
from mini_trainer_b200.ops import get_ops
from mini_trainer_b200.parallel.engine import ShardedEngine


def tiny(tied):
    return ModelConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, tie_word_embeddings=tied, attention_bias=True, model_type="qwen2",
                       architectures=["Qwen2ForCausalLM"])


def test_safetensors_interop_with_upstream(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int64), "c": torch.randn(2, 2)}
    st.save_file(t, str(tmp_path / "mine.safetensors"), metadata={"format": "pt"})
    up = load_file(str(tmp_path / "mine.safetensors"))
    assert all(torch.equal(up[k], t[k]) for k in t)
    save_file(t, str(tmp_path / "up.safetensors"))
    mine = st.load_file(str(tmp_path / "up.safetensors"))
    assert all(torch.equal(mine[k], t[k]) and mine[k].dtype == t[k].dtype for k in t)


def test_plan_shards():
    assert plan_shards([("a", 4), ("b", 4), ("c", 4)], 8) == [["a", "b"], ["c"]]
    assert plan_shards([("a", 40)], 8) == [["a"]]


def test_hf_checkpoint_roundtrip_single_and_sharded(tmp_path):
    for tied in (True, False):
        eng = ShardedEngine(tiny(tied), "cpu", get_ops("cpu"))
        eng.init_random(seed=5)
        d1 = str(tmp_path / f"one{tied}")
        save_hf_checkpoint(eng, d1)
        assert os.path.exists(os.path.join(d1, "model.safetensors")) and os.path.exists(os.path.join(d1, "config.json"))
        keys = set(st.load_file(os.path.join(d1, "model.safetensors")))
        assert ("lm_head.weight" in keys) == (not tied)
        assert "model.layers.1.self_attn.k_proj.bias" in keys and "model.layers.0.mlp.up_proj.weight" in keys
        d2 = str(tmp_path / f"many{tied}")
        save_hf_checkpoint(eng, d2, max_shard_bytes=6000)
        idx = json.load(open(os.path.join(d2, "model.safetensors.index.json")))
        assert set(idx["weight_map"]) == keys and idx["metadata"]["total_size"] > 0
        assert all(os.path.exists(os.path.join(d2, f)) for f in set(idx["weight_map"].values()))
        for d in (d1, d2):
            e2 = ShardedEngine(ModelConfig.from_pretrained(d), "cpu", get_ops("cpu"))
            load_hf_checkpoint(e2, d)
            for a, b in zip(eng.groups, e2.groups):
                assert torch.equal(a.master.bfloat16(), b.master.bfloat16())


def test_hf_transformers_loads_our_checkpoint(tmp_path):
    from transformers import AutoModelForCausalLM
    from mini_trainer_b200.models import decoder as D
    from mini_trainer_b200.data.sampler import mb_collate_fn
    cfg = tiny(True)
    eng = ShardedEngine(cfg, "cpu", get_ops("cpu"))
    eng.init_random(seed=2, std=0.05)
    path = save_model(eng, 8192.0, str(tmp_path), None)
    assert path.endswith("hf_format/samples_8192.0")
    hf = AutoModelForCausalLM.from_pretrained(path, torch_dtype=torch.float32)
    ids = torch.randint(0, cfg.vocab_size, (11,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    e2 = ShardedEngine(ModelConfig.from_pretrained(path), "cpu", get_ops("cpu"))
    load_hf_checkpoint(e2, path)
    mb = mb_collate_fn([{"input_ids": ids, "labels": ids, "len": 11, "num_loss_counted_tokens": 11}], 11)
    pb = D.make_packed_batch(mb, "cpu")
    blocks = [g.layout.views(g.shard) for g in e2.blocks]
    mine = D.forward_logits(e2.ops, e2.cfg, e2.embed.layout.views(e2.embed.shard)["embed"], blocks,
                            e2.head.layout.views(e2.head.shard)["norm"], e2.embed.layout.views(e2.embed.shard)["embed"], pb)
    assert torch.allclose(mine, ref, atol=2e-3, rtol=2e-3)


def test_train_state_resume(tmp_path):
    eng = ShardedEngine(tiny(False), "cpu", get_ops("cpu"))
    eng.init_random(seed=1)
    for g in eng.groups:
        g.m.normal_(); g.v.uniform_()
    eng.step_count = 7
    save_train_state(eng, str(tmp_path / "s"), {"scheduler": {"step": 8}})
    e2 = ShardedEngine(tiny(False), "cpu", get_ops("cpu"))
    meta = load_train_state(e2, str(tmp_path / "s"))
    assert e2.step_count == 7 and meta["scheduler"]["step"] == 8
    for a, b in zip(eng.groups, e2.groups):
        assert torch.equal(a.master, b.master) and torch.equal(a.m, b.m) and torch.equal(a.v, b.v)
    # a truncated shard is reported, not silently loaded
    shard = str(tmp_path / "s" / "rank0-of-1.safetensors")
    data = open(shard, "rb").read()
    open(shard, "wb").write(data[: len(data) // 2])
    try:
        load_train_state(e2, str(tmp_path / "s"))
        assert False, "corrupt shard must raise"
    except (RuntimeError, ValueError):
        pass


def test_property_safetensors_roundtrip_with_upstream(tmp_path_factory):
    """Any mix of dtypes and shapes (scalars, empty tensors, non-contiguous views): what this writer stores the upstream
    package reads back bit for bit, and the other way round."""
    import pytest
    pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as hs
    from safetensors.torch import load_file, save_file
    dtypes = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int32, torch.int16, torch.int8,
              torch.uint8, torch.bool]
    spec = hs.lists(hs.tuples(hs.sampled_from(range(len(dtypes))), hs.lists(hs.integers(0, 7), min_size=0, max_size=3),
                              hs.booleans()), min_size=1, max_size=8)
    root = tmp_path_factory.mktemp("st")

    @settings(max_examples=60, deadline=None)
    @given(spec=spec, seed=hs.integers(0, 10 ** 6))
    def run(spec, seed):
        g = torch.Generator().manual_seed(seed)
        tensors = {}
        for i, (d, shape, transpose) in enumerate(spec):
            r = torch.randn(tuple(shape), generator=g)
            t = (r * 50).to(dtypes[d]) if dtypes[d] != torch.bool else r > 0
            if transpose and t.dim() >= 2:
                t = t.transpose(0, 1)   # a non-contiguous view
            tensors[f"t{i}.weight"] = t
        st.save_file(tensors, str(root / "mine.safetensors"), metadata={"format": "pt"})
        up = load_file(str(root / "mine.safetensors"))
        save_file({k: v.contiguous() for k, v in tensors.items()}, str(root / "up.safetensors"))
        mine = st.load_file(str(root / "up.safetensors"))
        for k, t in tensors.items():
            for other in (up[k], mine[k]):
                assert other.dtype == t.dtype and other.shape == t.shape
                if t.numel():   # bit for bit (NaN-safe): compare the raw bytes
                    assert torch.equal(other.contiguous().reshape(-1).view(torch.uint8), t.contiguous().reshape(-1).view(torch.uint8))

    run()
