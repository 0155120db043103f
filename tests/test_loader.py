"""Model loading against real Hugging Face directories written by ``transformers`` (CPU).

For every supported family a tiny random model is saved with ``save_pretrained``, loaded through
``trainer.setup_model`` and its logits are compared with ``AutoModelForCausalLM``'s. Also: vocabulary
growth when the tokenizer is larger than the embedding, refusal of architectures whose math the
hand-written block does not implement, and hub-id resolution through the local cache only.
"""
import json
import os

import pytest
import torch

from mini_trainer_b200.data.sampler import mb_collate_fn
from mini_trainer_b200.models import decoder as D
from mini_trainer_b200.models.config import ModelConfig
from mini_trainer_b200.trainer import align_model_and_tokenizer, resolve_model_path, setup_model

transformers = pytest.importorskip("transformers")

COMMON = dict(vocab_size=96, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=512)


def _hf_dir(tmp_path, kind, **over):
    cls = {"llama": (transformers.LlamaConfig, {}), "qwen2": (transformers.Qwen2Config, {}),
           "mistral": (transformers.MistralConfig, {"sliding_window": None}),
           "granite": (transformers.GraniteConfig, {"embedding_multiplier": 12.0, "residual_multiplier": 0.22,
                                                    "attention_multiplier": 0.0625, "logits_scaling": 8.0}),
           "mixtral": (transformers.MixtralConfig, {"sliding_window": None, "num_local_experts": 4,
                                                    "num_experts_per_tok": 2}),
           "phi3": (transformers.Phi3Config, {"pad_token_id": 0, "eos_token_id": 2}),
           "qwen3": (transformers.Qwen3Config, {"head_dim": 32}),
           "gemma": (transformers.GemmaConfig, {"head_dim": 32}),
           "qwen3_moe": (transformers.Qwen3MoeConfig, {"head_dim": 32, "num_experts": 4, "num_experts_per_tok": 2,
                                                       "moe_intermediate_size": 48}),
           "granitemoe": (transformers.GraniteMoeConfig, {"num_local_experts": 4, "num_experts_per_tok": 2,
                                                         "embedding_multiplier": 12.0, "residual_multiplier": 0.22,
                                                         "attention_multiplier": 0.0625, "logits_scaling": 8.0}),
           "smollm3": (transformers.SmolLM3Config, {"num_hidden_layers": 4, "no_rope_layer_interval": 2, "pad_token_id": 0}),
           "qwen2_moe": (transformers.Qwen2MoeConfig, {"num_experts": 4, "num_experts_per_tok": 2, "moe_intermediate_size": 48,
                                                       "shared_expert_intermediate_size": 80}),
           "olmo2": (transformers.Olmo2Config, {"pad_token_id": 0}),
           "starcoder2": (transformers.Starcoder2Config, {"sliding_window": None, "bos_token_id": 1, "eos_token_id": 2})}[kind]
    kw = dict(COMMON, **cls[1])
    kw.update(over)
    cfg = cls[0](**kw)
    torch.manual_seed(0)
    model = transformers.AutoModelForCausalLM.from_config(cfg).to(torch.float32)
    path = str(tmp_path / kind)
    model.save_pretrained(path)
    return path, model


def _our_logits(eng, ids):
    mb = mb_collate_fn([{"input_ids": ids, "labels": ids, "len": len(ids), "num_loss_counted_tokens": len(ids)}], len(ids))
    pb = D.make_packed_batch(mb, "cpu")
    blocks = [g.layout.views(g.master) for g in eng.blocks]
    emb = eng.embed.layout.views(eng.embed.master)["embed"]
    head = eng.head.layout.views(eng.head.master)
    return D.forward_logits(eng.ops, eng.cfg, emb, blocks, head["norm"], head.get("lm_head", emb), pb, norm_b=head.get("bnorm"))


@pytest.mark.parametrize("kind", ["llama", "qwen2", "mistral", "granite", "mixtral", "phi3", "qwen3", "gemma", "starcoder2", "qwen3_moe", "granitemoe", "smollm3", "qwen2_moe", "olmo2"])
def test_setup_model_matches_transformers(tmp_path, kind):
    path, hf = _hf_dir(tmp_path, kind)
    eng = setup_model(path, device="cpu")
    ids = torch.randint(0, COMMON["vocab_size"], (23,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    mine = _our_logits(eng, ids)
    assert torch.allclose(mine, ref, atol=2e-4, rtol=2e-4), float((mine - ref).abs().max())


def test_granite_multipliers_reach_the_gradients(tmp_path):
    """The hand-written backward with all four Granite scalars agrees with autograd through transformers."""
    path, hf = _hf_dir(tmp_path, "granite")
    eng = setup_model(path, device="cpu")
    ids = torch.randint(0, COMMON["vocab_size"], (19,))
    labels = ids.clone()
    labels[:5] = -100
    mb = mb_collate_fn([{"input_ids": ids, "labels": labels, "len": 19, "num_loss_counted_tokens": 14}], 14)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 14, last=True)
    out = hf(input_ids=ids[None], labels=labels[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 14 - float(out.loss)) < 1e-4
    got = eng.blocks[1].layout.views(eng.blocks[1].gacc)
    want = dict(hf.named_parameters())
    assert torch.allclose(got["wd"], want["model.layers.1.mlp.down_proj.weight"].grad, atol=1e-5, rtol=1e-3)
    assert torch.allclose(got["wo"], want["model.layers.1.self_attn.o_proj.weight"].grad, atol=1e-5, rtol=1e-3)
    q = eng.cfg.q_size
    assert torch.allclose(got["wqkv"][:q], want["model.layers.1.self_attn.q_proj.weight"].grad, atol=1e-5, rtol=1e-3)
    emb = eng.embed.layout.views(eng.embed.gacc)["embed"]
    assert torch.allclose(emb, want["model.embed_tokens.weight"].grad, atol=1e-5, rtol=1e-3)


def test_mixture_of_experts_gradients_and_export_against_transformers(tmp_path):
    """Mixtral: router and expert gradients of the hand-written backward against autograd through transformers, and
    the exported checkpoint (published tensor names) loads there and gives the same logits."""
    path, hf = _hf_dir(tmp_path, "mixtral")
    eng = setup_model(path, device="cpu")
    assert eng.cfg.is_moe and not eng.region_overlap
    ids = torch.randint(0, COMMON["vocab_size"], (26,))
    labels = ids.clone()
    labels[:6] = -100
    mb = mb_collate_fn([{"input_ids": ids, "labels": labels, "len": 26, "num_loss_counted_tokens": 20}], 20)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 20, last=True)
    out = hf(input_ids=ids[None], labels=labels[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 20 - float(out.loss)) < 1e-4
    got = eng.blocks[0].layout.views(eng.blocks[0].gacc)
    want = {n: p_.grad for n, p_ in hf.named_parameters()}
    f = eng.cfg.intermediate_size
    L = "model.layers.0.mlp."
    assert torch.allclose(got["router"], want[L + "gate.weight"], atol=1e-5, rtol=1e-3)
    for e in range(4):
        assert torch.allclose(got[f"wgu{e}"], want[L + "experts.gate_up_proj"][e], atol=1e-5, rtol=1e-3)
        assert torch.allclose(got[f"wd{e}"], want[L + "experts.down_proj"][e], atol=1e-5, rtol=1e-3)
    assert torch.allclose(got["wo"], want["model.layers.0.self_attn.o_proj.weight"], atol=1e-5, rtol=1e-3)
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    out_dir = str(tmp_path / "export")
    save_hf_checkpoint(eng, out_dir)
    back = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32)
    with torch.no_grad():
        ref, again = hf(input_ids=ids[None]).logits[0], back(input_ids=ids[None]).logits[0]
    assert torch.allclose(again, ref, atol=0.05, rtol=0.05)   # the export is bf16


def test_qwen3_head_norm_gradients_and_export_against_transformers(tmp_path):
    """Qwen3's RMSNorm over head_dim on every q and k head (before the rotary embedding): gradients of both norm weights
    and of the q/k projections against autograd through transformers; the export loads there."""
    path, hf = _hf_dir(tmp_path, "qwen3")
    with torch.no_grad():   # transformers initialises norm weights to one
        for n, p_ in hf.named_parameters():
            if "q_norm" in n or "k_norm" in n:
                p_.uniform_(0.5, 1.5)
    hf.save_pretrained(path)
    eng = setup_model(path, device="cpu")
    assert eng.cfg.qk_norm and eng.cfg.head_dim == 32
    ids = torch.randint(0, COMMON["vocab_size"], (22,))
    labels = ids.clone()
    labels[:3] = -100
    mb = mb_collate_fn([{"input_ids": ids, "labels": labels, "len": 22, "num_loss_counted_tokens": 19}], 19)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 19, last=True)
    out = hf(input_ids=ids[None], labels=labels[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 19 - float(out.loss)) < 1e-4
    got = eng.blocks[0].layout.views(eng.blocks[0].gacc)
    want = {n: p_.grad for n, p_ in hf.named_parameters()}
    L, q, kv = "model.layers.0.self_attn.", eng.cfg.q_size, eng.cfg.kv_size
    for a, b in [(got["qn"], want[L + "q_norm.weight"]), (got["kn"], want[L + "k_norm.weight"]),
                 (got["wqkv"][:q], want[L + "q_proj.weight"]), (got["wqkv"][q: q + kv], want[L + "k_proj.weight"]),
                 (got["wqkv"][q + kv:], want[L + "v_proj.weight"])]:
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-3), float((a - b).abs().max())
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    out_dir = str(tmp_path / "export")
    save_hf_checkpoint(eng, out_dir)
    back = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32)
    with torch.no_grad():
        ref, again = hf(input_ids=ids[None]).logits[0], back(input_ids=ids[None]).logits[0]
    assert torch.allclose(again, ref, atol=0.05, rtol=0.05)   # the export is bf16


def test_gemma_gradients_and_export_against_transformers(tmp_path):
    """Gemma: norms that multiply by (1 + weight), GeGLU with the tanh GELU, embeddings scaled by sqrt(hidden), tied head.
    Norm-weight, MLP and embedding gradients against autograd through transformers; the export holds ``weight`` itself."""
    path, hf = _hf_dir(tmp_path, "gemma")
    with torch.no_grad():   # transformers initialises Gemma's norm weights to zero
        for n, p_ in hf.named_parameters():
            if "norm" in n:
                p_.normal_(0.0, 0.3)
    hf.save_pretrained(path)
    eng = setup_model(path, device="cpu")
    assert eng.cfg.mlp_act == "gelu_tanh" and eng.cfg.norm_weight_offset == 1.0 and eng.cfg.tie_word_embeddings
    assert abs(eng.cfg.embedding_multiplier - 8.0) < 1e-6
    ids = torch.randint(0, COMMON["vocab_size"], (24,))
    labels = ids.clone()
    labels[:5] = -100
    mb = mb_collate_fn([{"input_ids": ids, "labels": labels, "len": 24, "num_loss_counted_tokens": 19}], 19)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 19, last=True)
    out = hf(input_ids=ids[None], labels=labels[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 19 - float(out.loss)) < 1e-4
    got = eng.blocks[1].layout.views(eng.blocks[1].gacc)
    want = {n: p_.grad for n, p_ in hf.named_parameters()}
    L, f = "model.layers.1.", eng.cfg.intermediate_size
    for a, b in [(got["ln1"], want[L + "input_layernorm.weight"]), (got["ln2"], want[L + "post_attention_layernorm.weight"]),
                 (got["wgu"][:f], want[L + "mlp.gate_proj.weight"]), (got["wgu"][f:], want[L + "mlp.up_proj.weight"]),
                 (got["wd"], want[L + "mlp.down_proj.weight"]),
                 (eng.head.layout.views(eng.head.gacc)["norm"], want["model.norm.weight"]),
                 (eng.embed.layout.views(eng.embed.gacc)["embed"], want["model.embed_tokens.weight"])]:
        assert torch.allclose(a, b, atol=2e-5, rtol=1e-3), float((a - b).abs().max())
    from mini_trainer_b200.ckpt import safetensors_io as st
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    out_dir = str(tmp_path / "export")
    save_hf_checkpoint(eng, out_dir)
    saved = st.load_file(os.path.join(out_dir, "model.safetensors"))
    assert torch.allclose(saved["model.norm.weight"].float(), hf.model.norm.weight.detach(), atol=5e-3)
    back = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32)
    with torch.no_grad():
        ref, again = hf(input_ids=ids[None]).logits[0], back(input_ids=ids[None]).logits[0]
    assert torch.allclose(again, ref, atol=0.08, rtol=0.05)   # the export is bf16


def test_starcoder2_gradients_and_export_against_transformers(tmp_path):
    """Starcoder2: LayerNorm with bias, an MLP without a gate (c_fc, tanh GELU, c_proj), a bias on every projection, tied
    head. Gradients of norms, biases and MLP matrices against autograd through transformers; the export loads there."""
    path, hf = _hf_dir(tmp_path, "starcoder2")
    with torch.no_grad():   # biases start at zero and norm weights at one in transformers
        for n, p_ in hf.named_parameters():
            if n.endswith(".bias"):
                p_.normal_(0.0, 0.3)
            elif "norm" in n:
                p_.uniform_(0.5, 1.5)
    hf.save_pretrained(path)
    eng = setup_model(path, device="cpu")
    cfg = eng.cfg
    assert cfg.norm_type == "layernorm" and not cfg.mlp_gated and cfg.o_proj_bias and cfg.mlp_bias and cfg.tie_word_embeddings
    ids = torch.randint(0, COMMON["vocab_size"], (25,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    assert torch.allclose(_our_logits(eng, ids), ref, atol=3e-4, rtol=3e-4)
    labels = ids.clone()
    labels[:4] = -100
    mb = mb_collate_fn([{"input_ids": ids, "labels": labels, "len": 25, "num_loss_counted_tokens": 21}], 21)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 21, last=True)
    out = hf(input_ids=ids[None], labels=labels[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 21 - float(out.loss)) < 1e-4
    got = eng.blocks[0].layout.views(eng.blocks[0].gacc)
    hg = eng.head.layout.views(eng.head.gacc)
    want = {n: p_.grad for n, p_ in hf.named_parameters()}
    L = "model.layers.0."
    for a, b in [(got["ln1"], want[L + "input_layernorm.weight"]), (got["bln1"], want[L + "input_layernorm.bias"]),
                 (got["ln2"], want[L + "post_attention_layernorm.weight"]), (got["bln2"], want[L + "post_attention_layernorm.bias"]),
                 (got["wgu"], want[L + "mlp.c_fc.weight"]), (got["bgu"], want[L + "mlp.c_fc.bias"]),
                 (got["wd"], want[L + "mlp.c_proj.weight"]), (got["bd"], want[L + "mlp.c_proj.bias"]),
                 (got["bo"], want[L + "self_attn.o_proj.bias"]), (hg["norm"], want["model.norm.weight"]),
                 (hg["bnorm"], want["model.norm.bias"])]:
        assert torch.allclose(a, b, atol=2e-5, rtol=1e-3), float((a - b).abs().max())
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    out_dir = str(tmp_path / "export")
    save_hf_checkpoint(eng, out_dir)
    saved_cfg = json.load(open(os.path.join(out_dir, "config.json")))
    assert saved_cfg["use_bias"] is True and "norm_epsilon" in saved_cfg and "rms_norm_eps" not in saved_cfg
    back = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32)
    with torch.no_grad():
        again = back(input_ids=ids[None]).logits[0]
    assert torch.allclose(again, ref, atol=0.08, rtol=0.05)   # the export is bf16


@pytest.mark.parametrize("rope", [
    {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 128, "rope_theta": 10000.0},
    {"rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 64, "rope_theta": 10000.0, "beta_fast": 16, "beta_slow": 2,
     "attention_factor": 1.3},
    {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64,
     "rope_theta": 10000.0},
    {"rope_type": "linear", "factor": 2.0, "rope_theta": 10000.0},
])
def test_rope_scaling_kinds_match_transformers(tmp_path, rope):
    """YaRN (frequencies and the attention factor on q and k), llama3 and linear scaling: logits of a 300-token sample,
    long enough for the scaled frequencies to matter, against transformers."""
    path, hf = _hf_dir(tmp_path, "llama", rope_parameters=rope)
    eng = setup_model(path, device="cpu")
    ids = torch.randint(0, COMMON["vocab_size"], (300,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    mine = _our_logits(eng, ids)
    assert torch.allclose(mine, ref, atol=5e-4, rtol=5e-4), float((mine - ref).abs().max())


def test_longrope_switches_tables_with_the_longest_sample(tmp_path):
    """Phi-3's long-context rope: per-frequency divisors from the short table up to the original context length, from
    the long table beyond (decided per minibatch by its longest sample), and a constant factor on q and k. Logits of a
    short and of a long sample against transformers, and a training step of each through the engine."""
    short, long = [1.0 + 0.05 * i for i in range(8)], [1.5 + 0.4 * i for i in range(8)]
    path, hf = _hf_dir(tmp_path, "phi3", max_position_embeddings=512, original_max_position_embeddings=64,
                       rope_parameters={"rope_type": "longrope", "short_factor": short, "long_factor": long, "rope_theta": 10000.0,
                                        "original_max_position_embeddings": 64})
    eng = setup_model(path, device="cpu")
    assert eng.cfg.rope_long_context_threshold() == 64 and eng.cfg.rope_attention_factor > 1.0
    for n in (40, 200):
        ids = torch.randint(0, COMMON["vocab_size"], (n,))
        with torch.no_grad():
            ref = hf(input_ids=ids[None]).logits[0]
        mine = _our_logits(eng, ids)
        assert torch.allclose(mine, ref, atol=5e-4, rtol=5e-4), (n, float((mine - ref).abs().max()))
        mb = mb_collate_fn([{"input_ids": ids, "labels": ids, "len": n, "num_loss_counted_tokens": n}], n)
        loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / (n - 1), last=True)
        hf.zero_grad()
        out = hf(input_ids=ids[None], labels=ids[None])
        out.loss.backward()
        assert abs(float(loss.sum()) / (n - 1) - float(out.loss)) < 1e-4
        got = eng.blocks[0].layout.views(eng.blocks[0].gacc)["wqkv"]
        assert torch.allclose(got, hf.model.layers[0].self_attn.qkv_proj.weight.grad, atol=1e-5, rtol=1e-3)
        for g in eng.groups:
            g.has_grad = False


def test_partial_rotary_embedding(tmp_path):
    """Phi-4-mini turns only the leading part of every head: logits and the q/k/v gradient against transformers."""
    path, hf = _hf_dir(tmp_path, "phi3", rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5})
    eng = setup_model(path, device="cpu")
    assert eng.cfg.rotary_dim == 8 and eng.cfg.head_dim == 16 and eng.inv_freq.numel() == 4
    ids = torch.randint(0, COMMON["vocab_size"], (31,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    assert torch.allclose(_our_logits(eng, ids), ref, atol=3e-4, rtol=3e-4)
    mb = mb_collate_fn([{"input_ids": ids, "labels": ids, "len": 31, "num_loss_counted_tokens": 31}], 31)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 30, last=True)
    out = hf(input_ids=ids[None], labels=ids[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 30 - float(out.loss)) < 1e-4
    got = eng.blocks[0].layout.views(eng.blocks[0].gacc)["wqkv"]
    assert torch.allclose(got, hf.model.layers[0].self_attn.qkv_proj.weight.grad, atol=1e-5, rtol=1e-3)


def test_olmo2_post_norm_block_gradients_against_transformers(tmp_path):
    """OLMo-2: norms behind the branches and an RMSNorm over the whole q and the whole k projection; every kind of
    gradient of a block against autograd through transformers, and the export."""
    path, hf = _hf_dir(tmp_path, "olmo2")
    with torch.no_grad():
        for n, p_ in hf.named_parameters():
            if "norm" in n:
                p_.uniform_(0.5, 1.5)
    hf.save_pretrained(path)
    eng = setup_model(path, device="cpu")
    assert eng.cfg.post_norm and tuple(eng.blocks[0].layout.specs["qn"].shape) == (eng.cfg.q_size,)
    ids = torch.randint(0, COMMON["vocab_size"], (27,))
    labels = ids.clone()
    labels[:5] = -100
    mb = mb_collate_fn([{"input_ids": ids, "labels": labels, "len": 27, "num_loss_counted_tokens": 22}], 22)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 22, last=True)
    out = hf(input_ids=ids[None], labels=labels[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 22 - float(out.loss)) < 1e-4
    got = eng.blocks[0].layout.views(eng.blocks[0].gacc)
    want = {n: p_.grad for n, p_ in hf.named_parameters()}
    L, q, f = "model.layers.0.", eng.cfg.q_size, eng.cfg.intermediate_size
    for a, b in [(got["qn"], want[L + "self_attn.q_norm.weight"]), (got["kn"], want[L + "self_attn.k_norm.weight"]),
                 (got["ln1"], want[L + "post_attention_layernorm.weight"]), (got["ln2"], want[L + "post_feedforward_layernorm.weight"]),
                 (got["wqkv"][:q], want[L + "self_attn.q_proj.weight"]), (got["wo"], want[L + "self_attn.o_proj.weight"]),
                 (got["wgu"][:f], want[L + "mlp.gate_proj.weight"]), (got["wd"], want[L + "mlp.down_proj.weight"])]:
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-3), float((a - b).abs().max())
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    out_dir = str(tmp_path / "export")
    save_hf_checkpoint(eng, out_dir)
    back = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32)
    with torch.no_grad():
        ref, again = hf(input_ids=ids[None]).logits[0], back(input_ids=ids[None]).logits[0]
    assert torch.allclose(again, ref, atol=0.05, rtol=0.05)   # the export is bf16


def test_smollm3_layers_without_rotary_embedding(tmp_path):
    """SmolLM3: every second layer of this tiny model applies no rotary embedding; gradients of a rotated and of a
    not rotated layer against autograd through transformers."""
    path, hf = _hf_dir(tmp_path, "smollm3")
    eng = setup_model(path, device="cpu")
    assert eng.cfg.no_rope_layers == [1, 0, 1, 0] and not eng.cfg.layer_uses_rope(1)
    ids = torch.randint(0, COMMON["vocab_size"], (20,))
    mb = mb_collate_fn([{"input_ids": ids, "labels": ids, "len": 20, "num_loss_counted_tokens": 20}], 20)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 19, last=True)
    out = hf(input_ids=ids[None], labels=ids[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 19 - float(out.loss)) < 1e-4
    want = {n: p_.grad for n, p_ in hf.named_parameters()}
    q = eng.cfg.q_size
    for layer in (0, 1):
        got = eng.blocks[layer].layout.views(eng.blocks[layer].gacc)
        assert torch.allclose(got["wqkv"][:q], want[f"model.layers.{layer}.self_attn.q_proj.weight"], atol=1e-5, rtol=1e-3)


def test_phi3_export_keeps_the_fused_tensor_names(tmp_path):
    """Phi-3 stores q|k|v and gate|up fused; the export writes them the same way and transformers loads it."""
    path, hf = _hf_dir(tmp_path, "phi3", sliding_window=64)
    eng = setup_model(path, device="cpu")
    assert eng.cfg.attention_window == 64
    from mini_trainer_b200.ckpt import safetensors_io as st
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    out_dir = str(tmp_path / "export")
    save_hf_checkpoint(eng, out_dir)
    names = set(st.load_file(os.path.join(out_dir, "model.safetensors")))
    assert "model.layers.0.self_attn.qkv_proj.weight" in names and "model.layers.1.mlp.gate_up_proj.weight" in names
    back = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32)
    ids = torch.randint(0, COMMON["vocab_size"], (17,))
    with torch.no_grad():
        ref, again = hf(input_ids=ids[None]).logits[0], back(input_ids=ids[None]).logits[0]
    assert torch.allclose(again, ref, atol=0.05, rtol=0.05)   # the export is bf16


@pytest.mark.parametrize("renorm", [False, True])
def test_qwen3_moe_gradients_against_transformers(tmp_path, renorm):
    """Qwen3-MoE: per-head q/k norm plus routed experts of their own width, with and without renormalising the chosen
    weights; router, expert and norm gradients against autograd through transformers; export under the published names."""
    path, hf = _hf_dir(tmp_path, "qwen3_moe", norm_topk_prob=renorm)
    eng = setup_model(path, device="cpu")
    cfg = eng.cfg
    assert cfg.is_moe and cfg.qk_norm and cfg.norm_topk_prob == renorm and cfg.expert_intermediate_size == 48
    ids = torch.randint(0, COMMON["vocab_size"], (26,))
    labels = ids.clone()
    labels[:6] = -100
    mb = mb_collate_fn([{"input_ids": ids, "labels": labels, "len": 26, "num_loss_counted_tokens": 20}], 20)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 20, last=True)
    out = hf(input_ids=ids[None], labels=labels[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 20 - float(out.loss)) < 1e-4
    got = eng.blocks[0].layout.views(eng.blocks[0].gacc)
    want = {n: p_.grad for n, p_ in hf.named_parameters()}
    L = "model.layers.0."
    assert torch.allclose(got["router"], want[L + "mlp.gate.weight"], atol=1e-5, rtol=1e-3)
    for e in range(4):
        assert torch.allclose(got[f"wgu{e}"], want[L + "mlp.experts.gate_up_proj"][e], atol=1e-5, rtol=1e-3)
        assert torch.allclose(got[f"wd{e}"], want[L + "mlp.experts.down_proj"][e], atol=1e-5, rtol=1e-3)
    assert torch.allclose(got["qn"], want[L + "self_attn.q_norm.weight"], atol=1e-5, rtol=1e-3)
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    out_dir = str(tmp_path / "export")
    save_hf_checkpoint(eng, out_dir)
    back = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32)
    with torch.no_grad():
        ref, again = hf(input_ids=ids[None]).logits[0], back(input_ids=ids[None]).logits[0]
    assert torch.allclose(again, ref, atol=0.05, rtol=0.05)   # the export is bf16


def test_granite_moe_gradients_and_stacked_export_against_transformers(tmp_path):
    """Granite-MoE: Granite's multipliers around routed experts whose checkpoint stacks every projection into one 3-D
    tensor. Router and expert gradients against autograd through transformers; the export stacks them again."""
    path, hf = _hf_dir(tmp_path, "granitemoe")
    eng = setup_model(path, device="cpu")
    assert eng.cfg.is_moe and eng.cfg.residual_multiplier == 0.22
    ids = torch.randint(0, COMMON["vocab_size"], (26,))
    labels = ids.clone()
    labels[:6] = -100
    mb = mb_collate_fn([{"input_ids": ids, "labels": labels, "len": 26, "num_loss_counted_tokens": 20}], 20)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 20, last=True)
    out = hf(input_ids=ids[None], labels=labels[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 20 - float(out.loss)) < 1e-4
    got = eng.blocks[1].layout.views(eng.blocks[1].gacc)
    want = {n: p_.grad for n, p_ in hf.named_parameters()}
    L = "model.layers.1.block_sparse_moe."
    assert torch.allclose(got["router"], want[L + "router.layer.weight"], atol=1e-5, rtol=1e-3)
    for e in range(4):
        assert torch.allclose(got[f"wgu{e}"], want[L + "input_linear.weight"][e], atol=1e-5, rtol=1e-3)
        assert torch.allclose(got[f"wd{e}"], want[L + "output_linear.weight"][e], atol=1e-5, rtol=1e-3)
    from mini_trainer_b200.ckpt import safetensors_io as st
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    out_dir = str(tmp_path / "export")
    save_hf_checkpoint(eng, out_dir)
    saved = st.load_file(os.path.join(out_dir, "model.safetensors"))
    assert tuple(saved[L + "input_linear.weight"].shape) == (4, 2 * COMMON["intermediate_size"], COMMON["hidden_size"])
    back = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32)
    with torch.no_grad():
        ref, again = hf(input_ids=ids[None]).logits[0], back(input_ids=ids[None]).logits[0]
    assert torch.allclose(again, ref, atol=0.05, rtol=0.05)   # the export is bf16


def test_qwen2_moe_shared_expert_gradients_against_transformers(tmp_path):
    """Qwen2-MoE: routed experts plus one shared expert weighted by a sigmoid gate; gradients of the gate vector, the
    shared expert, a routed expert and the router against autograd through transformers; the export loads there."""
    path, hf = _hf_dir(tmp_path, "qwen2_moe")
    eng = setup_model(path, device="cpu")
    assert eng.cfg.shared_expert_intermediate_size == 80 and eng.cfg.attention_bias and not eng.cfg.o_proj_bias
    ids = torch.randint(0, COMMON["vocab_size"], (26,))
    labels = ids.clone()
    labels[:6] = -100
    mb = mb_collate_fn([{"input_ids": ids, "labels": labels, "len": 26, "num_loss_counted_tokens": 20}], 20)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 20, last=True)
    out = hf(input_ids=ids[None], labels=labels[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 20 - float(out.loss)) < 1e-4
    got = eng.blocks[0].layout.views(eng.blocks[0].gacc)
    want = {n: p_.grad for n, p_ in hf.named_parameters()}
    L, fs = "model.layers.0.mlp.", 80
    for a, b in [(got["wsg"], want[L + "shared_expert_gate.weight"]), (got["wgus"][:fs], want[L + "shared_expert.gate_proj.weight"]),
                 (got["wgus"][fs:], want[L + "shared_expert.up_proj.weight"]), (got["wds"], want[L + "shared_expert.down_proj.weight"]),
                 (got["router"], want[L + "gate.weight"]), (got["wgu2"], want[L + "experts.gate_up_proj"][2]),
                 (got["wd2"], want[L + "experts.down_proj"][2]), (got["bqkv"][: eng.cfg.q_size], want["model.layers.0.self_attn.q_proj.bias"])]:
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-3), float((a - b).abs().max())
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    out_dir = str(tmp_path / "export")
    save_hf_checkpoint(eng, out_dir)
    back = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32)
    with torch.no_grad():
        ref, again = hf(input_ids=ids[None]).logits[0], back(input_ids=ids[None]).logits[0]
    assert torch.allclose(again, ref, atol=0.05, rtol=0.05)   # the export is bf16


def test_mixture_of_experts_with_auxiliary_loss_is_refused(tmp_path):
    path, _ = _hf_dir(tmp_path, "mixtral", output_router_logits=True)
    with pytest.raises(ValueError, match="load-balancing loss"):
        setup_model(path, device="cpu")


class _Tok:
    pad_token_id, bos_token_id, eos_token_id = 3, 1, 2

    def __init__(self, n):
        self.n = n

    def __len__(self):
        return self.n


def test_vocabulary_growth_keeps_old_rows_and_initialises_new_ones(tmp_path):
    path, hf = _hf_dir(tmp_path, "llama")
    cfg = ModelConfig.from_pretrained(path)
    cfg.bos_token_id, cfg.pad_token_id = 7, None
    cfg = align_model_and_tokenizer(cfg, _Tok(101))
    # next multiple of 8; an id both sides define is synced, one the model leaves unset stays unset (as the reference)
    assert cfg.vocab_size == 104 and cfg.bos_token_id == 1 and cfg.pad_token_id is None
    from mini_trainer_b200.ckpt.hf_checkpoint import load_hf_checkpoint
    from mini_trainer_b200.ops import get_ops
    from mini_trainer_b200.parallel.engine import ShardedEngine
    eng = ShardedEngine(cfg, "cpu", get_ops("cpu"))
    load_hf_checkpoint(eng, path)
    emb = eng.embed.layout.views(eng.embed.master)["embed"]
    old = hf.model.embed_tokens.weight.detach()
    assert emb.shape == (104, 64) and torch.equal(emb[:96], old)
    assert torch.allclose(emb[96:], old.mean(0, keepdim=True).expand(8, -1), atol=1e-6)
    lm = eng.head.layout.views(eng.head.master)["lm_head"]
    assert torch.equal(lm[:96], hf.lm_head.weight.detach()) and lm.shape[0] == 104
    # the old tokens' logits are unchanged by the growth
    ids = torch.randint(0, 96, (9,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    assert torch.allclose(_our_logits(eng, ids)[:, :96], ref, atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("kind", ["llama", "granite"])
def test_projection_biases_reach_logits_gradients_and_exports(tmp_path, kind):
    """``attention_bias`` (q, k, v and o_proj) and ``mlp_bias`` (gate, up, down), as the Granite code models have them:
    logits and every bias gradient against transformers (for Granite with its residual multiplier scaling the
    biased branch), and the exported checkpoint carries the biases under their Hugging Face names."""
    path, hf = _hf_dir(tmp_path, kind, attention_bias=True, mlp_bias=True)
    with torch.no_grad():   # transformers initialises biases to zero; give them values
        for n, p_ in hf.named_parameters():
            if n.endswith(".bias"):
                p_.normal_(0.0, 0.5)
    hf.save_pretrained(path)
    eng = setup_model(path, device="cpu")
    assert eng.cfg.o_proj_bias and {"bqkv", "bo", "bgu", "bd"} <= set(eng.blocks[0].layout.specs)
    ids = torch.randint(0, COMMON["vocab_size"], (21,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    mine = _our_logits(eng, ids)
    assert torch.allclose(mine, ref, atol=3e-4, rtol=3e-4), float((mine - ref).abs().max())
    labels = ids.clone()
    labels[:4] = -100
    mb = mb_collate_fn([{"input_ids": ids, "labels": labels, "len": 21, "num_loss_counted_tokens": 17}], 17)
    loss = eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 17, last=True)
    out = hf(input_ids=ids[None], labels=labels[None])
    out.loss.backward()
    assert abs(float(loss.sum()) / 17 - float(out.loss)) < 1e-4
    got = eng.blocks[0].layout.views(eng.blocks[0].gacc)
    want = {n: p_.grad for n, p_ in hf.named_parameters()}
    L, q, kv, f = "model.layers.0.", eng.cfg.q_size, eng.cfg.kv_size, eng.cfg.intermediate_size
    pairs = [(got["bo"], want[L + "self_attn.o_proj.bias"]), (got["bd"], want[L + "mlp.down_proj.bias"]),
             (got["bgu"][:f], want[L + "mlp.gate_proj.bias"]), (got["bgu"][f:], want[L + "mlp.up_proj.bias"]),
             (got["bqkv"][:q], want[L + "self_attn.q_proj.bias"]), (got["bqkv"][q + kv:], want[L + "self_attn.v_proj.bias"]),
             (got["wd"], want[L + "mlp.down_proj.weight"]), (got["wo"], want[L + "self_attn.o_proj.weight"])]
    for a, b in pairs:
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-3), float((a - b).abs().max())
    from mini_trainer_b200.ckpt.hf_checkpoint import save_hf_checkpoint
    out_dir = str(tmp_path / "export")
    save_hf_checkpoint(eng, out_dir)
    back = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32)
    with torch.no_grad():
        again = back(input_ids=ids[None]).logits[0]
    assert torch.allclose(again, ref, atol=0.05, rtol=0.05)   # the export is bf16
    assert back.model.layers[1].mlp.down_proj.bias.abs().sum() > 0


@pytest.mark.parametrize("kind,over,needle", [
    ("llama", {"hidden_act": "gelu"}, "hidden_act"),
    ("llama", {"attention_dropout": 0.1}, "attention_dropout"),
    ("phi3", {"resid_pdrop": 0.1}, "resid_pdrop"),
    ("starcoder2", {"residual_dropout": 0.1}, "residual_dropout"),
    ("llama", {"rope_parameters": {"rope_type": "dynamic", "factor": 4.0, "rope_theta": 10000.0}}, "rope scaling"),
])
def test_models_the_block_cannot_compute_are_refused(tmp_path, kind, over, needle):
    path, _ = _hf_dir(tmp_path, kind, **over)
    with pytest.raises(ValueError, match=needle):
        setup_model(path, device="cpu")


def test_sliding_window_model_is_trained_up_to_the_window_and_refused_beyond(tmp_path):
    """A Mistral with a 32-token window: a 23-token sample gives transformers' logits (the window changes nothing up to
    its length), a 40-token sample is refused instead of being run through full causal attention."""
    path, hf = _hf_dir(tmp_path, "mistral", sliding_window=32)
    eng = setup_model(path, device="cpu")
    assert eng.cfg.attention_window == 32
    ids = torch.randint(0, COMMON["vocab_size"], (23,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    assert torch.allclose(_our_logits(eng, ids), ref, atol=2e-4, rtol=2e-4)
    long = torch.randint(0, COMMON["vocab_size"], (40,))
    mb = mb_collate_fn([{"input_ids": long, "labels": long, "len": 40, "num_loss_counted_tokens": 40}], 40)
    with pytest.raises(ValueError, match="sliding window of 32"):
        eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / 40, last=True)
    # Qwen2 carries a window in its config but only applies it with use_sliding_window
    assert ModelConfig.from_hf_dict({**COMMON, "model_type": "qwen2", "sliding_window": 32}).attention_window is None
    assert ModelConfig.from_hf_dict({**COMMON, "model_type": "qwen2", "sliding_window": 32,
                                     "use_sliding_window": True}).attention_window == 32


def test_dropout_can_be_waived_and_the_export_keeps_the_models_value(tmp_path):
    path, _ = _hf_dir(tmp_path, "starcoder2", residual_dropout=0.1)
    eng = setup_model(path, device="cpu", no_dropout=True)
    assert eng.cfg.to_hf_dict()["residual_dropout"] == 0.1 and "ignore_dropout" not in eng.cfg.to_hf_dict()


def test_unknown_architecture_is_refused(tmp_path):
    path, _ = _hf_dir(tmp_path, "llama")
    cfg = json.load(open(os.path.join(path, "config.json")))
    cfg["architectures"], cfg["model_type"] = ["FalconForCausalLM"], "falcon"
    json.dump(cfg, open(os.path.join(path, "config.json"), "w"))
    with pytest.raises(ValueError, match="FalconForCausalLM"):
        setup_model(path, device="cpu")


def test_hub_id_resolves_through_the_local_cache_only(tmp_path, monkeypatch):
    monkeypatch.setenv("HF_HOME", str(tmp_path / "hf_home"))
    monkeypatch.setenv("HF_HUB_OFFLINE", "1")
    with pytest.raises(FileNotFoundError, match="local Hugging Face cache"):
        resolve_model_path("nobody/not-a-cached-model")
    path, _ = _hf_dir(tmp_path, "llama")
    assert resolve_model_path(path) == path


def test_granite_config_round_trips_its_scalars(tmp_path):
    path, _ = _hf_dir(tmp_path, "granite")
    cfg = ModelConfig.from_pretrained(path)
    assert (cfg.embedding_multiplier, cfg.residual_multiplier, cfg.attention_multiplier, cfg.logits_scaling) == (12.0, 0.22, 0.0625, 8.0)
    out = str(tmp_path / "again.json")
    cfg.to_json_file(out)
    d = json.load(open(out))
    assert d["logits_scaling"] == 8.0 and d["model_type"] == "granite"
    llama = ModelConfig.from_pretrained(_hf_dir(tmp_path, "llama")[0]).to_hf_dict()
    assert "logits_scaling" not in llama and "embedding_multiplier" not in llama
