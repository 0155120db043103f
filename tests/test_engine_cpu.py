"""Hand-written backward + sharding engine against the autograd oracle (CPU, fp32)."""
import torch

from mini_trainer_b200.data.sampler import mb_collate_fn
from mini_trainer_b200.models import decoder as D
from mini_trainer_b200.models.config import ModelConfig, get_preset
from mini_trainer_b200.models.torch_oracle import oracle_per_token_loss
from mini_trainer_b200.ops import get_ops
from mini_trainer_b200.parallel.engine import OptimConfig, ShardedEngine


def small_cfg(tied: bool, bias: bool) -> ModelConfig:
    return ModelConfig(vocab_size=97, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, rope_theta=1e4,
                       tie_word_embeddings=tied, attention_bias=bias, rms_norm_eps=1e-6)


def make_mb(lens, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    samples = []
    for n in lens:
        ids = torch.randint(0, vocab, (n,), generator=g)
        labels = ids.clone()
        labels[: max(1, n // 3)] = -100
        samples.append({"input_ids": ids, "labels": labels, "len": n,
                        "num_loss_counted_tokens": int((labels != -100).sum())})
    total = sum(s["num_loss_counted_tokens"] for s in samples)
    return mb_collate_fn(samples, total)


def hf_state(engine):
    return {k: v.clone() for k, v in engine.iter_hf_tensors(dtype=torch.float32)}


def moe_cfg(experts: int = 4, top_k: int = 2) -> ModelConfig:
    return ModelConfig(vocab_size=97, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, rope_theta=1e4, rms_norm_eps=1e-6,
                       model_type="mixtral", architectures=["MixtralForCausalLM"],
                       num_local_experts=experts, num_experts_per_tok=top_k)


def check_grads(tied, bias, cfg=None):
    torch.manual_seed(0)
    cfg = cfg or small_cfg(tied, bias)
    eng = ShardedEngine(cfg, "cpu", get_ops("cpu"), optim=OptimConfig(lr=1e-3))
    eng.init_random(seed=3, std=0.2)
    mb = make_mb([7, 1, 12, 5], cfg.vocab_size)
    sd = {k: v.double().requires_grad_(True) for k, v in hf_state(eng).items()}
    # oracle (fp32 math inside, fp64 leaves would change dtype; keep fp32)
    sd = {k: v.float().detach().requires_grad_(True) for k, v in sd.items()}
    loss_o = oracle_per_token_loss(cfg, sd, mb["input_ids"][0], mb["labels"][0], mb["position_ids"][0])
    scale = 1.0 / mb["batch_num_loss_counted_tokens"]
    (loss_o.sum() * scale).backward()

    batch = D.make_packed_batch(mb, "cpu")
    loss_e = eng.forward_backward(batch, scale)
    assert torch.allclose(loss_e, loss_o.detach(), atol=1e-4, rtol=1e-4)
    # compare gradients through the HF-name mapping
    from mini_trainer_b200.models import layout as L
    for grp, it in eng._hf_iters():
        views = grp.layout.views(grp.gacc)
        for name, gview in it(views):
            ref = sd[name].grad
            assert ref is not None, name
            err = (gview - ref).abs().max().item()
            assert err < 2e-4 * max(1.0, ref.abs().max().item()), (name, err)


def test_grads_untied_nobias():
    check_grads(False, False)


def test_grads_tied_bias():
    check_grads(True, True)


def test_grads_head_norm():
    """Qwen3's per-head q/k norm against the autograd oracle, in all three checkpoint levels."""
    import dataclasses
    cfg = dataclasses.replace(small_cfg(False, False), model_type="qwen3", architectures=["Qwen3ForCausalLM"], qk_norm=True)
    check_grads(False, False, cfg)
    _check_levels(cfg)


def starcoder2_cfg() -> ModelConfig:
    return ModelConfig.from_hf_dict(dict(model_type="starcoder2", architectures=["Starcoder2ForCausalLM"], vocab_size=97,
                                         hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                                         num_key_value_heads=2, norm_epsilon=1e-5, use_bias=True))


def test_grads_layernorm_and_plain_gelu_mlp():
    """Starcoder2's block (LayerNorm with bias, c_proj(gelu(c_fc(x))), biases everywhere, tied head) against the
    autograd oracle, in all three checkpoint levels."""
    check_grads(True, True, starcoder2_cfg())
    _check_levels(starcoder2_cfg())


def test_grads_post_norm_block():
    """OLMo-2's block against the autograd oracle, in all three checkpoint levels."""
    cfg = ModelConfig.from_hf_dict(dict(model_type="olmo2", architectures=["Olmo2ForCausalLM"], vocab_size=97, hidden_size=32,
                                        intermediate_size=48, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2))
    check_grads(False, False, cfg)
    _check_levels(cfg)


def test_grads_mixture_of_experts():
    """Router (softmax, top-k, renormalisation) and routed SwiGLU experts against a dense autograd restatement."""
    check_grads(False, False, moe_cfg())


def test_grads_mixture_of_experts_with_an_idle_expert(monkeypatch):
    """16 experts for 25 tokens x 1 choice: several experts get no token; their gradients must be zero, not what the
    (here NaN-poisoned) gradient buffer held before."""
    monkeypatch.setenv("MTB200_POISON", "1")
    check_grads(False, False, moe_cfg(experts=16, top_k=1))


def test_adamw_matches_torch():
    cfg = small_cfg(False, True)
    eng = ShardedEngine(cfg, "cpu", get_ops("cpu"), optim=OptimConfig(lr=1e-2, max_grad_norm=1.0))
    eng.init_random(seed=1, std=0.2)
    sd = {k: v.float().detach().requires_grad_(True) for k, v in hf_state(eng).items()}
    opt = torch.optim.AdamW(list(sd.values()), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.0)
    for step in range(3):
        mb = make_mb([9, 4, 6], cfg.vocab_size, seed=step)
        out = eng.train_step([mb], lr=1e-2)
        loss = oracle_per_token_loss(cfg, sd, mb["input_ids"][0], mb["labels"][0], mb["position_ids"][0])
        (loss.sum() / mb["batch_num_loss_counted_tokens"]).backward()
        gn = torch.nn.utils.clip_grad_norm_(list(sd.values()), 1.0)
        opt.step()
        opt.zero_grad()
        assert abs(out["grad_norm"].item() - gn.item()) < 1e-3 * max(1.0, gn.item())
        assert abs(out["loss_sum"].item() - loss.sum().item()) < 1e-3 * abs(loss.sum().item())
    new = hf_state(eng)
    for k, v in sd.items():
        assert torch.allclose(new[k], v.detach(), atol=2e-4, rtol=1e-3), k


def test_checkpoint_levels_give_identical_gradients():
    """Keeping the attention output (level 1) or every GEMM output (level 0) must not change the math."""
    _check_levels(small_cfg(False, True))


def test_checkpoint_levels_give_identical_gradients_mixture_of_experts():
    _check_levels(moe_cfg())


def test_grads_and_checkpoint_levels_with_a_shared_expert():
    """Qwen2-MoE's block (q/k/v biases, routed experts of their own width without renormalisation, a sigmoid-gated
    shared expert) against the autograd oracle and across the checkpoint levels."""
    cfg = ModelConfig.from_hf_dict(dict(model_type="qwen2_moe", architectures=["Qwen2MoeForCausalLM"], vocab_size=97,
                                        hidden_size=32, intermediate_size=48, moe_intermediate_size=24,
                                        shared_expert_intermediate_size=40, num_hidden_layers=2, num_attention_heads=4,
                                        num_key_value_heads=2, num_experts=4, num_experts_per_tok=2))
    check_grads(False, True, cfg)
    _check_levels(cfg)


def _check_levels(cfg):
    mb = make_mb([11, 3, 8], cfg.vocab_size, seed=4)
    grads = []
    for budget in (0, None, 10 ** 12):
        eng = ShardedEngine(cfg, "cpu", get_ops("cpu"), optim=OptimConfig(), activation_budget_bytes=budget)
        eng.init_random(seed=6, std=0.2)
        if budget is None:   # force level 1 everywhere
            eng.plan_checkpointing = lambda tokens: [1] * cfg.num_hidden_layers
        else:
            assert set(eng.plan_checkpointing(22)) == ({2} if budget == 0 else {0})
        eng.forward_backward(D.make_packed_batch(mb, "cpu"), 1.0 / mb["batch_num_loss_counted_tokens"])
        grads.append([g.gacc.clone() for g in eng.groups])
    for other in grads[1:]:
        for a, b in zip(grads[0], other):
            assert torch.allclose(a, b, atol=1e-6, rtol=1e-5)


def test_head_on_counted_rows_only_matches_full_head():
    """The LM head runs on the rows whose target is not -100; loss and gradients equal the all-rows path."""
    import dataclasses
    cfg = small_cfg(False, False)
    mb = make_mb([9, 3, 14], cfg.vocab_size, seed=5)
    outs = []
    for full in (False, True):
        eng = ShardedEngine(cfg, "cpu", get_ops("cpu"), optim=OptimConfig(lr=1e-3))
        eng.init_random(seed=3, std=0.2)
        batch = D.make_packed_batch(mb, "cpu")
        assert batch.loss_rows is not None and 0 < batch.loss_rows.numel() < batch.num_tokens
        if full:
            batch = dataclasses.replace(batch, loss_rows=None, loss_targets=None)
        loss = eng.forward_backward(batch, 0.1)
        outs.append((loss, [g.gacc.clone() for g in eng.groups]))
    assert torch.allclose(outs[0][0], outs[1][0], atol=1e-6)
    for a, b in zip(outs[0][1], outs[1][1]):
        assert torch.allclose(a, b, atol=1e-6, rtol=1e-5)


def test_minibatch_without_counted_tokens_gives_zero_loss_and_head_gradient():
    cfg = small_cfg(True, True)
    eng = ShardedEngine(cfg, "cpu", get_ops("cpu"), optim=OptimConfig(lr=1e-3))
    eng.init_random(seed=3, std=0.2)
    ids = torch.tensor([15, 14, 13, 12, 11])
    mb = mb_collate_fn([{"input_ids": ids, "labels": torch.full((5,), -100), "len": 5, "num_loss_counted_tokens": 0}], 7)
    batch = D.make_packed_batch(mb, "cpu")
    assert batch.loss_rows.numel() == 0
    loss = eng.forward_backward(batch, 1.0 / 7)
    assert float(loss.abs().sum()) == 0.0
    assert all(float(g.gacc.abs().sum()) == 0.0 for g in eng.groups)
