"""End-to-end on a GPU: the native-kernel engine against the fp32 PyTorch-op engine."""
import pytest
import torch

from mini_trainer_b200.data.sampler import mb_collate_fn
from mini_trainer_b200.models import decoder as D
from mini_trainer_b200.models.config import get_preset
from mini_trainer_b200.ops import get_ops
from mini_trainer_b200.parallel.engine import OptimConfig, ShardedEngine

pytestmark = pytest.mark.gpu


def make_mb(lens, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    samples = []
    for n in lens:
        ids = torch.randint(0, vocab, (n,), generator=g)
        labels = ids.clone()
        labels[: max(1, n // 3)] = -100
        samples.append({"input_ids": ids, "labels": labels, "len": n, "num_loss_counted_tokens": int((labels != -100).sum())})
    return mb_collate_fn(samples, sum(s["num_loss_counted_tokens"] for s in samples))


@pytest.mark.parametrize("attention", ["native", "flash_attn"])
def test_native_engine_matches_fp32_reference(attention):
    from mini_trainer_b200.ops.native import NativeOps
    cfg = get_preset("smoke-llama")
    ops = NativeOps("cuda:0", attention=attention)
    if attention == "native" and not hasattr(ops.lib, "mtb200_attn_fwd"):
        pytest.skip("attention kernel not built")
    eng = ShardedEngine(cfg, "cuda:0", ops, optim=OptimConfig())
    eng.init_random(seed=11, std=0.05)
    ref = ShardedEngine(cfg, "cuda:0", get_ops("cuda:0", "torch"), param_dtype=torch.float32, optim=OptimConfig())
    for a, b in zip(eng.groups, ref.groups):     # identical (bf16-rounded) starting weights
        b.master.copy_(a.shard.float()); b.shard.copy_(b.master)
    mb = make_mb([300, 17, 129, 1, 640], cfg.vocab_size)
    batch = D.make_packed_batch(mb, "cuda:0")
    scale = 1.0 / mb["batch_num_loss_counted_tokens"]
    l1 = eng.forward_backward(batch, scale)
    l2 = ref.forward_backward(batch, scale)
    torch.cuda.synchronize()
    ops.check_status()
    assert abs(l1.sum().item() - l2.sum().item()) < 2e-2 * abs(l2.sum().item())
    for a, b in zip(eng.groups, ref.groups):
        err = (a.gacc - b.gacc).norm() / (b.gacc.norm() + 1e-12)
        assert err < 5e-2, (a.layout.name, err.item())
    n1, n2 = eng.optimizer_step(1e-4), ref.optimizer_step(1e-4)
    assert abs(n1.item() - n2.item()) < 3e-2 * n2.item()
    assert ops.launches > 0


@pytest.mark.parametrize("residual_multiplier", [1.0, 0.25])
def test_native_engine_with_projection_biases_matches_fp32_reference(residual_multiplier):
    """``attention_bias`` (q, k, v, o_proj) and ``mlp_bias`` (gate, up, down): bias and residual in one GEMM epilogue,
    bias gradients by the column-sum kernel, with and without Granite's scaling of the biased branch."""
    import dataclasses
    from mini_trainer_b200.ops.native import NativeOps
    cfg = dataclasses.replace(get_preset("smoke-llama"), attention_bias=True, mlp_bias=True)
    if residual_multiplier != 1.0:
        cfg = dataclasses.replace(cfg, model_type="granite", architectures=["GraniteForCausalLM"],
                                  residual_multiplier=residual_multiplier)
    ops = NativeOps("cuda:0")
    eng = ShardedEngine(cfg, "cuda:0", ops, optim=OptimConfig())
    eng.init_random(seed=12, std=0.05)
    biases = ("bqkv", "bo", "bgu", "bd")
    gen = torch.Generator(device="cuda:0").manual_seed(3)
    for grp in eng.blocks:     # random initialisation leaves biases at zero
        views = grp.layout.views(grp.master)
        for n in biases:
            views[n].normal_(0.0, 0.3, generator=gen)
        grp.shard.copy_(grp.master)
    ref = ShardedEngine(cfg, "cuda:0", get_ops("cuda:0", "torch"), param_dtype=torch.float32, optim=OptimConfig())
    for a, b in zip(eng.groups, ref.groups):
        b.master.copy_(a.shard.float()); b.shard.copy_(b.master)
    mb = make_mb([300, 17, 129, 1, 640], cfg.vocab_size)
    batch = D.make_packed_batch(mb, "cuda:0")
    scale = 1.0 / mb["batch_num_loss_counted_tokens"]
    l1 = eng.forward_backward(batch, scale)
    l2 = ref.forward_backward(batch, scale)
    torch.cuda.synchronize()
    ops.check_status()
    assert abs(l1.sum().item() - l2.sum().item()) < 2e-2 * abs(l2.sum().item())
    for a, b in zip(eng.groups, ref.groups):
        err = (a.gacc - b.gacc).norm() / (b.gacc.norm() + 1e-12)
        assert err < 5e-2, (a.layout.name, err.item())
    for a, b in zip(eng.blocks, ref.blocks):
        ga, gb = a.layout.views(a.gacc), b.layout.views(b.gacc)
        for n in biases:
            err = (ga[n] - gb[n]).norm() / (gb[n].norm() + 1e-12)
            assert gb[n].norm() > 0 and err < 5e-2, (a.layout.name, n, err.item())


def test_native_engine_starcoder2_matches_fp32_reference():
    """A Starcoder2-shaped model on the kernels: LayerNorm forward / backward, plain tanh GELU, a bias on every projection,
    tied head; recompute and kept-activation schedules."""
    from mini_trainer_b200.models.config import ModelConfig
    from mini_trainer_b200.ops.native import NativeOps
    cfg = ModelConfig.from_hf_dict(dict(model_type="starcoder2", architectures=["Starcoder2ForCausalLM"], vocab_size=4096,
                                        hidden_size=512, intermediate_size=1536, num_hidden_layers=2, num_attention_heads=4,
                                        num_key_value_heads=1, norm_epsilon=1e-5, use_bias=True, rope_theta=1e5))
    cfg.validate_supported()
    mb = make_mb([300, 17, 129, 1, 640], cfg.vocab_size)
    batch = D.make_packed_batch(mb, "cuda:0")
    scale = 1.0 / mb["batch_num_loss_counted_tokens"]
    for budget in (0, 10 ** 12):
        ops = NativeOps("cuda:0")
        eng = ShardedEngine(cfg, "cuda:0", ops, optim=OptimConfig(), activation_budget_bytes=budget)
        eng.init_random(seed=16, std=0.05)
        gen = torch.Generator(device="cuda:0").manual_seed(7)
        for grp in eng.blocks + [eng.head]:     # random initialisation leaves biases at zero and norm weights at one
            views = grp.layout.views(grp.master)
            for n, v in views.items():
                if n.startswith("b"):
                    v.normal_(0.0, 0.3, generator=gen)
                elif v.dim() == 1:
                    v.uniform_(0.5, 1.5, generator=gen)
            grp.shard.copy_(grp.master)
        ref = ShardedEngine(cfg, "cuda:0", get_ops("cuda:0", "torch"), param_dtype=torch.float32, optim=OptimConfig(),
                            activation_budget_bytes=budget)
        for a, b in zip(eng.groups, ref.groups):
            b.master.copy_(a.shard.float()); b.shard.copy_(b.master)
        l1 = eng.forward_backward(batch, scale)
        l2 = ref.forward_backward(batch, scale)
        torch.cuda.synchronize()
        ops.check_status()
        assert abs(l1.sum().item() - l2.sum().item()) < 2e-2 * abs(l2.sum().item())
        for a, b in zip(eng.groups, ref.groups):
            err = (a.gacc - b.gacc).norm() / (b.gacc.norm() + 1e-12)
            assert err < 5e-2, (a.layout.name, err.item())
        for a, b in zip(eng.blocks, ref.blocks):
            ga, gb = a.layout.views(a.gacc), b.layout.views(b.gacc)
            for n in ("ln1", "bln1", "ln2", "bln2", "bgu", "bd"):
                err = (ga[n] - gb[n]).norm() / (gb[n].norm() + 1e-12)
                assert gb[n].norm() > 0 and err < 5e-2, (a.layout.name, n, err.item())


def test_native_engine_gemma_matches_fp32_reference():
    """A Gemma-shaped model: GeGLU kernel, norms that multiply by (1 + weight), scaled tied embeddings, and head_dim 256,
    for which attention runs through the library kernel (the tcgen05 attention kernels are built for 64 and 128)."""
    from mini_trainer_b200.models.config import ModelConfig
    from mini_trainer_b200.ops.native import NativeOps
    cfg = ModelConfig.from_hf_dict(dict(model_type="gemma", architectures=["GemmaForCausalLM"], vocab_size=4096, hidden_size=512,
                                        intermediate_size=1536, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                                        head_dim=256, rope_theta=1e4, rms_norm_eps=1e-6))
    cfg.validate_supported()
    ops = NativeOps("cuda:0")
    eng = ShardedEngine(cfg, "cuda:0", ops, optim=OptimConfig())
    eng.init_random(seed=15, std=0.05)
    gen = torch.Generator(device="cuda:0").manual_seed(6)
    for grp in eng.blocks:     # random initialisation leaves Gemma's norm weights at zero
        views = grp.layout.views(grp.master)
        for n in ("ln1", "ln2"):
            views[n].normal_(0.0, 0.3, generator=gen)
        grp.shard.copy_(grp.master)
    ref = ShardedEngine(cfg, "cuda:0", get_ops("cuda:0", "torch"), param_dtype=torch.float32, optim=OptimConfig())
    for a, b in zip(eng.groups, ref.groups):
        b.master.copy_(a.shard.float()); b.shard.copy_(b.master)
    mb = make_mb([300, 17, 129, 1, 640], cfg.vocab_size)
    batch = D.make_packed_batch(mb, "cuda:0")
    scale = 1.0 / mb["batch_num_loss_counted_tokens"]
    l1 = eng.forward_backward(batch, scale)
    l2 = ref.forward_backward(batch, scale)
    torch.cuda.synchronize()
    ops.check_status()
    assert abs(l1.sum().item() - l2.sum().item()) < 2e-2 * abs(l2.sum().item())
    for a, b in zip(eng.groups, ref.groups):
        err = (a.gacc - b.gacc).norm() / (b.gacc.norm() + 1e-12)
        assert err < 5e-2, (a.layout.name, err.item())


def test_native_engine_with_head_norm_matches_fp32_reference():
    """Qwen3's per-head q/k norm through the engine on the kernels (recompute and kept-activation schedules)."""
    import dataclasses
    from mini_trainer_b200.ops.native import NativeOps
    cfg = dataclasses.replace(get_preset("smoke-llama"), model_type="qwen3", architectures=["Qwen3ForCausalLM"], qk_norm=True)
    mb = make_mb([300, 17, 129, 1, 640], cfg.vocab_size)
    batch = D.make_packed_batch(mb, "cuda:0")
    scale = 1.0 / mb["batch_num_loss_counted_tokens"]
    for budget in (0, 10 ** 12):
        ops = NativeOps("cuda:0")
        eng = ShardedEngine(cfg, "cuda:0", ops, optim=OptimConfig(), activation_budget_bytes=budget)
        eng.init_random(seed=14, std=0.05)
        gen = torch.Generator(device="cuda:0").manual_seed(5)
        for grp in eng.blocks:     # random initialisation leaves norm weights at one
            views = grp.layout.views(grp.master)
            for n in ("qn", "kn"):
                views[n].uniform_(0.5, 1.5, generator=gen)
            grp.shard.copy_(grp.master)
        ref = ShardedEngine(cfg, "cuda:0", get_ops("cuda:0", "torch"), param_dtype=torch.float32, optim=OptimConfig(),
                            activation_budget_bytes=budget)
        for a, b in zip(eng.groups, ref.groups):
            b.master.copy_(a.shard.float()); b.shard.copy_(b.master)
        l1 = eng.forward_backward(batch, scale)
        l2 = ref.forward_backward(batch, scale)
        torch.cuda.synchronize()
        ops.check_status()
        assert abs(l1.sum().item() - l2.sum().item()) < 2e-2 * abs(l2.sum().item())
        for a, b in zip(eng.groups, ref.groups):
            err = (a.gacc - b.gacc).norm() / (b.gacc.norm() + 1e-12)
            assert err < 5e-2, (a.layout.name, err.item())
        for a, b in zip(eng.blocks, ref.blocks):
            ga, gb = a.layout.views(a.gacc), b.layout.views(b.gacc)
            for n in ("qn", "kn"):
                err = (ga[n] - gb[n]).norm() / (gb[n].norm() + 1e-12)
                assert gb[n].norm() > 0 and err < 5e-2, (a.layout.name, n, err.item())


def test_native_engine_mixture_of_experts_matches_fp32_reference(monkeypatch):
    """A small Mixtral on the kernels: expert slabs of uneven height through the tcgen05 GEMM (row slices of shared
    buffers), row gathers by the embedding kernel, router in torch. The fp32 reference replays the experts the native run
    selected (a near-tie in bf16 may otherwise pick another expert) while its weights follow its own logits."""
    from mini_trainer_b200.models import moe as M
    from mini_trainer_b200.ops.native import NativeOps
    cfg = get_preset("tiny-mixtral")
    ops = NativeOps("cuda:0")
    eng = ShardedEngine(cfg, "cuda:0", ops, optim=OptimConfig(), activation_budget_bytes=0)
    eng.init_random(seed=13, std=0.05)
    ref = ShardedEngine(cfg, "cuda:0", get_ops("cuda:0", "torch"), param_dtype=torch.float32, optim=OptimConfig(),
                        activation_budget_bytes=0)
    for a, b in zip(eng.groups, ref.groups):
        b.master.copy_(a.shard.float()); b.shard.copy_(b.master)
    mb = make_mb([300, 17, 129, 1, 640], cfg.vocab_size)
    batch = D.make_packed_batch(mb, "cuda:0")
    scale = 1.0 / mb["batch_num_loss_counted_tokens"]
    chosen, orig = [], M.route

    def record(cfg_, w, n2):
        r = orig(cfg_, w, n2)
        chosen.append(r[1])
        return r

    monkeypatch.setattr(M, "route", record)
    l1 = eng.forward_backward(batch, scale)
    replay = list(chosen)
    monkeypatch.setattr(M, "route", lambda cfg_, w, n2: orig(cfg_, w, n2, topi=replay.pop(0)))
    l2 = ref.forward_backward(batch, scale)
    torch.cuda.synchronize()
    ops.check_status()
    assert not replay and len(chosen) == 2 * cfg.num_hidden_layers      # forward + recompute of every block
    counts = torch.bincount(chosen[0].reshape(-1), minlength=cfg.num_local_experts)
    assert counts.sum() == 2 * batch.num_tokens and (counts > 0).all()
    assert abs(l1.sum().item() - l2.sum().item()) < 2e-2 * abs(l2.sum().item())
    for a, b in zip(eng.groups, ref.groups):
        err = (a.gacc - b.gacc).norm() / (b.gacc.norm() + 1e-12)
        assert err < 5e-2, (a.layout.name, err.item())
    for a, b in zip(eng.blocks, ref.blocks):
        ga, gb = a.layout.views(a.gacc), b.layout.views(b.gacc)
        for n in ("router", "wgu0", "wd3"):
            err = (ga[n] - gb[n]).norm() / (gb[n].norm() + 1e-12)
            assert err < 6e-2, (a.layout.name, n, err.item())
    n1, n2 = eng.optimizer_step(1e-4), ref.optimizer_step(1e-4)
    assert abs(n1.item() - n2.item()) < 3e-2 * n2.item()


def test_osft_step_runs_with_native_kernels():
    from mini_trainer_b200.ops.native import NativeOps
    from mini_trainer_b200.parallel.osft import enable_osft
    cfg = get_preset("smoke-llama")
    ops = NativeOps("cuda:0")
    eng = ShardedEngine(cfg, "cuda:0", ops, optim=OptimConfig(), activation_budget_bytes=0)
    eng.init_random(seed=2, std=0.05)
    before = [g.master.clone() for g in eng.groups]
    ctl = enable_osft(eng, rank_ratio=0.5)
    mb = make_mb([200, 56, 384], cfg.vocab_size)
    losses = []
    for _ in range(3):
        out = eng.train_step([mb], lr=2e-3)
        losses.append(out["loss_sum"].item())
    ops.check_status()
    assert losses[-1] < losses[0]
    assert any(not torch.equal(a, g.master) for a, g in zip(before, eng.groups))
    assert len(ctl.mats) == 7 * cfg.num_hidden_layers


def test_gpu_engine_exports_hf_checkpoint_that_transformers_loads(tmp_path):
    """bf16 safetensors written from the GPU engine load in transformers and give the same logits
    as the engine's own kernels (bf16 tolerance)."""
    from transformers import AutoModelForCausalLM
    from mini_trainer_b200.ckpt.hf_checkpoint import save_model
    from mini_trainer_b200.ops.native import NativeOps
    cfg = get_preset("smoke-llama")
    ops = NativeOps("cuda:0")
    eng = ShardedEngine(cfg, "cuda:0", ops, optim=OptimConfig())
    eng.init_random(seed=9, std=0.05)
    path = save_model(eng, 64.0, str(tmp_path), None)
    hf = AutoModelForCausalLM.from_pretrained(path, torch_dtype=torch.float32)
    ids = torch.randint(0, cfg.vocab_size, (200,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    mb = mb_collate_fn([{"input_ids": ids, "labels": ids, "len": 200, "num_loss_counted_tokens": 200}], 200)
    pb = D.make_packed_batch(mb, "cuda:0")
    blocks = [g.layout.views(g.shard) for g in eng.blocks]
    head = eng.head.layout.views(eng.head.shard)
    mine = D.forward_logits(ops, cfg, eng.embed.layout.views(eng.embed.shard)["embed"], blocks, head["norm"], head["lm_head"], pb)
    ops.check_status()
    err = ((mine.cpu() - ref).norm() / ref.norm()).item()
    assert err < 3e-2, err


def test_block_inputs_offloaded_to_host_give_identical_gradients(monkeypatch):
    """Checkpoint level 3 (block input parked in pinned host memory during forward, staged back one block
    ahead in backward) changes where a tensor lives, not what is computed: same loss and gradients, bit for bit."""
    from mini_trainer_b200.ops.native import NativeOps
    cfg = get_preset("smoke-llama")
    cfg.num_hidden_layers = 4
    mbs = [make_mb([300, 17, 129, 1, 640], cfg.vocab_size), make_mb([900, 40], cfg.vocab_size, seed=1)]

    def run(offload):
        monkeypatch.setenv("MTB200_OFFLOAD_BLOCKS", "3" if offload else "0")
        eng = ShardedEngine(cfg, "cuda:0", NativeOps("cuda:0"), optim=OptimConfig(), activation_budget_bytes=0)
        eng.init_random(seed=3, std=0.05)
        losses = []
        for k, mb in enumerate(mbs):       # two microbatches of different sizes: the host and staging buffers are reused
            batch = D.make_packed_batch(mb, "cuda:0")
            assert eng.plan_checkpointing(batch.num_tokens) == ([3, 3, 3, 2] if offload else [2, 2, 2, 2])
            losses.append(eng.forward_backward(batch, 1.0 / mb["batch_num_loss_counted_tokens"], last=k == 1).sum().item())
        torch.cuda.synchronize()
        eng.ops.check_status()
        return losses, [g.gacc.clone() for g in eng.groups]

    l0, g0 = run(False)
    l1, g1 = run(True)
    assert l0 == l1
    # the attention backward adds dQ tiles in arrival order (fp32), everything else is deterministic
    for a, b in zip(g0, g1):
        assert ((a - b).norm() / (a.norm() + 1e-12)).item() < 1e-5
