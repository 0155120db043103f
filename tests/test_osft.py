"""OSFT: factor gradients, orthogonal projection and the recomposed update against a float64
autograd oracle that trains the same low-subspace factors directly."""
import torch

from mini_trainer_b200.models.config import ModelConfig
from mini_trainer_b200.models.torch_oracle import oracle_per_token_loss
from mini_trainer_b200.ops import get_ops
from mini_trainer_b200.parallel import osft as O
from mini_trainer_b200.parallel.engine import OptimConfig, ShardedEngine
from tests.test_engine_cpu import make_mb


def test_projection_removes_frozen_subspace():
    torch.manual_seed(0)
    w = torch.randn(24, 40, dtype=torch.float64)
    u_hi, s_hi, v_hi, u_lo, s_lo, v_lo = O.svd_split(w, 0.5)
    assert torch.allclose((u_hi * s_hi) @ v_hi + (u_lo * s_lo) @ v_lo, w, atol=1e-10)
    g = torch.randn_like(w)
    du, ds, dv = O.factor_grads(g, u_lo, s_lo, v_lo)
    # chain rule check against autograd
    ul, sl, vl = (t.clone().requires_grad_(True) for t in (u_lo, s_lo, v_lo))
    (((ul * sl) @ vl) * g).sum().backward()
    assert torch.allclose(du, ul.grad) and torch.allclose(ds, sl.grad) and torch.allclose(dv, vl.grad)
    du, dv = O.project_orthogonal(du + u_hi @ torch.randn(u_hi.shape[1], du.shape[1], dtype=torch.float64), dv, u_hi, v_hi)
    assert (u_hi.t() @ du).abs().max() < 1e-10 and (dv @ v_hi.t()).abs().max() < 1e-10


import pytest


def _llama_with_biases():
    return ModelConfig(vocab_size=61, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, tie_word_embeddings=False, attention_bias=True)


def _starcoder2():   # LayerNorm, an MLP without a gate (six projections per block), biases everywhere, tied head
    return ModelConfig.from_hf_dict(dict(model_type="starcoder2", architectures=["Starcoder2ForCausalLM"], vocab_size=61,
                                         hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                                         num_key_value_heads=2, norm_epsilon=1e-5, use_bias=True))


@pytest.mark.parametrize("make_cfg", [_llama_with_biases, _starcoder2])
def test_osft_training_matches_float64_oracle(make_cfg):
    cfg = make_cfg()
    eng = ShardedEngine(cfg, "cpu", get_ops("cpu"), optim=OptimConfig(max_grad_norm=1.0))
    eng.init_random(seed=4, std=0.2)
    ctl = O.enable_osft(eng, rank_ratio=0.5)

    # oracle parameters: the controller's own factors (an SVD is only unique up to signs) in float64
    base = {k: v.double() for k, v in eng.iter_hf_tensors(dtype=torch.float32)}
    label = {(n, r0): lab for n, r0, r1, lab in O.osft_targets(cfg)}
    fac = {}
    for mt in ctl.mats:
        pre = f"model.layers.{mt.block}." + ("self_attn." if "proj" in label[(mt.name, mt.r0)] and label[(mt.name, mt.r0)][0] in "qkvo" else "mlp.")
        key = pre + label[(mt.name, mt.r0)] + ".weight"
        fac[key] = dict(w_hi=mt.w_hi.double(), u_hi=mt.u_hi.double(), v_hi=mt.v_hi.double(),
                        p=[t.double().clone().requires_grad_(True) for t in ctl.factors(mt)])
        del base[key]
    others = {k: v.clone().requires_grad_(True) for k, v in base.items()}
    leaves = [t for f in fac.values() for t in f["p"]] + list(others.values())
    opt = torch.optim.AdamW(leaves, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.0)

    for step in range(2):
        mb = make_mb([9, 5, 7], cfg.vocab_size, seed=step)
        out = eng.train_step([mb], lr=1e-2)
        sd = dict(others)
        for k, f in fac.items():
            u, s, v = f["p"]
            sd[k] = f["w_hi"] + (u * s) @ v
        loss = oracle_per_token_loss(cfg, sd, mb["input_ids"][0], mb["labels"][0], mb["position_ids"][0]).double()
        (loss.sum() / mb["batch_num_loss_counted_tokens"]).backward()
        for f in fac.values():
            u, s, v = f["p"]
            du, dv = O.project_orthogonal(u.grad, v.grad, f["u_hi"], f["v_hi"])
            u.grad, v.grad = du, dv
        gn = torch.nn.utils.clip_grad_norm_(leaves, 1.0)
        opt.step(); opt.zero_grad()
        assert abs(out["grad_norm"].item() - gn.item()) < 2e-3 * gn.item()
        assert abs(out["loss_sum"].item() - loss.sum().item()) < 1e-3 * loss.sum().item()

    new = {k: v for k, v in eng.iter_hf_tensors(dtype=torch.float32)}
    for k, f in fac.items():
        u, s, v = f["p"]
        ref = (f["w_hi"] + (u * s) @ v).detach().float()
        assert torch.allclose(new[k], ref, atol=3e-4, rtol=1e-3), k
    # AdamW moves an element by about lr * g / (|g| + eps): where a gradient is of the order of eps (1e-8) the fp32 run and
    # the float64 oracle may take visibly different steps, so a stray element per tensor is tolerated, a wrong tensor is not
    for k, v in others.items():
        ref = v.detach().float()
        bad = ((new[k] - ref).abs() > 3e-4 + 1e-3 * ref.abs()).float().mean().item()
        assert bad < 2e-3, (k, bad)


def _osft_worker(rank, world, port, out_path):
    import os
    import torch.distributed as dist
    from mini_trainer_b200.parallel.comm import make_comm
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = ModelConfig(vocab_size=61, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, tie_word_embeddings=False, attention_bias=True)
    eng = ShardedEngine(cfg, "cpu", get_ops("cpu"), comm=make_comm("auto"), optim=OptimConfig(max_grad_norm=1.0))
    eng.init_random(seed=4, std=0.2)
    ctl = O.enable_osft(eng, rank_ratio=0.5)
    assert {m.owner for m in ctl.mats} == set(range(world))          # the factor state is spread over the ranks
    norms = []
    for step in range(3):
        # every rank sees the same three samples; rank r trains on samples r, r + world, ... (disjoint shares)
        lens = [9, 5, 7, 6]
        mbs = [make_mb([n], cfg.vocab_size, seed=10 * step + j) for j, n in enumerate(lens)]
        total = sum(mb["num_loss_counted_tokens"] for mb in mbs)
        mine = mbs[rank::world]
        for mb in mine:
            mb["batch_num_loss_counted_tokens"] = total
        out = eng.train_step(mine, lr=1e-2)
        norms.append(out["grad_norm"].item())
    weights = {k: v.clone() for k, v in eng.iter_hf_tensors(dtype=torch.float32)}
    if rank == 0:
        torch.save({"norms": norms, "weights": weights}, out_path)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def test_osft_two_gloo_ranks_match_one_rank(tmp_path):
    """Ownership by matrix across two ranks (gradients gathered, owners update, recomposed weights handed back)
    reproduces the single-rank run: same gradient norms, same weights after three steps."""
    import socket
    import torch.multiprocessing as mp
    f1, f2 = str(tmp_path / "one.pt"), str(tmp_path / "two.pt")
    _osft_worker(0, 1, 0, f1)
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mp.spawn(_osft_worker, args=(2, port, f2), nprocs=2, join=True)
    a, b = torch.load(f1), torch.load(f2)
    for x, y in zip(a["norms"], b["norms"]):
        assert abs(x - y) < 1e-4 * max(1.0, abs(x)), (a["norms"], b["norms"])
    for k in a["weights"]:
        assert torch.allclose(a["weights"][k], b["weights"][k], atol=2e-5, rtol=1e-4), k


def test_gram_svd_reconstructs_and_spans_the_same_top_subspace():
    """The fast decomposition (eigenproblem of the small Gram matrix) against the exact SVD: same singular
    values, same frozen subspace, exact reconstruction; tall and wide matrices."""
    torch.manual_seed(1)
    for shape in ((96, 40), (40, 96), (64, 64)):
        w = torch.randn(*shape, dtype=torch.float64)
        u, s, vh = O.svd_thin(w, "gram")
        ue, se, vhe = O.svd_thin(w, "exact")
        assert torch.allclose(s, se, rtol=1e-8, atol=1e-10)
        assert torch.allclose((u * s) @ vh, w, atol=1e-10)
        k = s.numel() // 2
        # projectors onto the top-k left / right singular subspaces agree
        assert torch.allclose(u[:, :k] @ u[:, :k].t(), ue[:, :k] @ ue[:, :k].t(), atol=1e-7)
        assert torch.allclose(vh[:k].t() @ vh[:k], vhe[:k].t() @ vhe[:k], atol=1e-7)
    w32 = torch.randn(80, 48)
    u, s, vh = O.svd_thin(w32, "gram")
    assert ((u * s) @ vh - w32).abs().max() < 1e-4


def test_training_state_carries_the_osft_factors(tmp_path):
    """A training-state checkpoint of an OSFT run holds the trainable factors and their moments; loading it into a
    fresh engine (which decomposes the ORIGINAL weights again) restores them, so the resumed run continues the
    same trajectory instead of restarting the low subspace from the export."""
    from mini_trainer_b200.ckpt.train_state import load_train_state, save_train_state
    cfg = ModelConfig(vocab_size=61, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, tie_word_embeddings=False, attention_bias=True)

    def fresh():
        eng = ShardedEngine(cfg, "cpu", get_ops("cpu"), optim=OptimConfig(max_grad_norm=1.0))
        eng.init_random(seed=4, std=0.2)
        return eng, O.enable_osft(eng, rank_ratio=0.5)

    eng, ctl = fresh()
    mbs = [make_mb([9, 5, 7], cfg.vocab_size, seed=s) for s in range(3)]
    for mb in mbs[:2]:
        eng.train_step([mb], lr=1e-2)
    save_train_state(eng, str(tmp_path / "state"))
    out_a = eng.train_step([mbs[2]], lr=1e-2)
    wa = {k: v.clone() for k, v in eng.iter_hf_tensors(dtype=torch.float32)}

    eng2, ctl2 = fresh()
    load_train_state(eng2, str(tmp_path / "state"))
    assert eng2.step_count == 2 and ctl2.fac_m.abs().sum() > 0          # moments restored, not zero as after a fresh start
    out_b = eng2.train_step([mbs[2]], lr=1e-2)
    assert abs(out_a["grad_norm"].item() - out_b["grad_norm"].item()) < 1e-5
    wb = {k: v for k, v in eng2.iter_hf_tensors(dtype=torch.float32)}
    for k in wa:
        assert torch.allclose(wa[k], wb[k], atol=1e-6), k
