"""Every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

from mini_trainer_b200.ops.torch_ref import TorchOps

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from mini_trainer_b200.ops.native import NativeOps
    return NativeOps("cuda:0")


REF = TorchOps()


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def max_err(a, b, rtol=2e-2):
    """Largest elementwise error beyond ``rtol * |reference|``, in units of the reference's RMS value: a
    handful of wrong elements in a large output barely moves the Frobenius norm but shows up here."""
    a, b = a.float(), b.float()
    excess = ((a - b).abs() - rtol * b.abs()).clamp_min(0.0)
    return (excess.max() / (b.pow(2).mean().sqrt() + 1e-12)).item()


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


GEMM_SHAPES = [(128, 256, 64), (128, 256, 128), (256, 512, 256), (300, 520, 200), (5, 64, 72), (1000, 1024, 4096),
               (777, 2048, 1000), (4096, 6144, 4096), (129, 264, 8)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_forward_layout(ops, M, N, K):
    torch.manual_seed(M + N + K)
    x, w = bf(M, K), bf(N, K, scale=0.05)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.gemm(x, False, w, False, out, M, N, K)
    ref = x.float() @ w.float().t()
    assert rel_err(out, ref) < 6e-3 and max_err(out, ref) < 5e-2
    ops.check_status()


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_dgrad_layout(ops, M, N, K):
    # out[M, N] = A[M, K] @ B[K, N]  (B stored [K, N]: MN-major)
    torch.manual_seed(1 + M + N + K)
    a, b = bf(M, K), bf(K, N, scale=0.05)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.gemm(a, False, b, True, out, M, N, K)
    assert rel_err(out, a.float() @ b.float()) < 6e-3 and max_err(out, a.float() @ b.float()) < 5e-2
    ops.check_status()


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_wgrad_layout(ops, M, N, K):
    # out[M, N] = A[K, M]^T @ B[K, N]  (both MN-major)
    torch.manual_seed(2 + M + N + K)
    if M % 8:
        pytest.skip("leading dimension of an MN-major A must be a multiple of 8")
    a, b = bf(K, M), bf(K, N, scale=0.05)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.gemm(a, True, b, True, out, M, N, K)
    assert rel_err(out, a.float().t() @ b.float()) < 6e-3 and max_err(out, a.float().t() @ b.float()) < 5e-2
    ops.check_status()


def test_gemm_epilogues(ops):
    M, N, K = 384, 776, 320
    x, w, bias, res = bf(M, K), bf(N, K, scale=0.05), bf(N), bf(M, N)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.gemm(x, False, w, False, out, M, N, K, residual=res, bias=bias)
    ref = x.float() @ w.float().t() + bias.float() + res.float()
    assert rel_err(out, ref) < 6e-3
    o32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.gemm(x, False, w, False, o32, M, N, K)
    assert rel_err(o32, x.float() @ w.float().t()) < 1e-5 + 1e-3
    ops.gemm(x, False, w, False, o32, M, N, K, residual=o32)   # accumulate in place
    assert rel_err(o32, 2 * (x.float() @ w.float().t())) < 2e-3
    # alpha scales the product before bias and residual are added
    ops.gemm(x, False, w, False, out, M, N, K, residual=res, bias=bias, alpha=0.25)
    assert rel_err(out, 0.25 * (x.float() @ w.float().t()) + bias.float() + res.float()) < 6e-3
    ops.check_status()


@pytest.mark.parametrize("two_cta", [False, True])
def test_gemm_strided_views(ops, two_cta):
    """Outputs, residuals and operands that are column or row slices of wider buffers, which is how
    the engine calls the kernel (dx[a:a+n], q/k/v column blocks of the fused qkv activation)."""
    M, N, K = 384, 520, 320
    xw = bf(M, K + 64)
    x = xw[:, 32:32 + K]                       # operand with a leading dimension larger than K
    w = bf(N, K, scale=0.05)
    ref = x.float() @ w.float().t()
    wide = torch.full((M, N + 64), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm(x, False, w, False, wide[:, 32:32 + N], M, N, K, two_cta=two_cta)
    assert rel_err(wide[:, 32:32 + N], ref) < 6e-3 and max_err(wide[:, 32:32 + N], ref) < 5e-2
    assert (wide[:, :32] == 7.0).all() and (wide[:, 32 + N:] == 7.0).all()      # nothing outside the view is touched
    tall = torch.full((M + 100, N), 7.0, dtype=torch.bfloat16, device="cuda")
    rw = bf(M, N + 8)
    ops.gemm(x, False, w, False, tall[50:50 + M], M, N, K, residual=rw[:, 8:], two_cta=two_cta)
    assert rel_err(tall[50:50 + M], ref + rw[:, 8:].float()) < 6e-3
    assert (tall[:50] == 7.0).all() and (tall[50 + M:] == 7.0).all()
    ops.check_status()


def test_linear_ops_match_reference(ops):
    T, K, N = 333, 256, 520
    x, w, b, r = bf(T, K), bf(N, K, scale=0.05), bf(N), bf(T, N)
    assert rel_err(ops.linear(x, w, b, r), REF.linear(x.float(), w.float(), b.float(), r.float())) < 6e-3
    dy = bf(T, N)
    assert rel_err(ops.linear_dgrad(dy, w), dy.float() @ w.float()) < 6e-3
    dw, db = torch.empty_like(w), torch.empty_like(b)
    ops.linear_wgrad(dy, x, dw, db)
    assert rel_err(dw, dy.float().t() @ x.float()) < 6e-3
    assert rel_err(db, dy.float().sum(0)) < 6e-3


@pytest.mark.parametrize("T,H", [(1, 256), (37, 1536), (500, 4096), (64, 8192), (300, 3584)])
def test_rmsnorm(ops, T, H):
    x, w, dy, res = bf(T, H), (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16(), bf(T, H), bf(T, H)
    y, rstd = ops.rmsnorm(x, w, 1e-5)
    yr, rr = REF.rmsnorm(x, w, 1e-5)
    assert rel_err(y, yr) < 4e-3 and rel_err(rstd, rr) < 1e-5
    dw, dwr = torch.empty_like(w), torch.empty(H, dtype=torch.float32, device="cuda")
    dx = ops.rmsnorm_bwd(dy, x, rstd, w, dw, add_to=res)
    dxr = REF.rmsnorm_bwd(dy.float(), x.float(), rr, w.float(), dwr, add_to=res.float())
    assert rel_err(dx, dxr) < 6e-3 and rel_err(dw, dwr) < 1e-2
    dx2 = ops.rmsnorm_bwd(dy, x, rstd, w, dw)
    assert rel_err(dx2, REF.rmsnorm_bwd(dy.float(), x.float(), rr, w.float(), dwr)) < 6e-3


@pytest.mark.parametrize("D,hq,hkv", [(128, 4, 1), (64, 4, 2), (128, 28, 4)])
def test_rope_forward_and_inverse(ops, D, hq, hkv):
    from mini_trainer_b200.models.config import ModelConfig
    T = 257
    cfg = ModelConfig(vocab_size=8, hidden_size=hq * D, intermediate_size=8, num_hidden_layers=1,
                      num_attention_heads=hq, num_key_value_heads=hkv, head_dim=D, rope_theta=5e5)
    inv = cfg.rope_inv_freq().cuda()
    pos = torch.randint(0, 60000, (T,), device="cuda", dtype=torch.int32)
    qkv = bf(T, (hq + 2 * hkv) * D)
    orig = qkv.clone()
    ref = REF.rope_(qkv.float().clone(), pos, inv, hq, hkv, D)
    ops.rope_(qkv, pos, inv, hq, hkv, D)
    assert rel_err(qkv, ref) < 4e-3
    assert torch.equal(qkv[:, (hq + hkv) * D:], orig[:, (hq + hkv) * D:])  # v untouched
    ops.rope_(qkv, pos, inv, hq, hkv, D, inverse=True)
    assert rel_err(qkv, orig) < 8e-3


@pytest.mark.parametrize("T,H", [(77, 512), (33, 3072), (9, 6144), (130, 200)])
def test_layernorm_forward_and_backward(ops, T, H):
    """LayerNorm with bias (Starcoder2): statistics, output, input gradient (+ residual gradient), weight and bias
    gradients; partial sums without atomics (run twice: bitwise equal)."""
    x, dy, res = bf(T, H, scale=2.0) + 0.5, bf(T, H), bf(T, H)
    w, b = (1.0 + 0.3 * torch.randn(H, device="cuda")).bfloat16(), (0.3 * torch.randn(H, device="cuda")).bfloat16()
    y, stats = ops.layernorm(x, w, b, 1e-5)
    y_ref, stats_ref = REF.layernorm(x.float(), w.float(), b.float(), 1e-5)
    assert rel_err(y, y_ref) < 4e-3 and max_err(y, y_ref) < 5e-2
    assert rel_err(stats[0], stats_ref[0]) < 1e-4 and rel_err(stats[1], stats_ref[1]) < 1e-4
    gw_ref, gb_ref = torch.empty(H, device="cuda"), torch.empty(H, device="cuda")
    dx_ref = REF.layernorm_bwd(dy.float(), x.float(), stats_ref, w.float(), gw_ref, gb_ref, add_to=res.float())
    outs = []
    for _ in range(2):
        gw, gb = torch.empty(H, dtype=torch.bfloat16, device="cuda"), torch.empty(H, dtype=torch.bfloat16, device="cuda")
        dx = ops.layernorm_bwd(dy, x, stats, w, gw, gb, add_to=res)
        outs.append((dx, gw, gb))
    dx, gw, gb = outs[0]
    assert rel_err(dx, dx_ref) < 5e-3 and max_err(dx, dx_ref) < 5e-2
    assert rel_err(gw, gw_ref) < 6e-3 and rel_err(gb, gb_ref) < 6e-3
    assert all(torch.equal(a, c) for a, c in zip(outs[0], outs[1]))
    ops.check_status()


def test_geglu_and_gelu(ops):
    """The tanh-approximated GELU as the gate of a gated MLP (Gemma) and as a plain activation (Starcoder2)."""
    T, F = 123, 688
    gu, da = bf(T, 2 * F), bf(T, F)
    assert rel_err(ops.swiglu(gu, "gelu_tanh"), REF.swiglu(gu.float(), "gelu_tanh")) < 4e-3
    assert rel_err(ops.swiglu_bwd(da, gu, "gelu_tanh"), REF.swiglu_bwd(da.float(), gu.float(), "gelu_tanh")) < 5e-3
    assert max_err(ops.swiglu_bwd(da, gu, "gelu_tanh"), REF.swiglu_bwd(da.float(), gu.float(), "gelu_tanh")) < 5e-2
    act_ref, dgu_ref = ops.swiglu(gu, "gelu_tanh"), ops.swiglu_bwd(da, gu, "gelu_tanh")
    buf = da.clone()
    dgu, act = ops.swiglu_bwd_act(buf, gu, "gelu_tanh")
    assert act.data_ptr() == buf.data_ptr() and torch.equal(act, act_ref) and torch.equal(dgu, dgu_ref)
    x, dy = bf(T, F, scale=2.0), bf(T, F)
    assert rel_err(ops.gelu(x), REF.gelu(x.float())) < 4e-3 and max_err(ops.gelu(x), REF.gelu(x.float())) < 5e-2
    assert rel_err(ops.gelu_bwd(dy, x), REF.gelu_bwd(dy.float(), x.float())) < 5e-3
    ops.check_status()


@pytest.mark.parametrize("D,hq,hkv,T", [(128, 4, 1, 257), (64, 4, 2, 33), (256, 2, 1, 100), (128, 28, 4, 1031)])
def test_head_rmsnorm_forward_and_backward(ops, D, hq, hkv, T):
    """Per-head RMSNorm of the q and k heads inside the fused qkv rows (Qwen3), in place, v untouched; backward in place
    on the gradient with the pre-norm heads as input, weight gradients without atomics (run twice: bitwise equal)."""
    nh = hq + hkv
    qkv = bf(T, (hq + 2 * hkv) * D)
    wq, wk = (1.0 + 0.3 * torch.randn(D, device="cuda")).bfloat16(), (1.0 + 0.3 * torch.randn(D, device="cuda")).bfloat16()
    orig = qkv.clone()
    pre = qkv[:, : nh * D].clone()
    ref = qkv.float().clone()
    rstd_ref = REF.head_rmsnorm_(ref, wq.float(), wk.float(), 1e-6, hq, hkv, D)
    rstd = ops.head_rmsnorm_(qkv, wq, wk, 1e-6, hq, hkv, D)
    assert rel_err(qkv, ref) < 4e-3 and max_err(qkv, ref) < 5e-2 and rel_err(rstd, rstd_ref) < 1e-5
    assert torch.equal(qkv[:, nh * D:], orig[:, nh * D:])
    dy = bf(T, (hq + 2 * hkv) * D)
    dref = dy.float().clone()
    gq_ref, gk_ref = torch.empty(D, device="cuda"), torch.empty(D, device="cuda")
    REF.head_rmsnorm_bwd_(dref, pre.float(), rstd_ref, wq.float(), wk.float(), gq_ref, gk_ref, hq, hkv, D)
    outs = []
    for _ in range(2):
        d = dy.clone()
        gq, gk = torch.empty(D, dtype=torch.bfloat16, device="cuda"), torch.empty(D, dtype=torch.bfloat16, device="cuda")
        ops.head_rmsnorm_bwd_(d, pre, rstd, wq, wk, gq, gk, hq, hkv, D)
        outs.append((d, gq, gk))
    d, gq, gk = outs[0]
    assert rel_err(d, dref) < 5e-3 and max_err(d, dref) < 5e-2
    assert torch.equal(d[:, nh * D:], dy[:, nh * D:])
    assert rel_err(gq, gq_ref) < 6e-3 and rel_err(gk, gk_ref) < 6e-3
    assert all(torch.equal(a, b) for a, b in zip(outs[0], outs[1]))
    ops.check_status()


def test_swiglu(ops):
    T, F = 123, 688
    gu, da = bf(T, 2 * F), bf(T, F)
    assert rel_err(ops.swiglu(gu), REF.swiglu(gu.float())) < 4e-3
    assert rel_err(ops.swiglu_bwd(da, gu), REF.swiglu_bwd(da.float(), gu.float())) < 5e-3
    # fused form: the gradient and the forward output (written over the incoming gradient) in one pass
    act_ref, dgu_ref = ops.swiglu(gu), ops.swiglu_bwd(da, gu)
    buf = da.clone()
    dgu, act = ops.swiglu_bwd_act(buf, gu)
    assert act.data_ptr() == buf.data_ptr() and torch.equal(act, act_ref) and torch.equal(dgu, dgu_ref)


def test_embedding(ops):
    V, H, T = 1000, 256, 4000
    w = bf(V, H)
    ids = torch.randint(0, 50, (T,), device="cuda")  # many collisions
    assert torch.equal(ops.embedding(w, ids), w[ids])
    dx = bf(T, H, scale=0.01)
    base = bf(V, H, scale=0.01)   # what the buffer already holds (the LM-head gradient when embeddings are tied)
    dw = base.clone()
    ops.embedding_bwd(dw, ids, dx)
    ref = base.float().index_add_(0, ids, dx.float())
    assert rel_err(dw, ref) < 3e-3  # fp32 sum of ~80 addends per row, one bf16 rounding
    assert torch.equal(dw[50:], base[50:])   # rows of ids that do not occur are untouched
    dw2 = base.clone()
    ops.embedding_bwd(dw2, ids, dx)
    assert torch.equal(dw, dw2)   # no atomics: bitwise reproducible


@pytest.mark.parametrize("T,H,V", [(300, 256, 32000), (70, 512, 4104)])
def test_linear_ce(ops, T, H, V):
    torch.manual_seed(0)
    x, w = bf(T, H), bf(V, H, scale=0.05)
    tg = torch.randint(0, V, (T,), device="cuda")
    tg[::3] = -100
    dw, dwr = torch.zeros(V, H, dtype=torch.bfloat16, device="cuda"), torch.zeros(V, H, device="cuda")
    ops.ce_chunk = 128
    loss, dx = ops.linear_ce(x, w, tg, 0.01, dw)
    ref = TorchOps(ce_chunk=128)
    lr, dxr = ref.linear_ce(x.float(), w.float(), tg, 0.01, dwr)
    assert rel_err(loss, lr) < 1e-3
    assert (loss[::3] == 0).all()
    assert rel_err(dx, dxr) < 1e-2 and rel_err(dw, dwr) < 1e-2
    dw2 = dw.clone()
    ops.linear_ce(x, w, tg, 0.01, dw2, accumulate_dw=True)
    assert rel_err(dw2, 2 * dwr) < 1e-2


def test_optimizer_kernels(ops):
    n = 128 * 1000
    for sdt in (torch.float32, torch.bfloat16):
        master = torch.randn(n, device="cuda")
        m, v = torch.randn(n, device="cuda").mul(0.01).to(sdt), torch.rand(n, device="cuda").mul(0.001).to(sdt)
        g = torch.randn(n, device="cuda")
        p = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        rm, rmm, rv, rp = master.clone(), m.clone(), v.clone(), torch.empty(n, device="cuda")
        coef = torch.tensor(0.5, device="cuda")
        ops.adamw_step(master, m, v, g, p, 1e-3, 0.9, 0.95, 1e-8, 0.01, 3, coef)
        REF.adamw_step(rm, rmm, rv, g, rp, 1e-3, 0.9, 0.95, 1e-8, 0.01, 3, coef)
        assert rel_err(master, rm) < 1e-5 and rel_err(m, rmm) < 1e-2 and rel_err(v, rv) < 1e-2
        assert torch.equal(p, master.bfloat16())
    g = torch.randn(n, device="cuda")
    assert abs(ops.sumsq(g).item() - g.pow(2).sum().item()) < 1e-3 * n
    acc, src = torch.randn(n, device="cuda"), bf(n)
    ref = acc + src.float()
    ops.accumulate(acc, src, True)
    assert torch.allclose(acc, ref)
    ops.accumulate(acc, src, False)
    assert torch.equal(acc, src.float())


ATTN_CASES = [(128, 4, 1, [300, 17, 129, 1, 640]), (64, 4, 2, [128, 256, 5]), (128, 8, 2, [1000]), (128, 4, 4, [127, 128, 129]),
              # the GQA ratios of the benchmark models (1.5B: 6, 7B: 7, 70B: 8) and sequences of many key tiles
              (128, 6, 1, [4097, 200]), (128, 7, 1, [513, 2050]), (128, 8, 1, [3000])]


def _cu(lens):
    cu_host = [0]
    for n in lens:
        cu_host.append(cu_host[-1] + n)
    return cu_host, torch.tensor(cu_host, dtype=torch.int32, device="cuda")


def _attn_ref_one_head(q, k, v, do=None):
    """fp32 causal attention of ONE head of ONE sequence in query chunks: (out, lse[, dq, dk, dv])."""
    n, d = q.shape
    scale = d ** -0.5
    out = torch.empty_like(q)
    lse = torch.empty(n, device=q.device)
    dq = torch.zeros_like(q) if do is not None else None
    dk = torch.zeros_like(k) if do is not None else None
    dv = torch.zeros_like(v) if do is not None else None
    for a in range(0, n, 2048):
        b = min(n, a + 2048)
        s = (q[a:b] @ k[:b].t()) * scale
        s = s.masked_fill(torch.arange(b, device=q.device)[None, :] > torch.arange(a, b, device=q.device)[:, None], float("-inf"))
        l = torch.logsumexp(s, -1)
        p = torch.exp(s - l[:, None])
        out[a:b] = p @ v[:b]
        lse[a:b] = l
        if do is not None:
            dp = do[a:b] @ v[:b].t()
            delta = (do[a:b] * out[a:b]).sum(-1, keepdim=True)
            ds = p * (dp - delta) * scale
            dq[a:b] = ds @ k[:b]
            dk[:b] += ds.t() @ q[a:b]
            dv[:b] += p.t() @ do[a:b]
    return out, lse, dq, dk, dv


@pytest.mark.parametrize("n,hq,hkv", [(16384, 8, 1), (65536, 2, 1)])
def test_attention_long_sequences(ops, n, hq, hkv):
    """Sequences as long as the benchmark's (hundreds of key tiles per query block: the S/P double
    buffers and the rescale path run many times) against an fp32 reference computed head by head."""
    D = 128
    torch.manual_seed(n)
    qkv = bf(n, (hq + 2 * hkv) * D)
    dout = bf(n, hq * D)
    cu_host, cu = _cu([n])
    out, lse = ops.attention(qkv, cu, cu_host, n, hq, hkv, D)
    out2, lse2 = ops.attention(qkv, cu, cu_host, n, hq, hkv, D)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)          # forward has no order-dependent accumulation
    dqkv = ops.attention_bwd(dout, qkv, out, lse, cu, cu_host, n, hq, hkv, D)
    ops.check_status()
    g = hq // hkv
    for h in (0, hq - 1):
        hk = h // g
        q = qkv[:, h * D:(h + 1) * D].float()
        k = qkv[:, (hq + hk) * D:(hq + hk + 1) * D].float()
        v = qkv[:, (hq + hkv + hk) * D:(hq + hkv + hk + 1) * D].float()
        ro, rl, rdq, _, _ = _attn_ref_one_head(q, k, v, dout[:, h * D:(h + 1) * D].float())
        assert rel_err(out[:, h * D:(h + 1) * D], ro) < 1e-2 and max_err(out[:, h * D:(h + 1) * D], ro) < 0.1
        assert (lse[h] - rl).abs().max() < 2e-2
        assert rel_err(dqkv[:, h * D:(h + 1) * D], rdq) < 2e-2
    # dK / dV of kv head 0 sum over its whole query-head group
    rdk = torch.zeros(n, D, device="cuda")
    rdv = torch.zeros(n, D, device="cuda")
    k = qkv[:, hq * D:(hq + 1) * D].float()
    v = qkv[:, (hq + hkv) * D:(hq + hkv + 1) * D].float()
    for h in range(g):
        _, _, _, dk, dv = _attn_ref_one_head(qkv[:, h * D:(h + 1) * D].float(), k, v, dout[:, h * D:(h + 1) * D].float())
        rdk += dk
        rdv += dv
    assert rel_err(dqkv[:, hq * D:(hq + 1) * D], rdk) < 2e-2 and rel_err(dqkv[:, (hq + hkv) * D:(hq + hkv + 1) * D], rdv) < 2e-2


@pytest.mark.parametrize("D,hq,hkv,lens", ATTN_CASES)
def test_attention_forward(ops, D, hq, hkv, lens):
    torch.manual_seed(sum(lens))
    T = sum(lens)
    qkv = bf(T, (hq + 2 * hkv) * D)
    cu_host = [0]
    for n in lens:
        cu_host.append(cu_host[-1] + n)
    cu = torch.tensor(cu_host, dtype=torch.int32, device="cuda")
    out, lse = ops.attention(qkv, cu, cu_host, max(lens), hq, hkv, D)
    ro, rl = REF.attention(qkv.float(), cu, cu_host, max(lens), hq, hkv, D)
    ops.check_status()
    assert rel_err(lse, rl) < 2e-3 and (lse - rl).abs().max() < 2e-2
    assert rel_err(out, ro) < 1e-2 and max_err(out, ro) < 0.1
    out2, lse2 = ops.attention(qkv, cu, cu_host, max(lens), hq, hkv, D)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)   # run twice: bitwise identical


@pytest.mark.parametrize("D,hq,hkv,lens", ATTN_CASES)
def test_attention_backward(ops, D, hq, hkv, lens):
    if not hasattr(ops.lib, "mtb200_attn_bwd"):
        pytest.skip("attention backward kernel not built")
    torch.manual_seed(1 + sum(lens))
    T = sum(lens)
    qkv = bf(T, (hq + 2 * hkv) * D)
    dout = bf(T, hq * D)
    cu_host = [0]
    for n in lens:
        cu_host.append(cu_host[-1] + n)
    cu = torch.tensor(cu_host, dtype=torch.int32, device="cuda")
    out, lse = ops.attention(qkv, cu, cu_host, max(lens), hq, hkv, D)
    dqkv = ops.attention_bwd(dout, qkv, out, lse, cu, cu_host, max(lens), hq, hkv, D)
    ro, rl = REF.attention(qkv.float(), cu, cu_host, max(lens), hq, hkv, D)
    rd = REF.attention_bwd(dout.float(), qkv.float(), ro, rl, cu, cu_host, max(lens), hq, hkv, D)
    ops.check_status()
    q_end, k_end = hq * D, (hq + hkv) * D
    assert rel_err(dqkv[:, :q_end], rd[:, :q_end]) < 2e-2 and max_err(dqkv[:, :q_end], rd[:, :q_end]) < 0.25
    assert rel_err(dqkv[:, q_end:k_end], rd[:, q_end:k_end]) < 2e-2 and max_err(dqkv[:, q_end:k_end], rd[:, q_end:k_end]) < 0.25
    assert rel_err(dqkv[:, k_end:], rd[:, k_end:]) < 2e-2 and max_err(dqkv[:, k_end:], rd[:, k_end:]) < 0.25


def test_bounded_wait_expires_with_status_and_context_stays_usable(ops):
    """A wait on a flag that nothing sets must run out, record {code, peer} and return."""
    import ctypes
    lib = ops.lib
    fn = lib.mtb200_symm_wait
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_uint, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    flags[0] = 5                                   # "peer 0" already signalled epoch 5, "peer 1" never does
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = fn(flags.data_ptr(), 2, 5, 2000, 42, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    code = int(status.item())
    assert code & 0xff == 42 and code >> 8 == 1
    x = torch.ones(1024, device="cuda")
    assert x.sum().item() == 1024                  # the context is still healthy


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 256), (300, 520, 200), (1000, 1024, 4096), (4096, 6144, 4096), (264, 264, 72)])
@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_gemm_two_cta(ops, M, N, K, layout):
    """cta_group::2 kernel (256x256 tiles per CTA pair) against the fp32 reference, all three layouts."""
    torch.manual_seed(3 + M + N + K)
    if layout == "tn" and M % 8:
        pytest.skip("leading dimension of an MN-major A must be a multiple of 8")
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    if layout == "nt":
        a, b = bf(M, K), bf(N, K, scale=0.05)
        ref = a.float() @ b.float().t()
        ops.gemm(a, False, b, False, out, M, N, K, two_cta=True)
    elif layout == "nn":
        a, b = bf(M, K), bf(K, N, scale=0.05)
        ref = a.float() @ b.float()
        ops.gemm(a, False, b, True, out, M, N, K, two_cta=True)
    else:
        a, b = bf(K, M), bf(K, N, scale=0.05)
        ref = a.float().t() @ b.float()
        ops.gemm(a, True, b, True, out, M, N, K, two_cta=True)
    torch.cuda.synchronize()
    ops.check_status()
    assert rel_err(out, ref) < 6e-3
    res, bias = bf(M, N), bf(N)
    if layout == "nt":
        ops.gemm(a, False, b, False, out, M, N, K, residual=res, bias=bias, two_cta=True)
        assert rel_err(out, ref + res.float() + bias.float()) < 6e-3
    # fp32 output accumulated in place (the form the linear+CE weight gradient uses), scaled product
    o32 = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    for _ in range(2):
        ops.gemm(a, layout == "tn", b, layout != "nt", o32, M, N, K, residual=o32, two_cta=True, alpha=0.5)
    assert rel_err(o32, ref) < 2e-3 and max_err(o32, ref) < 2e-2
    ops.check_status()


def test_osft_projection_on_tcgen05_gemm(ops):
    """G - U(U^T G) and G - (G V^T) V on the tcgen05 GEMM against float64 PyTorch."""
    from mini_trainer_b200.parallel import osft as O
    torch.manual_seed(0)
    w = torch.randn(512, 1024, device="cuda", dtype=torch.float64)
    u_hi, s_hi, v_hi, u_lo, s_lo, v_lo = O.svd_split(w, 0.5)
    du = torch.randn(512, u_lo.shape[1], device="cuda", dtype=torch.float64)
    dv = torch.randn(v_lo.shape[0], 1024, device="cuda", dtype=torch.float64)
    ref_u, ref_v = O.project_orthogonal(du, dv, u_hi, v_hi)
    got_u, got_v = O.project_orthogonal_tcgen05(ops, du.float(), dv.float(), u_hi.float(), v_hi.float())
    ops.check_status()
    assert rel_err(got_u, ref_u) < 1e-2 and rel_err(got_v, ref_v) < 1e-2
    # what is left inside the frozen subspace is at bf16 rounding level
    assert (u_hi.float().t() @ got_u).norm() < 2e-2 * du.float().norm()
    assert (got_v @ v_hi.float().t()).norm() < 2e-2 * dv.float().norm()


def test_out_of_range_inputs_are_reported_not_dereferenced(ops):
    """Bounds checks that record a status code and skip the access: a token id outside the embedding
    table, an attention work item outside the packed batch. The context stays usable."""
    w = bf(100, 64)
    ids = torch.tensor([3, 100, 7, -1], device="cuda")
    out = ops.embedding(w, ids)
    torch.cuda.synchronize()
    assert torch.equal(out[0], w[3]) and torch.equal(out[2], w[7]) and (out[1] == 0).all() and (out[3] == 0).all()
    with pytest.raises(RuntimeError, match="token id outside"):
        ops.check_status()
    dw = torch.zeros(100, 64, dtype=torch.bfloat16, device="cuda")
    ops.embedding_bwd(dw, ids, bf(4, 64))
    with pytest.raises(RuntimeError, match="token id outside"):
        ops.check_status()
    assert dw[3].abs().sum() > 0 and dw[7].abs().sum() > 0
    # an attention plan that claims a sequence longer than the batch
    T, hq, hkv, D = 256, 2, 1, 128
    qkv = bf(T, (hq + 2 * hkv) * D)
    cu_host = [0, 300]
    cu = torch.tensor(cu_host, dtype=torch.int32, device="cuda")
    ops.attention(qkv, cu, cu_host, 300, hq, hkv, D)
    with pytest.raises(RuntimeError, match="attention work item"):
        ops.check_status()
    ops.check_status()     # cleared; and the device still works
    assert torch.ones(8, device="cuda").sum().item() == 8
