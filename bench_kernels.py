"""Per-kernel microbenchmarks with roofline fractions.

    python bench_kernels.py --op gemm --layout nt --m 8192 --n 8192 --k 8192
    python bench_kernels.py --op attn_fwd --lens 16384,16384
    python bench_kernels.py --op all
    python bench_kernels.py --op families      # LayerNorm, per-head q/k norm, GeGLU / GELU
    (ops: gemm, attn_fwd, attn_bwd, rmsnorm, swiglu, rope, ce, linear_ce, embedding, adamw)

Each op is timed with CUDA events on the launching stream after warm-up, with a synchronize on
both sides. Inputs are larger than the 126 MB L2 (or an L2-sized buffer is rewritten between
iterations with ``--flush-l2``). The achieved figure is compared with the MEASURED peaks in
``MEASURED_PEAKS.json`` (cuBLAS bf16 burst throughput, STREAM-style copy bandwidth) when that file
is present, else with the fallback 1.59 PFLOP/s and 6.65 TB/s ("of fallback").
This script is also the small-case driver for ``ncu`` captures (``--iters 1 --warmup 1``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from mini_trainer_b200.ops.native import NativeOps  # noqa: E402


def peaks():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d["bf16_tflops"], d["hbm_gbs"], "of measured"
    return 1590.0, 6650.0, "of fallback"


def timeit(fn, iters, warmup, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def sustained(fn, seconds):
    """Mean time per call (ms) over back-to-back calls for ``seconds`` of device time, measured on the
    second half only: the regime of a long training step, where the 1000 W power cap, not the burst
    clock, sets the pace. Returns (ms per call, median SM MHz over the measured half)."""
    import subprocess
    fn(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); fn(); e1.record(); torch.cuda.synchronize()
    n = max(4, int(seconds * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
    for _ in range(n // 2):
        fn()
    smi = subprocess.Popen(["nvidia-smi", "--query-gpu=clocks.sm", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                            str(torch.cuda.current_device())], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    e0.record()
    for _ in range(n - n // 2):
        fn()
    e1.record()
    torch.cuda.synchronize()
    smi.terminate()
    mhz = sorted(float(x) for x in smi.stdout.read().split() if x.strip().replace(".", "").isdigit())
    return e0.elapsed_time(e1) / (n - n // 2), (mhz[len(mhz) // 2] if mhz else None)


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all")
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--lens", default="16384,16384")
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--adamw-n", type=int, default=512 * 1024 * 1024, help="elements of the AdamW shard (14 bytes each with fp32 moments)")
    ap.add_argument("--ce-chunk", type=int, default=0, help="token rows per linear+CE chunk (0 = library default)")
    ap.add_argument("--flush-l2", action="store_true")
    ap.add_argument("--sustain", type=float, default=0.0, help="--op shapes: also run every kernel back to back for this many "
                    "seconds and report the throughput under the power cap")
    ap.add_argument("--two-cta", action="store_true", help="use the cta_group::2 GEMM kernel (256x256 tiles per CTA pair)")
    a = ap.parse_args()
    ops = NativeOps("cuda:0")
    if a.ce_chunk:
        ops.ce_chunk = a.ce_chunk
    tf_peak, bw_peak, tag = peaks()
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda") if a.flush_l2 else None
    out = []

    def report(name, ms, flops=None, bytes_=None):
        rec = {"op": name, "ms": round(ms, 4)}
        if flops:
            rec["tflops"] = round(flops / ms / 1e9, 1)
            rec["frac_compute"] = f"{flops / ms / 1e9 / tf_peak:.3f} {tag} cuBLAS bf16"
        if bytes_:
            rec["gbs"] = round(bytes_ / ms / 1e6, 1)
            rec["frac_hbm"] = f"{bytes_ / ms / 1e6 / bw_peak:.3f} {tag} copy bandwidth"
        out.append(rec)
        print(json.dumps(rec), flush=True)

    EW = ("rmsnorm", "swiglu", "rope", "ce", "embedding", "adamw")   # --op ew: the bandwidth-bound kernels

    def want(n):
        ok = a.op in ("all", n) or (a.op == "ew" and n in EW)
        if ok:
            torch.cuda.empty_cache()   # the previous op's tensors are gone: keep the resident set small
        return ok

    if want("gemm"):
        M, N, K = a.m, a.n, a.k
        for lay in (["nt", "nn", "tn"] if a.op == "all" else [a.layout]):
            if lay == "nt":
                x, w = bf(M, K), bf(N, K, scale=0.02)
                o = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
                fn = lambda: ops.gemm(x, False, w, False, o, M, N, K, two_cta=a.two_cta)
            elif lay == "nn":
                x, w = bf(M, K), bf(K, N, scale=0.02)
                o = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
                fn = lambda: ops.gemm(x, False, w, True, o, M, N, K, two_cta=a.two_cta)
            else:
                x, w = bf(K, M), bf(K, N, scale=0.02)
                o = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
                fn = lambda: ops.gemm(x, True, w, True, o, M, N, K, two_cta=a.two_cta)
            report(f"gemm{2 if a.two_cta else 1}cta_{lay}_{M}x{N}x{K}", timeit(fn, a.iters, a.warmup, flush), flops=2.0 * M * N * K)
    if a.op == "shapes":
        # the GEMMs of one Llama-3.1-8B block at --tokens tokens: one-CTA kernel, CTA-pair kernel and cuBLAS (torch.matmul)
        T, H, F, Q = min(a.tokens, 16384), 4096, 14336, 6144
        cases = [("qkv_fwd", "nt", T, Q, H), ("gate_up_fwd", "nt", T, 2 * F, H), ("down_fwd", "nt", T, H, F), ("o_fwd", "nt", T, H, H),
                 ("gate_up_dgrad", "nn", T, H, 2 * F), ("down_dgrad", "nn", T, F, H),
                 ("gate_up_wgrad", "tn", 2 * F, H, T), ("down_wgrad", "tn", H, F, T), ("qkv_wgrad", "tn", Q, H, T)]
        for name, lay, M, N, K in cases:
            torch.cuda.empty_cache()
            o = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            if lay == "nt":
                x, w = bf(M, K), bf(N, K, scale=0.02)
                lib = lambda: torch.matmul(x, w.t(), out=o)
            elif lay == "nn":
                x, w = bf(M, K), bf(K, N, scale=0.02)
                lib = lambda: torch.matmul(x, w, out=o)
            else:
                x, w = bf(K, M), bf(K, N, scale=0.02)
                lib = lambda: torch.matmul(x.t(), w, out=o)
            fl = 2.0 * M * N * K
            variants = [("1cta", lambda: ops.gemm(x, lay == "tn", w, lay != "nt", o, M, N, K, two_cta=False)),
                        ("2cta", lambda: ops.gemm(x, lay == "tn", w, lay != "nt", o, M, N, K, two_cta=True)), ("cublas", lib)]
            for vname, fn in variants:
                report(f"{name}_{lay}_{M}x{N}x{K}_{vname}", timeit(fn, a.iters, a.warmup, flush), flops=fl)
                if a.sustain > 0:
                    ms, mhz = sustained(fn, a.sustain)
                    rec = {"op": f"{name}_{lay}_{M}x{N}x{K}_{vname}_sustained", "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
                           "sm_mhz_median": mhz}
                    print(json.dumps(rec), flush=True)
    if want("attn_fwd") or want("attn_bwd"):
        lens = [int(v) for v in a.lens.split(",")]
        T = sum(lens)
        qkv, dout = bf(T, (a.hq + 2 * a.hkv) * a.d), bf(T, a.hq * a.d)
        cu_host = [0]
        for n in lens:
            cu_host.append(cu_host[-1] + n)
        cu = torch.tensor(cu_host, dtype=torch.int32, device="cuda")
        fl = sum(4.0 * n * n / 2 * a.hq * a.d for n in lens)
        o, lse = ops.attention(qkv, cu, cu_host, max(lens), a.hq, a.hkv, a.d)
        if want("attn_fwd"):
            report(f"attn_fwd_T{T}", timeit(lambda: ops.attention(qkv, cu, cu_host, max(lens), a.hq, a.hkv, a.d), a.iters, a.warmup, flush), flops=fl)
        if want("attn_bwd"):
            report(f"attn_bwd_T{T}", timeit(lambda: ops.attention_bwd(dout, qkv, o, lse, cu, cu_host, max(lens), a.hq, a.hkv, a.d), a.iters, a.warmup, flush), flops=2.5 * fl)
    def op_rmsnorm():
        T, H = a.tokens, a.hidden
        x, w, dy = bf(T, H), bf(H), bf(T, H)
        y, rstd = ops.rmsnorm(x, w, 1e-5)
        dw = torch.empty_like(w)
        report(f"rmsnorm_fwd_{T}x{H}", timeit(lambda: ops.rmsnorm(x, w, 1e-5), a.iters, a.warmup, flush), bytes_=2.0 * T * H * 2)
        report(f"rmsnorm_bwd_{T}x{H}", timeit(lambda: ops.rmsnorm_bwd(dy, x, rstd, w, dw, add_to=dy), a.iters, a.warmup, flush), bytes_=4.0 * T * H * 2)
    def op_swiglu():
        T, F = a.tokens, 14336
        gu, da = bf(T, 2 * F), bf(T, F)
        report(f"swiglu_fwd_{T}x{F}", timeit(lambda: ops.swiglu(gu), a.iters, a.warmup, flush), bytes_=3.0 * T * F * 2)
        report(f"swiglu_bwd_{T}x{F}", timeit(lambda: ops.swiglu_bwd(da, gu), a.iters, a.warmup, flush), bytes_=5.0 * T * F * 2)
    def op_rope():
        T = a.tokens
        qkv = bf(T, (a.hq + 2 * a.hkv) * a.d)
        pos = (torch.arange(T, device="cuda") % 4096).to(torch.int32)
        inv = (1.0 / (5e5 ** (torch.arange(0, a.d, 2, device="cuda", dtype=torch.float32) / a.d))).contiguous()
        # reads and rewrites the q and k heads in place
        report(f"rope_{T}x{a.hq}+{a.hkv}x{a.d}", timeit(lambda: ops.rope_(qkv, pos, inv, a.hq, a.hkv, a.d), a.iters, a.warmup, flush),
               bytes_=2.0 * T * (a.hq + a.hkv) * a.d * 2)
    def op_ce():
        R, V = 2048, a.vocab
        logits = torch.randn(R, V, device="cuda").bfloat16()
        tg = torch.randint(0, V, (R,), device="cuda")
        loss = torch.empty(R, device="cuda")
        dlog = torch.empty(R, V, dtype=torch.bfloat16, device="cuda")
        fn = lambda: ops._call("mtb200_ce_fwd_bwd", logits.data_ptr(), V, 1, tg.data_ptr(), loss.data_ptr(), dlog.data_ptr(), V, R, V,
                               1.0, -100, ops._st())
        # two passes over the bf16 logits (online max/sum, then gradient) + the bf16 gradient write
        report(f"ce_fwd_bwd_{R}x{V}", timeit(fn, a.iters, a.warmup, flush), bytes_=R * V * (2.0 + 2.0 + 2.0))
    def op_linear_ce():
        T, H, V = min(a.tokens, 8192), a.hidden, a.vocab
        x, w = bf(T, H), bf(V, H, scale=0.02)
        tg = torch.randint(0, V, (T,), device="cuda")
        dw = torch.empty(V, H, dtype=torch.bfloat16, device="cuda")
        report(f"linear_ce_{T}x{H}x{V}_chunk{ops.ce_chunk}", timeit(lambda: ops.linear_ce(x, w, tg, 1.0, dw), a.iters, a.warmup, flush), flops=6.0 * T * H * V)
    def op_embedding():
        T, H, V = a.tokens, a.hidden, a.vocab
        w, dx = bf(V, H), bf(T, H)
        ids = torch.randint(0, V, (T,), device="cuda")
        dw = torch.zeros(V, H, dtype=torch.bfloat16, device="cuda")
        report(f"embedding_fwd_{T}x{H}", timeit(lambda: ops.embedding(w, ids), a.iters, a.warmup, flush), bytes_=2.0 * T * H * 2)
        # sort of the ids + read dx, read-modify-write the touched rows
        report(f"embedding_bwd_{T}x{H}", timeit(lambda: ops.embedding_bwd(dw, ids, dx), a.iters, a.warmup, flush), bytes_=3.0 * T * H * 2)
    def op_adamw():
        n = a.adamw_n
        master, m, v, g = (torch.zeros(n, device="cuda") for _ in range(4))
        p = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        coef = torch.ones(1, device="cuda")
        report(f"adamw_{n}", timeit(lambda: ops.adamw_step(master, m, v, g, p, 1e-4, 0.9, 0.95, 1e-8, 0.0, 2, coef), a.iters, a.warmup, flush),
               bytes_=n * (4 * 4 + 3 * 4 + 2.0))
    def op_layernorm():
        T, H = a.tokens, min(a.hidden, 6144)
        x, w, b, dy = bf(T, H), bf(H), bf(H), bf(T, H)
        y, stats = ops.layernorm(x, w, b, 1e-5)
        dw, db = torch.empty_like(w), torch.empty_like(b)
        report(f"layernorm_fwd_{T}x{H}", timeit(lambda: ops.layernorm(x, w, b, 1e-5), a.iters, a.warmup, flush), bytes_=2.0 * T * H * 2)
        report(f"layernorm_bwd_{T}x{H}", timeit(lambda: ops.layernorm_bwd(dy, x, stats, w, dw, db, add_to=dy), a.iters, a.warmup, flush),
               bytes_=4.0 * T * H * 2)
    def op_head_rmsnorm():
        T, nh = a.tokens, a.hq + a.hkv
        qkv, dqkv = bf(T, (a.hq + 2 * a.hkv) * a.d), bf(T, (a.hq + 2 * a.hkv) * a.d)
        wq, wk = bf(a.d), bf(a.d)
        pre = qkv[:, : nh * a.d].clone()
        rstd = ops.head_rmsnorm_(qkv.clone(), wq, wk, 1e-6, a.hq, a.hkv, a.d)
        gq, gk = torch.empty_like(wq), torch.empty_like(wk)
        # in place on the q and k heads: read + write (forward), read gradient and pre-norm heads + write (backward)
        report(f"head_rmsnorm_fwd_{T}x{a.hq}+{a.hkv}x{a.d}", timeit(lambda: ops.head_rmsnorm_(qkv, wq, wk, 1e-6, a.hq, a.hkv, a.d), a.iters, a.warmup, flush),
               bytes_=2.0 * T * nh * a.d * 2)
        report(f"head_rmsnorm_bwd_{T}x{a.hq}+{a.hkv}x{a.d}",
               timeit(lambda: ops.head_rmsnorm_bwd_(dqkv, pre, rstd, wq, wk, gq, gk, a.hq, a.hkv, a.d), a.iters, a.warmup, flush),
               bytes_=3.0 * T * nh * a.d * 2)
    def op_geglu():
        T, F = a.tokens, 14336
        gu, da = bf(T, 2 * F), bf(T, F)
        report(f"geglu_fwd_{T}x{F}", timeit(lambda: ops.swiglu(gu, "gelu_tanh"), a.iters, a.warmup, flush), bytes_=3.0 * T * F * 2)
        report(f"geglu_bwd_{T}x{F}", timeit(lambda: ops.swiglu_bwd(da, gu, "gelu_tanh"), a.iters, a.warmup, flush), bytes_=5.0 * T * F * 2)
        x = bf(T, F)
        report(f"gelu_fwd_{T}x{F}", timeit(lambda: ops.gelu(x), a.iters, a.warmup, flush), bytes_=2.0 * T * F * 2)
        report(f"gelu_bwd_{T}x{F}", timeit(lambda: ops.gelu_bwd(da, x), a.iters, a.warmup, flush), bytes_=3.0 * T * F * 2)
    for name, fn in (("layernorm", op_layernorm), ("head_rmsnorm", op_head_rmsnorm), ("geglu", op_geglu)):
        if a.op in (name, "families"):   # kernels of the model families beyond the Llama block; not part of --op all
            torch.cuda.empty_cache()
            fn()
    for name, fn in (("rmsnorm", op_rmsnorm), ("swiglu", op_swiglu), ("rope", op_rope), ("ce", op_ce), ("linear_ce", op_linear_ce),
                     ("embedding", op_embedding), ("adamw", op_adamw)):
        if want(name):
            fn()   # the op's tensors die with its frame
    ops.check_status()


if __name__ == "__main__":
    main()
