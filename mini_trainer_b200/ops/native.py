"""sm_100a kernel backend: ctypes bindings over ``_native/libmtb200_cuda.so``.

Same method set as ``TorchOps``; tensors are bf16 on a CUDA device, 2-D, row-major. Every call
launches on the current torch CUDA stream. A missing library or a non-zero return code raises —
there is no silent fallback to PyTorch on a GPU machine.

``launches`` counts kernels launched through this backend (reported by the benchmark).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .. import build as _build
from ..utils import nvtx

_LIB = None


def load_library():
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _build.CUDA_LIB
    if not path.exists() or os.environ.get("MTB200_REBUILD"):
        _build.build_cuda()
    if not path.exists():
        raise RuntimeError(f"native CUDA library {path} is missing and could not be built (nvcc not found)")
    lib = ctypes.CDLL(str(path))
    for name in dir(_Sig):
        if name.startswith("mtb200_") and hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = c_int
            fn.argtypes = getattr(_Sig, name)
    _LIB = lib
    return lib


P, I, L, F = c_void_p, c_int, c_longlong, c_float


class _Sig:
    mtb200_gemm_bf16 = [P, L, I, P, L, I, P, L, I, P, L, P, I, I, I, F, P, P]
    mtb200_gemm2_bf16 = [P, L, I, P, L, I, P, L, I, P, L, P, I, I, I, F, P, P]
    mtb200_rmsnorm_fwd = [P, P, P, P, F, I, I, P]
    mtb200_rmsnorm_bwd_blocks = [I]
    mtb200_rmsnorm_bwd = [P, P, P, P, P, P, P, P, I, I, P]
    mtb200_layernorm_fwd = [P, P, P, P, P, P, F, I, I, P]
    mtb200_layernorm_bwd = [P, P, P, P, P, P, P, P, P, P, I, I, P]
    mtb200_rope = [P, P, P, I, L, I, I, I, P]
    mtb200_head_rmsnorm_fwd = [P, P, P, P, F, I, L, I, I, I, P]
    mtb200_head_rmsnorm_bwd_blocks = [I, I]
    mtb200_head_rmsnorm_bwd = [P, P, P, P, P, P, P, P, I, L, L, I, I, I, P]
    mtb200_swiglu_fwd = [P, P, L, I, P]
    mtb200_swiglu_bwd = [P, P, P, L, I, P]
    mtb200_swiglu_bwd_act = [P, P, P, L, I, P]
    mtb200_geglu_fwd = [P, P, L, I, P]
    mtb200_geglu_bwd = [P, P, P, L, I, P]
    mtb200_geglu_bwd_act = [P, P, P, L, I, P]
    mtb200_gelu_fwd = [P, P, L, P]
    mtb200_gelu_bwd = [P, P, P, L, P]
    mtb200_embedding_fwd = [P, P, P, I, I, I, P, P]
    mtb200_embedding_bwd = [P, P, P, P, I, I, I, P, P]
    mtb200_ce_fwd_bwd = [P, L, I, P, P, P, L, I, I, F, L, P]
    mtb200_colsum = [P, L, P, P, I, I, P]
    mtb200_accumulate = [P, P, L, I, I, P]
    mtb200_f32_to_bf16 = [P, P, L, I, P]
    mtb200_sumsq = [P, L, P, P]
    mtb200_adamw = [P, P, P, I, P, P, L, F, F, F, F, F, I, P, P]
    mtb200_attn_fwd = [P, L, P, L, P, P, I, I, I, I, I, I, F, P, P]
    mtb200_attn_bwd = [P, L, P, L, P, L, P, L, P, P, P, P, I, I, I, I, I, I, F, P, P]


_GLU = {"silu": "mtb200_swiglu", "gelu_tanh": "mtb200_geglu"}
NATIVE_HEAD_DIMS = (64, 128)   # head dimensions of the hand-written attention kernels


def _ptr(t):
    return None if t is None else t.data_ptr()


class NativeOps:
    name = "native"

    def __init__(self, device, ce_chunk: int = 8192, attention: str | None = None):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("NativeOps needs a CUDA device")
        self.lib = load_library()
        self.ce_chunk = ce_chunk
        self.attention_impl = attention or os.environ.get("MTB200_ATTENTION", "native")
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # MTB200_GEMM2=1: two-CTA (cta_group::2, 256x256 tiles) GEMM for problems with about a full wave of such
        # tiles or more. It is the faster kernel in isolation (0.92-0.95 of the cuBLAS burst figure against
        # 0.74-0.90), but a training step runs at the 1000 W power cap, where the clock settles at what the GEMMs
        # draw: with the CTA-pair kernel the SM clock drops by 12-16 % for EVERY kernel of the step, and the
        # latency-bound ones (attention, normalisation) lose more than the GEMMs gain: measured end to end on
        # one GPU 25.2 s against 23.9 s per step. So the one-CTA kernel is the default.
        self.use_gemm2 = os.environ.get("MTB200_GEMM2", "0") == "1"
        # bit 0: attention forward keeps P in a shared-memory tile instead of tensor memory (A/B timing)
        self.attn_fwd_flags = int(os.environ.get("MTB200_ATTN_P_SMEM", "0"))
        self.launches = 0
        self.profile = [] if os.environ.get("MTB200_PROFILE") else None
        self._scratch = {}
        self._attn_plan_cache = {}

    # -- plumbing ---------------------------------------------------------------------
    def _st(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def _call(self, name, *args, n=1, tag=None):
        if self.profile is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        if nvtx.ENABLED:
            nvtx.push(tag or name)
        rc = getattr(self.lib, name)(*args)
        if nvtx.ENABLED:
            nvtx.pop()
        if rc != 0:
            raise RuntimeError(f"{name} failed with code {rc}")
        self.launches += n
        if self.profile is not None:
            e1.record()
            self.profile.append((tag or name, e0, e1))

    def profile_summary(self) -> dict:
        """Device time per op (ms) since profiling was switched on (``MTB200_PROFILE=1``)."""
        torch.cuda.synchronize(self.device)
        out = {}
        for name, e0, e1 in self.profile or []:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        self.profile = [] if self.profile is not None else None
        return dict(sorted(out.items(), key=lambda kv: -kv[1]))

    def _buf(self, key, numel, dtype):
        b = self._scratch.get(key)
        if b is None or b.numel() < numel or b.dtype != dtype:
            b = torch.empty(numel, dtype=dtype, device=self.device)
            self._scratch[key] = b
        return b[:numel]

    def _ev(self):
        if self.profile is None:
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def _ev_end(self, name, e0):
        if e0 is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            self.profile.append((name, e0, e1))

    def check_status(self):
        """Raises if any kernel recorded an expired bounded wait (one host sync)."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            what = {60: "a token id outside the embedding table", 61: "an attention work item outside the packed batch"}.get(
                code, "a device-side bounded wait expired")
            raise RuntimeError(f"{what} (status code {code})")

    # -- GEMM -------------------------------------------------------------------------
    def gemm(self, a, a_mn, b, b_mn, out, M, N, K, residual=None, bias=None, tag=None, two_cta=None, alpha=1.0):
        """out[M,N] = alpha*A*B (+bias) (+residual). ``a_mn``/``b_mn``: operand stored [K, rows].
        ``two_cta``: force (True) or forbid (False) the cta_group::2 kernel; default by problem size."""
        out_f32 = out.dtype == torch.float32
        assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
        assert residual is None or residual.dtype == out.dtype
        if two_cta is None:
            two_cta = self.use_gemm2 and (-(-M // 256)) * (-(-N // 256)) >= 64
        self._call("mtb200_gemm2_bf16" if two_cta else "mtb200_gemm_bf16", a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(), b.stride(0), int(b_mn),
                   out.data_ptr(), out.stride(0), int(out_f32), _ptr(residual),
                   residual.stride(0) if residual is not None else 0, _ptr(bias), M, N, K, float(alpha),
                   self.status.data_ptr(), self._st(), tag=tag or f"gemm_{'t' if a_mn else 'n'}{'n' if b_mn else 't'}")
        return out

    # -- embedding --------------------------------------------------------------------
    def embedding(self, weight, ids):
        T, H = ids.shape[0], weight.shape[1]
        out = torch.empty(T, H, dtype=weight.dtype, device=self.device)
        self._call("mtb200_embedding_fwd", weight.data_ptr(), ids.data_ptr(), out.data_ptr(), T, H, weight.shape[0],
                   self.status.data_ptr(), self._st())
        return out

    def embedding_bwd(self, dweight, ids, dx):
        """dweight[ids] += dx, deterministic: a stable sort groups equal ids; one block sums each group in fp32."""
        sorted_ids, order = torch.sort(ids, stable=True)
        self._call("mtb200_embedding_bwd", dweight.data_ptr(), sorted_ids.data_ptr(), order.data_ptr(), dx.data_ptr(),
                   ids.shape[0], dweight.shape[1], dweight.shape[0], self.status.data_ptr(), self._st())

    # -- rmsnorm ----------------------------------------------------------------------
    def rmsnorm(self, x, w, eps):
        T, H = x.shape
        y = torch.empty_like(x)
        rstd = torch.empty(T, dtype=torch.float32, device=self.device)
        self._call("mtb200_rmsnorm_fwd", x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), eps, T, H, self._st())
        return y, rstd

    def rmsnorm_bwd(self, dy, x, rstd, w, dw_out, add_to=None):
        T, H = x.shape
        dx = torch.empty_like(x)
        blocks = self.lib.mtb200_rmsnorm_bwd_blocks(T)
        part = self._buf("rms_part", blocks * H, torch.float32)
        self._call("mtb200_rmsnorm_bwd", dy.data_ptr(), x.data_ptr(), rstd.data_ptr(), w.data_ptr(), _ptr(add_to),
                   dx.data_ptr(), part.data_ptr(), dw_out.data_ptr(), T, H, self._st(), n=2)
        return dx

    # -- layernorm (Starcoder2) -----------------------------------------------------------
    def layernorm(self, x, w, b, eps):
        """``((x - mean) * rstd) * w + b``; returns ``(y, (mean, rstd))`` with fp32 row statistics."""
        T, H = x.shape
        y = torch.empty_like(x)
        mean = torch.empty(T, dtype=torch.float32, device=self.device)
        rstd = torch.empty(T, dtype=torch.float32, device=self.device)
        self._call("mtb200_layernorm_fwd", x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr(),
                   rstd.data_ptr(), eps, T, H, self._st())
        return y, (mean, rstd)

    def layernorm_bwd(self, dy, x, stats, w, dw_out, db_out, add_to=None):
        T, H = x.shape
        dx = torch.empty_like(x)
        blocks = self.lib.mtb200_rmsnorm_bwd_blocks(T)
        part = self._buf("layernorm_dw", blocks * 2 * H, torch.float32)
        self._call("mtb200_layernorm_bwd", dy.data_ptr(), x.data_ptr(), stats[0].data_ptr(), stats[1].data_ptr(), w.data_ptr(),
                   _ptr(add_to), dx.data_ptr(), part.data_ptr(), dw_out.data_ptr(), db_out.data_ptr(), T, H, self._st(), n=2)
        return dx

    # -- linear -----------------------------------------------------------------------
    def linear(self, x, w, bias=None, residual=None, gather=None, alpha=1.0, out=None):
        """``alpha * x @ w.T (+bias) (+residual)``. ``gather = (GatherPlan, stage)`` runs the projection with the all-gather of its parameter
        group fused into the same kernel (symmetric-memory backend only). ``out``: write into this ``[T, N]`` view (rows of a
        larger buffer) instead of a new tensor."""
        T, K = x.shape
        N = w.shape[0]
        if out is None:
            out = torch.empty(T, N, dtype=x.dtype, device=self.device)
        if gather is not None:
            assert residual is None and alpha == 1.0
            ev = self._ev()
            gather[0].launch(self, x, w, bias, out, gather[1])
            self._ev_end("gemm_nt_allgather", ev)
            return out
        return self.gemm(x, False, w, False, out, T, N, K, residual=residual, bias=bias, alpha=alpha)

    def linear_dgrad(self, dy, w, alpha=1.0, out=None):
        T, N = dy.shape
        K = w.shape[1]
        if out is None:
            out = torch.empty(T, K, dtype=dy.dtype, device=self.device)
        return self.gemm(dy, False, w, True, out, T, K, N, alpha=alpha)

    def linear_wgrad(self, dy, x, dw_out, dbias_out=None, alpha=1.0):
        T, N = dy.shape
        K = x.shape[1]
        self.gemm(dy, True, x, True, dw_out, N, K, T, alpha=alpha)
        if dbias_out is not None:
            scratch = self._buf("colsum", 32 * N, torch.float32)
            self._call("mtb200_colsum", dy.data_ptr(), dy.stride(0), dbias_out.data_ptr(), scratch.data_ptr(), T, N,
                       self._st(), n=2)

    # -- rope -------------------------------------------------------------------------
    def rope_(self, qkv, position_ids, inv_freq, n_q_heads, n_kv_heads, head_dim, inverse=False, rot_dim=None):
        if rot_dim is not None and rot_dim != head_dim:
            # A partial rotary embedding (Phi-4-mini) pairs dimension i with i + rot_dim / 2 and leaves the tail of the head
            # alone; the kernel pairs i with i + head_dim / 2. Such models take the PyTorch-op form of the rotation.
            from .torch_ref import TorchOps
            return TorchOps.rope_(self, qkv, position_ids, inv_freq, n_q_heads, n_kv_heads, head_dim, inverse, rot_dim)
        assert position_ids.dtype == torch.int32
        self._call("mtb200_rope", qkv.data_ptr(), position_ids.data_ptr(), inv_freq.data_ptr(), qkv.shape[0],
                   qkv.stride(0), n_q_heads + n_kv_heads, head_dim, int(inverse), self._st())
        return qkv

    # -- per-head RMSNorm of q and k (Qwen3) -----------------------------------------------
    def head_rmsnorm_(self, qkv, wq, wk, eps, n_q_heads, n_kv_heads, head_dim):
        """Normalises every q head (weight ``wq``) and k head (``wk``) of ``qkv`` over ``head_dim``, in place;
        returns the reciprocal RMS per (token, head), ``[T * (n_q + n_kv)]`` fp32."""
        T, nh = qkv.shape[0], n_q_heads + n_kv_heads
        rstd = torch.empty(T * nh, dtype=torch.float32, device=self.device)
        self._call("mtb200_head_rmsnorm_fwd", qkv.data_ptr(), wq.data_ptr(), wk.data_ptr(), rstd.data_ptr(), eps, T,
                   qkv.stride(0), n_q_heads, nh, head_dim, self._st())
        return rstd

    def head_rmsnorm_bwd_(self, dqkv, pre, rstd, wq, wk, dwq_out, dwk_out, n_q_heads, n_kv_heads, head_dim):
        """In place on the q and k columns of ``dqkv``: gradient of the normalised heads in, gradient of the projection
        output out. ``pre``: the q|k heads before the norm, ``[T, (n_q + n_kv) * head_dim]``."""
        T, nh = dqkv.shape[0], n_q_heads + n_kv_heads
        blocks = self.lib.mtb200_head_rmsnorm_bwd_blocks(T, nh)
        part = self._buf("head_rmsnorm_dw", blocks * 2 * head_dim, torch.float32)
        self._call("mtb200_head_rmsnorm_bwd", dqkv.data_ptr(), pre.data_ptr(), rstd.data_ptr(), wq.data_ptr(), wk.data_ptr(),
                   part.data_ptr(), dwq_out.data_ptr(), dwk_out.data_ptr(), T, dqkv.stride(0), pre.stride(0), n_q_heads, nh,
                   head_dim, self._st(), n=2)
        return dqkv

    # -- attention --------------------------------------------------------------------
    def _attn_plan(self, cu_host, block, most_work_last_block: bool):
        """Work table for the attention kernels: one row (seq_start, seq_len, block_start) per
        128-row block of every sequence, most work first (forward: late query blocks see the most
        keys; backward: early key blocks are seen by the most queries). Built once per minibatch
        and reused by every layer."""
        key = (id(cu_host), block, most_work_last_block)
        hit = self._attn_plan_cache.get(key)
        if hit is not None and hit[0] is cu_host:
            return hit[1]
        items = []
        for a, b in zip(cu_host[:-1], cu_host[1:]):
            n = b - a
            for s0 in range(0, n, block):
                work = s0 if most_work_last_block else n - s0
                items.append((work, a, n, s0))
        items.sort(key=lambda it: -it[0])
        table = torch.tensor([it[1:] for it in items], dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        if len(self._attn_plan_cache) > 8:
            self._attn_plan_cache.clear()
        self._attn_plan_cache[key] = (cu_host, table)
        return table

    def attention(self, qkv, cu_seqlens, cu_host, max_seqlen, hq, hkv, d, scale=None):
        T = qkv.shape[0]
        scale = d ** -0.5 if scale is None else float(scale)
        if self.attention_impl == "flash_attn" or d not in NATIVE_HEAD_DIMS:
            return self._fa_fwd(qkv, cu_seqlens, max_seqlen, hq, hkv, d, scale)
        out = torch.empty(T, hq * d, dtype=qkv.dtype, device=self.device)
        lse = torch.empty(hq, T, dtype=torch.float32, device=self.device)
        plan = self._attn_plan(cu_host, 128, True)
        self._call("mtb200_attn_fwd", qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), lse.data_ptr(),
                   plan.data_ptr(), plan.shape[0], T, hq, hkv, d, self.attn_fwd_flags, scale, self.status.data_ptr(), self._st())
        return out, lse

    def attention_bwd(self, dout, qkv, out, lse, cu_seqlens, cu_host, max_seqlen, hq, hkv, d, scale=None):
        T = qkv.shape[0]
        scale = d ** -0.5 if scale is None else float(scale)
        if self.attention_impl == "flash_attn" or d not in NATIVE_HEAD_DIMS:
            return self._fa_bwd(dout, qkv, out, lse, cu_seqlens, max_seqlen, hq, hkv, d, scale)
        dqkv = torch.empty_like(qkv)
        plan = self._attn_plan(cu_host, 128, False)
        delta = torch.empty(hq, T, dtype=torch.float32, device=self.device)
        dq_acc = torch.zeros(T, hq * d, dtype=torch.float32, device=self.device)
        self._call("mtb200_attn_bwd", qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), dout.data_ptr(),
                   dout.stride(0), dqkv.data_ptr(), dqkv.stride(0), lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(),
                   plan.data_ptr(), plan.shape[0], T, hq, hkv, d, 0, scale,
                   self.status.data_ptr(), self._st(), n=3)
        return dqkv

    # Library attention (flash-attn 2): selectable for A/B comparisons, and the path of head dimensions the
    # tcgen05 kernels are not built for (Gemma's 256: S plus a 256-column output accumulator would fill tensor memory
    # with no second S buffer to overlap softmax and MMA, so it needs a kernel of its own design).
    def _fa_fwd(self, qkv, cu, max_seqlen, hq, hkv, d, scale):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_forward
        T = qkv.shape[0]
        q = qkv[:, : hq * d].view(T, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].view(T, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
        ev = self._ev()
        out, lse, _, _ = _flash_attn_varlen_forward(q, k, v, cu, cu, max_seqlen, max_seqlen, 0.0, scale, causal=True)
        self._ev_end("flash_attn_fwd", ev)
        return out.reshape(T, hq * d), lse

    def _fa_bwd(self, dout, qkv, out, lse, cu, max_seqlen, hq, hkv, d, scale):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward
        T = qkv.shape[0]
        q = qkv[:, : hq * d].view(T, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].view(T, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
        dqkv = torch.empty_like(qkv)
        dq = dqkv[:, : hq * d].view(T, hq, d)
        dk = dqkv[:, hq * d: (hq + hkv) * d].view(T, hkv, d)
        dv = dqkv[:, (hq + hkv) * d:].view(T, hkv, d)
        ev = self._ev()
        _flash_attn_varlen_backward(dout.view(T, hq, d), q, k, v, out.view(T, hq, d), lse, dq, dk, dv, cu, cu,
                                    max_seqlen, max_seqlen, 0.0, scale, True, -1, -1, 0.0, None, False)
        self._ev_end("flash_attn_bwd", ev)
        return dqkv

    # -- swiglu -----------------------------------------------------------------------
    def swiglu(self, gate_up, act="silu"):
        """``act(gate) * up`` over ``[gate | up]``: SiLU (SwiGLU) or the tanh-approximated GELU (GeGLU)."""
        T, F2 = gate_up.shape
        out = torch.empty(T, F2 // 2, dtype=gate_up.dtype, device=self.device)
        self._call(_GLU[act] + "_fwd", gate_up.data_ptr(), out.data_ptr(), T, F2 // 2, self._st())
        return out

    def swiglu_bwd(self, dact, gate_up, act="silu"):
        T, F2 = gate_up.shape
        dgu = torch.empty_like(gate_up)
        self._call(_GLU[act] + "_bwd", dact.data_ptr(), gate_up.data_ptr(), dgu.data_ptr(), T, F2 // 2, self._st())
        return dgu

    def swiglu_bwd_act(self, dact, gate_up, act="silu"):
        """Returns ``(dgate_up, act)``; ``act`` (the forward output) is written over ``dact``."""
        T, F2 = gate_up.shape
        dgu = torch.empty_like(gate_up)
        self._call(_GLU[act] + "_bwd_act", dact.data_ptr(), gate_up.data_ptr(), dgu.data_ptr(), T, F2 // 2, self._st())
        return dgu, dact

    # -- plain GELU (tanh approximation) of a not gated MLP ----------------------------------
    def gelu(self, x):
        y = torch.empty_like(x)
        self._call("mtb200_gelu_fwd", x.data_ptr(), y.data_ptr(), x.numel(), self._st())
        return y

    def gelu_bwd(self, dy, x):
        dx = torch.empty_like(x)
        self._call("mtb200_gelu_bwd", dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), self._st())
        return dx

    # -- fused linear + cross-entropy ---------------------------------------------------
    def linear_ce(self, x, w, targets, grad_scale, dw_out, accumulate_dw=False, ignore_index=-100, logit_scale=1.0):
        """Per-token CE of ``logit_scale * x @ w.T``. Chunked over tokens (8192 rows): bf16 logits chunk
        by the tcgen05 GEMM (fp32 accumulation, one rounding: what the reference's fused linear-CE holds
        too) -> per-row softmax statistics, loss and the bf16 gradient written over the logits -> dX
        chunk and dW accumulation, again on the tcgen05 GEMM. Only ``[chunk, V]`` logits ever exist.
        dW is accumulated in fp32 and rounded to bf16 once at the end."""
        T, H = x.shape
        V = w.shape[0]
        loss = torch.empty(T, dtype=torch.float32, device=self.device)
        dx = torch.empty_like(x)
        ck = min(self.ce_chunk, T)
        logits = self._buf("ce_logits", ck * V, torch.bfloat16).view(ck, V)
        dw32 = self._buf("ce_dw", V * H, torch.float32).view(V, H)
        first = True
        for a in range(0, T, ck):
            n = min(ck, T - a)
            self.gemm(x[a:a + n], False, w, False, logits, n, V, H, alpha=logit_scale)
            self._call("mtb200_ce_fwd_bwd", logits.data_ptr(), V, 1, targets[a:a + n].data_ptr(), loss[a:a + n].data_ptr(),
                       logits.data_ptr(), V, n, V, float(grad_scale), ignore_index, self._st())
            self.gemm(logits, False, w, True, dx[a:a + n], n, H, V, alpha=logit_scale)
            self.gemm(logits, True, x[a:a + n], True, dw32, V, H, n, residual=None if first else dw32, alpha=logit_scale)
            first = False
        self._call("mtb200_f32_to_bf16", dw_out.data_ptr(), dw32.data_ptr(), V * H, int(accumulate_dw), self._st())
        return loss, dx

    # -- optimizer --------------------------------------------------------------------
    def sumsq(self, g):
        out = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._call("mtb200_sumsq", g.data_ptr(), g.numel(), out.data_ptr(), self._st())
        return out

    def accumulate(self, acc, src, accumulate: bool):
        """acc(fp32) = (acc if accumulate else 0) + src (bf16 or fp32)."""
        self._call("mtb200_accumulate", acc.data_ptr(), src.data_ptr(), acc.numel(), int(src.dtype == torch.float32),
                   int(accumulate), self._st())

    def adamw_step(self, master, m, v, grad, param_out, lr, beta1, beta2, eps, weight_decay, step, grad_coef):
        if not torch.is_tensor(grad_coef):
            grad_coef = torch.full((1,), float(grad_coef), dtype=torch.float32, device=self.device)
        grad_coef = grad_coef.reshape(1).float()
        self._call("mtb200_adamw", master.data_ptr(), m.data_ptr(), v.data_ptr(), int(m.dtype == torch.float32),
                   grad.data_ptr(), param_out.data_ptr(), master.numel(), lr, beta1, beta2, eps, weight_decay, step,
                   grad_coef.data_ptr(), self._st())
