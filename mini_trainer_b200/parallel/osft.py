"""Orthogonal-subspace fine-tuning (OSFT) on top of the sharding engine.

Every attention and MLP projection ``W [out, in]`` (q, k, v, o, gate, up, down of every block) is
decomposed once with an SVD, ``W = U diag(S) V`` (``V`` is ``[k, in]``). The top ``rank_ratio`` of
the singular directions ``(U_hi, S_hi, V_hi)`` is frozen; the remaining low subspace
``(U_lo, S_lo, V_lo)`` is what training updates:

    W = U_hi diag(S_hi) V_hi + U_lo diag(S_lo) V_lo

The engine still runs dense GEMMs and produces the dense gradient ``G = dL/dW``; the factor
gradients follow from the chain rule

    dU_lo = G V_lo^T diag(S_lo)      dS_lo = diag(U_lo^T G V_lo^T)      dV_lo = diag(S_lo) U_lo^T G

and are then projected orthogonal to the frozen subspace so the update cannot move energy back
into it:

    dU_lo <- dU_lo - U_hi (U_hi^T dU_lo)           dV_lo <- dV_lo - (dV_lo V_hi^T) V_hi

AdamW runs on the factors, ``W`` is recomposed and written back into the engine's fp32 master /
bf16 working shards, so checkpoints stay plain HF safetensors.

Distribution: each projection matrix is OWNED by one rank (round robin over the 7 x L matrices, so
the factor state is sharded 1/world), which keeps its factors, their AdamW moments and the frozen
dense part. All other parameters (norms, biases, embedding, head) are updated by the engine's
ordinary sharded AdamW. The gradient norm that drives clipping is taken over the projected factor
gradients plus those other parameters.

On the symmetric (NVLink) backend nothing on the step path calls NCCL:

* backward: as soon as a projection's dense gradient is complete in the block's gradient buffer, ONE tcgen05
  GEMM kernel on the owning rank pulls that region from every rank, sums it in fp32 and multiplies it by
  ``V_lo^T`` (``SymmetricComm.reduce_gemm_to_owner``: the reduce-scatter with ownership by MATRIX, fused into
  the GEMM that consumes the reduced gradient), accumulating over microbatches into the gradient slot of
  ``U_lo``; ``U_lo^T G`` follows on the reduced gradient the kernel leaves behind. ``MTB200_OSFT_FUSED=0`` runs
  the reduction as a kernel of its own into an fp32 matrix gradient (``reduce_to_owner``). The small tensors of
  the block go through the ordinary slice reduction restricted to their region;
* optimizer: on the owner the two projections (applied twice, which squares the bf16 rounding residue left
  inside the frozen subspace) and the recomposition ``W_hi + (U_lo S_lo) V_lo`` are tcgen05 GEMMs (bf16 operands, fp32 accumulate and output); AdamW on
  all factors of a rank is ONE launch of the fused kernel over a flat buffer; the norm scalar is
  all-reduced by the arena's scalar kernel;
* the recomposed fp32 matrices sit in a symmetric staging buffer; every rank pulls exactly the part
  that lies in its own flat slice (``SymmetricComm.pull``) into its master weights.

On the other backends (one rank, NCCL, gloo: tests and the baseline-grade path) the engine reduces as
usual, each block's reduced gradient is gathered once, owners update and broadcast their matrices.

The reference snapshot contains no OSFT code; this module defines the behaviour from the
description above, and ``tests/test_osft.py`` pins it against a float64 autograd oracle.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..models.config import ModelConfig


def osft_targets(cfg: ModelConfig) -> list:
    """(param name in the block layout, first row, last row, HF-style label) of every projection."""
    q, kv, f, h = cfg.q_size, cfg.kv_size, cfg.intermediate_size, cfg.hidden_size
    attn = [("wqkv", 0, q, "q_proj"), ("wqkv", q, q + kv, "k_proj"), ("wqkv", q + kv, q + 2 * kv, "v_proj"), ("wo", 0, h, "o_proj")]
    if not cfg.mlp_gated:
        return attn + [("wgu", 0, f, "c_fc"), ("wd", 0, h, "c_proj")]
    return attn + [("wgu", 0, f, "gate_proj"), ("wgu", f, 2 * f, "up_proj"), ("wd", 0, h, "down_proj")]


def svd_thin(w: torch.Tensor, method: str = "auto"):
    """Thin SVD ``w = U diag(S) Vh`` with singular values in descending order.

    ``exact``: ``torch.linalg.svd``. ``gram``: eigendecomposition of the smaller Gram matrix (``w^T w`` or
    ``w w^T``) and one GEMM for the other side: a few GEMMs and one symmetric eigenproblem of the small
    dimension instead of a full bidiagonalisation, which is what makes decomposing the 196 projections
    of a 7B model at start-up a matter of seconds. The side that comes from the eigenproblem is
    orthonormal to working precision; the other side is ``w v / s``, so ``U diag(S) Vh`` reproduces ``w``
    to that same precision whatever the conditioning, but its columns for singular values below about
    ``sqrt(eps) * s_max`` are only approximately orthonormal. ``auto``: ``gram`` for fp32 matrices on a GPU
    whose small dimension exceeds 1024, ``exact`` otherwise."""
    rows, cols = w.shape
    if method == "auto":
        method = "gram" if (w.is_cuda and w.dtype == torch.float32 and min(rows, cols) > 1024) else "exact"
    if method == "exact":
        return torch.linalg.svd(w, full_matrices=False)
    if rows >= cols:
        lam, v = torch.linalg.eigh(w.t() @ w)                 # ascending
        lam, v = lam.flip(0).clamp_min(0), v.flip(1)
        s = lam.sqrt()
        u = (w @ v) / s.clamp_min(torch.finfo(w.dtype).tiny)
        return u, s, v.t().contiguous()
    lam, u = torch.linalg.eigh(w @ w.t())
    lam, u = lam.flip(0).clamp_min(0), u.flip(1)
    s = lam.sqrt()
    vh = (u.t() @ w) / s.clamp_min(torch.finfo(w.dtype).tiny).unsqueeze(1)
    return u.contiguous(), s, vh


def svd_split(w: torch.Tensor, rank_ratio: float, method: str = "exact"):
    """Returns ``(U_hi, S_hi, V_hi, U_lo, S_lo, V_lo)`` of ``w`` (float32/float64 input)."""
    u, s, vh = svd_thin(w, method)
    k = s.numel()
    k_hi = max(0, min(k - 1, int(round(k * rank_ratio))))
    return u[:, :k_hi], s[:k_hi], vh[:k_hi], u[:, k_hi:].clone(), s[k_hi:].clone(), vh[k_hi:].clone()


def factor_grads(g, u_lo, s_lo, v_lo):
    """Chain rule from the dense gradient ``g`` to the low-subspace factors."""
    gv = g @ v_lo.t()                       # [out, k_lo]
    du = gv * s_lo
    ds = (u_lo * gv).sum(0)
    dv = (u_lo.t() @ g) * s_lo.unsqueeze(1)
    return du, ds, dv


def project_orthogonal(du, dv, u_hi, v_hi):
    """Removes the components of the factor gradients that lie in the frozen subspace."""
    if u_hi.shape[1]:
        du = du - u_hi @ (u_hi.t() @ du)
        dv = dv - (dv @ v_hi.t()) @ v_hi
    return du, dv


def project_orthogonal_tcgen05(ops, du, dv, u_hi, v_hi):
    """Same projection with the four products on the tcgen05 GEMM (bf16 operands, fp32 accumulate
    and fp32 results; the subtraction is the GEMM's residual epilogue):

        P = U_hi^T dU   (both operands read MN-major)      dU <- dU + U_hi (-P)
        R = dV V_hi^T   (both K-major)                     dV <- dV + (-R) V_hi

    Requires every dimension to be a multiple of 8 (TMA strides); callers fall back to
    ``project_orthogonal`` otherwise.
    """
    k_hi = u_hi.shape[1]
    if k_hi == 0:
        return du, dv
    bf = torch.bfloat16
    rows, k_lo = du.shape
    cols = dv.shape[1]
    u16, v16 = u_hi.to(bf).contiguous(), v_hi.to(bf).contiguous()
    du32, dv32 = du.float().contiguous(), dv.float().contiguous()
    pmat = torch.empty(k_hi, k_lo, dtype=torch.float32, device=du.device)
    ops.gemm(u16, True, du32.to(bf), True, pmat, k_hi, k_lo, rows)
    du_out = torch.empty_like(du32)
    ops.gemm(u16, False, (-pmat).to(bf), True, du_out, rows, k_lo, k_hi, residual=du32)
    rmat = torch.empty(k_lo, k_hi, dtype=torch.float32, device=du.device)
    ops.gemm(dv32.to(bf), False, v16, False, rmat, k_lo, k_hi, cols)
    dv_out = torch.empty_like(dv32)
    ops.gemm((-rmat).to(bf), False, v16, True, dv_out, k_lo, cols, k_hi, residual=dv32)
    return du_out.to(du.dtype), dv_out.to(dv.dtype)




@dataclass
class _Matrix:
    index: int
    block: int
    name: str           # tensor of the block layout that holds it (wqkv / wo / wgu / wd)
    r0: int
    r1: int
    owner: int
    elem_lo: int = 0    # extent inside the block's flat buffer
    elem_hi: int = 0
    out: int = 0
    cols: int = 0
    k_hi: int = 0
    k_lo: int = 0
    # owner-only state
    w_hi: torch.Tensor = None      # frozen dense part, fp32 [out, cols]
    u_hi: torch.Tensor = None      # [out, k_hi]  (bf16 on the kernel path, factor dtype otherwise)
    v_hi: torch.Tensor = None      # [k_hi, cols]
    fac_off: int = 0               # offset of (U_lo | S_lo | V_lo) in the rank's flat factor buffers
    g_acc: torch.Tensor = None     # fp32 [out, cols] reduced dense gradient (matrix-owned reduction only)
    has_grad: bool = False
    stage_off: int = 0             # offset of the recomposed matrix in the staging buffer


class OSFT:
    """Controller that replaces ``engine.optimizer_step`` (and, on the symmetric backend, the
    reduction of the projection gradients) once ``enable_osft`` has run."""

    def __init__(self, engine, rank_ratio: float = 0.5, factor_dtype=torch.float32, projection: str = "auto",
                 projection_passes: int = 2, svd_method: str = "auto"):
        self.eng, self.rank_ratio, self.dtype = engine, rank_ratio, factor_dtype
        self.svd_method = svd_method
        self.world, self.rank = engine.world, engine.rank
        # kernel path: every product on the tcgen05 GEMM (bf16 operands, fp32 out); torch path: PyTorch matmuls in the
        # factor dtype (CPU, float64 oracle runs)
        self.kernels = hasattr(engine.ops, "gemm") and projection in ("auto", "tcgen05") and factor_dtype == torch.float32
        self.projection = "tcgen05" if self.kernels else "torch"
        self.passes = projection_passes if self.kernels else 1
        # ownership by matrix inside the reduction itself needs the symmetric backend's kernels
        self.owner_reduce = bool(engine.symmetric) and self.world > 1 and self.kernels
        # the reduction of a projection's gradient runs INSIDE the tcgen05 GEMM that forms G V_lo^T (up to 8 ranks)
        import os as _os
        self.fused = self.owner_reduce and self.world <= 8 and _os.environ.get("MTB200_OSFT_FUSED", "1") != "0"
        self._want_fused = self.fused
        self.mats: list[_Matrix] = []
        cfg = engine.cfg
        lay = engine.blocks[0].layout
        idx = 0
        for b in range(len(engine.blocks)):
            for name, r0, r1, _ in osft_targets(cfg):
                spec = lay.specs[name]
                cols = spec.shape[1]
                k = min(r1 - r0, cols)
                k_hi = max(0, min(k - 1, int(round(k * rank_ratio))))
                self.mats.append(_Matrix(idx, b, name, r0, r1, idx % self.world, spec.offset + r0 * cols, spec.offset + r1 * cols,
                                         r1 - r0, cols, k_hi, k - k_hi))
                idx += 1
        self.by_block = [[m for m in self.mats if m.block == b] for b in range(len(engine.blocks))]
        if any(m.out % 8 or m.cols % 8 or m.k_lo % 8 for m in self.mats):   # TMA strides of the fused kernel's operands
            self.fused = False
        self._alloc_and_decompose()

    # -- set-up ---------------------------------------------------------------------------
    def _mine(self):
        return [m for m in self.mats if m.owner == self.rank]

    def _fac_views(self, mt: _Matrix, flat: torch.Tensor):
        a = mt.fac_off
        u = flat[a: a + mt.out * mt.k_lo].view(mt.out, mt.k_lo)
        a += mt.out * mt.k_lo
        s = flat[a: a + mt.k_lo]
        a += mt.k_lo
        v = flat[a: a + mt.k_lo * mt.cols].view(mt.k_lo, mt.cols)
        return u, s, v

    def factors(self, mt: _Matrix):
        """``(U_lo, S_lo, V_lo)`` views of a matrix this rank owns."""
        return self._fac_views(mt, self.fac)

    def _alloc_and_decompose(self) -> None:
        eng, dev = self.eng, self.eng.device
        total = 0
        for mt in self._mine():
            mt.fac_off = total
            total += -(-(mt.out * mt.k_lo + mt.k_lo + mt.k_lo * mt.cols) // 8) * 8
        self.fac = torch.zeros(total, dtype=self.dtype, device=dev)        # U_lo | S_lo | V_lo of every owned matrix
        self.fac_m = torch.zeros_like(self.fac)
        self.fac_v = torch.zeros_like(self.fac)
        self.fac_g = torch.zeros_like(self.fac)
        self.fac16 = torch.zeros(total, dtype=torch.bfloat16, device=dev) if self.kernels else None
        # staging of the recomposed matrices: the same size and offsets on every rank (peers pull from it)
        per_rank = [0] * self.world
        for mt in self.mats:
            mt.stage_off = per_rank[mt.owner]
            per_rank[mt.owner] += mt.out * mt.cols
        n_stage = max(per_rank) if per_rank else 0
        if self.owner_reduce:
            self.stage = eng.comm.alloc_region(n_stage, torch.float32)
        else:
            self.stage = torch.zeros(n_stage, dtype=torch.float32, device=dev)
        for b, grp in enumerate(eng.blocks):
            mine = [m for m in self.by_block[b] if m.owner == self.rank]
            full = self._gather_fp32(grp.master, grp) if (mine or self.world > 1) else None
            for mt in mine:
                w = full[mt.elem_lo: mt.elem_hi].view(mt.out, mt.cols).to(self.dtype)
                u_hi, s_hi, v_hi, u_lo, s_lo, v_lo = svd_split(w, self.rank_ratio, self.svd_method)
                assert u_hi.shape[1] == mt.k_hi and u_lo.shape[1] == mt.k_lo
                mt.w_hi = ((u_hi * s_hi) @ v_hi).float().contiguous()
                hdt = torch.bfloat16 if self.kernels else self.dtype
                mt.u_hi, mt.v_hi = u_hi.to(hdt).contiguous(), v_hi.to(hdt).contiguous()
                u, s, v = self._fac_views(mt, self.fac)
                u.copy_(u_lo); s.copy_(s_lo); v.copy_(v_lo)
                if self.owner_reduce and not self.fused:
                    mt.g_acc = torch.zeros(mt.out, mt.cols, dtype=torch.float32, device=dev)
            del full
        if self.kernels:
            self.fac16.copy_(self.fac)
        if self.fused:
            # one staging buffer for the reduced bf16 gradient of whichever projection is being processed, and the
            # completion words of its 128 KB chunks
            biggest = max((m.out * m.cols for m in self._mine()), default=8)
            self.g_red = torch.empty(biggest, dtype=torch.bfloat16, device=dev)
            self.red_flags = torch.zeros(-(-biggest * 2 // (128 * 1024)) + 1, dtype=torch.int32, device=dev)
            self.red_epoch = 0
        if self.owner_reduce:
            # the slice reduction never touches the projections' regions of the accumulators again: they must
            # read as zero gradient for the engine's AdamW pass from now on
            for grp in eng.blocks:
                grp.gacc.zero_()

    def _gather_fp32(self, shard: torch.Tensor, grp) -> torch.Tensor:
        if self.world == 1:
            return shard
        full = torch.empty(grp.layout.padded_numel, dtype=shard.dtype, device=shard.device)
        try:
            dist.all_gather_into_tensor(full, shard.contiguous())
        except RuntimeError:   # a backend without the flat form
            parts = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(parts, shard.contiguous())
            full = torch.cat(parts)
        return full

    # -- backward-time reduction (symmetric backend) --------------------------------------------
    def reducer(self, i: int, gbuf: torch.Tensor, gslot: int, last: bool):
        """``(notify, finish)`` for block ``i`` (see ``ShardedEngine._region_reducer``): every projection's
        region is reduced to its owner as soon as backward has written it; the block's small tensors go
        through the slice reduction restricted to their region. Region numbers index the flag channels."""
        eng, grp = self.eng, self.eng.blocks[i]
        specs = grp.layout.specs
        mats = {m.index: m for m in self.by_block[i]}
        order = {"wd": ["wd"], "wgu": ["wgu"], "wo": ["wo"]}
        state = {"k": 0}

        def reduce_tensor(name):
            for mt in (m for m in mats.values() if m.name == name):
                k = state["k"]; state["k"] += 1
                eng.comm.grad_ready(gbuf, k)
                mine = mt.owner == self.rank
                with eng.side.run(wait_current=True):
                    if not self.fused:
                        eng.comm.reduce_to_owner(gbuf, mt.g_acc, mt.has_grad, mt.owner, mt.elem_lo, mt.elem_hi, region=k)
                    elif not mine:
                        eng.comm.reduce_gemm_to_owner(eng.ops, gbuf, mt.owner, mt.elem_lo, mt.out, mt.cols, k, None, None, None, False, None, 0)
                    else:
                        # G V_lo^T with the reduction fused in (accumulated over microbatches in the gradient slot of
                        # U_lo), then U_lo^T G on the reduced gradient the kernel left behind (slot of V_lo)
                        u16, _, v16 = self._fac_views(mt, self.fac16)
                        gu, _, gv = self._fac_views(mt, self.fac_g)
                        self.red_epoch += 1
                        staged = self.g_red[: mt.out * mt.cols].view(mt.out, mt.cols)
                        eng.comm.reduce_gemm_to_owner(eng.ops, gbuf, mt.owner, mt.elem_lo, mt.out, mt.cols, k, staged, v16, gu,
                                                      mt.has_grad, self.red_flags, self.red_epoch)
                        self._mm(u16, True, staged, False, residual=gv if mt.has_grad else None, out=gv)
                if mine:
                    mt.has_grad = True

        def reduce_small(lo, hi, final):
            """The tensors that are not projections (norm weights, biases) between two element offsets: plain
            reduce-scatter by flat slice, like a region of a dense block."""
            k = state["k"]; state["k"] += 1
            eng._reduce(grp, gbuf, gslot, last, region=k, elem_lo=lo, elem_hi=hi, final=final)

        names = list(specs)

        def end(n):   # where the tensor laid out after ``n`` starts: tensor starts are 256-byte aligned, tensor ends need not be
            k = names.index(n) + 1
            return specs[names[k]].offset if k < len(names) else grp.layout.numel

        def notify(name):
            if name in order:
                reduce_tensor(name)
            if name == "wd" and end("wd") < grp.layout.numel:   # the down projection's bias lies behind it
                reduce_small(end("wd"), grp.layout.numel, final=False)
            if name == "wo":    # o_proj bias | post-attention norm | gate/up bias
                reduce_small(end("wo"), specs["wgu"].offset, final=False)

        def finish():
            reduce_tensor("wqkv")
            reduce_small(0, specs["wqkv"].offset, final=True)   # input norm | q/k/v bias

        return notify, finish

    @property
    def last_region(self) -> int:
        """Index of the region a block reduces last (what ``wait_consumed`` must wait for)."""
        return len(self.by_block[0]) + 1 + int("bd" in self.eng.blocks[0].layout.specs)

    # -- products -----------------------------------------------------------------------------
    def _mm(self, x, x_t: bool, y, y_t: bool, alpha: float = 1.0, residual=None, out=None):
        """fp32 ``alpha * op(x) @ op(y) (+ residual)`` with ``op`` = transpose when the flag is set. Kernel
        path: bf16 operands on the tcgen05 GEMM; torch path: a plain matmul in the factor dtype."""
        m = x.shape[1] if x_t else x.shape[0]
        kk = x.shape[0] if x_t else x.shape[1]
        n = y.shape[0] if y_t else y.shape[1]
        if not self.kernels or m % 8 or n % 8 or kk % 8:   # TMA strides need multiples of 8 elements
            x, y = (x.float(), y.float()) if self.kernels else (x, y)
            r = (x.t() if x_t else x) @ (y.t() if y_t else y)
            r = r * alpha if alpha != 1.0 else r
            r = r + residual if residual is not None else r
            if out is not None:
                out.copy_(r)
                return out
            return r
        bf = torch.bfloat16
        x16 = x if x.dtype == bf else x.to(bf)
        y16 = y if y.dtype == bf else y.to(bf)
        if out is None:
            out = torch.empty(m, n, dtype=torch.float32, device=x.device)
        # A operand: [M, K] row-major (a_mn = 0) or [K, M] (a_mn = 1); B operand: [N, K] (b_mn = 0) or [K, N] (b_mn = 1)
        self.eng.ops.gemm(x16.contiguous(), x_t, y16.contiguous(), not y_t, out, m, n, kk, residual=residual, alpha=alpha, tag="osft_gemm")
        return out

    def _factor_grads(self, mt: _Matrix, g: torch.Tensor) -> None:
        """Writes the projected gradients of (U_lo, S_lo, V_lo) of ``mt`` into ``fac_g`` from its dense gradient."""
        u, s, v = self._fac_views(mt, self.fac)
        u16, _, v16 = self._fac_views(mt, self.fac16) if self.kernels else (u, None, v)
        gu, gs, gv = self._fac_views(mt, self.fac_g)
        g = g.to(torch.bfloat16) if self.kernels else g.to(self.dtype)
        a = self._mm(g, False, v16, True)                       # G V_lo^T   [out, k_lo]
        gs.copy_((u * a).sum(0))
        du = a * s
        dv = self._mm(u16, True, g, False) * s.unsqueeze(1)     # S U_lo^T G [k_lo, cols]
        if mt.k_hi:
            for _ in range(self.passes):
                p = self._mm(mt.u_hi, True, du, False)          # U_hi^T dU
                du = self._mm(mt.u_hi, False, p, False, alpha=-1.0, residual=du.float() if self.kernels else du)
                r = self._mm(dv, False, mt.v_hi, True)          # dV V_hi^T
                dv = self._mm(r, False, mt.v_hi, False, alpha=-1.0, residual=dv.float() if self.kernels else dv)
        gu.copy_(du)
        gv.copy_(dv)

    def _finish_factor_grads(self, mt: _Matrix) -> None:
        """Fused path: the gradient slots of U_lo and V_lo hold the raw products ``G V_lo^T`` and ``U_lo^T G``
        accumulated during backward; turns them into the projected factor gradients in place."""
        u, s, v = self._fac_views(mt, self.fac)
        gu, gs, gv = self._fac_views(mt, self.fac_g)
        gs.copy_((u * gu).sum(0))
        du = gu * s
        dv = gv * s.unsqueeze(1)
        if mt.k_hi:
            for _ in range(self.passes):
                p = self._mm(mt.u_hi, True, du, False)
                du = self._mm(mt.u_hi, False, p, False, alpha=-1.0, residual=du)
                r = self._mm(dv, False, mt.v_hi, True)
                dv = self._mm(r, False, mt.v_hi, False, alpha=-1.0, residual=dv)
        gu.copy_(du)
        gv.copy_(dv)

    def _recompose(self, mt: _Matrix) -> torch.Tensor:
        """fp32 ``W_hi + (U_lo S_lo) V_lo`` written into this rank's staging slot of ``mt``."""
        u, s, v = self._fac_views(mt, self.fac)
        out = self.stage[mt.stage_off: mt.stage_off + mt.out * mt.cols].view(mt.out, mt.cols)
        if self.kernels:
            self._mm((u * s), False, self._fac_views(mt, self.fac16)[2], False, residual=mt.w_hi, out=out)
        else:
            out.copy_((mt.w_hi.to(self.dtype) + (u * s) @ v).float())
        return out

    # -- training-state checkpoints ------------------------------------------------------------
    def state_tensors(self) -> dict:
        """Trainable factors and their AdamW moments of the matrices this rank owns, as three flat
        tensors (the frozen part is rebuilt from the weights at start-up and is not stored)."""
        return {"osft.factors": self.fac, "osft.m": self.fac_m, "osft.v": self.fac_v}

    def load_state_tensors(self, tensors: dict) -> None:
        for key, dst in (("osft.factors", self.fac), ("osft.m", self.fac_m), ("osft.v", self.fac_v)):
            dst.copy_(tensors[key].to(dst.dtype))
        if self.kernels:
            self.fac16.copy_(self.fac)

    def _factor_layout(self, world: int) -> dict:
        """``{matrix index: (owner, offset in the owner's flat factor buffers, elements)}`` for a run of ``world`` ranks
        (round-robin ownership, offsets in matrix order, sizes rounded up to 8 elements: what ``_alloc_and_decompose`` does)."""
        out, total = {}, [0] * world
        for mt in self.mats:
            n = mt.out * mt.k_lo + mt.k_lo + mt.k_lo * mt.cols
            owner = mt.index % world
            out[mt.index] = (owner, total[owner], n)
            total[owner] += -(-n // 8) * 8
        return out

    def load_state_from(self, files: list, old_world: int) -> None:
        """Factors and moments from a training state written by ``old_world`` ranks (``files``: one open reader per
        old rank): every matrix this rank owns now is read from the flat buffers of the rank that owned it then."""
        then = self._factor_layout(old_world)
        for mt in self._mine():
            owner, off, n = then[mt.index]
            for key, dst in (("osft.factors", self.fac), ("osft.m", self.fac_m), ("osft.v", self.fac_v)):
                src = files[owner].get_slice(key, off, off + n)
                if src.numel() != n:
                    raise RuntimeError(f"{key}: matrix {mt.index} not found in the state of rank {owner} of {old_world}")
                dst[mt.fac_off: mt.fac_off + n].copy_(src.to(dst.dtype))
        if self.kernels:
            self.fac16.copy_(self.fac)

    # -- the optimizer step -----------------------------------------------------------------
    def _mask_targets(self, grp, block: int, tensor: torch.Tensor, value: float = 0.0) -> None:
        """Sets this rank's slice of every projection's region of ``tensor`` (a shard) to ``value``."""
        s = grp.layout.shard_numel
        lo = self.rank * s
        for mt in self.by_block[block]:
            a, b = max(mt.elem_lo, lo), min(mt.elem_hi, lo + s)
            if a < b:
                tensor[a - lo: b - lo] = value

    def _adamw_factors(self, lr: float, coef: torch.Tensor, t: int) -> None:
        o = self.eng.optim
        if self.fac.numel() == 0:
            return
        if self.kernels:   # one launch of the fused kernel over every factor this rank owns; refreshes the bf16 copies
            self.eng.ops.adamw_step(self.fac, self.fac_m, self.fac_v, self.fac_g, self.fac16, lr, o.beta1, o.beta2, o.eps,
                                    o.weight_decay, t, coef)
            return
        g = self.fac_g * coef.to(self.dtype)
        if o.weight_decay:
            self.fac.mul_(1.0 - lr * o.weight_decay)
        self.fac_m.mul_(o.beta1).add_(g, alpha=1.0 - o.beta1)
        self.fac_v.mul_(o.beta2).addcmul_(g, g, value=1.0 - o.beta2)
        bc1, bc2 = 1.0 - o.beta1 ** t, 1.0 - o.beta2 ** t
        self.fac.addcdiv_(self.fac_m, (self.fac_v.sqrt() / (bc2 ** 0.5)).add_(o.eps), value=-lr / bc1)

    @torch.no_grad()
    def optimizer_step(self, lr: float) -> torch.Tensor:
        eng, o = self.eng, self.eng.optim
        if eng.side.cuda:
            torch.cuda.current_stream().wait_stream(eng.side.stream)   # the last reductions have landed
        dev = eng.device
        sq = eng._sq if self.owner_reduce else torch.zeros(1, dtype=torch.float32, device=dev)
        stepped = False
        # 1. projected factor gradients on the owners
        if not self.fused:
            self.fac_g.zero_()
        for b, grp in enumerate(eng.blocks):
            if self.owner_reduce:
                for mt in (m for m in self.by_block[b] if m.owner == self.rank):
                    gu, gs, gv = self._fac_views(mt, self.fac_g)
                    if not mt.has_grad:
                        if self.fused:
                            gu.zero_(); gs.zero_(); gv.zero_()
                        continue
                    if self.fused:
                        self._finish_factor_grads(mt)
                    else:
                        self._factor_grads(mt, mt.g_acc)
                    mt.has_grad = False
                    stepped = True
                continue
            if not grp.has_grad:
                continue
            stepped = True
            full = self._gather_fp32(grp.gacc, grp)
            for mt in (m for m in self.by_block[b] if m.owner == self.rank):
                self._factor_grads(mt, full[mt.elem_lo: mt.elem_hi].view(mt.out, mt.cols))
            self._mask_targets(grp, b, grp.gacc, 0.0)   # the dense gradients of the projections are not applied
            del full
        if self.fac_g.numel():
            sq += (eng.ops.sumsq(self.fac_g) if self.kernels else self.fac_g.float().pow(2).sum()).reshape(1)
        # 2. global norm over factor gradients + every other parameter
        for grp in eng.groups:
            if grp.has_grad and not grp.sq_done:
                sq += eng.ops.sumsq(grp.gacc).reshape(1)
        eng.comm.all_reduce_sum(sq)
        norm = sq.sqrt().squeeze(0)
        coef = torch.clamp(o.max_grad_norm / (norm + 1e-6), max=1.0) if o.max_grad_norm and o.max_grad_norm > 0 \
            else torch.ones((), dtype=torch.float32, device=dev)
        eng.step_count += 1
        t = eng.step_count
        # 3. the engine's AdamW for everything (the projections' regions see zero gradients and are overwritten below)
        for grp in eng.groups:
            if grp.has_grad:
                eng.ops.adamw_step(grp.master, grp.m, grp.v, grp.gacc, grp.shard, lr, o.beta1, o.beta2, o.eps,
                                   o.weight_decay, t, coef)
                grp.has_grad = False
                grp.sq_done = False
        # 4. AdamW on the factors, recomposition into the staging buffer
        if stepped or self.world > 1:
            self._adamw_factors(lr, coef, t)
            for mt in self._mine():
                self._recompose(mt)
        # 5. every rank takes the part of each recomposed matrix that lies in its flat slice
        if self.owner_reduce:
            eng.comm.barrier()    # all staging buffers are complete
        for b, grp in enumerate(eng.blocks):
            s = grp.layout.shard_numel
            lo = self.rank * s
            for mt in self.by_block[b]:
                x0, x1 = max(mt.elem_lo, lo), min(mt.elem_hi, lo + s)
                if self.owner_reduce:
                    if x0 < x1:
                        eng.comm.pull(mt.owner, self.stage, mt.stage_off + (x0 - mt.elem_lo), grp.master[x0 - lo: x1 - lo])
                    continue
                n = mt.out * mt.cols
                w = self.stage[mt.stage_off: mt.stage_off + n]
                if self.world > 1:
                    if mt.owner != self.rank:
                        w = torch.empty(n, dtype=torch.float32, device=dev)
                    dist.broadcast(w, src=mt.owner)
                if x0 < x1:
                    grp.master[x0 - lo: x1 - lo] = w[x0 - mt.elem_lo: x1 - mt.elem_lo]
            grp.shard.copy_(grp.master.to(grp.shard.dtype))
        eng._sq = torch.zeros(1, dtype=torch.float32, device=dev)
        if eng.symmetric:    # nobody pulls a shard (or overwrites a staging buffer) before every rank is done
            eng.comm.barrier()
        if eng.side.cuda:
            eng.side.stream.wait_stream(torch.cuda.current_stream())
        return norm


def enable_osft(engine, rank_ratio: float = 0.5, **kw) -> OSFT:
    """Switches ``engine.optimizer_step`` (and the reduction of the projection gradients, where the
    backend supports ownership by matrix) to the OSFT update. Returns the controller."""
    if engine.cfg.is_moe:
        raise ValueError("OSFT is defined here for the seven dense projections of a block; a mixture-of-experts model "
                         "is trained with the plain AdamW update")
    ctl = OSFT(engine, rank_ratio, **kw)
    engine.osft = ctl
    engine.optimizer_step = ctl.optimizer_step
    return ctl
