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

Distribution: each projection matrix is OWNED by one rank (round robin), which keeps its factors,
their AdamW moments and the frozen dense part. Per step the block's reduced gradient is gathered
once (the engine's reduce-scatter has already summed it over ranks), owners update their matrices
and broadcast the recomposed weights; every rank copies the slice it shards. All other parameters
(norms, biases, embedding, head) are updated by the engine's ordinary sharded AdamW. The gradient
norm that drives clipping is taken over the projected factor gradients plus those other
parameters.

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
    return [("wqkv", 0, q, "q_proj"), ("wqkv", q, q + kv, "k_proj"), ("wqkv", q + kv, q + 2 * kv, "v_proj"),
            ("wo", 0, h, "o_proj"), ("wgu", 0, f, "gate_proj"), ("wgu", f, 2 * f, "up_proj"), ("wd", 0, h, "down_proj")]


def svd_split(w: torch.Tensor, rank_ratio: float):
    """Returns ``(U_hi, S_hi, V_hi, U_lo, S_lo, V_lo)`` of ``w`` (float32/float64 input)."""
    u, s, vh = torch.linalg.svd(w, full_matrices=False)
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
    block: int
    name: str
    r0: int
    r1: int
    owner: int
    # owner-only state
    w_hi: torch.Tensor = None
    u_hi: torch.Tensor = None
    v_hi: torch.Tensor = None
    factors: list = None      # [U_lo, S_lo, V_lo]
    m: list = None
    v: list = None
    grads: list = None


class OSFT:
    def __init__(self, engine, rank_ratio: float = 0.5, factor_dtype=torch.float32, projection: str = "auto"):
        self.eng, self.rank_ratio, self.dtype = engine, rank_ratio, factor_dtype
        # "tcgen05": projection GEMMs on the hand-written kernel (GPU, dims multiple of 8); "torch": PyTorch matmuls
        self.projection = projection if projection != "auto" else ("tcgen05" if hasattr(engine.ops, "gemm") else "torch")
        self.world, self.rank = engine.world, engine.rank
        self.mats: list[_Matrix] = []
        idx = 0
        for b in range(len(engine.blocks)):
            for name, r0, r1, _ in osft_targets(engine.cfg):
                self.mats.append(_Matrix(b, name, r0, r1, idx % self.world))
                idx += 1
        self._decompose()

    # -- helpers ------------------------------------------------------------------------
    def _gather_fp32(self, shard: torch.Tensor, grp) -> torch.Tensor:
        if self.world == 1:
            return shard
        full = torch.empty(grp.layout.padded_numel, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard.contiguous())
        return full

    def _decompose(self) -> None:
        for b, grp in enumerate(self.eng.blocks):
            full = self._gather_fp32(grp.master, grp)
            views = grp.layout.views(full)
            for mt in (m for m in self.mats if m.block == b and m.owner == self.rank):
                w = views[mt.name][mt.r0:mt.r1].to(self.dtype)
                u_hi, s_hi, v_hi, u_lo, s_lo, v_lo = svd_split(w, self.rank_ratio)
                mt.u_hi, mt.v_hi = u_hi.contiguous(), v_hi.contiguous()
                mt.w_hi = (u_hi * s_hi) @ v_hi
                mt.factors = [u_lo, s_lo, v_lo]
                mt.m = [torch.zeros_like(t) for t in mt.factors]
                mt.v = [torch.zeros_like(t) for t in mt.factors]

    def _mask_targets(self, grp, block: int, tensor: torch.Tensor, value: float = 0.0) -> None:
        """Sets this rank's slice of every target matrix region of ``tensor`` (a shard) to ``value``."""
        s = grp.layout.shard_numel
        lo = self.rank * s
        for mt in (m for m in self.mats if m.block == block):
            spec = grp.layout.specs[mt.name]
            cols = spec.shape[1]
            a, bnd = spec.offset + mt.r0 * cols, spec.offset + mt.r1 * cols
            a, bnd = max(a, lo), min(bnd, lo + s)
            if a < bnd:
                tensor[a - lo: bnd - lo] = value

    # -- training-state checkpoints ------------------------------------------------------------
    def state_tensors(self) -> dict:
        """Trainable factors and their AdamW moments of the matrices this rank owns (the frozen part
        is rebuilt from the weights at start-up and is not stored)."""
        out = {}
        for i, mt in enumerate(self.mats):
            if mt.owner == self.rank:
                for kind, lst in (("f", mt.factors), ("m", mt.m), ("v", mt.v)):
                    for j, t in enumerate(lst):
                        out[f"osft.{i}.{kind}{j}"] = t
        return out

    def load_state_tensors(self, tensors: dict) -> None:
        for i, mt in enumerate(self.mats):
            if mt.owner == self.rank:
                for kind, lst in (("f", mt.factors), ("m", mt.m), ("v", mt.v)):
                    for j, t in enumerate(lst):
                        t.copy_(tensors[f"osft.{i}.{kind}{j}"].to(t.dtype))

    # -- the optimizer step -----------------------------------------------------------------
    @torch.no_grad()
    def optimizer_step(self, lr: float) -> torch.Tensor:
        eng, o = self.eng, self.eng.optim
        if eng.side.cuda:
            torch.cuda.current_stream().wait_stream(eng.side.stream)
        dev = eng.device
        sq = torch.zeros(1, dtype=torch.float32, device=dev)
        # 1. factor gradients (owners), projected; dense target gradients are then dropped from the shards
        for b, grp in enumerate(eng.blocks):
            if not grp.has_grad:
                continue
            full = self._gather_fp32(grp.gacc, grp)
            views = grp.layout.views(full)
            for mt in (m for m in self.mats if m.block == b and m.owner == self.rank):
                g = views[mt.name][mt.r0:mt.r1].to(self.dtype)
                du, ds, dv = factor_grads(g, *mt.factors)
                dims = (du.shape[0], du.shape[1], dv.shape[1], mt.u_hi.shape[1])
                if self.projection == "tcgen05" and all(d % 8 == 0 and d > 0 for d in dims):
                    du, dv = project_orthogonal_tcgen05(eng.ops, du, dv, mt.u_hi, mt.v_hi)
                else:
                    du, dv = project_orthogonal(du, dv, mt.u_hi, mt.v_hi)
                mt.grads = [du, ds, dv]
                sq += sum(t.float().pow(2).sum() for t in mt.grads).to(dev)
            self._mask_targets(grp, b, grp.gacc, 0.0)
            del full, views
        # 2. global norm over factor gradients + every non-target parameter
        for grp in eng.groups:
            if grp.has_grad:
                sq += eng.ops.sumsq(grp.gacc).reshape(1)
        if self.world > 1:
            dist.all_reduce(sq)
        norm = sq.sqrt().squeeze(0)
        coef = torch.clamp(o.max_grad_norm / (norm + 1e-6), max=1.0) if o.max_grad_norm and o.max_grad_norm > 0 \
            else torch.ones((), dtype=torch.float32, device=dev)
        eng.step_count += 1
        t = eng.step_count
        # 3. engine AdamW for everything (target regions see zero gradients and are overwritten below)
        for grp in eng.groups:
            if grp.has_grad:
                eng.ops.adamw_step(grp.master, grp.m, grp.v, grp.gacc, grp.shard, lr, o.beta1, o.beta2, o.eps,
                                   o.weight_decay, t, coef)
                grp.has_grad = False
                grp.sq_done = False
        # 4. AdamW on the factors, recompose, distribute
        bc1, bc2 = 1.0 - o.beta1 ** t, 1.0 - o.beta2 ** t
        c = coef.to(self.dtype)
        for b, grp in enumerate(eng.blocks):
            s = grp.layout.shard_numel
            lo = self.rank * s
            for mt in (m for m in self.mats if m.block == b):
                spec = grp.layout.specs[mt.name]
                cols = spec.shape[1]
                if mt.owner == self.rank:
                    if mt.grads is not None:
                        for p, g, m1, v1 in zip(mt.factors, mt.grads, mt.m, mt.v):
                            g = g * c
                            if o.weight_decay:
                                p.mul_(1.0 - lr * o.weight_decay)
                            m1.mul_(o.beta1).add_(g, alpha=1.0 - o.beta1)
                            v1.mul_(o.beta2).addcmul_(g, g, value=1.0 - o.beta2)
                            p.addcdiv_(m1, (v1.sqrt() / (bc2 ** 0.5)).add_(o.eps), value=-lr / bc1)
                        mt.grads = None
                    u_lo, s_lo, v_lo = mt.factors
                    w = (mt.w_hi + (u_lo * s_lo) @ v_lo).float().contiguous()
                else:
                    w = torch.empty(mt.r1 - mt.r0, cols, dtype=torch.float32, device=dev)
                if self.world > 1:
                    dist.broadcast(w, src=mt.owner)
                a, bnd = spec.offset + mt.r0 * cols, spec.offset + mt.r1 * cols
                x0, x1 = max(a, lo), min(bnd, lo + s)
                if x0 < x1:
                    grp.master[x0 - lo: x1 - lo] = w.reshape(-1)[x0 - a: x1 - a]
            grp.shard.copy_(grp.master.to(grp.shard.dtype))
        eng._sq.zero_()
        if eng.symmetric:
            eng.comm.barrier()
        if eng.side.cuda:
            eng.side.stream.wait_stream(torch.cuda.current_stream())
        return norm


def enable_osft(engine, rank_ratio: float = 0.5) -> OSFT:
    """Switches ``engine.optimizer_step`` to the OSFT update. Returns the controller."""
    ctl = OSFT(engine, rank_ratio)
    engine.osft = ctl
    engine.optimizer_step = ctl.optimizer_step
    return ctl
