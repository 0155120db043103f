"""Sparse mixture-of-experts MLP (Mixtral) with a hand-written backward.

The reference trains Mixtral through ``AutoModelForCausalLM`` (it is on the allow-list of
setup_model_for_training.py:111-123); the function reproduced here is transformers'
``MixtralSparseMoeBlock`` (modeling_mixtral.py) and ``Qwen3MoeSparseMoeBlock`` (modeling_qwen3_moe.py):
router logits in the compute dtype, softmax in fp32, top-k, weights renormalised over the chosen
experts (optional for Qwen3-MoE), each expert a SwiGLU MLP, outputs combined with the weights. No auxiliary load-balancing loss (transformers only adds one with
``output_router_logits``; a config that asks for it is refused at load time).

Schedule: the (token, slot) pairs are sorted by expert once per block, so every expert sees one
contiguous slab of gathered rows and its three projections are plain GEMMs on row slices of shared
buffers (the same tcgen05 kernel as the dense model; slabs of any height, empty ones skipped).
The slab boundaries are the one device-to-host read of a block. Contributions of a token's
experts are put back in token order by the inverse permutation and summed in fp32, so forward and
backward are deterministic (no atomics).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class MoeState:
    """What the backward of the expert MLP reads."""
    probs: torch.Tensor          # [T, E] fp32 softmax of the router logits
    topi: torch.Tensor           # [T, k] experts chosen per token
    w: torch.Tensor              # [T, k] fp32 weights, renormalised over the chosen experts
    order: torch.Tensor          # [T*k] routed row -> index of its (token, slot) pair, grouped by expert
    tok: torch.Tensor            # [T*k] token of each routed row
    bounds: list                 # E+1 host ints: routed rows [bounds[e], bounds[e+1]) belong to expert e
    gu: torch.Tensor             # [T*k, 2F] gate/up pre-activations of the routed rows
    act: Optional[torch.Tensor]  # [T*k, F] SwiGLU output (None: rebuilt in backward)
    gu_s: Optional[torch.Tensor] = None    # [T, 2Fs] gate/up pre-activations of the shared expert (Qwen2-MoE)
    act_s: Optional[torch.Tensor] = None   # [T, Fs] its SwiGLU output (None: rebuilt in backward)


def route(cfg, router_w: torch.Tensor, n2: torch.Tensor, topi: Optional[torch.Tensor] = None):
    """Router of one block: ``(probs, topi, w, order, tok, bounds)``. With ``topi`` given, those experts
    are used instead of the top-k while the weights still follow this call's logits (comparisons
    between backends of different precision, where a near-tie may otherwise select differently)."""
    E, k = cfg.num_local_experts, cfg.num_experts_per_tok
    probs = torch.softmax((n2 @ router_w.t()).float(), dim=-1)
    if topi is None:
        topv, topi = torch.topk(probs, k, dim=-1)
    else:
        topv = probs.gather(1, topi)
    w = topv / topv.sum(-1, keepdim=True) if cfg.norm_topk_prob else topv
    flat = topi.reshape(-1)
    order = torch.argsort(flat, stable=True)
    bounds = [0] + torch.cumsum(torch.bincount(flat, minlength=E), 0).tolist()   # the block's one host read
    tok = torch.div(order, k, rounding_mode="floor")
    return probs, topi, w, order, tok, bounds


def _slabs(bounds: list):
    for e in range(len(bounds) - 1):
        yield e, bounds[e], bounds[e + 1]


def _combine(rows: torch.Tensor, order: torch.Tensor, T: int, k: int) -> torch.Tensor:
    """Routed rows ``[T*k, H]`` back to token order and summed over a token's experts: ``[T, H]`` fp32."""
    buf = torch.empty_like(rows)
    buf[order] = rows
    return buf.view(T, k, rows.shape[1]).float().sum(1)


def moe_forward(ops, cfg, p: dict, n2: torch.Tensor, h1: torch.Tensor, need_out: bool, keep_act: bool):
    """``(h1 + residual_multiplier * MoE(n2), state)``; the output is ``None`` when ``need_out`` is false
    (a recompute inside backward stops after the gate/up projections)."""
    T, H = n2.shape
    k, fe = cfg.num_experts_per_tok, cfg.expert_intermediate_size
    probs, topi, w, order, tok, bounds = route(cfg, p["router"], n2)
    xs = ops.embedding(n2, tok)                       # rows gathered expert by expert
    gu = torch.empty(T * k, 2 * fe, dtype=n2.dtype, device=n2.device)
    for e, a, b in _slabs(bounds):
        if b > a:
            ops.linear(xs[a:b], p[f"wgu{e}"], out=gu[a:b])
    del xs
    st = MoeState(probs, topi, w, order, tok, bounds, gu, None)
    shared = "wgus" in p   # Qwen2-MoE: every token also goes through one shared expert, weighted by a sigmoid gate
    if shared:
        st.gu_s = ops.linear(n2, p["wgus"])
    if not need_out:
        return None, st
    # activation and down projection slab by slab: only the slab's activation is alive unless backward wants all of it
    act = torch.empty(T * k, fe, dtype=n2.dtype, device=n2.device) if keep_act else None
    yr = torch.empty(T * k, H, dtype=n2.dtype, device=n2.device)
    for e, a, b in _slabs(bounds):
        if b > a:
            act_e = ops.swiglu(gu[a:b], cfg.mlp_act)
            ops.linear(act_e, p[f"wd{e}"], out=yr[a:b])
            if keep_act:
                act[a:b] = act_e
    wr = w.reshape(-1)[order]
    y = _combine((yr.float() * wr[:, None]).to(yr.dtype), order, T, k)
    if shared:
        act_s = ops.swiglu(st.gu_s, cfg.mlp_act)
        y += torch.sigmoid((n2 @ p["wsg"].t()).float()) * ops.linear(act_s, p["wds"]).float()
        st.act_s = act_s if keep_act else None
    st.act = act
    return (h1.float() + cfg.residual_multiplier * y).to(h1.dtype), st


def moe_backward(ops, cfg, p: dict, g: dict, st: MoeState, n2: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    """Writes the gradients of the router and of every expert into ``g`` and returns the gradient of
    ``n2`` (the normalised MLP input). ``dout`` is the gradient of the block output.

    Everything between the gathered output gradient and the gathered input gradient runs slab by slab, so the
    intermediates (activation, its gradient, the gate/up gradient) only ever exist for one expert's rows."""
    T, H = n2.shape
    k = cfg.num_experts_per_tok
    rm = cfg.residual_multiplier
    order, tok, bounds = st.order, st.tok, st.bounds
    gr = ops.embedding(dout, tok)                     # output gradient of every routed row, before its weight
    if rm != 1.0:
        gr = gr * rm
    xs = ops.embedding(n2, tok)
    wr = st.w.reshape(-1)[order]
    dwr = torch.zeros(T * k, dtype=torch.float32, device=n2.device)
    dxs = torch.empty(T * k, H, dtype=n2.dtype, device=n2.device)
    for e, a, b in _slabs(bounds):
        if b == a:   # an expert no token chose: its gradients are zero, not what the buffer held before
            g[f"wd{e}"].zero_()
            g[f"wgu{e}"].zero_()
            continue
        gu_e, w_e = st.gu[a:b], wr[a:b, None]
        act = st.act[a:b] if st.act is not None else ops.swiglu(gu_e, cfg.mlp_act)
        # y_row = wd act, weighted by w: d(weight) = dout . y_row = (wd^T dout) . act, so the unweighted data
        # gradient of the down projection gives both the weight's and (scaled) the activation's gradient
        du = ops.linear_dgrad(gr[a:b], p[f"wd{e}"])
        duf, actf = du.float(), act.float()
        dwr[a:b] = (duf * actf).sum(-1)
        ops.linear_wgrad(gr[a:b], (actf * w_e).to(act.dtype), g[f"wd{e}"])
        dgu = ops.swiglu_bwd((duf * w_e).to(du.dtype), gu_e, cfg.mlp_act)
        del du, duf, actf, act
        ops.linear_dgrad(dgu, p[f"wgu{e}"], out=dxs[a:b])
        ops.linear_wgrad(dgu, xs[a:b], g[f"wgu{e}"])
        del dgu
    dn2 = _combine(dxs, order, T, k)
    del xs, dxs, gr
    if "wgus" in p:   # shared expert: y_s = sigmoid(n2 wsg^T) * MLP_s(n2)
        act_s = st.act_s if st.act_s is not None else ops.swiglu(st.gu_s, cfg.mlp_act)
        ys = ops.linear(act_s, p["wds"]).float()          # its output again: the gate's gradient needs it
        sg = torch.sigmoid((n2 @ p["wsg"].t()).float())   # [T, 1]
        df = dout.float() * rm
        dz = ((df * ys).sum(-1, keepdim=True) * sg * (1 - sg)).to(n2.dtype)
        g["wsg"].copy_(dz.t() @ n2)
        dn2 += (dz @ p["wsg"]).float()
        dys = (df * sg).to(n2.dtype)
        del ys, df
        dact_s = ops.linear_dgrad(dys, p["wds"])
        ops.linear_wgrad(dys, act_s, g["wds"])
        dgu_s = ops.swiglu_bwd(dact_s, st.gu_s, cfg.mlp_act)
        del dact_s, act_s, dys
        dn2 += ops.linear_dgrad(dgu_s, p["wgus"]).float()
        ops.linear_wgrad(dgu_s, n2, g["wgus"])
        del dgu_s
    # router: weights -> renormalisation -> top-k selection -> softmax -> logits
    dw = torch.empty(T * k, dtype=torch.float32, device=n2.device)
    dw[order] = dwr
    dw = dw.view(T, k)
    if cfg.norm_topk_prob:
        s = st.probs.gather(1, st.topi).sum(-1, keepdim=True)
        dtop = (dw - (dw * st.w).sum(-1, keepdim=True)) / s
    else:   # Qwen3-MoE may use the chosen probabilities as they are
        dtop = dw
    dprobs = torch.zeros_like(st.probs).scatter_(1, st.topi, dtop)
    dlogits = (st.probs * (dprobs - (dprobs * st.probs).sum(-1, keepdim=True))).to(n2.dtype)
    g["router"].copy_(dlogits.t() @ n2)
    dn2 += (dlogits @ p["router"]).float()
    return dn2.to(n2.dtype)
