"""Decoder math with hand-written forward AND backward passes.

There is no autograd graph on the training path: each decoder block is a pair of functions over
explicit tensors, which is what lets the sharding engine decide exactly when parameters are
gathered, what is kept between forward and backward, and when each gradient buffer is complete
and can be reduced. The same functions run on the PyTorch reference ops (CPU, tests) and on the
sm_100a kernels; ``ops`` is the backend object.

Architecture (HF Llama/Qwen2, modeling_llama.py:303-332): ``x + Attn(RMSNorm(x))`` followed by
``h + MLP(RMSNorm(h))`` with rotary GQA attention and a SwiGLU MLP; every projection may carry a bias
(``attention_bias``, ``mlp_bias``), added in the GEMM epilogue, its gradient a column sum of the
output gradient. Activation checkpointing is per block as in the reference
(setup_model_for_training.py:28-29): forward keeps only the block input; backward first re-runs
the block forward (``block_forward(..., keep=True)``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from .config import ModelConfig
from .moe import moe_backward, moe_forward
from . import postnorm


@dataclass
class PackedBatch:
    """One padding-free minibatch on the compute device."""
    input_ids: torch.Tensor      # [T] int64
    targets: torch.Tensor        # [T] int64, labels shifted left by one, -100 = no loss
    position_ids: torch.Tensor   # [T] int64/int32, restarts at 0 per sample
    cu_seqlens: torch.Tensor     # [n+1] int32 (device)
    cu_seqlens_host: list        # same values as Python ints
    max_seqlen: int
    # Positions whose target is not -100 and their targets, found on the host where the labels are
    # known (None when every position counts): the LM head only runs on these rows.
    loss_rows: Optional[torch.Tensor] = None     # [T'] int64
    loss_targets: Optional[torch.Tensor] = None  # [T'] int64
    h2d_bytes: int = 0           # bytes of the host tensors copied to the device for this minibatch

    @property
    def num_tokens(self) -> int:
        return int(self.input_ids.shape[0])


def shift_labels(labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Target of position t is label t+1 over the whole packed row (HF causal-LM convention)."""
    out = torch.full_like(labels, ignore_index)
    out[..., :-1] = labels[..., 1:]
    return out


def make_packed_batch(mb: dict, device, non_blocking: bool = True) -> PackedBatch:
    """Moves a collated minibatch (see ``data.sampler.mb_collate_fn``) to ``device``."""
    ids = mb["input_ids"].reshape(-1)
    targets = shift_labels(mb["labels"].reshape(-1))
    pos = mb["position_ids"].reshape(-1)
    if "cu_seqlens" in mb:
        cu = mb["cu_seqlens"].to(torch.int32)
    else:  # recover sample boundaries from restarting position ids (host side, once)
        starts = (pos == 0).nonzero().flatten().to(torch.int32)
        cu = torch.cat([starts, torch.tensor([pos.numel()], dtype=torch.int32)])
    cu_host = cu.tolist()
    max_seqlen = int(mb.get("max_seqlen", max(b - a for a, b in zip(cu_host[:-1], cu_host[1:]))))
    moved = [0]

    def mv(t):
        moved[0] += t.numel() * t.element_size()
        return t.to(device, non_blocking=non_blocking)

    rows = sel = None
    counted = (targets != -100).nonzero().flatten()
    # MTB200_HEAD_ALL_ROWS=1 runs the head on every row, as the reference does (for A/B timing)
    if counted.numel() < targets.numel() and os.environ.get("MTB200_HEAD_ALL_ROWS", "0") != "1":
        rows, sel = mv(counted), mv(targets[counted])
    batch = PackedBatch(mv(ids), mv(targets), mv(pos.to(torch.int32)), mv(cu), cu_host, max_seqlen, rows, sel)
    batch.h2d_bytes = moved[0]
    return batch


def _nw(cfg: ModelConfig, w: torch.Tensor) -> torch.Tensor:
    """Weight a norm multiplies by: the stored tensor, or ``offset + weight`` for Gemma (whose checkpoints, master
    weights and exports all hold ``weight``; its gradient is the same as that of the sum)."""
    return w if cfg.norm_weight_offset == 0.0 else (w.float() + cfg.norm_weight_offset).to(w.dtype)


def _norm(ops, cfg: ModelConfig, x: torch.Tensor, p: dict, w: str, b: str):
    """The model's normalisation of ``x`` with the weight (and bias) named ``w`` (``b``) in ``p``: ``(y, stats)``."""
    if cfg.norm_type == "layernorm":
        return ops.layernorm(x, p[w], p[b], cfg.rms_norm_eps)
    return ops.rmsnorm(x, _nw(cfg, p[w]), cfg.rms_norm_eps)


def _norm_bwd(ops, cfg: ModelConfig, dy, x, stats, p: dict, g: dict, w: str, b: str, add_to=None):
    if cfg.norm_type == "layernorm":
        return ops.layernorm_bwd(dy, x, stats, p[w], g[w], g[b], add_to=add_to)
    return ops.rmsnorm_bwd(dy, x, stats, _nw(cfg, p[w]), g[w], add_to=add_to)


@dataclass
class BlockActs:
    """Everything the block backward reads, produced by ``block_forward(keep=True)``."""
    x: torch.Tensor
    n1: torch.Tensor
    rstd1: torch.Tensor
    qkv: torch.Tensor
    attn: torch.Tensor
    lse: torch.Tensor
    h1: torch.Tensor
    n2: torch.Tensor
    rstd2: torch.Tensor
    gu: torch.Tensor
    act: torch.Tensor
    qk_pre: Optional[torch.Tensor] = None    # q|k heads before the per-head norm (Qwen3), [T, (Hq + Hkv) * D]
    rstd_qk: Optional[torch.Tensor] = None   # reciprocal RMS per (token, head)
    moe: Optional[object] = None   # routing and expert pre-activations of a mixture-of-experts block (``moe.MoeState``)


def block_forward(ops, cfg: ModelConfig, p: dict, x: torch.Tensor, batch: PackedBatch, inv_freq, keep: bool = False,
                  saved_attn=None, want_attn: bool = False, need_out: bool = True):
    """Returns ``(out, acts, attn_state)``.

    ``need_out=False`` (recompute inside backward) stops before the down projection: backward reads
    the block's intermediates, never its output, so that GEMM (27 % of the block's forward FLOPs for
    Llama-3.1-8B) would be wasted work.

    ``acts`` is a ``BlockActs`` when ``keep`` (everything backward reads), else ``None``.
    ``saved_attn = (attn, lse)`` from an earlier forward skips the attention kernel (used by the
    recompute of blocks whose attention output was kept); ``want_attn`` returns that pair.
    """
    if cfg.post_norm:
        return postnorm.block_forward(ops, cfg, p, x, batch, inv_freq, keep, saved_attn, want_attn, need_out)
    plan = p.get("_gather")   # all-gather of this block's parameters fused into its first GEMMs
    if plan is not None:
        plan.prefetch_small()
    n1, rstd1 = _norm(ops, cfg, x, p, "ln1", "bln1")
    qkv = ops.linear(n1, p["wqkv"], p.get("bqkv"), gather=None if plan is None else (plan, 0))
    qk_pre = rstd_qk = None
    if cfg.qk_norm:   # the backward of the norm needs its input; the qkv tensor itself goes on normalised and rotated
        qk_pre = qkv[:, : cfg.q_size + cfg.kv_size].clone()
        rstd_qk = ops.head_rmsnorm_(qkv, p["qn"], p["kn"], cfg.rms_norm_eps, cfg.num_attention_heads,
                                    cfg.num_key_value_heads, cfg.head_dim)
    if inv_freq is not None:   # None: a layer without positional rotation (SmolLM3's NoPE layers)
        ops.rope_(qkv, batch.position_ids, inv_freq, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                  rot_dim=cfg.rotary_dim)
    rm = cfg.residual_multiplier   # Granite scales every branch output before the residual add (1.0 elsewhere)
    # the GEMM epilogue computes alpha * product + bias + residual; the models scale (product + bias)
    bo, bd = p.get("bo"), p.get("bd")
    if rm != 1.0:
        bo, bd = (None if bo is None else bo * rm), (None if bd is None else bd * rm)
    if saved_attn is not None:
        attn, lse = saved_attn
    else:
        attn, lse = ops.attention(qkv, batch.cu_seqlens, batch.cu_seqlens_host, batch.max_seqlen,
                                  cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, scale=cfg.attention_scale)
    h1 = ops.linear(attn, p["wo"], bo, x, alpha=rm)
    n2, rstd2 = _norm(ops, cfg, h1, p, "ln2", "bln2")
    if cfg.is_moe:
        out, st = moe_forward(ops, cfg, p, n2, h1, need_out, keep_act=keep is True)
        acts = None
        if keep == "compact":
            acts = BlockActs(x, None, rstd1, qkv, attn, lse, h1, None, rstd2, None, None, qk_pre, rstd_qk, st)
        elif keep:
            acts = BlockActs(x, n1, rstd1, qkv, attn, lse, h1, n2, rstd2, None, None, qk_pre, rstd_qk, st)
        return out, acts, ((attn, lse) if want_attn else None)
    gu = ops.linear(n2, p["wgu"], p.get("bgu"), gather=None if plan is None else (plan, 1))
    # a recompute that stops before the down projection does not need the SwiGLU output: backward rebuilds it
    # inside the SwiGLU-gradient kernel
    act = (ops.swiglu(gu, cfg.mlp_act) if cfg.mlp_gated else ops.gelu(gu)) if need_out else None
    out = ops.linear(act, p["wd"], bd, h1, alpha=rm) if need_out else None
    acts = None
    if keep == "compact":   # kept from forward to backward: drop what one elementwise kernel can rebuild
        acts = BlockActs(x, None, rstd1, qkv, attn, lse, h1, None, rstd2, gu, None, qk_pre, rstd_qk)
    elif keep:
        acts = BlockActs(x, n1, rstd1, qkv, attn, lse, h1, n2, rstd2, gu, act, qk_pre, rstd_qk)
    return out, acts, ((attn, lse) if want_attn else None)


def block_backward(ops, cfg: ModelConfig, p: dict, g: dict, acts: BlockActs, dout: torch.Tensor,
                   batch: PackedBatch, inv_freq, notify=None) -> torch.Tensor:
    """Writes every parameter gradient of the block into ``g`` (views of the block's flat
    gradient buffer, same names as ``p``) and returns the gradient of the block input.

    ``notify(name)`` is called right after the weight gradient of ``wd``, ``wgu`` and ``wo`` has been
    queued: everything laid out from that tensor to the end of the buffer (to the previous
    notification) is then complete, and the engine starts reducing that region while the rest of
    the block's backward still runs."""
    if cfg.post_norm:
        return postnorm.block_backward(ops, cfg, p, g, acts, dout, batch, inv_freq, notify)
    a = acts
    notify = notify or (lambda name: None)
    rm = cfg.residual_multiplier
    # activations kept in compact form: the normalised inputs and the SwiGLU output are rebuilt by
    # bandwidth-bound kernels (about 1 ms per block) instead of being held for the whole step
    # MLP
    if cfg.is_moe:
        n2 = a.n2 if a.n2 is not None else _norm(ops, cfg, a.h1, p, "ln2", "bln2")[0]
        dn2 = moe_backward(ops, cfg, p, g, a.moe, n2, dout)
        del n2
        return _attention_backward(ops, cfg, p, g, a, dn2, dout, batch, inv_freq, notify, rm)
    dact = ops.linear_dgrad(dout, p["wd"], alpha=rm)
    if a.act is not None:
        ops.linear_wgrad(dout, a.act, g["wd"], g.get("bd"), alpha=rm)
        dgu = ops.swiglu_bwd(dact, a.gu, cfg.mlp_act) if cfg.mlp_gated else ops.gelu_bwd(dact, a.gu)
    elif not cfg.mlp_gated:
        act, dgu = ops.gelu(a.gu), ops.gelu_bwd(dact, a.gu)
        ops.linear_wgrad(dout, act, g["wd"], g.get("bd"), alpha=rm)
        del act
    else:   # one pass over gate/up gives its gradient and the SwiGLU output (written over dact)
        dgu, act = ops.swiglu_bwd_act(dact, a.gu, cfg.mlp_act)
        ops.linear_wgrad(dout, act, g["wd"], g.get("bd"), alpha=rm)
        del act
    if rm != 1.0 and "bd" in g:   # the bias sits inside the scaled branch; the column sum is not scaled by alpha
        g["bd"].mul_(rm)
    notify("wd")
    del dact
    dn2 = ops.linear_dgrad(dgu, p["wgu"])
    n2 = a.n2 if a.n2 is not None else _norm(ops, cfg, a.h1, p, "ln2", "bln2")[0]
    ops.linear_wgrad(dgu, n2, g["wgu"], g.get("bgu"))
    notify("wgu")
    del dgu, n2
    return _attention_backward(ops, cfg, p, g, a, dn2, dout, batch, inv_freq, notify, rm)


def _attention_backward(ops, cfg: ModelConfig, p: dict, g: dict, a: BlockActs, dn2: torch.Tensor, dout: torch.Tensor,
                        batch: PackedBatch, inv_freq, notify, rm: float) -> torch.Tensor:
    """The part of the block backward in front of the MLP: post-attention norm, o_proj, attention, rotary,
    q/k/v projection, input norm. ``dn2`` is the gradient of the normalised MLP input."""
    dh1 = _norm_bwd(ops, cfg, dn2, a.h1, a.rstd2, p, g, "ln2", "bln2", add_to=dout)
    del dn2
    # attention
    dattn = ops.linear_dgrad(dh1, p["wo"], alpha=rm)
    ops.linear_wgrad(dh1, a.attn, g["wo"], g.get("bo"), alpha=rm)
    if rm != 1.0 and "bo" in g:
        g["bo"].mul_(rm)
    notify("wo")     # ln2's gradient was written by the rmsnorm backward above, bgu's with wgu's
    dqkv = ops.attention_bwd(dattn, a.qkv, a.attn, a.lse, batch.cu_seqlens, batch.cu_seqlens_host,
                             batch.max_seqlen, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                             scale=cfg.attention_scale)
    del dattn
    if inv_freq is not None:
        ops.rope_(dqkv, batch.position_ids, inv_freq, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                  inverse=True, rot_dim=cfg.rotary_dim)
    if cfg.qk_norm:
        ops.head_rmsnorm_bwd_(dqkv, a.qk_pre, a.rstd_qk, p["qn"], p["kn"], g["qn"], g["kn"], cfg.num_attention_heads,
                              cfg.num_key_value_heads, cfg.head_dim)
    dn1 = ops.linear_dgrad(dqkv, p["wqkv"])
    n1 = a.n1 if a.n1 is not None else _norm(ops, cfg, a.x, p, "ln1", "bln1")[0]
    ops.linear_wgrad(dqkv, n1, g["wqkv"], g.get("bqkv"))
    del dqkv, n1
    dx = _norm_bwd(ops, cfg, dn1, a.x, a.rstd1, p, g, "ln1", "bln1", add_to=dh1)
    return dx


def head_forward_backward(ops, cfg: ModelConfig, head_p: dict, head_g: dict, lm_w: torch.Tensor, lm_g: torch.Tensor,
                          accumulate_lm_grad: bool, x: torch.Tensor, batch: PackedBatch, grad_scale: float):
    """Final norm + fused linear/CE. Returns ``(per_token_loss [T] fp32, dx)``.

    The CE op produces its gradients in the same pass, scaled by ``grad_scale`` (the reciprocal
    of the global batch's loss-token count), so backward starts here without a separate call.
    """
    rows = batch.loss_rows
    ls = 1.0 / cfg.logits_scaling   # Granite divides the logits by a constant
    if rows is None:
        n, rstd = _norm(ops, cfg, x, head_p, "norm", "bnorm")
        loss, dn = ops.linear_ce(n, lm_w, batch.targets, grad_scale, lm_g, accumulate_dw=accumulate_lm_grad, logit_scale=ls)
        dx = _norm_bwd(ops, cfg, dn, x, rstd, head_p, head_g, "norm", "bnorm")
        return loss, dx
    # Masked positions (prompt tokens, the last token of every sample) have zero loss and zero
    # gradient, so the final norm, the three vocabulary-sized GEMMs and the CE kernel only see the
    # rows that count; their input gradient is scattered back into a zero tensor. Exact, not an
    # approximation; the reference's fused linear-CE computes logits for every row.
    loss = torch.zeros(x.shape[0], dtype=torch.float32, device=x.device)
    dx = torch.zeros_like(x)
    if rows.numel() == 0:   # nothing to learn from in this minibatch (e.g. only the idle-rank dummy sample);
        return loss, dx     # the gradient buffers of the head were zeroed by the caller
    xs = ops.embedding(x, rows)   # row gather
    n, rstd = _norm(ops, cfg, xs, head_p, "norm", "bnorm")
    loss_s, dn = ops.linear_ce(n, lm_w, batch.loss_targets, grad_scale, lm_g, accumulate_dw=accumulate_lm_grad,
                               logit_scale=ls)
    dxs = _norm_bwd(ops, cfg, dn, xs, rstd, head_p, head_g, "norm", "bnorm")
    loss.index_copy_(0, rows, loss_s)
    dx.index_copy_(0, rows, dxs)
    return loss, dx


@torch.no_grad()
def forward_logits(ops, cfg: ModelConfig, embed_w, blocks: list, norm_w, lm_w, batch: PackedBatch, norm_b=None) -> torch.Tensor:
    """Plain inference forward returning ``[T, V]`` logits (tests, checkpoint round-trips)."""
    inv_freq = cfg.rope_inv_freq(seq_len=batch.max_seqlen).to(embed_w.device)
    x = ops.embedding(embed_w, batch.input_ids)
    if cfg.embedding_multiplier != 1.0:
        x = x * cfg.embed_scale(x.dtype)
    for i, p in enumerate(blocks):
        x, _, _ = block_forward(ops, cfg, p, x, batch, inv_freq if cfg.layer_uses_rope(i) else None)
    n, _ = _norm(ops, cfg, x, {"norm": norm_w, "bnorm": norm_b}, "norm", "bnorm")
    return (n.float() @ lm_w.float().t()) / cfg.logits_scaling
