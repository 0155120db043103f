"""Decoder block with the norms BEHIND its branches (OLMo-2), forward and hand-written backward.

transformers' ``Olmo2DecoderLayer`` (modeling_olmo2.py): ``x + RMSNorm(Attn(x))`` followed by
``h + RMSNorm(MLP(h))`` with no norm in front of either branch, and inside attention an RMSNorm
over the WHOLE query projection and over the whole key projection (not per head) before the rotary
embedding. The residual therefore cannot ride in a GEMM epilogue (a norm sits between) and the
backward of each branch starts with the backward of its norm, which needs the branch output: a
recompute cannot stop before the down projection as it does for the pre-norm block.

Everything runs on the kernels the pre-norm block uses (GEMM, RMSNorm forward / backward with the
residual gradient folded in, rotary, attention, SwiGLU); the q and k column blocks of the fused qkv
tensor are copied out for their norm and written back.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class PostNormActs:
    """Everything the backward reads."""
    x: torch.Tensor
    q_pre: torch.Tensor          # query projection before its norm, [T, Hq * D]
    k_pre: torch.Tensor          # key projection before its norm, [T, Hkv * D]
    rq: torch.Tensor
    rk: torch.Tensor
    qkv: torch.Tensor            # normalised and rotated q, k and v: what attention saw
    attn: torch.Tensor
    lse: torch.Tensor
    ao: torch.Tensor             # o_proj output before the post-attention norm
    r1: torch.Tensor
    h1: torch.Tensor
    gu: torch.Tensor
    act: Optional[torch.Tensor]  # SwiGLU output (None: rebuilt in backward)
    mo: torch.Tensor             # down projection output before the post-feedforward norm
    r2: torch.Tensor


def block_forward(ops, cfg, p: dict, x: torch.Tensor, batch, inv_freq, keep=False, saved_attn=None, want_attn: bool = False,
                  need_out: bool = True):
    """Same contract as ``decoder.block_forward``; ``need_out`` is ignored (see the module docstring)."""
    plan = p.get("_gather")
    if plan is not None:
        plan.prefetch_small()
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    q, kv = cfg.q_size, cfg.kv_size
    qkv = ops.linear(x, p["wqkv"], p.get("bqkv"), gather=None if plan is None else (plan, 0))
    q_pre, k_pre = qkv[:, :q].contiguous(), qkv[:, q: q + kv].contiguous()
    qn, rq = ops.rmsnorm(q_pre, p["qn"], cfg.rms_norm_eps)
    kn, rk = ops.rmsnorm(k_pre, p["kn"], cfg.rms_norm_eps)
    qkv[:, :q] = qn
    qkv[:, q: q + kv] = kn
    del qn, kn
    if inv_freq is not None:
        ops.rope_(qkv, batch.position_ids, inv_freq, hq, hkv, d, rot_dim=cfg.rotary_dim)
    if saved_attn is not None:
        attn, lse = saved_attn
    else:
        attn, lse = ops.attention(qkv, batch.cu_seqlens, batch.cu_seqlens_host, batch.max_seqlen, hq, hkv, d,
                                  scale=cfg.attention_scale)
    ao = ops.linear(attn, p["wo"], p.get("bo"))
    aon, r1 = ops.rmsnorm(ao, p["ln1"], cfg.rms_norm_eps)
    h1 = x + aon
    del aon
    gu = ops.linear(h1, p["wgu"], p.get("bgu"), gather=None if plan is None else (plan, 1))
    act = ops.swiglu(gu, cfg.mlp_act)
    mo = ops.linear(act, p["wd"], p.get("bd"))
    mon, r2 = ops.rmsnorm(mo, p["ln2"], cfg.rms_norm_eps)
    out = h1 + mon
    acts = None
    if keep:
        acts = PostNormActs(x, q_pre, k_pre, rq, rk, qkv, attn, lse, ao, r1, h1, gu, None if keep == "compact" else act, mo, r2)
    return out, acts, ((attn, lse) if want_attn else None)


def block_backward(ops, cfg, p: dict, g: dict, a: PostNormActs, dout: torch.Tensor, batch, inv_freq, notify=None) -> torch.Tensor:
    """Same contract as ``decoder.block_backward``."""
    notify = notify or (lambda name: None)
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    q, kv = cfg.q_size, cfg.kv_size
    # MLP branch: out = h1 + RMSNorm(mo)
    dmo = ops.rmsnorm_bwd(dout, a.mo, a.r2, p["ln2"], g["ln2"])
    dact = ops.linear_dgrad(dmo, p["wd"])
    act = a.act if a.act is not None else ops.swiglu(a.gu, cfg.mlp_act)
    ops.linear_wgrad(dmo, act, g["wd"], g.get("bd"))
    notify("wd")
    dgu = ops.swiglu_bwd(dact, a.gu, cfg.mlp_act)
    del dact, act, dmo
    dh1 = ops.linear_dgrad(dgu, p["wgu"])
    ops.linear_wgrad(dgu, a.h1, g["wgu"], g.get("bgu"))
    notify("wgu")
    del dgu
    dh1 = dh1 + dout                                  # the residual path around the MLP
    # attention branch: h1 = x + RMSNorm(ao)
    dao = ops.rmsnorm_bwd(dh1, a.ao, a.r1, p["ln1"], g["ln1"])
    dattn = ops.linear_dgrad(dao, p["wo"])
    ops.linear_wgrad(dao, a.attn, g["wo"], g.get("bo"))
    notify("wo")
    del dao
    dqkv = ops.attention_bwd(dattn, a.qkv, a.attn, a.lse, batch.cu_seqlens, batch.cu_seqlens_host, batch.max_seqlen,
                             hq, hkv, d, scale=cfg.attention_scale)
    del dattn
    if inv_freq is not None:
        ops.rope_(dqkv, batch.position_ids, inv_freq, hq, hkv, d, inverse=True, rot_dim=cfg.rotary_dim)
    dq = ops.rmsnorm_bwd(dqkv[:, :q].contiguous(), a.q_pre, a.rq, p["qn"], g["qn"])
    dk = ops.rmsnorm_bwd(dqkv[:, q: q + kv].contiguous(), a.k_pre, a.rk, p["kn"], g["kn"])
    dqkv[:, :q] = dq
    dqkv[:, q: q + kv] = dk
    del dq, dk
    dx = ops.linear_dgrad(dqkv, p["wqkv"])
    ops.linear_wgrad(dqkv, a.x, g["wqkv"], g.get("bqkv"))
    return dx + dh1                                   # the residual path around attention
