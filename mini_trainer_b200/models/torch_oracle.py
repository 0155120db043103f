"""Autograd reference of the decoder, written independently of ``decoder.py``.

Used only by tests: it takes HF-named tensors, runs a plain differentiable forward with stock
PyTorch functions (``scaled_dot_product_attention`` per sample, ``F.cross_entropy`` with
``reduction='none'`` as the reference's unfused path does, none_reduction_losses.py:27-36) and
lets autograd produce the gradients the hand-written backward must match.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .config import ModelConfig


def _rms(x, w, eps, offset=0.0):
    xf = x.float()
    return ((xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)) * (w + offset)


def _norm(cfg, sd, name, x):
    if cfg.norm_type == "layernorm":
        return F.layer_norm(x, (x.shape[-1],), sd[name + ".weight"], sd[name + ".bias"], cfg.rms_norm_eps)
    return _rms(x, sd[name + ".weight"], cfg.rms_norm_eps, cfg.norm_weight_offset)


def _rope(x, pos, inv_freq):
    # x: [T, heads, D]; the first 2 * len(inv_freq) dimensions of every head are turned
    ang = pos.float()[:, None] * inv_freq[None, :]
    cos = torch.cat([ang.cos(), ang.cos()], -1)[:, None, :]
    sin = torch.cat([ang.sin(), ang.sin()], -1)[:, None, :]
    r = 2 * inv_freq.shape[0]
    xr, rest = x[..., :r], x[..., r:]
    rot = torch.cat([-xr[..., r // 2:], xr[..., : r // 2]], -1)
    return torch.cat([(xr.float() * cos + rot.float() * sin).to(x.dtype), rest], -1)


def oracle_per_token_loss(cfg: ModelConfig, sd: dict, input_ids, labels, position_ids, return_logits=False):
    """``sd``: HF-named tensors (requires_grad as needed). Inputs are 1-D packed rows."""
    T = input_ids.shape[0]
    inv_freq = cfg.rope_inv_freq(seq_len=int(position_ids.max()) + 1).to(input_ids.device)
    starts = (position_ids == 0).nonzero().flatten().tolist() + [T]
    x = sd["model.embed_tokens.weight"][input_ids] * cfg.embed_scale(sd["model.embed_tokens.weight"].dtype)
    rm = cfg.residual_multiplier
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    mlp_act = F.silu if cfg.mlp_act == "silu" else (lambda t: F.gelu(t, approximate="tanh"))
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        n = x if cfg.post_norm else _norm(cfg, sd, p + "input_layernorm", x)
        q = F.linear(n, sd[p + "self_attn.q_proj.weight"], sd.get(p + "self_attn.q_proj.bias")).view(T, hq, d)
        k = F.linear(n, sd[p + "self_attn.k_proj.weight"], sd.get(p + "self_attn.k_proj.bias")).view(T, hkv, d)
        v = F.linear(n, sd[p + "self_attn.v_proj.weight"], sd.get(p + "self_attn.v_proj.bias")).view(T, hkv, d)
        if cfg.post_norm:   # over the whole projection, not per head
            q = _rms(q.reshape(T, hq * d), sd[p + "self_attn.q_norm.weight"], cfg.rms_norm_eps).view(T, hq, d)
            k = _rms(k.reshape(T, hkv * d), sd[p + "self_attn.k_norm.weight"], cfg.rms_norm_eps).view(T, hkv, d)
        if cfg.qk_norm:
            q = _rms(q, sd[p + "self_attn.q_norm.weight"], cfg.rms_norm_eps)
            k = _rms(k, sd[p + "self_attn.k_norm.weight"], cfg.rms_norm_eps)
        if cfg.layer_uses_rope(i):
            q, k = _rope(q, position_ids, inv_freq), _rope(k, position_ids, inv_freq)
        outs = []
        for a, b in zip(starts[:-1], starts[1:]):
            o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None],
                                               v[a:b].transpose(0, 1)[None], is_causal=True, enable_gqa=True,
                                               scale=cfg.attention_scale)
            outs.append(o[0].transpose(0, 1).reshape(b - a, hq * d))
        ao = F.linear(torch.cat(outs, 0), sd[p + "self_attn.o_proj.weight"], sd.get(p + "self_attn.o_proj.bias"))
        if cfg.post_norm:
            x = x + _rms(ao, sd[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
            a = F.silu(F.linear(x, sd[p + "mlp.gate_proj.weight"])) * F.linear(x, sd[p + "mlp.up_proj.weight"])
            x = x + _rms(F.linear(a, sd[p + "mlp.down_proj.weight"]), sd[p + "post_feedforward_layernorm.weight"], cfg.rms_norm_eps)
            continue
        x = x + rm * ao
        n = _norm(cfg, sd, p + "post_attention_layernorm", x)
        if cfg.is_moe:   # dense restatement: every expert on every token, masked by the routing weights
            fe = cfg.expert_intermediate_size
            if cfg.model_type == "mixtral":
                m = p + "block_sparse_moe."
                router = sd[m + "gate.weight"]
                experts = [(sd[m + f"experts.{e}.w1.weight"], sd[m + f"experts.{e}.w3.weight"], sd[m + f"experts.{e}.w2.weight"])
                           for e in range(cfg.num_local_experts)]
            elif cfg.model_type == "granitemoe":   # stacked [E, 2F, H] and [E, H, F]
                m = p + "block_sparse_moe."
                router = sd[m + "router.layer.weight"]
                experts = [(sd[m + "input_linear.weight"][e, :fe], sd[m + "input_linear.weight"][e, fe:],
                            sd[m + "output_linear.weight"][e]) for e in range(cfg.num_local_experts)]
            else:
                m = p + "mlp."
                router = sd[m + "gate.weight"]
                experts = [(sd[m + f"experts.{e}.gate_proj.weight"], sd[m + f"experts.{e}.up_proj.weight"],
                            sd[m + f"experts.{e}.down_proj.weight"]) for e in range(cfg.num_local_experts)]
            probs = F.softmax(F.linear(n, router).float(), -1)
            topv, topi = probs.topk(cfg.num_experts_per_tok, -1)
            gatew = torch.zeros_like(probs).scatter(1, topi, topv / topv.sum(-1, keepdim=True) if cfg.norm_topk_prob else topv)
            y = 0
            for e, (wg, wu, wdn) in enumerate(experts):
                y = y + gatew[:, e: e + 1].to(n.dtype) * F.linear(F.silu(F.linear(n, wg)) * F.linear(n, wu), wdn)
            if cfg.shared_expert_intermediate_size:
                se = m + "shared_expert."
                ys = F.linear(F.silu(F.linear(n, sd[se + "gate_proj.weight"])) * F.linear(n, sd[se + "up_proj.weight"]),
                              sd[se + "down_proj.weight"])
                y = y + torch.sigmoid(F.linear(n, sd[m + "shared_expert_gate.weight"])) * ys
            x = x + rm * y
            continue
        if not cfg.mlp_gated:
            act = mlp_act(F.linear(n, sd[p + "mlp.c_fc.weight"], sd.get(p + "mlp.c_fc.bias")))
            x = x + rm * F.linear(act, sd[p + "mlp.c_proj.weight"], sd.get(p + "mlp.c_proj.bias"))
            continue
        act = mlp_act(F.linear(n, sd[p + "mlp.gate_proj.weight"], sd.get(p + "mlp.gate_proj.bias"))) \
            * F.linear(n, sd[p + "mlp.up_proj.weight"], sd.get(p + "mlp.up_proj.bias"))
        x = x + rm * F.linear(act, sd[p + "mlp.down_proj.weight"], sd.get(p + "mlp.down_proj.bias"))
    n = _norm(cfg, sd, "model.norm", x)
    lm = sd["model.embed_tokens.weight"] if cfg.tie_word_embeddings else sd["lm_head.weight"]
    logits = F.linear(n, lm).float() / cfg.logits_scaling
    if return_logits:
        return logits
    targets = torch.full_like(labels, -100)
    targets[:-1] = labels[1:]
    return F.cross_entropy(logits, targets, ignore_index=-100, reduction="none")
