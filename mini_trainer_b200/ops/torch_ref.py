"""Plain-PyTorch implementation of every op the decoder needs, forward and backward.

This backend is the numerical oracle for the CUDA kernels and the execution path on machines
without a GPU (CPU/gloo tests). Every op works on token-major 2-D tensors ``[T, features]`` of
one padding-free packed row; sequence boundaries come from ``cu_seqlens``.

Math is done in fp32 internally and cast back to the tensor dtype, mirroring what the
hand-written kernels do (fp32 accumulation, storage-dtype outputs).

Operation semantics follow the modules the reference runs (HF Llama/Qwen2 + Liger):
RMSNorm with fp32 variance (modeling_llama.py:62-67), rotate-half RoPE indexed by position ids
that restart per sample (modeling_llama.py:146-168), causal varlen GQA attention scaled by
``head_dim**-0.5``, SwiGLU ``silu(gate) * up``, and a chunked linear + cross-entropy that never
holds ``[T, V]`` logits and returns per-token losses (none_reduction_losses.py:5-25).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


class TorchOps:
    name = "torch"

    def __init__(self, ce_chunk: int = 2048):
        self.ce_chunk = ce_chunk

    # -- embedding --------------------------------------------------------------------
    def embedding(self, weight, ids):
        return weight.index_select(0, ids)

    def embedding_bwd(self, dweight, ids, dx):
        """Scatter-adds ``dx`` rows into ``dweight`` (which already holds other contributions)."""
        dweight.index_add_(0, ids, dx.to(dweight.dtype))

    # -- rmsnorm ----------------------------------------------------------------------
    def rmsnorm(self, x, w, eps):
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        y = (xf * rstd).to(x.dtype) * w
        return y, rstd.squeeze(-1)

    def rmsnorm_bwd(self, dy, x, rstd, w, dw_out, add_to=None):
        """Returns ``dx`` (+ ``add_to`` when given, the residual-stream gradient); writes ``dw_out``."""
        xf, dyf = x.float(), dy.float()
        r = rstd.unsqueeze(-1)
        xhat = xf * r
        dw_out.copy_((dyf * xhat.to(x.dtype).float()).sum(0).to(dw_out.dtype))
        g = dyf * w.float()
        dx = r * (g - xhat * (g * xhat).mean(-1, keepdim=True))
        if add_to is not None:
            dx = dx + add_to.float()
        return dx.to(x.dtype)

    # -- layernorm (Starcoder2) -----------------------------------------------------------
    def layernorm(self, x, w, b, eps):
        xf = x.float()
        mean = xf.mean(-1, keepdim=True)
        rstd = torch.rsqrt((xf - mean).pow(2).mean(-1, keepdim=True) + eps)
        y = ((xf - mean) * rstd * w.float() + b.float()).to(x.dtype)
        return y, (mean.squeeze(-1), rstd.squeeze(-1))

    def layernorm_bwd(self, dy, x, stats, w, dw_out, db_out, add_to=None):
        xf, dyf = x.float(), dy.float()
        mean, r = stats[0].unsqueeze(-1), stats[1].unsqueeze(-1)
        xhat = (xf - mean) * r
        dw_out.copy_((dyf * xhat).sum(0).to(dw_out.dtype))
        db_out.copy_(dyf.sum(0).to(db_out.dtype))
        g = dyf * w.float()
        dx = r * (g - g.mean(-1, keepdim=True) - xhat * (g * xhat).mean(-1, keepdim=True))
        if add_to is not None:
            dx = dx + add_to.float()
        return dx.to(x.dtype)

    # -- linear -----------------------------------------------------------------------
    def linear(self, x, w, bias=None, residual=None, gather=None, alpha=1.0, out=None):
        y = x @ w.t()
        if alpha != 1.0:
            y = y * alpha
        if bias is not None:
            y = y + bias
        if residual is not None:
            y = y + residual
        return y if out is None else out.copy_(y)

    def linear_dgrad(self, dy, w, alpha=1.0, out=None):
        y = dy @ w if alpha == 1.0 else (dy @ w) * alpha
        return y if out is None else out.copy_(y)

    def linear_wgrad(self, dy, x, dw_out, dbias_out=None, alpha=1.0):
        dw_out.copy_(((dy.float().t() @ x.float()) * alpha).to(dw_out.dtype))
        if dbias_out is not None:
            dbias_out.copy_(dy.float().sum(0).to(dbias_out.dtype))

    # -- rope (in place on the q and k column blocks of the fused qkv tensor) ------------
    def rope_(self, qkv, position_ids, inv_freq, n_q_heads, n_kv_heads, head_dim, inverse=False, rot_dim=None):
        """``rot_dim``: leading dimensions of each head that are turned (default: the whole head)."""
        T = qkv.shape[0]
        rot = head_dim if rot_dim is None else rot_dim
        ang = position_ids.to(torch.float32).unsqueeze(-1) * inv_freq.to(qkv.device).unsqueeze(0)  # [T, rot/2]
        cos, sin = ang.cos(), ang.sin()
        if inverse:
            sin = -sin
        nh = n_q_heads + n_kv_heads
        v = qkv[:, : nh * head_dim].reshape(T, nh, head_dim)
        x1, x2 = v[..., : rot // 2].float(), v[..., rot // 2: rot].float()
        c, s = cos.unsqueeze(1), sin.unsqueeze(1)
        o1 = x1 * c - x2 * s
        o2 = x2 * c + x1 * s
        out = torch.cat([o1.to(qkv.dtype), o2.to(qkv.dtype), v[..., rot:]], -1)
        qkv[:, : nh * head_dim] = out.reshape(T, nh * head_dim)
        return qkv

    # -- per-head RMSNorm of q and k (Qwen3 q_norm / k_norm) --------------------------------
    def head_rmsnorm_(self, qkv, wq, wk, eps, n_q_heads, n_kv_heads, head_dim):
        T, nh = qkv.shape[0], n_q_heads + n_kv_heads
        v = qkv[:, : nh * head_dim].reshape(T, nh, head_dim).float()
        rstd = torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
        w = torch.cat([wq.expand(n_q_heads, head_dim), wk.expand(n_kv_heads, head_dim)], 0)
        y = (v * rstd).to(qkv.dtype) * w
        qkv[:, : nh * head_dim] = y.reshape(T, nh * head_dim).to(qkv.dtype)
        return rstd.reshape(-1)

    def head_rmsnorm_bwd_(self, dqkv, pre, rstd, wq, wk, dwq_out, dwk_out, n_q_heads, n_kv_heads, head_dim):
        T, nh = dqkv.shape[0], n_q_heads + n_kv_heads
        dy = dqkv[:, : nh * head_dim].reshape(T, nh, head_dim).float()
        r = rstd.reshape(T, nh, 1)
        xhat = pre.reshape(T, nh, head_dim).float() * r
        c = dy * xhat.to(dqkv.dtype).float()
        dwq_out.copy_(c[:, :n_q_heads].sum((0, 1)).to(dwq_out.dtype))
        dwk_out.copy_(c[:, n_q_heads:].sum((0, 1)).to(dwk_out.dtype))
        w = torch.cat([wq.expand(n_q_heads, head_dim), wk.expand(n_kv_heads, head_dim)], 0).float()
        g = dy * w
        dx = r * (g - xhat * (g * xhat).mean(-1, keepdim=True))
        dqkv[:, : nh * head_dim] = dx.reshape(T, nh * head_dim).to(dqkv.dtype)
        return dqkv

    # -- attention --------------------------------------------------------------------
    @staticmethod
    def _split(qkv, hq, hkv, d):
        T = qkv.shape[0]
        q = qkv[:, : hq * d].reshape(T, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].reshape(T, hkv, d)
        v = qkv[:, (hq + hkv) * d:].reshape(T, hkv, d)
        return q, k, v

    def attention(self, qkv, cu_seqlens, cu_host, max_seqlen, hq, hkv, d, scale=None):
        """Causal attention inside each ``cu_seqlens`` segment. Returns ``out [T, hq*d]``, ``lse [hq, T]``."""
        T = qkv.shape[0]
        q, k, v = self._split(qkv, hq, hkv, d)
        g = hq // hkv
        scale = d ** -0.5 if scale is None else float(scale)
        out = torch.empty(T, hq, d, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(hq, T, dtype=torch.float32, device=qkv.device)
        bounds = list(cu_host) if cu_host is not None else cu_seqlens.tolist()
        for a, b in zip(bounds[:-1], bounds[1:]):
            n = b - a
            qs = q[a:b].float().transpose(0, 1)                                 # [hq, n, d]
            ks = k[a:b].float().transpose(0, 1).repeat_interleave(g, 0)
            vs = v[a:b].float().transpose(0, 1).repeat_interleave(g, 0)
            s = (qs @ ks.transpose(1, 2)) * scale
            mask = torch.ones(n, n, dtype=torch.bool, device=qkv.device).tril_()
            s = s.masked_fill(~mask, float("-inf"))
            l = torch.logsumexp(s, -1)
            p = torch.exp(s - l.unsqueeze(-1))
            out[a:b] = (p @ vs).transpose(0, 1).to(qkv.dtype)
            lse[:, a:b] = l
        return out.reshape(T, hq * d), lse

    def attention_bwd(self, dout, qkv, out, lse, cu_seqlens, cu_host, max_seqlen, hq, hkv, d, scale=None):
        T = qkv.shape[0]
        q, k, v = self._split(qkv, hq, hkv, d)
        g = hq // hkv
        scale = d ** -0.5 if scale is None else float(scale)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = self._split(dqkv, hq, hkv, d)
        do = dout.reshape(T, hq, d)
        o = out.reshape(T, hq, d)
        bounds = list(cu_host) if cu_host is not None else cu_seqlens.tolist()
        for a, b in zip(bounds[:-1], bounds[1:]):
            n = b - a
            qs = q[a:b].float().transpose(0, 1)
            ks = k[a:b].float().transpose(0, 1).repeat_interleave(g, 0)
            vs = v[a:b].float().transpose(0, 1).repeat_interleave(g, 0)
            dos = do[a:b].float().transpose(0, 1)
            os_ = o[a:b].float().transpose(0, 1)
            s = (qs @ ks.transpose(1, 2)) * scale
            mask = torch.ones(n, n, dtype=torch.bool, device=qkv.device).tril_()
            p = torch.exp(s - lse[:, a:b].unsqueeze(-1)).masked_fill(~mask, 0.0)
            dvs = p.transpose(1, 2) @ dos                                       # [hq, n, d]
            dp = dos @ vs.transpose(1, 2)
            delta = (dos * os_).sum(-1, keepdim=True)
            ds = p * (dp - delta) * scale
            dqs = ds @ ks
            dks = ds.transpose(1, 2) @ qs
            dq[a:b] = dqs.transpose(0, 1).to(qkv.dtype)
            dk[a:b] = dks.reshape(hkv, g, n, d).sum(1).transpose(0, 1).to(qkv.dtype)
            dv[a:b] = dvs.reshape(hkv, g, n, d).sum(1).transpose(0, 1).to(qkv.dtype)
        return dqkv

    # -- swiglu -----------------------------------------------------------------------
    def swiglu(self, gate_up, act="silu"):
        f = gate_up.shape[1] // 2
        g, u = gate_up[:, :f].float(), gate_up[:, f:].float()
        a = F.silu(g) if act == "silu" else F.gelu(g, approximate="tanh")
        return (a * u).to(gate_up.dtype)

    def swiglu_bwd(self, dact, gate_up, act="silu"):
        f = gate_up.shape[1] // 2
        g, u = gate_up[:, :f].float(), gate_up[:, f:].float()
        da = dact.float()
        if act == "silu":
            sig = torch.sigmoid(g)
            dg = da * u * sig * (1 + g * (1 - sig))
            du = da * g * sig
        else:
            dg = da * u * self._gelu_tanh_grad(g)
            du = da * F.gelu(g, approximate="tanh")
        return torch.cat([dg, du], 1).to(gate_up.dtype)

    def swiglu_bwd_act(self, dact, gate_up, act="silu"):
        """``(dgate_up, act)``: the gradient and the forward output in one call."""
        return self.swiglu_bwd(dact, gate_up, act), self.swiglu(gate_up, act)

    @staticmethod
    def _gelu_tanh_grad(x):
        k = 0.7978845608028654
        th = torch.tanh(k * (x + 0.044715 * x ** 3))
        return 0.5 * (1 + th) + 0.5 * x * (1 - th * th) * k * (1 + 3 * 0.044715 * x * x)

    def gelu(self, x):
        return F.gelu(x.float(), approximate="tanh").to(x.dtype)

    def gelu_bwd(self, dy, x):
        return (dy.float() * self._gelu_tanh_grad(x.float())).to(x.dtype)

    # -- fused linear + cross-entropy ---------------------------------------------------
    def linear_ce(self, x, w, targets, grad_scale, dw_out, accumulate_dw=False, ignore_index=-100, logit_scale=1.0):
        """Per-token CE of ``logit_scale * x @ w.T`` against ``targets`` without materialising all logits.

        Returns ``(loss [T] fp32, dx [T, H])``; ``dw_out`` receives (or accumulates) ``dW``.
        Gradients are those of ``grad_scale * sum(loss)``, the uniform upstream scale the
        training loop applies (reference train.py:98-102).
        """
        T = x.shape[0]
        loss = torch.zeros(T, dtype=torch.float32, device=x.device)
        dx = torch.empty_like(x)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=x.device)
        wf = w.float()
        for a in range(0, T, self.ce_chunk):
            b = min(T, a + self.ce_chunk)
            xc, tc = x[a:b].float(), targets[a:b]
            logits = (xc @ wf.t()) * logit_scale
            valid = tc != ignore_index
            safe = tc.clamp_min(0)
            lse = torch.logsumexp(logits, -1)
            picked = logits.gather(1, safe.unsqueeze(1)).squeeze(1)
            loss[a:b] = torch.where(valid, lse - picked, torch.zeros_like(lse))
            dl = torch.softmax(logits, -1)
            dl[torch.arange(b - a, device=x.device), safe] -= 1.0
            dl = dl * (valid.float() * grad_scale).unsqueeze(1)
            dl = dl.to(x.dtype).float() * logit_scale  # the kernels round dlogits to the storage dtype
            dx[a:b] = (dl @ wf).to(x.dtype)
            dw += dl.t() @ xc
        if accumulate_dw:
            dw_out.add_(dw.to(dw_out.dtype))
        else:
            dw_out.copy_(dw.to(dw_out.dtype))
        return loss, dx

    # -- optimizer --------------------------------------------------------------------
    def sumsq(self, g):
        return g.float().pow(2).sum()

    def adamw_step(self, master, m, v, grad, param_out, lr, beta1, beta2, eps, weight_decay, step, grad_coef):
        """AdamW on fp32 master weights with the clip coefficient folded into the gradient.

        ``grad_coef`` is a 0-dim tensor (kept on device so no host sync is needed) or a float.
        ``param_out`` (the low-precision working shard) is refreshed from the master copy.
        """
        g = grad.float() * grad_coef
        if weight_decay:
            master.mul_(1.0 - lr * weight_decay)
        mf = m.float().mul_(beta1).add_(g, alpha=1.0 - beta1)
        vf = v.float().mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
        m.copy_(mf.to(m.dtype))
        v.copy_(vf.to(v.dtype))
        bc1 = 1.0 - beta1 ** step
        bc2 = 1.0 - beta2 ** step
        denom = (vf.sqrt() / (bc2 ** 0.5)).add_(eps)
        master.addcdiv_(mf, denom, value=-lr / bc1)
        param_out.copy_(master.to(param_out.dtype))
