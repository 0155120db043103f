"""Decoder configuration, read from / written to Hugging Face ``config.json``.

Covers the Llama / Qwen2 / Qwen3 / Qwen3-MoE / Mistral / Phi-3 / Gemma / Granite / Granite-MoE / Mixtral / Starcoder2 families the reference trains through
``AutoModelForCausalLM`` (setup_model_for_training.py:86-130): pre-norm decoder blocks with
RMSNorm, rotary GQA attention (optional biases, optional per-head q/k norm), a SwiGLU MLP or Mixtral's routed SwiGLU experts,
tied or untied LM head, plus Granite's four scalars (embedding, residual, attention and logits
multipliers).

The reference's allow-list (setup_model_for_training.py:111-123) also names GPTDolomite
and merely warns for anything else, because whatever
``AutoModelForCausalLM`` loads brings its own forward. Here the forward and backward are
hand-written for ONE block structure, so an architecture whose math differs (LayerNorm or
GeGLU blocks) is refused by ``validate_supported`` instead of being trained with the wrong
function. Llama-style ``attention_bias`` (q/k/v AND o_proj) and ``mlp_bias`` (gate, up, down), which
the Granite code models use, are part of the block. Sliding-window models are accepted for samples no longer than the
window, where the window changes nothing (``attention_window``).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Optional


@dataclass
class ModelConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: Optional[int] = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    attention_bias: bool = False
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 131072
    model_type: str = "llama"
    architectures: list = field(default_factory=lambda: ["LlamaForCausalLM"])
    pad_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    # Granite (modeling_granite.py): embeddings * embedding_multiplier, block outputs * residual_multiplier
    # before the residual add, softmax scale = attention_multiplier, logits / logits_scaling
    embedding_multiplier: float = 1.0
    residual_multiplier: float = 1.0
    attention_multiplier: Optional[float] = None
    logits_scaling: float = 1.0
    sliding_window: Optional[int] = None
    use_sliding_window: Optional[bool] = None
    mlp_bias: bool = False
    hidden_act: str = "silu"
    # Mixtral (modeling_mixtral.py): the MLP of every block is num_local_experts SwiGLU experts, of which a
    # softmax router picks num_experts_per_tok per token; 0 experts = dense MLP
    # Starcoder2 (modeling_starcoder2.py): LayerNorm with bias instead of RMSNorm, and an MLP without a gate,
    # c_proj(gelu(c_fc(x))); its config spells the epsilon ``norm_epsilon`` and has one ``use_bias`` for every projection
    norm_type: str = "rmsnorm"
    mlp_gated: bool = True
    # dropout is not implemented: a config that sets one is refused unless the user asks to train without it
    ignore_dropout: bool = False
    # Gemma (modeling_gemma.py): the norms multiply by (1 + weight); embeddings are scaled by sqrt(hidden_size),
    # a constant that is first rounded to the embedding's dtype (55.4256 becomes 55.5 in bf16)
    norm_weight_offset: float = 0.0
    embedding_multiplier_in_param_dtype: bool = False
    # OLMo-2 (modeling_olmo2.py): no norm in front of a branch but one behind it (x + Norm(Attn(x)), h + Norm(MLP(h))),
    # and an RMSNorm over the whole query and the whole key projection
    post_norm: bool = False
    # SmolLM3 (modeling_smollm3.py): layers whose entry is 0 apply no rotary embedding (NoPE); None = every layer rotates
    no_rope_layers: Optional[list] = None
    # Qwen3 (modeling_qwen3.py): RMSNorm over head_dim on every q and k head before the rotary embedding
    qk_norm: bool = False
    # Qwen3-MoE (modeling_qwen3_moe.py): experts of their own width, optional renormalisation of the chosen weights,
    # experts stored as mlp.experts.N.{gate,up,down}_proj; Mixtral always renormalises and stores w1 / w3 / w2
    num_local_experts: int = 0
    num_experts_per_tok: int = 2
    moe_intermediate_size: Optional[int] = None
    norm_topk_prob: bool = True
    # Qwen2-MoE (modeling_qwen2_moe.py): next to the routed experts one shared SwiGLU expert of this width, whose output
    # is weighted by sigmoid(shared_expert_gate(x))
    shared_expert_intermediate_size: Optional[int] = None
    output_router_logits: bool = False
    router_jitter_noise: float = 0.0
    extra: dict = field(default_factory=dict)  # unknown keys of config.json, written back verbatim

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")

    @property
    def attention_scale(self) -> float:
        """Scale applied to q.k before the softmax (with YaRN's / longrope's factor on q and k folded in)."""
        base = float(self.attention_multiplier) if self.attention_multiplier is not None else self.head_dim ** -0.5
        return base * self.rope_attention_factor ** 2

    @property
    def attention_window(self) -> Optional[int]:
        """Sliding-window length where the model applies one (Mistral, Mixtral, Phi-3 always; Qwen2 with ``use_sliding_window``), else
        ``None``. A query sees the last ``window`` keys including itself (masking_utils.sliding_window_overlay), so for
        samples of at most ``window`` tokens windowed and full causal attention are the same function. The attention
        kernels here are full causal: the engine accepts such a model and refuses a minibatch that holds a longer sample."""
        if self.sliding_window is None or self.sliding_window >= self.max_position_embeddings:
            return None
        # (SmolLM3 windows only its NoPE layers; treating the window as model-wide is the stricter reading)
        on = self.use_sliding_window if self.use_sliding_window is not None else \
            self.model_type in ("mistral", "mixtral", "phi3", "starcoder2")
        return int(self.sliding_window) if on else None

    def embed_scale(self, dtype) -> float:
        """Factor applied to the embedding output (1.0 for most models) as the model itself computes it in ``dtype``."""
        m = float(self.embedding_multiplier)
        if self.embedding_multiplier_in_param_dtype and m != 1.0:
            import torch
            m = float(torch.tensor(m, dtype=dtype))
        return m

    @property
    def rotary_dim(self) -> int:
        """Leading dimensions of every head the rotary embedding turns (``partial_rotary_factor``: Phi-4-mini turns
        three quarters of a head); the rest passes through."""
        prf = (self.extra.get("rope_parameters") or {}).get("partial_rotary_factor", self.extra.get("partial_rotary_factor"))
        return self.head_dim if prf in (None, 1.0) else int(self.head_dim * float(prf))

    def layer_uses_rope(self, layer: int) -> bool:
        return self.no_rope_layers is None or bool(self.no_rope_layers[layer])

    @property
    def mlp_act(self) -> str:
        """Activation of the gated MLP: ``silu`` (SwiGLU) or ``gelu_tanh`` (GeGLU)."""
        return "gelu_tanh" if self.hidden_act == "gelu_pytorch_tanh" else "silu"

    @property
    def fused_hf_names(self) -> bool:
        """Phi-3 checkpoints store q|k|v and gate|up already fused (``qkv_proj``, ``gate_up_proj``), in the order
        the flat layout uses."""
        return self.model_type == "phi3"

    @property
    def is_moe(self) -> bool:
        return self.num_local_experts > 0

    @property
    def expert_intermediate_size(self) -> int:
        return int(self.moe_intermediate_size or self.intermediate_size)

    def validate_supported(self) -> None:
        """Raises ``ValueError`` when the hand-written block would not compute this model's function."""
        arch = (self.architectures or ["?"])[0]
        problems = []
        if self.no_rope_layers is not None and len(self.no_rope_layers) != self.num_hidden_layers:
            problems.append(f"no_rope_layers has {len(self.no_rope_layers)} entries for {self.num_hidden_layers} layers")
        if self.post_norm and (self.is_moe or self.norm_type != "rmsnorm" or not self.mlp_gated or self.qk_norm
                               or self.norm_weight_offset or self.residual_multiplier != 1.0):
            problems.append("the post-norm block is implemented for OLMo-2's combination only (dense gated MLP, RMSNorm)")
        if self.is_moe:
            if self.output_router_logits:
                problems.append("output_router_logits=true adds the router's load-balancing loss, which is not implemented")
            if self.router_jitter_noise:
                problems.append(f"router_jitter_noise={self.router_jitter_noise} (input jitter is not implemented)")
            if self.mlp_bias:
                problems.append("mlp_bias=true with experts")
            if self.shared_expert_intermediate_size and self.model_type != "qwen2_moe":
                problems.append("a shared expert outside Qwen2-MoE")
            if self.extra.get("decoder_sparse_step", 1) != 1 or self.extra.get("mlp_only_layers"):
                problems.append("dense and expert layers mixed (decoder_sparse_step / mlp_only_layers): every block must have "
                                "the same layout")
            if not 0 < self.num_experts_per_tok <= self.num_local_experts:
                problems.append(f"num_experts_per_tok={self.num_experts_per_tok} of {self.num_local_experts} experts")
        if arch not in SUPPORTED_ARCHITECTURES:
            problems.append(f"architecture {arch} is not one of {', '.join(SUPPORTED_ARCHITECTURES)}")
        for k in ("attention_dropout", "resid_pdrop", "embd_pdrop", "residual_dropout", "embedding_dropout", "hidden_dropout"):
            if self.extra.get(k) and not self.ignore_dropout:
                problems.append(f"{k}={self.extra[k]} (dropout is not implemented; pass --no-dropout to train without it)")
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            problems.append(f"partial_rotary_factor gives a rotary width of {self.rotary_dim} for head_dim {self.head_dim}")
        if not self.mlp_gated and (self.hidden_act != "gelu_pytorch_tanh" or self.is_moe):
            problems.append(f"an MLP without a gate is implemented with the tanh-approximated GELU only (hidden_act={self.hidden_act!r})")
        if self.hidden_act not in ("silu", "swish", "gelu_pytorch_tanh"):
            problems.append(f"hidden_act={self.hidden_act!r} (the gated MLP is implemented with SiLU and with the "
                            "tanh-approximated GELU)")
        try:
            self.rope_inv_freq()
        except ValueError as e:   # e.g. Phi-3's "longrope" or "yarn": per-position frequency rescaling is not implemented
            problems.append(str(e))
        if problems:
            raise ValueError("this model cannot be trained faithfully: " + "; ".join(problems))

    # sizes -------------------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_size(self) -> int:
        return self.q_size + 2 * self.kv_size

    @property
    def o_proj_bias(self) -> bool:
        """``attention_bias`` covers q, k, v and o_proj in the Llama-style classes (modeling_llama.py,
        modeling_granite.py); Qwen2 has the q/k/v biases only (modeling_qwen2.py)."""
        return self.attention_bias and self.model_type not in ("qwen2", "qwen2_moe")

    @property
    def mlp_mats(self) -> int:
        """Matrices of one MLP: gate, up, down, or up and down only."""
        return 3 if self.mlp_gated else 2

    @property
    def mlp_rows_factor(self) -> int:
        """Rows that go through an MLP per token: the number of experts a token is sent to (1 for a dense MLP)."""
        return self.num_experts_per_tok if self.is_moe else 1

    def block_param_count(self) -> int:
        h, f = self.hidden_size, (self.expert_intermediate_size if self.is_moe else self.intermediate_size)
        n = 2 * h + self.qkv_size * h + self.q_size * h + self.mlp_mats * h * f * max(1, self.num_local_experts)
        n += 2 * h if self.norm_type == "layernorm" else 0
        n += self.num_local_experts * h   # router
        if self.shared_expert_intermediate_size:
            n += 3 * h * self.shared_expert_intermediate_size + h
        n += self.qkv_size if self.attention_bias else 0
        n += 2 * self.head_dim if self.qk_norm else 0
        n += self.q_size + self.kv_size if self.post_norm else 0
        n += h if self.o_proj_bias else 0
        return n + ((self.mlp_mats - 1) * f + h if self.mlp_bias else 0)

    def param_count(self) -> int:
        emb = self.vocab_size * self.hidden_size
        final_norm = self.hidden_size * (2 if self.norm_type == "layernorm" else 1)
        return self.num_hidden_layers * self.block_param_count() + final_norm + emb * (1 if self.tie_word_embeddings else 2)

    def flops_per_token(self, avg_context: float = 0.0, recompute: bool = True) -> float:
        """Training FLOPs per token: 6 x matmul params (+2 x with full recompute) + attention. With experts
        only the ``num_experts_per_tok`` chosen ones (and the router) count."""
        h, f = self.hidden_size, (self.expert_intermediate_size if self.is_moe else self.intermediate_size)
        mm = self.num_hidden_layers * (self.qkv_size * h + self.q_size * h + self.mlp_mats * h * f * self.mlp_rows_factor
                                       + self.num_local_experts * h)
        head = self.vocab_size * h
        k = 8 if recompute else 6
        attn = self.num_hidden_layers * 2 * 2 * self.q_size * avg_context  # QK^T and PV, forward
        return k * mm + 6 * head + (4 if recompute else 3) * attn

    def attention_cost_length(self, recompute: bool = True, gemm_rate: float = 1.25e15, attn_rate: float = 0.75e15) -> float:
        """Sequence length at which the causal attention of a token costs as much time as its GEMMs.

        Used by the cost-aware packer. GEMM work per token: 6 (8 with recompute) FLOPs per matmul
        parameter; attention work per token and per context token: forward 2*2*q_size per layer, halved
        by causality, times 3.5 for forward + backward. The rates are typical sustained throughputs of
        the two kernel families on a power-capped B200.
        """
        h, f = self.hidden_size, (self.expert_intermediate_size if self.is_moe else self.intermediate_size)
        mm = self.num_hidden_layers * (self.qkv_size * h + self.q_size * h + self.mlp_mats * h * f * self.mlp_rows_factor)
        gemm = (8 if recompute else 6) * mm + 6 * self.vocab_size * h
        attn = 3.5 * 2 * self.q_size * self.num_hidden_layers
        return (gemm / gemm_rate) / (attn / attn_rate)

    # rotary ------------------------------------------------------------------------
    def rope_long_context_threshold(self) -> Optional[int]:
        """``longrope`` (Phi-3 128k) rescales the frequencies with one table up to this many tokens and with another
        beyond; ``None`` for every other kind of rope."""
        rs = self.rope_scaling or {}
        if rs.get("rope_type", rs.get("type")) != "longrope":
            return None
        return int(rs.get("original_max_position_embeddings") or self.extra.get("original_max_position_embeddings")
                   or self.max_position_embeddings)

    def rope_inv_freq(self, seq_len: Optional[int] = None):
        """fp32 inverse frequencies [rotary_dim/2], with ``linear``, ``llama3``, ``yarn`` and ``longrope`` scaling.
        ``seq_len``: the longest sample of the minibatch (only ``longrope`` looks at it)."""
        import torch
        d = self.rotary_dim
        inv = 1.0 / (self.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        rs = self.rope_scaling or {}
        kind = rs.get("rope_type", rs.get("type", "default"))
        if kind in (None, "default"):
            pass
        elif kind == "linear":
            inv = inv / float(rs["factor"])
        elif kind == "llama3":
            factor = float(rs["factor"])
            lo, hi = float(rs.get("low_freq_factor", 1.0)), float(rs.get("high_freq_factor", 4.0))
            old = float(rs.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv
            smooth = (old / wavelen - lo) / (hi - lo)
            mid = (1 - smooth) * inv / factor + smooth * inv
            inv = torch.where(wavelen > old / lo, inv / factor, torch.where(wavelen < old / hi, inv, mid))
        elif kind == "longrope":   # modeling_rope_utils._compute_longrope_parameters: one divisor per frequency
            long_ctx = seq_len is not None and seq_len > self.rope_long_context_threshold()
            ext = torch.tensor(rs["long_factor"] if long_ctx else rs["short_factor"], dtype=torch.float64)
            if ext.numel() != inv.numel():
                raise ValueError(f"longrope factors have {ext.numel()} entries for {inv.numel()} frequencies")
            inv = inv / ext
        elif kind == "yarn":   # modeling_rope_utils._compute_yarn_parameters: interpolate low frequencies, keep high ones
            factor = float(rs["factor"])
            old = float(rs.get("original_max_position_embeddings") or self.max_position_embeddings)
            fast, slow = float(rs.get("beta_fast") or 32), float(rs.get("beta_slow") or 1)

            def corr_dim(rot):
                return d * math.log(old / (rot * 2 * math.pi)) / (2 * math.log(self.rope_theta))

            lo, hi = corr_dim(fast), corr_dim(slow)
            if rs.get("truncate", True):
                lo, hi = math.floor(lo), math.ceil(hi)
            lo, hi = max(lo, 0), min(hi, d - 1)
            if lo == hi:
                hi += 0.001
            ramp = ((torch.arange(d // 2, dtype=torch.float32) - lo) / (hi - lo)).clamp(0, 1)
            pos = self.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d)
            keep = 1 - ramp
            inv = (1.0 / (factor * pos)) * (1 - keep) + (1.0 / pos) * keep
        else:
            raise ValueError(f"unsupported rope scaling {kind!r}")
        return inv.to(torch.float32)

    @property
    def rope_attention_factor(self) -> float:
        """YaRN and longrope multiply the rotary cosines and sines by this factor, i.e. q and k each, i.e. the scores by
        its square (1.0 for every other kind of rope)."""
        rs = self.rope_scaling or {}
        kind = rs.get("rope_type", rs.get("type"))
        if kind not in ("yarn", "longrope"):
            return 1.0
        if rs.get("attention_factor") is not None:
            return float(rs["attention_factor"])
        if kind == "longrope":
            old = self.rope_long_context_threshold()
            factor = float(rs.get("factor") or self.max_position_embeddings / old)
            return 1.0 if factor <= 1.0 else math.sqrt(1 + math.log(factor) / math.log(old))
        factor = float(rs["factor"])

        def mscale(scale, m=1.0):
            return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

        if rs.get("mscale") and rs.get("mscale_all_dim"):
            return float(mscale(factor, rs["mscale"]) / mscale(factor, rs["mscale_all_dim"]))
        return float(mscale(factor))

    # HF I/O -------------------------------------------------------------------------
    _KNOWN = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
              "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "rope_scaling", "attention_bias",
              "tie_word_embeddings", "max_position_embeddings", "model_type", "architectures",
              "pad_token_id", "bos_token_id", "eos_token_id", "embedding_multiplier", "residual_multiplier",
              "attention_multiplier", "logits_scaling", "sliding_window", "use_sliding_window", "mlp_bias", "hidden_act",
              "num_local_experts", "num_experts_per_tok", "output_router_logits", "router_jitter_noise",
              "moe_intermediate_size", "norm_topk_prob", "no_rope_layers", "shared_expert_intermediate_size")
    _MOE_ONLY = ("num_local_experts", "num_experts_per_tok", "output_router_logits", "router_jitter_noise",
                 "moe_intermediate_size", "norm_topk_prob", "shared_expert_intermediate_size")
    _GRANITE_ONLY = ("embedding_multiplier", "residual_multiplier", "attention_multiplier", "logits_scaling")

    @classmethod
    def from_hf_dict(cls, d: dict) -> "ModelConfig":
        d = dict(d)
        kw = {k: d.pop(k) for k in list(d) if k in cls._KNOWN}
        kw.setdefault("num_key_value_heads", kw.get("num_attention_heads"))
        rp = d.get("rope_parameters")  # transformers >= 5 nests rope settings
        if isinstance(rp, dict):
            kw.setdefault("rope_theta", rp.get("rope_theta", 10000.0))
            if rp.get("rope_type", "default") != "default":
                kw.setdefault("rope_scaling", rp)
        if kw.get("model_type") in ("qwen2", "qwen2_moe"):
            kw.setdefault("attention_bias", True)  # Qwen2 always has q/k/v biases
        if kw.get("model_type") in ("qwen3", "qwen3_moe"):
            kw["qk_norm"] = True
        if kw.get("model_type") in ("qwen3_moe", "qwen2_moe"):
            if "num_experts" in d:   # the published configs' key; transformers also writes num_local_experts
                kw["num_local_experts"] = d["num_experts"]
            kw.setdefault("norm_topk_prob", False)
            qwen3 = kw["model_type"] == "qwen3_moe"   # the defaults of the two config classes
            kw.setdefault("moe_intermediate_size", 768 if qwen3 else 1408)
            kw.setdefault("num_experts_per_tok", 8 if qwen3 else 4)
            if not qwen3:
                kw.setdefault("shared_expert_intermediate_size", 5632)
        if kw.get("model_type") in ("mixtral", "granitemoe"):
            # GraniteMoe takes the softmax over the chosen logits only, which is the softmax over all of them
            # renormalised over the chosen ones: the same weights as Mixtral's
            kw.pop("moe_intermediate_size", None)
            kw["norm_topk_prob"] = True
        if kw.get("model_type") == "smollm3" and kw.get("no_rope_layers") is None:   # the config class's default rule
            step = int(d.get("no_rope_layer_interval", 4))
            kw["no_rope_layers"] = [int((i + 1) % step != 0) for i in range(int(kw["num_hidden_layers"]))]
        if kw.get("model_type") == "olmo2":
            kw["post_norm"] = True
        if kw.get("model_type") == "starcoder2":
            use_bias = bool(d.pop("use_bias", True))
            kw.update(norm_type="layernorm", mlp_gated=False, attention_bias=use_bias, mlp_bias=use_bias,
                      rms_norm_eps=float(d.pop("norm_epsilon", 1e-5)))
            kw.setdefault("hidden_act", "gelu_pytorch_tanh")
            kw.setdefault("tie_word_embeddings", True)
        if kw.get("model_type") == "gemma":
            kw.update(norm_weight_offset=1.0, embedding_multiplier_in_param_dtype=True,
                      embedding_multiplier=float(kw["hidden_size"]) ** 0.5)
            kw.setdefault("hidden_act", "gelu_pytorch_tanh")
            kw.setdefault("tie_word_embeddings", True)
            if d.get("hidden_activation"):   # older Gemma configs carry the real activation under this key
                kw["hidden_act"] = d["hidden_activation"]
        for k in ("bos_token_id", "eos_token_id", "pad_token_id"):
            if isinstance(kw.get(k), list):
                d[k + "_list"] = kw[k]
                kw[k] = kw[k][0]
        return cls(**kw, extra=d)

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_dict(json.load(f))

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        extra = d.pop("extra")
        for k in ("qk_norm", "norm_weight_offset", "embedding_multiplier_in_param_dtype", "norm_type", "mlp_gated", "ignore_dropout", "post_norm"):
            d.pop(k)   # implied by the model type, not keys of any Hugging Face config
        if d["no_rope_layers"] is None:
            d.pop("no_rope_layers")
        if self.model_type == "starcoder2":   # back to its own spelling
            d["norm_epsilon"], d["use_bias"] = d.pop("rms_norm_eps"), d.pop("attention_bias")
            d["mlp_bias"] = False
        out = dict(extra)
        for k in ("bos_token_id", "eos_token_id", "pad_token_id"):
            lst = out.pop(k + "_list", None)
            if lst is not None:
                d[k] = lst
        for k in self._GRANITE_ONLY:   # only Granite's config class knows these keys
            if self.model_type not in ("granite", "granitemoe"):
                d.pop(k)
        for k in self._MOE_ONLY:
            if not self.is_moe or d[k] is None or (self.model_type in ("mixtral", "granitemoe")
                                                   and k in ("moe_intermediate_size", "norm_topk_prob")):
                d.pop(k)
        if self.model_type in ("qwen3_moe", "qwen2_moe"):
            d["num_experts"] = self.num_local_experts
        if self.model_type == "qwen2_moe":
            d.pop("attention_bias", None)
        for k in ("sliding_window", "use_sliding_window"):
            if d[k] is None:
                d.pop(k)
        if not d["mlp_bias"]:
            d.pop("mlp_bias")
        out.update(d)
        out.setdefault("hidden_act", "silu")
        out.setdefault("torch_dtype", "bfloat16")
        out["use_cache"] = False
        if self.model_type == "qwen2":
            out.pop("attention_bias", None)
        return out

    def to_json_file(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_hf_dict(), f, indent=2, sort_keys=True)
            f.write("\n")


SUPPORTED_ARCHITECTURES = ("LlamaForCausalLM", "Qwen2ForCausalLM", "MistralForCausalLM", "GraniteForCausalLM",
                           "MixtralForCausalLM", "Phi3ForCausalLM", "Qwen3ForCausalLM", "GemmaForCausalLM",
                           "Starcoder2ForCausalLM", "Qwen3MoeForCausalLM", "GraniteMoeForCausalLM", "SmolLM3ForCausalLM",
                           "Qwen2MoeForCausalLM", "Olmo2ForCausalLM")


def _llama(**kw):
    return ModelConfig(model_type="llama", architectures=["LlamaForCausalLM"], **kw)


def _qwen2(**kw):
    return ModelConfig(model_type="qwen2", architectures=["Qwen2ForCausalLM"], attention_bias=True, **kw)


PRESETS = {
    # the five benchmark architectures (random-init; sizes only)
    "tiny-qwen2": lambda: _qwen2(vocab_size=32000, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                                 num_attention_heads=4, num_key_value_heads=2, rope_theta=1e6,
                                 tie_word_embeddings=True, rms_norm_eps=1e-6),
    "qwen2.5-1.5b": lambda: _qwen2(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
                                   num_attention_heads=12, num_key_value_heads=2, rope_theta=1e6,
                                   tie_word_embeddings=True, rms_norm_eps=1e-6),
    "llama-3.1-8b": lambda: _llama(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                                   num_attention_heads=32, num_key_value_heads=8, rope_theta=5e5, rms_norm_eps=1e-5),
    "qwen2.5-7b": lambda: _qwen2(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                                 num_attention_heads=28, num_key_value_heads=4, rope_theta=1e6, rms_norm_eps=1e-6),
    "llama-3.1-70b": lambda: _llama(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                                    num_attention_heads=64, num_key_value_heads=8, rope_theta=5e5, rms_norm_eps=1e-5),
    "mixtral-8x7b": lambda: ModelConfig(model_type="mixtral", architectures=["MixtralForCausalLM"], vocab_size=32000,
                                        hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                                        num_attention_heads=32, num_key_value_heads=8, rope_theta=1e6, rms_norm_eps=1e-5,
                                        num_local_experts=8, num_experts_per_tok=2),
    # a small Mixtral (4 experts, 2 per token) for CPU and GPU tests (head_dim 128 on the GPU kernels' account)
    "tiny-mixtral": lambda: ModelConfig(model_type="mixtral", architectures=["MixtralForCausalLM"], vocab_size=4096,
                                        hidden_size=256, intermediate_size=384, num_hidden_layers=2, num_attention_heads=2,
                                        num_key_value_heads=1, rope_theta=1e6, rms_norm_eps=1e-5, num_local_experts=4,
                                        num_experts_per_tok=2),
    # the smallest useful Llama: command-line and resume tests on CPU
    "nano-llama": lambda: _llama(vocab_size=2048, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                 num_attention_heads=4, num_key_value_heads=2, rope_theta=1e4, rms_norm_eps=1e-5),
    # a small Llama used by GPU smoke tests (head_dim 128, GQA 4:1)
    "smoke-llama": lambda: _llama(vocab_size=4096, hidden_size=512, intermediate_size=1536, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=1, rope_theta=5e5, rms_norm_eps=1e-5),
}


def get_preset(name: str) -> ModelConfig:
    return PRESETS[name]()
