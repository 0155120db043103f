"""Flat parameter layouts and the mapping to Hugging Face tensor names.

The sharding engine keeps each parameter *group* (one decoder block, the embedding, the head)
in ONE flat buffer; a rank owns one contiguous ``1/world`` slice of it. This replaces FSDP2's
per-parameter dim-0 sharding and its copy-in / copy-out glue
(torch/distributed/fsdp/_fully_shard/_fsdp_collectives.py:175-233): the all-gather target IS the
buffer the GEMMs read, with every tensor starting on a 256-byte boundary so that TMA descriptors
can point straight at it.

Within a block, q/k/v are stored as one ``[Hq*D + 2*Hkv*D, H]`` matrix and gate/up as one
``[2F, H]`` matrix, so each pair of projections is a single GEMM. Checkpoints split and merge
them back to the HF names (``q_proj``, ``k_proj``, ``v_proj``, ``gate_proj``, ``up_proj``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator

import torch

from .config import ModelConfig

ALIGN_ELEMS = 128  # every tensor starts at a multiple of 128 elements (256 B in bf16)


@dataclass(frozen=True)
class ParamSpec:
    name: str            # engine-local name, e.g. "wqkv"
    shape: tuple
    offset: int          # element offset in the group's flat buffer

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class GroupLayout:
    """Ordered tensors of one group inside a flat buffer padded to ``world * ALIGN_ELEMS``."""

    def __init__(self, name: str, entries: list, world: int):
        self.name = name
        self.specs: dict[str, ParamSpec] = {}
        off = 0
        for pname, shape in entries:
            spec = ParamSpec(pname, tuple(shape), off)
            self.specs[pname] = spec
            off += -(-spec.numel // ALIGN_ELEMS) * ALIGN_ELEMS
        self.numel = off
        q = world * ALIGN_ELEMS
        self.padded_numel = -(-off // q) * q
        self.shard_numel = self.padded_numel // world

    def views(self, flat: torch.Tensor) -> dict:
        """Named tensor views into a full (gathered) flat buffer."""
        return {n: flat[s.offset: s.offset + s.numel].view(s.shape) for n, s in self.specs.items()}


def block_entries(cfg: ModelConfig) -> list:
    h, f = cfg.hidden_size, cfg.intermediate_size
    # the small tensors needed before the first GEMM come first (see parallel.symmetric.GatherPlan)
    ln = cfg.norm_type == "layernorm"   # LayerNorm carries a bias next to its weight
    gu = (2 if cfg.mlp_gated else 1) * f   # rows of the first MLP matrix: gate|up, or c_fc alone
    e = [("ln1", (h,))]
    if ln:
        e.append(("bln1", (h,)))
    if cfg.attention_bias:
        e.append(("bqkv", (cfg.qkv_size,)))
    if cfg.qk_norm:
        e += [("qn", (cfg.head_dim,)), ("kn", (cfg.head_dim,))]
    if cfg.post_norm:   # OLMo-2 normalises the whole query and the whole key projection
        e += [("qn", (cfg.q_size,)), ("kn", (cfg.kv_size,))]
    e += [("wqkv", (cfg.qkv_size, h)), ("wo", (h, cfg.q_size))]
    # Optional biases sit where both schedules want them: ``bo`` and ``bgu`` in front of ``wgu``, so the
    # gather fused into the QKV projection has brought them in before o_proj / gate-up run and backward has
    # written their gradients before the region that starts at ``wo`` is reduced; ``bd`` behind ``wd``, inside
    # the gather fused into gate/up and inside the first region backward completes.
    if cfg.o_proj_bias:
        e.append(("bo", (h,)))
    e.append(("ln2", (h,)))
    if ln:
        e.append(("bln2", (h,)))
    if cfg.is_moe:   # router, then every expert's fused gate/up and down matrices
        fe = cfg.expert_intermediate_size
        e.append(("router", (cfg.num_local_experts, h)))
        for x in range(cfg.num_local_experts):
            e += [(f"wgu{x}", (2 * fe, h)), (f"wd{x}", (h, fe))]
        if cfg.shared_expert_intermediate_size:   # Qwen2-MoE: a shared expert and the vector that gates it
            fs = cfg.shared_expert_intermediate_size
            e += [("wgus", (2 * fs, h)), ("wds", (h, fs)), ("wsg", (1, h))]
        return e
    if cfg.mlp_bias:
        e.append(("bgu", (gu,)))
    e += [("wgu", (gu, h)), ("wd", (h, f))]
    if cfg.mlp_bias:
        e.append(("bd", (h,)))
    return e


def embed_entries(cfg: ModelConfig) -> list:
    return [("embed", (cfg.vocab_size, cfg.hidden_size))]


def head_entries(cfg: ModelConfig) -> list:
    e = [("norm", (cfg.hidden_size,))]
    if cfg.norm_type == "layernorm":
        e.append(("bnorm", (cfg.hidden_size,)))
    if not cfg.tie_word_embeddings:
        e.append(("lm_head", (cfg.vocab_size, cfg.hidden_size)))
    return e


# ------------------------------------------------------------------------------------------
# HF name mapping
# ------------------------------------------------------------------------------------------
def hf_tensors_of_block(cfg: ModelConfig, layer: int, views: dict) -> Iterator[tuple]:
    """Yields ``(hf_name, tensor_view)`` for one block, in HF ``state_dict`` order. Where the checkpoint stacks
    the experts of a projection into one 3-D tensor (Granite-MoE) the second item is a tuple of views, one per expert."""
    p = f"model.layers.{layer}."
    q, kv = cfg.q_size, cfg.kv_size
    if cfg.fused_hf_names:   # Phi-3: the checkpoint's tensors are the layout's
        yield p + "self_attn.qkv_proj.weight", views["wqkv"]
        yield p + "self_attn.o_proj.weight", views["wo"]
        yield p + "mlp.gate_up_proj.weight", views["wgu"]
        yield p + "mlp.down_proj.weight", views["wd"]
        yield p + "input_layernorm.weight", views["ln1"]
        yield p + "post_attention_layernorm.weight", views["ln2"]
        return
    w = views["wqkv"]
    yield p + "self_attn.q_proj.weight", w[:q]
    if cfg.attention_bias:
        yield p + "self_attn.q_proj.bias", views["bqkv"][:q]
    yield p + "self_attn.k_proj.weight", w[q: q + kv]
    if cfg.attention_bias:
        yield p + "self_attn.k_proj.bias", views["bqkv"][q: q + kv]
    yield p + "self_attn.v_proj.weight", w[q + kv:]
    if cfg.attention_bias:
        yield p + "self_attn.v_proj.bias", views["bqkv"][q + kv:]
    yield p + "self_attn.o_proj.weight", views["wo"]
    if cfg.qk_norm or cfg.post_norm:
        yield p + "self_attn.q_norm.weight", views["qn"]
        yield p + "self_attn.k_norm.weight", views["kn"]
    if cfg.o_proj_bias:
        yield p + "self_attn.o_proj.bias", views["bo"]
    f = cfg.intermediate_size
    if cfg.is_moe:   # names of the published checkpoints
        fe = cfg.expert_intermediate_size
        if cfg.model_type == "mixtral":   # w1 = gate, w3 = up, w2 = down
            m = p + "block_sparse_moe."
            for x in range(cfg.num_local_experts):
                yield m + f"experts.{x}.w1.weight", views[f"wgu{x}"][:fe]
                yield m + f"experts.{x}.w2.weight", views[f"wd{x}"]
                yield m + f"experts.{x}.w3.weight", views[f"wgu{x}"][fe:]
            yield m + "gate.weight", views["router"]
        elif cfg.model_type == "granitemoe":   # one 3-D tensor per projection: a tuple of views, one per expert
            m = p + "block_sparse_moe."
            yield m + "input_linear.weight", tuple(views[f"wgu{x}"] for x in range(cfg.num_local_experts))
            yield m + "output_linear.weight", tuple(views[f"wd{x}"] for x in range(cfg.num_local_experts))
            yield m + "router.layer.weight", views["router"]
        else:   # Qwen3-MoE
            for x in range(cfg.num_local_experts):
                yield p + f"mlp.experts.{x}.gate_proj.weight", views[f"wgu{x}"][:fe]
                yield p + f"mlp.experts.{x}.up_proj.weight", views[f"wgu{x}"][fe:]
                yield p + f"mlp.experts.{x}.down_proj.weight", views[f"wd{x}"]
            yield p + "mlp.gate.weight", views["router"]
            if cfg.shared_expert_intermediate_size:
                fs = cfg.shared_expert_intermediate_size
                yield p + "mlp.shared_expert.gate_proj.weight", views["wgus"][:fs]
                yield p + "mlp.shared_expert.up_proj.weight", views["wgus"][fs:]
                yield p + "mlp.shared_expert.down_proj.weight", views["wds"]
                yield p + "mlp.shared_expert_gate.weight", views["wsg"]
        yield p + "input_layernorm.weight", views["ln1"]
        yield p + "post_attention_layernorm.weight", views["ln2"]
        return
    if not cfg.mlp_gated:   # Starcoder2: c_fc, c_proj and LayerNorm biases
        yield p + "mlp.c_fc.weight", views["wgu"]
        if cfg.mlp_bias:
            yield p + "mlp.c_fc.bias", views["bgu"]
        yield p + "mlp.c_proj.weight", views["wd"]
        if cfg.mlp_bias:
            yield p + "mlp.c_proj.bias", views["bd"]
        yield p + "input_layernorm.weight", views["ln1"]
        yield p + "post_attention_layernorm.weight", views["ln2"]
        if cfg.norm_type == "layernorm":
            yield p + "input_layernorm.bias", views["bln1"]
            yield p + "post_attention_layernorm.bias", views["bln2"]
        return
    yield p + "mlp.gate_proj.weight", views["wgu"][:f]
    if cfg.mlp_bias:
        yield p + "mlp.gate_proj.bias", views["bgu"][:f]
    yield p + "mlp.up_proj.weight", views["wgu"][f:]
    if cfg.mlp_bias:
        yield p + "mlp.up_proj.bias", views["bgu"][f:]
    yield p + "mlp.down_proj.weight", views["wd"]
    if cfg.mlp_bias:
        yield p + "mlp.down_proj.bias", views["bd"]
    if cfg.post_norm:   # OLMo-2: the two norms sit behind the attention and the MLP branch
        yield p + "post_attention_layernorm.weight", views["ln1"]
        yield p + "post_feedforward_layernorm.weight", views["ln2"]
        return
    yield p + "input_layernorm.weight", views["ln1"]
    yield p + "post_attention_layernorm.weight", views["ln2"]


def hf_tensors_of_embed(cfg: ModelConfig, views: dict) -> Iterator[tuple]:
    yield "model.embed_tokens.weight", views["embed"]


def hf_tensors_of_head(cfg: ModelConfig, views: dict) -> Iterator[tuple]:
    yield "model.norm.weight", views["norm"]
    if cfg.norm_type == "layernorm":
        yield "model.norm.bias", views["bnorm"]
    if not cfg.tie_word_embeddings:
        yield "lm_head.weight", views["lm_head"]


def group_names(cfg: ModelConfig) -> list:
    return ["embed"] + [f"block{i}" for i in range(cfg.num_hidden_layers)] + ["head"]
