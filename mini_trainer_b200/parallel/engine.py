"""The sharding engine: fully sharded parameters, gradients and optimizer state.

Role of the reference's ``wrap_fsdp2`` + ``AdamW`` + ``clip_grad_norm_`` + ``take_gradient_step``
(setup_model_for_training.py:14-48,132-152; train.py:22-28), built as one explicit schedule
instead of hooks on an autograd graph:

* Parameters are grouped as ``embed | block0 .. blockL-1 | head``. Each group lives in one flat
  buffer; a rank permanently owns one contiguous ``1/world`` slice of it: the working copy in the
  compute dtype, an fp32 master copy, AdamW moments and an fp32 gradient accumulator.
* Forward walks the blocks, gathering block ``i+1`` on a side stream while block ``i`` computes,
  and keeps only each block's input (per-block activation checkpointing, as the reference).
* Backward walks them in reverse: gather, recompute the block forward, run the hand-written
  backward into the block's flat gradient buffer, then reduce-scatter that buffer (SUM) into the
  fp32 accumulator shard on the side stream while the next block computes.
* After the last microbatch: one sum of squares over the accumulator shards, one scalar
  all-reduce, the clip coefficient ``min(1, max_norm / (norm + 1e-6))`` kept on the device, and a
  fused AdamW pass that updates master weights and refreshes the working shard.

The gradient of a step is that of ``sum(token CE over all ranks and microbatches) /
batch_num_loss_counted_tokens`` (reference train.py:98-102 after FSDP's averaging).

Precision: compute dtype bf16 on GPUs (fp32 in the CPU oracle runs); gradients are produced in
the compute dtype per microbatch and accumulated in fp32; master weights fp32; moments fp32 or
bf16 (``state_dtype``). The reference keeps everything, moments included, in bf16.
"""
from __future__ import annotations

import contextlib
import math
import os
from dataclasses import dataclass, field
from typing import Iterator, Optional

import torch

from ..models import decoder as D
from ..models import layout as L
from ..models.config import ModelConfig
from ..utils import nvtx
from .comm import LocalComm


@dataclass
class OptimConfig:
    lr: float = 5e-6
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0


class ShardedGroup:
    """One parameter group: layout + this rank's shard of params, master, moments, grads."""

    def __init__(self, layout: L.GroupLayout, device, param_dtype, state_dtype, shard=None):
        self.layout = layout
        s = layout.shard_numel
        self.shard = shard if shard is not None else torch.zeros(s, dtype=param_dtype, device=device)
        self.master = torch.zeros(s, dtype=torch.float32, device=device)
        self.m = torch.zeros(s, dtype=state_dtype, device=device)
        self.v = torch.zeros(s, dtype=state_dtype, device=device)
        self.gacc = torch.zeros(s, dtype=torch.float32, device=device)
        self.has_grad = False
        self.sq_done = False   # sum of squares of gacc already added to the engine's norm scalar

    def state_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.shard, self.master, self.m, self.v, self.gacc))


class _Side:
    """A side CUDA stream with event hand-offs; degenerates to inline execution on CPU."""

    def __init__(self, device):
        self.cuda = device.type == "cuda"
        self.stream = torch.cuda.Stream(device=device, priority=-1) if self.cuda else None

    @contextlib.contextmanager
    def run(self, wait_current: bool = True):
        if not self.cuda:
            yield
            return
        if wait_current:
            self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            yield

    def record(self):
        if not self.cuda:
            return None
        ev = torch.cuda.Event()
        ev.record(self.stream)
        return ev

    # When a list is installed here, every wait of the compute stream on communication work is
    # bracketed by two events, so the time the compute stream really stalled can be summed later.
    stalls = None

    @staticmethod
    def wait(ev):
        if ev is not None:
            cur = torch.cuda.current_stream()
            if _Side.stalls is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(cur)
                cur.wait_event(ev)
                e1.record(cur)
                _Side.stalls.append((e0, e1))
            else:
                cur.wait_event(ev)


class _HostInput:
    """A block input that lives in pinned host memory between forward and backward."""

    def __init__(self, host: torch.Tensor, shape: tuple):
        self.host, self.shape = host, shape
        self.device = self.ready = self.slot = None


class ShardedEngine:
    def __init__(self, cfg: ModelConfig, device, ops, comm=None, param_dtype=None, state_dtype=None,
                 optim: Optional[OptimConfig] = None, activation_budget_bytes: Optional[int] = None):
        self.cfg, self.device, self.ops = cfg, torch.device(device), ops
        self.comm = comm if comm is not None else LocalComm()
        self.world, self.rank = self.comm.world, self.comm.rank
        self.param_dtype = param_dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.state_dtype = state_dtype or torch.float32
        self.optim = optim or OptimConfig()
        self.step_count = 0
        self.inv_freq = cfg.rope_inv_freq().to(self.device)
        # longrope: a second table for minibatches whose longest sample exceeds the original context length
        self._rope_threshold = cfg.rope_long_context_threshold()
        self.inv_freq_long = cfg.rope_inv_freq(seq_len=self._rope_threshold + 1).to(self.device) if self._rope_threshold else None

        layouts = ([L.GroupLayout("embed", L.embed_entries(cfg), self.world)]
                   + [L.GroupLayout(f"block{i}", L.block_entries(cfg), self.world) for i in range(cfg.num_hidden_layers)]
                   + [L.GroupLayout("head", L.head_entries(cfg), self.world)])
        blk = layouts[1].padded_numel
        nbuf = 2
        # Buffers that peers read (parameter shards, gradient buffers) live in the comm backend's
        # symmetric arena when it has one; otherwise they are ordinary device tensors.
        self.symmetric = hasattr(self.comm, "setup")
        # the fused gather resolves one shard boundary per 128 KB chunk, so shards must be at least that large
        # (a mixture-of-experts block has no single gate/up GEMM to carry the second half of the gather: its
        # parameters are prefetched by the stand-alone all-gather, one block ahead, on the side stream)
        self.fused_gather = (self.symmetric and os.environ.get("MTB200_FUSED_GATHER", "1") != "0" and not cfg.is_moe
                             and layouts[1].shard_numel * torch.empty(0, dtype=self.param_dtype).element_size() >= 128 * 1024)
        if self.symmetric:
            es = torch.empty(0, dtype=self.param_dtype).element_size()
            payload = sum(l.shard_numel for l in layouts) + nbuf * blk + layouts[0].padded_numel + layouts[-1].padded_numel
            self.comm.setup(payload * es + (len(layouts) + 8) * 512)
        salloc = (lambda n: self.comm.alloc(n, self.param_dtype)) if self.symmetric else \
                 (lambda n: torch.zeros(n, dtype=self.param_dtype, device=self.device))
        mk = lambda lay: ShardedGroup(lay, self.device, self.param_dtype, self.state_dtype,
                                      shard=salloc(lay.shard_numel) if self.symmetric else None)
        self.embed = mk(layouts[0])
        self.blocks = [mk(l) for l in layouts[1:-1]]
        self.head = mk(layouts[-1])
        self.groups = [self.embed] + self.blocks + [self.head]

        self.side = _Side(self.device)
        # rotating full-size buffers for gathered block parameters and block gradients
        self._pbufs = [] if self.world == 1 else [torch.zeros(blk, dtype=self.param_dtype, device=self.device) for _ in range(nbuf)]
        self._gbufs = [salloc(blk) for _ in range(nbuf)]
        self._eg_full = salloc(self.embed.layout.padded_numel)   # embedding gradient (full, reduced once per microbatch)
        self._hg_full = salloc(self.head.layout.padded_numel)    # final norm / lm_head gradient
        self._root_free = {"embed": None, "head": None}
        self._sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._pbuf_free = [None] * nbuf   # event after which the buffer may be overwritten
        self._gbuf_free = [None] * nbuf
        self._rs_scratch = None
        if self.world > 1:
            smax = max(g.layout.shard_numel for g in self.groups)
            self._rs_scratch = torch.empty(smax, dtype=self.param_dtype, device=self.device)
        # None = derive from free device memory; 0 = recompute every block like the reference
        self.activation_budget_bytes = activation_budget_bytes
        self._oom_retries = 0
        # Reduce a block's gradients tensor region by tensor region while its backward still runs
        # (MTB200_REGION_OVERLAP=0: one reduction per block, after its backward).
        # A mixture-of-experts block is reduced once: its experts' gradients complete in no fixed layout order.
        self.region_overlap = os.environ.get("MTB200_REGION_OVERLAP", "1") != "0" and not cfg.is_moe
        # checkpoint level 3: block inputs parked in pinned host memory, two device staging buffers for the way back
        self._copy_stream = None
        self._host_inputs = {}
        self._dev_inputs = [None, None]
        self._dev_input_free = [None, None]
        self._pending_input_slot = None
        # Test configuration: buffers that are about to be filled by a gather or by a block's weight
        # gradients are first filled with NaN, so data consumed before it arrived (or a gradient that
        # was never written) shows up as NaN in the loss / norm instead of as a plausible stale value.
        self.poison = os.environ.get("MTB200_POISON", "0") == "1" and self.param_dtype != torch.int8

    def _inv_freq(self, layer: int, batch=None):
        """Rotary frequencies of a layer for this minibatch, or ``None`` where the model applies no positional rotation."""
        if not self.cfg.layer_uses_rope(layer):
            return None
        if self.inv_freq_long is not None and batch is not None and batch.max_seqlen > self._rope_threshold:
            return self.inv_freq_long
        return self.inv_freq

    # ------------------------------------------------------------------------------------
    # initialisation / state exchange
    # ------------------------------------------------------------------------------------
    def _set_group_from_full(self, grp: ShardedGroup, full: torch.Tensor) -> None:
        s = grp.layout.shard_numel
        sl = full[self.rank * s:(self.rank + 1) * s]
        grp.master.copy_(sl.float())
        grp.shard.copy_(grp.master.to(self.param_dtype))

    def init_random(self, seed: int = 0, std: float = 0.02, on_device: bool = False) -> None:
        """Same weights on every world size: each group is generated in full from its own seeded
        generator and the rank keeps its slice. ``on_device`` draws with the device generator
        (fast for multi-billion-parameter benchmarks; a different stream than the CPU one)."""
        dev = self.device if on_device else torch.device("cpu")
        for gi, grp in enumerate(self.groups):
            gen = torch.Generator(device=dev).manual_seed(seed * 1000003 + gi)
            full = torch.zeros(grp.layout.padded_numel, dtype=torch.float32, device=dev)
            for name, spec in grp.layout.specs.items():
                v = full[spec.offset: spec.offset + spec.numel]
                if len(spec.shape) == 1:
                    v.fill_(0.0 if name.startswith("b") else 1.0 - self.cfg.norm_weight_offset)   # biases 0, norms identity
                else:
                    v.normal_(0.0, std, generator=gen)
            self._set_group_from_full(grp, full.to(self.device))
            del full

    def load_hf_tensors(self, get_tensor) -> None:
        """``get_tensor(hf_name) -> torch.Tensor`` (any dtype, CPU). Every rank reads the tensors
        of one group at a time, so host memory holds one block, not the model.

        A vocabulary larger than the checkpoint's (``align_model_and_tokenizer`` grew it to fit the
        tokenizer, reference setup_model_for_training.py:54-60 ``resize_token_embeddings``) keeps
        the checkpoint's rows and initialises every new row of the embedding and of the LM head
        with the mean of the existing rows."""
        for grp, it in self._hf_iters():
            full = torch.zeros(grp.layout.padded_numel, dtype=torch.float32)
            views = grp.layout.views(full)
            for name, view in it(views):
                src = get_tensor(name).to(torch.float32)
                if isinstance(view, tuple):   # experts stacked along the first dimension of one checkpoint tensor
                    if src.shape[0] != len(view) or src[0].numel() != view[0].numel():
                        raise ValueError(f"{name}: checkpoint shape {tuple(src.shape)} does not fit {len(view)} x {tuple(view[0].shape)}")
                    for x, v in enumerate(view):
                        v.copy_(src[x].reshape(v.shape))
                    continue
                if src.dim() == 2 and src.shape[0] < view.shape[0] and src.shape[1:] == view.shape[1:] \
                        and name in ("model.embed_tokens.weight", "lm_head.weight"):
                    view[: src.shape[0]].copy_(src)
                    view[src.shape[0]:].copy_(src.mean(0, keepdim=True).expand(view.shape[0] - src.shape[0], -1))
                    continue
                if src.numel() != view.numel():
                    raise ValueError(f"{name}: checkpoint shape {tuple(src.shape)} does not fit {tuple(view.shape)}")
                view.copy_(src.reshape(view.shape))
            self._set_group_from_full(grp, full.to(self.device))

    def _hf_iters(self):
        cfg = self.cfg
        yield self.embed, (lambda v: L.hf_tensors_of_embed(cfg, v))
        for i, b in enumerate(self.blocks):
            yield b, (lambda v, i=i: L.hf_tensors_of_block(cfg, i, v))
        yield self.head, (lambda v: L.hf_tensors_of_head(cfg, v))

    @torch.no_grad()
    def iter_hf_tensors(self, dtype=torch.bfloat16, source: str = "master", host_ranks=None) -> Iterator[tuple]:
        """Yields ``(hf_name, cpu_tensor)`` group by group on every rank (collective call). Ranks not
        in ``host_ranks`` (default: all) take part in the gathers but get ``None`` instead of a host
        copy, so an export in which only rank 0 writes does not convert and copy the model on every rank.

        Only one gathered group is alive at a time, so exporting a 70B model needs one block
        of device memory, not a full replica per rank as the reference's
        ``get_model_state_dict(full_state_dict=True)`` does (train.py:41-42).
        """
        for grp, it in self._hf_iters():
            src = grp.master if source == "master" and not self.symmetric else grp.shard  # peers can only read arena tensors
            if self.world == 1:
                full = src
            else:
                full = torch.empty(grp.layout.padded_numel, dtype=src.dtype, device=self.device)
                self.comm.all_gather(src, full)
            views = grp.layout.views(full)
            to_host = host_ranks is None or self.rank in host_ranks
            for name, view in it(views):
                if isinstance(view, tuple):
                    yield name, (torch.stack([v.to(dtype) for v in view]).cpu() if to_host else None)
                else:
                    yield name, (view.to(dtype).cpu() if to_host else None)
            del full, views

    # ------------------------------------------------------------------------------------
    # gather / reduce plumbing
    # ------------------------------------------------------------------------------------
    def _gather_block(self, i: int, fused: bool = False):
        """Starts gathering block ``i`` on the side stream; returns (views, ready_event, slot).

        ``fused`` (symmetric backend): nothing is launched here; the views carry a gather plan and
        the block's QKV and gate/up GEMMs pull the parameters from the peers while they run."""
        grp = self.blocks[i]
        if self.world == 1:
            return grp.layout.views(grp.shard), None, -1
        slot = i % len(self._pbufs)
        buf = self._pbufs[slot]
        if fused and self.fused_gather:
            _Side.wait(self._pbuf_free[slot])
            if self.poison:
                buf.fill_(float("nan"))
            views = grp.layout.views(buf)
            views["_gather"] = self.comm.gather_plan(grp.shard, buf, grp.layout, split_before="wgu", small_until="wqkv")
            return views, None, slot
        with self.side.run(wait_current=False):
            if self.side.cuda and self._pbuf_free[slot] is not None:
                self.side.stream.wait_event(self._pbuf_free[slot])
            if self.poison:
                buf.fill_(float("nan"))
            self.comm.all_gather(grp.shard, buf)
            ev = self.side.record()
        return grp.layout.views(buf), ev, slot

    def _release_pbuf(self, slot: int):
        if slot >= 0 and self.side.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self._pbuf_free[slot] = ev

    def _gather_group(self, grp: ShardedGroup, prefetch: bool = False):
        """Gathers the embed / head group into a fresh buffer; returns ``(views, buffer, event)``.

        ``prefetch``: the gather runs on the side stream (which first waits for the work already
        queued on the compute stream, so the fresh buffer cannot be written while its memory's
        previous owner is still being read) and the caller waits on ``event`` before the first use.
        Otherwise it runs on the compute stream inside an exposed-communication bracket."""
        if self.world == 1:
            return grp.layout.views(grp.shard), grp.shard, None
        full = torch.empty(grp.layout.padded_numel, dtype=self.param_dtype, device=self.device)
        if self.poison:
            full.fill_(float("nan"))
        if prefetch and self.side.cuda:
            with self.side.run(wait_current=True):
                self.comm.all_gather(grp.shard, full)
                ev = self.side.record()
            full.record_stream(self.side.stream)
            return grp.layout.views(full), full, ev
        self._timed_comm(lambda: self.comm.all_gather(grp.shard, full))
        return grp.layout.views(full), full, None

    # Tensor regions of a block's gradient buffer in the order backward completes them. The layout is
    # ln1 | bqkv | wqkv | wo | ln2 | wgu | wd and backward writes from the back: region k spans from the
    # named tensor to the start of the previous region; the last region is what is left at the front.
    REGION_STARTS = ("wd", "wgu", "wo")

    def _reduce(self, grp: ShardedGroup, gfull: torch.Tensor, slot: int = -1, last: bool = False,
                region: int = 0, elem_lo: int = 0, elem_hi: Optional[int] = None, final: bool = True):
        """Reduce-scatter ``gfull`` (or elements [elem_lo, elem_hi) of it, one tensor region) into the
        group's fp32 accumulator on the side stream.

        With the symmetric backend the compute stream first publishes "this region of my buffer is
        complete" to the peers; the reduction kernel itself waits for the peers' matching signals. On
        the last microbatch of a step that kernel also adds the sum of squares of the finished
        accumulator to the step's norm scalar, so the optimizer does not have to read the accumulator
        again. ``final`` marks the last region of the buffer (bookkeeping of the group and the slot)."""
        if self.symmetric:
            self.comm.grad_ready(gfull, region)
        with self.side.run(wait_current=True):
            if self.world == 1 and hasattr(self.ops, "accumulate"):
                hi = grp.gacc.numel() if elem_hi is None else min(elem_hi, grp.gacc.numel())
                if hi > elem_lo:
                    self.ops.accumulate(grp.gacc[elem_lo:hi], gfull[elem_lo:hi], grp.has_grad)
            elif self.symmetric:
                self.comm.reduce_scatter_accumulate(gfull, grp.gacc, grp.has_grad, sumsq=self._sq if last else None,
                                                    region=region, elem_lo=elem_lo, elem_hi=elem_hi)
                if final:
                    grp.sq_done = last
            else:
                self.comm.reduce_scatter_accumulate(gfull, grp.gacc, grp.has_grad, self._rs_scratch)
            ev = self.side.record()
        if final:
            grp.has_grad = True
            if slot >= 0:
                self._gbuf_free[slot] = ev
        return ev

    def _region_reducer(self, i: int, gbuf: torch.Tensor, gslot: int, last: bool):
        """Returns ``(notify, finish)`` for block ``i``: ``notify(name)`` reduces the region that ends
        where the previous one started as soon as backward has written it; ``finish()`` reduces the
        rest. Backends whose reduction is a collective over the whole buffer (NCCL, gloo) reduce once,
        in ``finish``."""
        osft = getattr(self, "osft", None)
        if osft is not None and osft.owner_reduce:
            return osft.reducer(i, gbuf, gslot, last)
        grp = self.blocks[i]
        per_region = self.region_overlap and (self.symmetric or (self.world == 1 and hasattr(self.ops, "accumulate")))
        state = {"hi": grp.layout.padded_numel, "k": 0}

        def notify(name):
            if not per_region or name not in self.REGION_STARTS:
                return
            lo = grp.layout.specs[name].offset
            with nvtx.range(f"reduce/block{i}/{name}"):
                self._reduce(grp, gbuf, gslot, last, region=state["k"], elem_lo=lo, elem_hi=state["hi"], final=False)
            state["hi"], state["k"] = lo, state["k"] + 1

        def finish():
            with nvtx.range(f"reduce/block{i}"):
                if per_region:
                    self._reduce(grp, gbuf, gslot, last, region=state["k"], elem_lo=0, elem_hi=state["hi"], final=True)
                else:
                    self._reduce(grp, gbuf, gslot, last)

        return notify, finish

    def _grad_buffer(self, i: int):
        slot = i % len(self._gbufs)
        _Side.wait(self._gbuf_free[slot])
        self._gbuf_free[slot] = None
        if self.symmetric:   # the region reduced last (the front of the buffer) covers the earlier ones
            osft = getattr(self, "osft", None)
            if osft is not None and osft.owner_reduce:
                last_region = osft.last_region
            else:
                last_region = len(self.REGION_STARTS) if self.region_overlap else 0
            self._timed_comm(lambda: self.comm.wait_consumed(self._gbufs[slot], last_region))
        if self.poison:   # only the tensors themselves: alignment gaps are never written and must stay zero
            for view in self.blocks[i].layout.views(self._gbufs[slot]).values():
                view.fill_(float("nan"))
        return self._gbufs[slot], slot

    def _root_grad_buffer(self, which: str) -> torch.Tensor:
        """Zeroed full gradient buffer of the embed / head group, once its previous reduction is over."""
        buf = self._eg_full if which == "embed" else self._hg_full
        _Side.wait(self._root_free[which])
        if self.symmetric:
            self._timed_comm(lambda: self.comm.wait_consumed(buf))
        buf.zero_()
        return buf

    # ------------------------------------------------------------------------------------
    # activation checkpointing plan
    # ------------------------------------------------------------------------------------
    def plan_checkpointing(self, tokens: int) -> list:
        """Per-block checkpoint level for a minibatch of ``tokens`` tokens.

        3 = as 2, with the block input parked in pinned host memory (only when even the inputs do not fit);
        2 = keep only the block input and recompute the whole block in backward (what the reference
        does for every block, setup_model_for_training.py:28-29); 1 = also keep the attention
        output and its log-sum-exp so the recompute skips the attention kernel; 0 = keep every GEMM
        output (qkv, attention, h1, gate/up), so backward runs no forward GEMM at all. Blocks are upgraded from the last one backwards (their
        activations are freed first in backward) while the estimated footprint fits in
        ``activation_budget_bytes``. ``activation_budget_bytes = 0`` gives the reference behaviour.
        """
        cfg, nL = self.cfg, len(self.blocks)
        levels = [2] * nL
        budget = self.activation_budget_bytes
        if budget is None:
            budget = self._auto_activation_budget(tokens)
        force = int(os.environ.get("MTB200_OFFLOAD_BLOCKS", "0"))
        if (budget < 0 or force) and self.device.type == "cuda":
            # Not even the block inputs fit next to the optimizer state (a 70B model with a sample far longer
            # than the per-GPU token budget): level 3 parks a block's input in pinned host memory during
            # forward and brings it back one block ahead of its use in backward. The earliest blocks go first:
            # their inputs would stay resident longest.
            per_block = tokens * cfg.hidden_size * (2 if self.param_dtype != torch.float32 else 4)
            n_off = max(force, -(-(-budget) // per_block) if budget < 0 else 0)
            for i in range(min(n_off, nL - 1)):
                levels[i] = 3
        if budget <= 0:
            return levels
        es = 2 if self.param_dtype != torch.float32 else 4
        h, f = cfg.hidden_size, (cfg.expert_intermediate_size if cfg.is_moe else cfg.intermediate_size) * cfg.mlp_rows_factor
        lvl1 = tokens * (cfg.q_size * es + cfg.num_attention_heads * 4)
        # level 0 keeps qkv, the attention output, h1 and gate/up (the normalised inputs and the SwiGLU
        # output are rebuilt in backward by elementwise kernels)
        lvl0 = lvl1 + tokens * ((h + cfg.qkv_size + 2 * f) * es + 8)
        if cfg.post_norm:   # both branch outputs before their norms and the q|k projections before theirs
            lvl0 += tokens * (2 * h + cfg.q_size + cfg.kv_size) * es
        if cfg.qk_norm:   # the q|k heads before their norm and one reciprocal RMS per head
            lvl0 += tokens * ((cfg.q_size + cfg.kv_size) * es + (cfg.num_attention_heads + cfg.num_key_value_heads) * 4)
        for i in range(nL - 1, -1, -1):      # cheapest upgrade first: keep attention everywhere it fits
            if budget >= lvl1:
                levels[i] = 1
                budget -= lvl1
        for i in range(nL - 1, -1, -1):
            if levels[i] == 1 and budget >= lvl0 - lvl1:
                levels[i] = 0
                budget -= lvl0 - lvl1
        return levels

    def _auto_activation_budget(self, tokens: int) -> int:
        """Memory that can hold extra saved activations. Two bounds, the smaller wins:

        * a static plan: 93 % of the device minus optimizer/parameter state, the per-block inputs,
          the working set of one block's backward and the loss buffers;
        * what is actually obtainable right now: free device memory as the driver reports it (this
          sees everything outside the caching allocator too: the symmetric arena's mappings, NCCL's
          buffers, another process) plus the allocator's cached-but-unused blocks, minus the same
          transient needs and a margin. Called at the start of a microbatch, when the previous one's
          activations have been returned to the allocator.
        """
        if self.device.type != "cuda":
            return 0
        cfg = self.cfg
        total = torch.cuda.get_device_properties(self.device).total_memory
        h, v = cfg.hidden_size, cfg.vocab_size
        f = (cfg.expert_intermediate_size if cfg.is_moe else cfg.intermediate_size) * cfg.mlp_rows_factor
        base = tokens * 2 * h * len(self.blocks)
        work = tokens * 2 * (7 * h + cfg.qkv_size + 6 * f)
        ce = getattr(self.ops, "ce_chunk", 2048) * v * 2 + v * h * 4
        root = 4 * v * h * 2
        bufs = sum(b.numel() * b.element_size() for b in self._pbufs + self._gbufs)
        transient = base + work + ce + root
        static = int(0.93 * total - (self.state_bytes() + transient + bufs + (4 << 30)))
        free, _ = torch.cuda.mem_get_info(self.device)
        cached = torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
        live = int(0.97 * (free + cached) - transient - (3 << 30))
        if self._oom_retries:   # an earlier microbatch ran out of memory: plan more cautiously from now on
            live -= self._oom_retries * (8 << 30)
        return min(static, live)

    # ------------------------------------------------------------------------------------
    # one microbatch
    # ------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_backward(self, batch: D.PackedBatch, grad_scale: float, last: bool = False) -> torch.Tensor:
        """Runs forward and backward of one packed minibatch; accumulates gradients.

        ``last`` marks the final minibatch before ``optimizer_step`` (lets the reduction kernels
        fold the gradient-norm partial sums in). Returns the per-token loss vector ``[T]``
        (fp32, on device)."""
        cfg, ops = self.cfg, self.ops
        nL = len(self.blocks)
        tied = cfg.tie_word_embeddings
        win = cfg.attention_window
        if win is not None and batch.max_seqlen > win:
            raise ValueError(f"a sample of {batch.max_seqlen} tokens exceeds the model's sliding window of {win}: attention "
                             "here is full causal attention, which equals the windowed one only up to that length")

        # ---- forward ----
        levels = self.plan_checkpointing(batch.num_tokens)
        try:
            x, saved, last_block, emb_views, head = self._forward(batch, levels)
        except torch.OutOfMemoryError:
            # Forward only pulls parameters and writes activations: nothing has been reduced or signalled
            # yet, so with one-sided gathers (one rank, or the symmetric backend) it can simply run again
            # with every block at the cheapest checkpoint level. Collective gathers cannot be re-issued.
            if not (self.world == 1 or self.symmetric):
                raise
            self._oom_retries += 1
            torch.cuda.empty_cache()
            x, saved, last_block, emb_views, head = self._forward(batch, [2] * nL)

        # ---- head: loss and its gradients in one pass ----
        head_views, head_full, head_ev = head
        _Side.wait(head_ev)
        hg_full = self._root_grad_buffer("head")
        head_g = self.head.layout.views(hg_full)
        nvtx.push("head")
        if tied:
            eg_full = self._root_grad_buffer("embed")
            emb_g = self.embed.layout.views(eg_full)
            loss, dx = D.head_forward_backward(ops, cfg, head_views, head_g, emb_views["embed"], emb_g["embed"], True,
                                               x, batch, grad_scale)
        else:
            loss, dx = D.head_forward_backward(ops, cfg, head_views, head_g, head_views["lm_head"], head_g["lm_head"],
                                               False, x, batch, grad_scale)
        nvtx.pop()
        del x, head_views, head_full, head
        self._root_free["head"] = self._reduce(self.head, hg_full, last=last)

        # ---- backward through the blocks ----
        cur = ({k: v for k, v in last_block[0].items() if k != "_gather"}, None, last_block[1])   # already gathered
        for i in range(nL - 1, -1, -1):
            p, ev, slot = cur
            _Side.wait(ev)
            # a block that will be recomputed gathers inside its recompute GEMMs; one whose activations
            # were all kept has no forward GEMM left, so its parameters are prefetched on the side stream
            cur = self._gather_block(i - 1, fused=saved[i - 1][1] is None) if i > 0 else None
            gbuf, gslot = self._grad_buffer(i)
            g = self.blocks[i].layout.views(gbuf)
            xin, acts, attn_state = saved.pop()
            if isinstance(xin, _HostInput):
                xin = self._fetch_input(i, xin)
            if i > 0 and isinstance(saved[i - 1][0], _HostInput):   # the next block's input travels while this block computes
                self._prefetch_input(i - 1, saved[i - 1][0])
            if acts is None:   # recompute the block forward (attention is skipped when its output was kept)
                with nvtx.range(f"recompute/block{i}"):
                    _, acts, _ = D.block_forward(ops, cfg, p, xin, batch, self._inv_freq(i, batch), keep=True, saved_attn=attn_state,
                                                 need_out=False)
            notify, finish = self._region_reducer(i, gbuf, gslot, last)
            with nvtx.range(f"backward/block{i}"):
                dx = D.block_backward(ops, cfg, p, g, acts, dx, batch, self._inv_freq(i, batch), notify=notify)
            del acts, xin, attn_state
            self._release_input()
            self._release_pbuf(slot)
            finish()

        # ---- embedding ----
        if not tied:
            eg_full = self._root_grad_buffer("embed")
            emb_g = self.embed.layout.views(eg_full)
        if cfg.embedding_multiplier != 1.0:
            dx.mul_(cfg.embed_scale(dx.dtype))
        ops.embedding_bwd(emb_g["embed"], batch.input_ids, dx)
        self._root_free["embed"] = self._reduce(self.embed, eg_full, last=last)
        return loss

    # ------------------------------------------------------------------------------------
    # block inputs parked in host memory (checkpoint level 3)
    # ------------------------------------------------------------------------------------
    def reserve_host_offload(self, tokens: int) -> int:
        """Allocates, ahead of training, the pinned host buffers a minibatch of ``tokens`` tokens would park
        its block inputs in (call it with the longest sample of the dataset, or the per-GPU token budget if
        that is larger). Page-locking tens of gigabytes takes tens of seconds; done lazily it would stall
        one rank in the middle of a step while every peer waits for it. Returns the number of blocks reserved."""
        if self.device.type != "cuda":
            return 0
        levels = self.plan_checkpointing(tokens)
        n = 0
        for i, lv in enumerate(levels):
            if lv == 3:
                need = tokens * self.cfg.hidden_size
                host = self._host_inputs.get(i)
                if host is None or host.numel() < need:
                    self._host_inputs[i] = torch.empty(need, dtype=self.param_dtype, pin_memory=True)
                n += 1
        return n

    def _offload_input(self, i: int, x: torch.Tensor) -> "_HostInput":
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        host = self._host_inputs.get(i)
        if host is None or host.numel() < x.numel():
            host = torch.empty(x.numel(), dtype=x.dtype, pin_memory=True)
            self._host_inputs[i] = host
        cur = torch.cuda.current_stream()
        self._copy_stream.wait_stream(cur)          # the block that reads x has been queued; x itself is complete
        with torch.cuda.stream(self._copy_stream):
            host[: x.numel()].view(x.shape).copy_(x, non_blocking=True)
        x.record_stream(self._copy_stream)          # its memory is not reused before the copy has read it
        return _HostInput(host, tuple(x.shape))

    def _prefetch_input(self, i: int, h: "_HostInput") -> None:
        if h.device is not None:
            return
        slot = i % 2
        n = 1
        for d in h.shape:
            n *= d
        buf = self._dev_inputs[slot]
        if buf is None or buf.numel() < n:
            if buf is not None:
                buf.record_stream(self._copy_stream)
            buf = torch.empty(n, dtype=h.host.dtype, device=self.device)
            self._dev_inputs[slot] = buf
            self._dev_input_free[slot] = None    # fresh memory: order the copy after everything queued so far
        if self._dev_input_free[slot] is not None:   # the block that last used this staging buffer has finished
            self._copy_stream.wait_event(self._dev_input_free[slot])
        else:
            self._copy_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._copy_stream):
            dev = buf[:n].view(h.shape)
            dev.copy_(h.host[:n].view(h.shape), non_blocking=True)
            h.ready = torch.cuda.Event()
            h.ready.record(self._copy_stream)
        h.device, h.slot = dev, slot

    def _fetch_input(self, i: int, h: "_HostInput") -> torch.Tensor:
        self._prefetch_input(i, h)
        _Side.wait(h.ready)      # counted as exposed time when the copy is late
        self._pending_input_slot = h.slot
        return h.device

    def _release_input(self) -> None:
        """Called after a block's backward has been queued: its staged input may be overwritten afterwards."""
        slot = self._pending_input_slot
        if slot is not None:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self._dev_input_free[slot] = ev
            self._pending_input_slot = None

    def _forward(self, batch: D.PackedBatch, levels: list):
        """Forward through the embedding and the blocks; returns the last hidden state, what each
        block kept for backward, the still-gathered last block, the embedding views (tied head) and
        the head group's ``(views, buffer, ready event)``."""
        cfg, ops = self.cfg, self.ops
        nL = len(self.blocks)
        emb_views, emb_full, _ = self._gather_group(self.embed)
        x = ops.embedding(emb_views["embed"], batch.input_ids)
        if cfg.embedding_multiplier != 1.0:   # Granite, Gemma
            x.mul_(cfg.embed_scale(x.dtype))
        if not cfg.tie_word_embeddings:
            emb_views = None
        del emb_full
        saved = []
        nxt = self._gather_block(0, fused=True)
        last_block = None
        head = None
        for i in range(nL):
            p, ev, slot = nxt
            _Side.wait(ev)
            nxt = self._gather_block(i + 1, fused=True) if i + 1 < nL else None
            if i == nL - 1:   # the head's parameters arrive while the last block computes
                head = self._gather_group(self.head, prefetch=True)
            xin = x
            with nvtx.range(f"forward/block{i}"):
                x, acts, attn_state = D.block_forward(ops, cfg, p, x, batch, self._inv_freq(i, batch),
                                                      keep="compact" if levels[i] == 0 else False, want_attn=levels[i] == 1)
            if levels[i] == 3:
                xin = self._offload_input(i, xin)
            saved.append((xin, acts, attn_state))
            if i + 1 < nL or self.world == 1:
                self._release_pbuf(slot)
            last_block = (p, slot)  # the last block stays gathered for backward (reshard_after_forward=False)
        return x, saved, last_block, emb_views, head

    # ------------------------------------------------------------------------------------
    # optimizer
    # ------------------------------------------------------------------------------------
    @torch.no_grad()
    def optimizer_step(self, lr: float) -> torch.Tensor:
        """Global-norm clip + AdamW on the shards. Returns the pre-clip gradient norm (0-dim)."""
        with nvtx.range("optimizer"):
            return self._optimizer_step(lr)

    def _optimizer_step(self, lr: float) -> torch.Tensor:
        if self.side.cuda:
            _Side.wait(self.side.record())   # the last reductions must have landed
        o = self.optim
        live = [g for g in self.groups if g.has_grad]
        sq = self._sq
        for g in live:
            if not g.sq_done:
                sq += self.ops.sumsq(g.gacc)
        self.comm.all_reduce_sum(sq)
        norm = sq.sqrt().squeeze(0)
        if o.max_grad_norm and o.max_grad_norm > 0:
            coef = torch.clamp(o.max_grad_norm / (norm + 1e-6), max=1.0)
        else:
            coef = torch.ones((), dtype=torch.float32, device=self.device)
        self.step_count += 1
        for g in live:
            self.ops.adamw_step(g.master, g.m, g.v, g.gacc, g.shard, lr, o.beta1, o.beta2, o.eps, o.weight_decay,
                                self.step_count, coef)
            g.has_grad = False
            g.sq_done = False
        self._sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        if self.symmetric:   # no peer may pull a shard before every rank has finished updating its own
            self._timed_comm(self.comm.barrier)
        if self.side.cuda:
            self.side.stream.wait_stream(torch.cuda.current_stream())
        return norm

    def measure_exposed_comm(self, on: bool = True) -> None:
        """Starts (or stops) recording how long the compute stream waits for communication: gathers
        that are not ready, gradient buffers still being reduced, peers' "consumed" signals, the
        reductions still running when the optimizer starts and the post-step barrier."""
        _Side.stalls = [] if on else None

    def exposed_comm_ms(self) -> dict:
        """Exposed communication since the last call, in milliseconds (synchronises the device; clears
        the record): ``stream_ms`` is the sum of the recorded compute-stream stalls, ``in_kernel_ms``
        the time the fused all-gather GEMMs' TMA producers spent waiting for weight chunks that had
        not arrived yet (mean over the CTAs of each launch, summed over launches)."""
        if _Side.stalls is None:
            return {"stream_ms": 0.0, "in_kernel_ms": 0.0}
        torch.cuda.synchronize(self.device)
        total = sum(a.elapsed_time(b) for a, b in _Side.stalls)
        _Side.stalls = []
        in_kernel = self.comm.take_gather_wait_ms() if hasattr(self.comm, "take_gather_wait_ms") else 0.0
        return {"stream_ms": total, "in_kernel_ms": in_kernel}

    def _timed_comm(self, fn):
        """Runs a device-side wait (a kernel that polls peers' flags) inside a stall bracket."""
        if _Side.stalls is None:
            return fn()
        cur = torch.cuda.current_stream()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(cur)
        fn()
        e1.record(cur)
        _Side.stalls.append((e0, e1))

    def zero_grad(self) -> None:
        for g in self.groups:
            g.has_grad = False
            g.sq_done = False
        self._sq.zero_()

    # ------------------------------------------------------------------------------------
    # convenience: a full training step over this rank's minibatches
    # ------------------------------------------------------------------------------------
    def train_step(self, minibatches: list, lr: float) -> dict:
        """``minibatches``: collated dicts (``data.sampler.mb_collate_fn``). One optimizer step.

        Device work is queued without host synchronisation; the returned tensors
        (``loss_sum``, ``grad_norm``) are read by the caller when it logs.
        """
        loss_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        ntok = h2d = 0
        for k, mb in enumerate(minibatches):
            batch = D.make_packed_batch(mb, self.device)
            h2d += batch.h2d_bytes
            denom = float(mb["batch_num_loss_counted_tokens"]) or 1.0
            loss = self.forward_backward(batch, 1.0 / denom, last=k == len(minibatches) - 1)
            loss_sum += loss.sum()
            ntok += batch.num_tokens
        gnorm = self.optimizer_step(lr)
        return {"loss_sum": loss_sum, "grad_norm": gnorm, "num_tokens": ntok, "h2d_bytes": h2d}

    def state_bytes(self) -> int:
        return sum(g.state_bytes() for g in self.groups)


def plan_state_dtype(cfg: ModelConfig, world: int, hbm_bytes: float, tokens: int) -> torch.dtype:
    """fp32 moments when they fit comfortably next to activations, else bf16.

    Per-parameter bytes on a rank: 2 (working) + 4 (master) + 4 (grad accumulator) + 2x moment.
    """
    p = cfg.param_count() / world
    act = tokens * cfg.hidden_size * 2 * (cfg.num_hidden_layers + 24) + tokens * cfg.intermediate_size * 2 * 8
    fixed = p * 10 + act + 3 * cfg.block_param_count() * 2 * (world > 1) + 6e9
    return torch.float32 if fixed + p * 8 < 0.85 * hbm_bytes else torch.bfloat16
