"""Single-node NVLink/NVSwitch communication backend over symmetric memory.

Every rank allocates one arena with ``torch.distributed._symmetric_memory`` (CUDA VMM allocation
whose handle is exchanged through the process group's store) and maps all peers' arenas. The
engine places parameter shards, gradient buffers and flag words in the arena; the hand-written
kernels in ``csrc/symm_comm.cu`` then move data with peer loads — there is no NCCL call in
``all_gather`` / ``reduce_scatter_accumulate`` / ``all_reduce_sum`` / ``barrier``.
NCCL (through ``torch.distributed``) is only used once, for the rendezvous.

Protocol (epochs are per-channel counters that advance identically on all ranks, because all
ranks execute the same sequence of collectives):

* ``grad_ready(buf)``      my gradient buffer (or one tensor region of it) is complete
                                                                  -> ``ready[ch][me] = epoch`` on all peers
* ``reduce_scatter_...``   waits ``ready[ch][p] >= epoch`` for all p, reads, then
                           ``consumed[ch][me] = epoch`` on all peers
* ``wait_consumed(buf)``   before overwriting my buffer: ``consumed[ch][p] >= last epoch`` for all p
* ``barrier()``            signal + wait on a dedicated channel (after the optimizer step, so that
                           no peer pulls a half-updated shard)

All device-side waits are bounded (``flag_spin_limit`` = time limit in microseconds, default three minutes:
long enough for the skew an over-length sample causes at 70B scale; ``MTB200_FLAG_TIMEOUT_US`` overrides);
an expired wait records a code in ``status`` which ``check_status()`` turns into an exception on the host.
"""
from __future__ import annotations

import ctypes
import os

# By default the arena is only accessed with plain peer loads/stores and is NOT bound to an NVLink
# multicast object: a rank that dies while its memory is bound to one can fault its peers' GPUs.
# MTB200_NVLS=1 opts in: the arena is bound, and the gradient reduce-scatter sums inside the switch
# (multimem.ld_reduce) instead of pulling every peer's copy. Failure-path tests never set it.
NVLS_REQUESTED = os.environ.get("MTB200_NVLS", "0") == "1"
if not NVLS_REQUESTED:
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

from ctypes import c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import torch
import torch.distributed as dist

from ..ops.native import load_library

MAX_CHANNELS = 64
MAX_RANKS = 16
_ALIGN = 256


class SymmetricComm:
    name = "symmetric"
    fused_sumsq = True

    def __init__(self, device, group=None, flag_spin_limit: int | None = None):
        self.device = torch.device(device)
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > MAX_RANKS:
            raise ValueError(f"symmetric backend supports up to {MAX_RANKS} ranks on one node")
        self.lib = load_library()
        self._bind()
        self.flag_spin_limit = int(flag_spin_limit or os.environ.get("MTB200_FLAG_TIMEOUT_US", 0))   # 0 = the library default
        self.arena = None
        self._off = 0
        self._chan = {}
        self._epoch = [0] * MAX_CHANNELS
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0
        self.nvls, self.mc_ptr = False, 0
        self._regions = []

    def _bind(self):
        P, I, L, U, UL = c_void_p, c_int, c_longlong, c_uint, c_ulonglong
        sig = {
            "mtb200_symm_allgather": [P, I, UL, UL, P, UL, UL, I, P],
            "mtb200_gemm_bf16_allgather": [P, L, P, L, P, I, I, I, P, I, UL, UL, P, UL, P, U, I, I, P, P, I, P, P],
            "mtb200_symm_signal": [P, I, I, UL, U, P],
            "mtb200_symm_wait": [P, I, U, U, I, P, P],
            "mtb200_symm_reduce_scatter": [P, I, I, UL, L, L, P, I, P, P, UL, U, U, P, P, I, P],
            "mtb200_symm_allreduce_scalar": [P, I, I, UL, UL, P, P, U, U, P, P, P],
            "mtb200_symm_pull": [P, I, I, UL, P, UL, I, P],
            "mtb200_gemm_bf16_reduce_a": [P, P, L, P, L, P, L, I, I, I, P, I, I, UL, P, U, P, P, P, UL, U, U, P, P],
            "mtb200_symm_reduce_scatter_nvls": [UL, P, I, I, UL, L, L, P, I, P, P, UL, U, U, P, P, I, P],
        }
        for name, args in sig.items():
            fn = getattr(self.lib, name)
            fn.restype = c_int
            fn.argtypes = args

    # -- arena ------------------------------------------------------------------------
    def setup(self, payload_bytes: int) -> None:
        """Allocates and rendezvouses the arena: ``payload_bytes`` for engine buffers + flag words."""
        import torch.distributed._symmetric_memory as symm_mem
        flag_bytes = MAX_CHANNELS * 3 * MAX_RANKS * 4 + 4096
        total = -(-(payload_bytes + flag_bytes + 64 * _ALIGN) // 4096) * 4096
        gname = self.group.group_name
        try:
            symm_mem.enable_symm_mem_for_group(gname)
        except Exception:
            pass
        self.arena = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.arena.zero_()
        self.handle = symm_mem.rendezvous(self.arena, gname)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._bases = (c_ulonglong * self.world)(*ptrs)
        assert ptrs[self.rank] == self.arena.data_ptr()
        # multicast address of the arena: non-zero only when binding was requested and the fabric supports it
        self.mc_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0) if NVLS_REQUESTED else 0
        self.nvls = self.mc_ptr != 0
        self._off = 0
        # flag rows: ready[ch][r], consumed[ch][r] (uint32) and vals[ch][r] (fp32 payload for scalar all-reduce)
        self._flags = self.alloc(MAX_CHANNELS * 3 * MAX_RANKS, torch.int32)
        self._counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._ticket = torch.zeros(1, dtype=torch.int32, device=self.device)       # chunk tickets of the fused gather
        self._gather_wait = torch.zeros(2, dtype=torch.int64, device=self.device)  # producer wait (ns) summed over CTAs, CTA count
        self._gather_launches = 0
        # the fused reduce + GEMM runs on the side stream next to gathering GEMMs of the compute stream: words of its own
        self._red_words = torch.zeros(2, dtype=torch.int32, device=self.device)    # chunk ticket, CTA counter
        self._barrier_ch = self._new_channel("barrier")
        self._scalar_ch = [self._new_channel("scalar0"), self._new_channel("scalar1")]
        self._scalar_calls = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)   # every arena is zeroed before anyone signals

    def alloc(self, numel: int, dtype) -> torch.Tensor:
        es = torch.empty(0, dtype=dtype).element_size()
        nbytes = numel * es
        start = -(-self._off // _ALIGN) * _ALIGN
        if self.arena is None or start + nbytes > self.arena.numel():
            raise RuntimeError("symmetric arena exhausted")
        self._off = start + nbytes
        return self.arena[start:start + nbytes].view(dtype)

    def alloc_region(self, numel: int, dtype) -> torch.Tensor:
        """A symmetric buffer of its own (same size on every rank, rendezvoused like the arena) for state
        that is sized after the engine has laid out the arena, e.g. the OSFT staging of recomposed
        matrices. Collective. Peers read it with ``pull``."""
        import torch.distributed._symmetric_memory as symm_mem
        es = torch.empty(0, dtype=dtype).element_size()
        nbytes = -(-max(1, numel) * es // 4096) * 4096
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        buf.zero_()
        handle = symm_mem.rendezvous(buf, self.group.group_name)
        bases = (c_ulonglong * self.world)(*[int(p) for p in handle.buffer_ptrs])
        self._regions.append((buf, handle, bases))
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        return buf[: numel * es].view(dtype)

    def _locate(self, t: torch.Tensor):
        """(peer base table, byte offset) of a tensor living in the arena or in one of the extra regions."""
        p = t.data_ptr()
        if self.arena is not None and 0 <= p - self.arena.data_ptr() < self.arena.numel():
            return self._bases, p - self.arena.data_ptr()
        for buf, _, bases in self._regions:
            if 0 <= p - buf.data_ptr() < buf.numel():
                return bases, p - buf.data_ptr()
        raise ValueError("tensor does not live in symmetric memory")

    def _offset(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.arena.data_ptr()
        if off < 0 or off >= self.arena.numel():
            raise ValueError("tensor does not live in the symmetric arena")
        return off

    def _new_channel(self, key) -> int:
        ch = len(self._chan)
        if ch >= MAX_CHANNELS:
            raise RuntimeError("out of flag channels")
        self._chan[key] = ch
        return ch

    def _channel(self, t: torch.Tensor, region: int = 0) -> int:
        """Flag channel of (buffer, region). A block's gradient buffer is reduced region by region as
        backward completes its tensors; each region has its own ready / consumed epochs."""
        key = (t.data_ptr(), region)
        ch = self._chan.get(key)
        return self._new_channel(key) if ch is None else ch

    def _ready_off(self, ch):
        return self._offset(self._flags) + (ch * 3 + 0) * MAX_RANKS * 4

    def _consumed_off(self, ch):
        return self._offset(self._flags) + (ch * 3 + 1) * MAX_RANKS * 4

    def _vals_off(self, ch):
        return self._offset(self._flags) + (ch * 3 + 2) * MAX_RANKS * 4

    def _st(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def _call(self, name, *args):
        rc = getattr(self.lib, name)(*args)
        if rc != 0:
            raise RuntimeError(f"{name} failed with code {rc}")
        self.launches += 1

    # -- collectives ------------------------------------------------------------------
    def all_gather(self, shard, full, blocks: int = 296, byte_lo: int = 0, byte_hi: int = 0):
        """Pulls every rank's shard into ``full`` (optionally only bytes [byte_lo, byte_hi) of it)."""
        self._call("mtb200_symm_allgather", self._bases, self.world, self._offset(shard),
                   shard.numel() * shard.element_size(), full.data_ptr(), byte_lo, byte_hi, blocks, self._st())

    def gather_plan(self, shard, full, layout, split_before: str, small_until: str):
        """Plan for gathering one parameter group INSIDE its consuming GEMMs (see ``GatherPlan``)."""
        return GatherPlan(self, shard, full, layout, split_before, small_until)

    def grad_ready(self, gfull, region: int = 0):
        ch = self._channel(gfull, region)
        self._epoch[ch] += 1
        self._call("mtb200_symm_signal", self._bases, self.world, self.rank, self._ready_off(ch), self._epoch[ch], self._st())

    def reduce_scatter_accumulate(self, gfull, acc, accumulate: bool, scratch=None, sumsq=None, blocks: int = 296,
                                  region: int = 0, elem_lo: int = 0, elem_hi: int | None = None):
        """acc (+)= sum over ranks of this rank's slice of ``gfull``. With ``elem_lo`` / ``elem_hi`` only the
        part of the slice inside elements [elem_lo, elem_hi) of the buffer is reduced (one tensor region;
        possibly empty for this rank, which then only takes part in the handshake)."""
        ch = self._channel(gfull, region)
        base = self.arena.data_ptr()
        s = acc.numel()
        lo = max(self.rank * s, elem_lo)
        hi = min((self.rank + 1) * s, gfull.numel() if elem_hi is None else elem_hi)
        n = max(0, hi - lo)
        acc_ptr = acc.data_ptr() + (lo - self.rank * s) * 4 if n else acc.data_ptr()
        if self.nvls:   # sum formed inside NVSwitch
            self._call("mtb200_symm_reduce_scatter_nvls", self.mc_ptr, self._bases, self.world, self.rank, self._offset(gfull),
                       lo if n else 0, n, acc_ptr, int(accumulate), None if sumsq is None else sumsq.data_ptr(),
                       base + self._ready_off(ch), self._consumed_off(ch), self._epoch[ch], self.flag_spin_limit,
                       self._counter.data_ptr(), self.status.data_ptr(), blocks, self._st())
            return
        self._call("mtb200_symm_reduce_scatter", self._bases, self.world, self.rank, self._offset(gfull), lo if n else 0, n,
                   acc_ptr, int(accumulate), None if sumsq is None else sumsq.data_ptr(),
                   base + self._ready_off(ch), self._consumed_off(ch), self._epoch[ch], self.flag_spin_limit,
                   self._counter.data_ptr(), self.status.data_ptr(), blocks, self._st())

    def reduce_to_owner(self, gfull, acc, accumulate: bool, owner: int, elem_lo: int, elem_hi: int, region: int,
                        sumsq=None, blocks: int = 296):
        """Sum of elements [elem_lo, elem_hi) of every rank's ``gfull``, delivered to rank ``owner`` only
        (``acc`` fp32, ``elem_hi - elem_lo`` elements there; ignored elsewhere): the reduce-scatter kernel
        with ownership by tensor instead of by flat slice. Every rank takes part in the handshake."""
        ch = self._channel(gfull, region)
        mine = self.rank == owner
        n = (elem_hi - elem_lo) if mine else 0
        fn = "mtb200_symm_reduce_scatter_nvls" if self.nvls else "mtb200_symm_reduce_scatter"
        args = (self._bases, self.world, self.rank, self._offset(gfull), elem_lo if mine else 0, n,
                acc.data_ptr() if mine else None, int(accumulate), None if (sumsq is None or not mine) else sumsq.data_ptr(),
                self.arena.data_ptr() + self._ready_off(ch), self._consumed_off(ch), self._epoch[ch], self.flag_spin_limit,
                self._counter.data_ptr(), self.status.data_ptr(), blocks, self._st())
        self._call(fn, *(((self.mc_ptr,) + args) if self.nvls else args))

    def reduce_gemm_to_owner(self, ops, gfull, owner: int, elem_lo: int, rows: int, cols: int, region: int, staged, b16, out32,
                             accumulate: bool, flags, epoch: int):
        """Fused gradient reduction + GEMM on rank ``owner``: ``out32 (+)= (sum over ranks of G) @ b16.T`` where ``G`` is
        the ``[rows, cols]`` tensor at element ``elem_lo`` of every rank's ``gfull``. The kernel's gather warps pull the
        region from all ranks, sum in fp32 and leave the reduced bf16 gradient in ``staged`` (the GEMM's A operand,
        consumed as its chunks complete; it stays valid afterwards for further products). The other ranks only take part
        in the ready / consumed handshake."""
        ch = self._channel(gfull, region)
        if self.rank != owner:
            self._call("mtb200_symm_reduce_scatter", self._bases, self.world, self.rank, self._offset(gfull), 0, 0, None, 0, None,
                       self.arena.data_ptr() + self._ready_off(ch), self._consumed_off(ch), self._epoch[ch], self.flag_spin_limit,
                       self._counter.data_ptr(), self.status.data_ptr(), 1, self._st())
            return
        n = out32.shape[1]
        rc = self.lib.mtb200_gemm_bf16_reduce_a(
            staged.data_ptr(), b16.data_ptr(), b16.stride(0), out32.data_ptr(), out32.stride(0),
            out32.data_ptr() if accumulate else None, out32.stride(0), rows, n, cols, self._bases, self.world, self.rank,
            self._offset(gfull) + elem_lo * 2, flags.data_ptr(), epoch, self._red_words.data_ptr(), self._red_words.data_ptr() + 4,
            self.arena.data_ptr() + self._ready_off(ch), self._consumed_off(ch), self._epoch[ch], self.flag_spin_limit,
            ops.status.data_ptr(), ops._st())
        if rc != 0:
            raise RuntimeError(f"mtb200_gemm_bf16_reduce_a failed with code {rc}")
        ops.launches += 1
        self.launches += 1

    def pull(self, owner: int, src: torch.Tensor, src_elem_off: int, dst: torch.Tensor, blocks: int = 64):
        """``dst[:] = owner's copy of src[src_elem_off : src_elem_off + dst.numel()]``. ``src`` is this rank's
        view of a tensor that every rank allocated at the same arena offset. Order it after the owner's
        writes with ``barrier()``."""
        es = src.element_size()
        assert dst.dtype == src.dtype and dst.is_contiguous()
        bases, off = self._locate(src)
        self._call("mtb200_symm_pull", bases, self.world, owner, off + src_elem_off * es, dst.data_ptr(),
                   dst.numel() * es, blocks, self._st())

    def wait_consumed(self, gfull, region: int = 0):
        """Blocks the stream until every peer has finished reading ``region`` of my buffer. Every peer
        reduces the regions of a buffer in the same order on one stream, so waiting for the region
        that is reduced last covers the earlier ones."""
        ch = self._channel(gfull, region)
        if self._epoch[ch] == 0:
            return
        self._call("mtb200_symm_wait", self.arena.data_ptr() + self._consumed_off(ch), self.world, self._epoch[ch],
                   self.flag_spin_limit, 42, self.status.data_ptr(), self._st())

    def barrier(self):
        ch = self._barrier_ch
        self._epoch[ch] += 1
        self._call("mtb200_symm_signal", self._bases, self.world, self.rank, self._ready_off(ch), self._epoch[ch], self._st())
        self._call("mtb200_symm_wait", self.arena.data_ptr() + self._ready_off(ch), self.world, self._epoch[ch],
                   self.flag_spin_limit, 43, self.status.data_ptr(), self._st())

    def all_reduce_sum(self, vec):
        """Sum of a 1-element fp32 tensor over ranks (the gradient-norm scalar), in rank order."""
        assert vec.numel() == 1 and vec.dtype == torch.float32
        ch = self._scalar_ch[self._scalar_calls & 1]   # alternate rows so a fast peer cannot overwrite an unread value
        self._scalar_calls += 1
        self._epoch[ch] += 1
        self._call("mtb200_symm_allreduce_scalar", self._bases, self.world, self.rank, self._vals_off(ch), self._ready_off(ch),
                   self.arena.data_ptr() + self._vals_off(ch), self.arena.data_ptr() + self._ready_off(ch), self._epoch[ch],
                   self.flag_spin_limit, vec.data_ptr(), self.status.data_ptr(), self._st())
        return vec

    def take_gather_wait_ms(self) -> float:
        """Time the TMA producers of the fused all-gather GEMMs spent waiting for weight chunks since
        the last call: mean over the CTAs of each launch, summed over launches (one host sync)."""
        ns, ctas = (int(x) for x in self._gather_wait.tolist())
        launches = self._gather_launches
        self._gather_wait.zero_()
        self._gather_launches = 0
        if not ctas or not launches:
            return 0.0
        return ns / (ctas / launches) / 1e6

    def check_status(self):
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise RuntimeError(f"symmetric comm: a bounded wait on a peer expired (code {code & 0xff}, peer {code >> 8})")


GATHER_CHUNK_BYTES = 128 * 1024


class GatherPlan:
    """All-gather of one parameter group fused into the GEMMs that first read it.

    The group's full buffer is cut into 128 KB chunks. Launch ``stage 0`` (the QKV projection)
    gathers the chunks up to the tensor named ``split_before`` while it multiplies; ``stage 1``
    (the gate/up projection) gathers the rest. Inside each launch, eight extra warps pull the chunks
    from the peers and flag them; one more warp polls the flags of the chunks under each weight tile
    (all of a tile's flags in parallel) and tells the GEMM's TMA producer how many tiles are ready. The few parameters needed BEFORE the first GEMM (the input norm weight and
    the q/k/v bias, laid out first in the buffer) are pulled by a tiny separate copy.
    """

    _state = {}   # per full buffer: (flags tensor, epoch)

    def __init__(self, comm, shard, full, layout, split_before, small_until):
        self.comm, self.shard, self.full, self.layout = comm, shard, full, layout
        es = full.element_size()
        total = full.numel() * es
        self.n_chunks = -(-total // GATHER_CHUNK_BYTES)
        self.split = min(self.n_chunks, -(-(layout.specs[split_before].offset * es) // GATHER_CHUNK_BYTES))
        self.small_bytes = -(-(layout.specs[small_until].offset * es) // 16) * 16
        key = full.data_ptr()
        st = GatherPlan._state.get(key)
        if st is None or st[0].numel() != self.n_chunks:
            st = [torch.zeros(self.n_chunks, dtype=torch.int32, device=full.device), 0]
            GatherPlan._state[key] = st
        st[1] += 1
        self.flags, self.epoch = st[0], st[1]

    def prefetch_small(self):
        if self.small_bytes:
            self.comm.all_gather(self.shard, self.full, blocks=1, byte_lo=0, byte_hi=self.small_bytes)

    def launch(self, ops, x, w, bias, out, stage: int):
        c = self.comm
        lo, hi = (0, self.split) if stage == 0 else (self.split, self.n_chunks)
        M, K = x.shape
        N = w.shape[0]
        rc = c.lib.mtb200_gemm_bf16_allgather(
            x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), None if bias is None else bias.data_ptr(), M, N, K,
            c._bases, c.world, c._offset(self.shard), self.shard.numel() * self.shard.element_size(), self.full.data_ptr(),
            w.data_ptr() - self.full.data_ptr(), self.flags.data_ptr(), self.epoch, lo, hi, c._ticket.data_ptr(),
            c._gather_wait.data_ptr(), int(getattr(ops, "use_gemm2", False) and M >= 4096), ops.status.data_ptr(), ops._st())
        if rc != 0:
            raise RuntimeError(f"mtb200_gemm_bf16_allgather failed with code {rc}")
        ops.launches += 1
        c.launches += 1
        c._gather_launches += 1
        return out
