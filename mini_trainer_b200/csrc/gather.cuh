// In-kernel all-gather shared by the one-CTA and the two-CTA GEMM: while the tensor cores work, eight
// extra warps per CTA pull this parameter group's shards from every peer's symmetric arena (plain
// peer loads over NVLink, no multicast of any kind) into the local full buffer that the B tensor map
// points at, 128 KB chunk by chunk, and publish each finished chunk in a flag array. One more warp
// (the flag checker) polls the flags of the chunks under each of the CTA's B tiles, one lane per
// chunk, and publishes a tile count in shared memory; the TMA producer loads a B tile only once that
// count covers it, then fences the async proxy (the chunk was written with ordinary stores).
//
// Chunks are handed out by a global ticket counter, not by blockIdx: whichever CTAs are resident
// pull the next chunk, so the transfer makes progress even while some CTAs of the grid are still
// waiting for an SM (another kernel of a side stream may occupy it). Every wait is bounded.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "flags.cuh"
#include "ptx.cuh"

namespace mtb {

constexpr int GATHER_THREADS = 256;
constexpr int GATHER_EXTRA_THREADS = GATHER_THREADS + 32;   // gather warps + one flag-checker warp
constexpr int GATHER_UNROLL = 8;     // 16-byte peer loads in flight per gather thread
constexpr int GATHER_CHUNK_BYTES = 128 * 1024;
constexpr int GATHER_MAX_RANKS = 16;

struct GatherParams {
  unsigned long long peer_base[GATHER_MAX_RANKS];  // every rank's arena, as mapped here
  unsigned long long shard_off;    // byte offset of this group's shard inside each arena
  unsigned long long shard_bytes;  // bytes per rank
  unsigned char* dst;              // local full buffer (world * shard_bytes)
  unsigned int* flags;             // [n_chunks] epoch per chunk, local
  unsigned int* ticket;            // chunk ticket counter, zeroed by the host before the launch
  unsigned long long* wait_ns;     // [2]: summed producer wait (ns) over CTAs and launches, CTA count
  unsigned int epoch;
  int world;
  int chunk_lo, chunk_hi;          // chunks this launch gathers
  int chunk_first;                 // gather order starts here (the chunks under B), wraps inside [lo, hi)
  unsigned long long b_byte_off;   // byte offset of the gathered GEMM operand's first element inside dst
  // ---- reduce mode (the gathered operand is the SUM over ranks of a region of their gradient buffers) ----
  unsigned long long src_off;      // byte offset of the region inside every rank's arena
  unsigned long long total_bytes;  // bytes of the region (= bytes of dst)
  const unsigned int* ready_flags; // local row of "my buffer is complete" epochs, one per rank
  unsigned long long consumed_off; // byte offset of the "consumed" row inside every rank's arena
  unsigned int* done;              // counter of CTAs whose gather warps have finished (zeroed by the host)
  unsigned int rs_epoch;           // epoch of the ready / consumed handshake
  unsigned int limit_us;           // bound of the wait for the peers' ready flags
  int rank;
  int* status;
};

__device__ __forceinline__ uint32_t ld_acquire_cta_shared(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_cta_shared(uint32_t* p, uint32_t v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const unsigned int* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Body of the eight gather warps. `gt` = thread index inside the gather group (0..255), `slot` a
// shared-memory word used to broadcast the ticket. Uses named barrier 1.
__device__ __forceinline__ void gather_chunks(const GatherParams& g, int gt, uint32_t* slot) {
  const int n_chunks = g.chunk_hi - g.chunk_lo;
  const unsigned long long total = g.shard_bytes * g.world;
  const unsigned long long vec_per_shard = g.shard_bytes >> 4;
  while (true) {
    if (gt == 0) *slot = atomicAdd(g.ticket, 1u);
    asm volatile("bar.sync 1, %0;" ::"n"(GATHER_THREADS) : "memory");
    const uint32_t k = *slot;
    asm volatile("bar.sync 1, %0;" ::"n"(GATHER_THREADS) : "memory");   // everyone has read the slot before it is rewritten
    if (k >= static_cast<uint32_t>(n_chunks)) break;
    int c = g.chunk_first + static_cast<int>(k);
    if (c >= g.chunk_hi) c -= n_chunks;
    const unsigned long long b0 = static_cast<unsigned long long>(c) * GATHER_CHUNK_BYTES;
    const unsigned long long b1 = min(b0 + GATHER_CHUNK_BYTES, total);
    const unsigned long long v0 = b0 >> 4, nv = (b1 - b0) >> 4;
    uint4* dst = reinterpret_cast<uint4*>(g.dst) + v0;
    // a chunk lies in one peer's shard, or straddles one boundary (shards are larger than a chunk);
    // the peer is resolved once per chunk, not per vector
    const unsigned long long pr0 = v0 / vec_per_shard;
    if (pr0 >= static_cast<unsigned long long>(g.world)) break;   // a chunk beyond the last shard: never dereference a peer that does not exist
    const unsigned long long first = min(nv, (pr0 + 1) * vec_per_shard - v0);   // vectors that belong to peer pr0
    const uint4* src0 = reinterpret_cast<const uint4*>(g.peer_base[pr0] + g.shard_off) + (v0 - pr0 * vec_per_shard);
    const uint4* src1 = first < nv ? reinterpret_cast<const uint4*>(g.peer_base[pr0 + 1] + g.shard_off) - first : src0;
    for (unsigned long long j = gt; j < nv; j += GATHER_UNROLL * GATHER_THREADS) {
      uint4 v[GATHER_UNROLL];
#pragma unroll
      for (int u = 0; u < GATHER_UNROLL; ++u) {
        const unsigned long long jj = j + u * GATHER_THREADS;
        if (jj < nv) v[u] = jj < first ? src0[jj] : src1[jj];
      }
#pragma unroll
      for (int u = 0; u < GATHER_UNROLL; ++u) {
        const unsigned long long jj = j + u * GATHER_THREADS;
        if (jj < nv) dst[jj] = v[u];
      }
    }
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"n"(GATHER_THREADS) : "memory");
    if (gt == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(g.flags + c), "r"(g.epoch) : "memory");
  }
}

// Reduce form of the gather warps: chunk by chunk, dst = bf16(sum over all ranks of their copy of the
// region), read with plain peer loads, summed in fp32. This is the gradient reduce-scatter with ownership
// by tensor, run inside the GEMM that consumes the reduced gradient: the handshake is the reduce-scatter's
// (wait for every rank's "ready" epoch before the first load, signal "consumed" to every rank after the
// last one). A wait that runs out records code 46 and the kernel carries on (the host raises).
template <int MAXW>
__device__ __forceinline__ void reduce_chunks(const GatherParams& g, int gt, uint32_t* slot) {
  if (gt < g.world && !wait_flag(g.ready_flags + gt, g.rs_epoch, g.limit_us)) atomicExch(g.status, 46 | (gt << 8));
  asm volatile("bar.sync 1, %0;" ::"n"(GATHER_THREADS) : "memory");
  const int n_chunks = g.chunk_hi - g.chunk_lo;
  while (true) {
    if (gt == 0) *slot = atomicAdd(g.ticket, 1u);
    asm volatile("bar.sync 1, %0;" ::"n"(GATHER_THREADS) : "memory");
    const uint32_t k = *slot;
    asm volatile("bar.sync 1, %0;" ::"n"(GATHER_THREADS) : "memory");
    if (k >= static_cast<uint32_t>(n_chunks)) break;
    const int c = g.chunk_lo + static_cast<int>(k);      // front to back: the GEMM consumes its operand in row order
    const unsigned long long b0 = static_cast<unsigned long long>(c) * GATHER_CHUNK_BYTES;
    const unsigned long long b1 = min(b0 + GATHER_CHUNK_BYTES, g.total_bytes);
    const unsigned long long nv = (b1 - b0) >> 4;
    uint4* dst = reinterpret_cast<uint4*>(g.dst + b0);
    for (unsigned long long j = gt; j < nv; j += 2 * GATHER_THREADS) {
      uint4 v[2][MAXW];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const unsigned long long jj = j + u * GATHER_THREADS;
        if (jj < nv) {
#pragma unroll
          for (int p = 0; p < MAXW; ++p)
            if (p < g.world) v[u][p] = *(reinterpret_cast<const uint4*>(g.peer_base[p] + g.src_off + b0) + jj);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const unsigned long long jj = j + u * GATHER_THREADS;
        if (jj >= nv) continue;
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int p = 0; p < MAXW; ++p) {
          if (p < g.world) {
            const float2 a = unpack_bf16(v[u][p].x), b = unpack_bf16(v[u][p].y), cc = unpack_bf16(v[u][p].z), d = unpack_bf16(v[u][p].w);
            f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y; f[4] += cc.x; f[5] += cc.y; f[6] += d.x; f[7] += d.y;
          }
        }
        dst[jj] = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
      }
    }
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"n"(GATHER_THREADS) : "memory");
    if (gt == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(g.flags + c), "r"(g.epoch) : "memory");
  }
  // The last CTA whose gather warps run out of chunks tells every rank that its buffer has been read.
  __shared__ int last_s;
  if (gt == 0) last_s = (atomicAdd(g.done, 1u) == gridDim.x - 1);
  asm volatile("bar.sync 1, %0;" ::"n"(GATHER_THREADS) : "memory");
  if (last_s && gt < g.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(g.peer_base[gt] + g.consumed_off) + g.rank, g.rs_epoch);
  }
}

// Flag checker (one warp): waits until every chunk that overlaps bytes [lo, hi] of the full buffer
// carries this launch's epoch. Returns false when the bound ran out or another role aborted.
// `limit_us` > 0: time bound instead of the poll count (reduce mode, see mbar_wait).
__device__ __forceinline__ bool wait_chunks(const GatherParams& g, unsigned long long lo, unsigned long long hi, int lane,
                                            volatile int* abort_flag, uint32_t limit_us = 0) {
  const unsigned long long t0 = globaltimer_ns(), budget = static_cast<unsigned long long>(limit_us) * 1000ull;
  const int c_hi = static_cast<int>(hi / GATHER_CHUNK_BYTES);
  for (int c0 = static_cast<int>(lo / GATHER_CHUNK_BYTES); c0 <= c_hi; c0 += 32) {
    const int c = c0 + lane;
    bool ok = c > c_hi;
    uint32_t spins = 0;
    while (true) {
      if (!ok) ok = ld_acquire_gpu(g.flags + c) == g.epoch;
      if (__all_sync(0xffffffffu, ok)) break;
      ++spins;
      bool stop;
      if (limit_us == 0) stop = spins > SPIN_LIMIT || ((spins & 1023u) == 0 && *abort_flag);
      else stop = (spins & 1023u) == 0 && (*abort_flag || globaltimer_ns() - t0 > budget);
      if (__any_sync(0xffffffffu, stop)) return false;
    }
  }
  return true;
}

// TMA producer side: waits until the checker has verified tile number `tl` of this CTA; adds the
// time spent waiting to `waited_ns`. Returns false on timeout / abort.
__device__ __forceinline__ bool wait_verified(const uint32_t* verified, uint32_t tl, volatile int* abort_flag,
                                              unsigned long long& waited_ns, uint32_t limit_us = 0) {
  if (ld_acquire_cta_shared(verified) > tl) return true;
  const unsigned long long t0 = globaltimer_ns(), budget = static_cast<unsigned long long>(limit_us) * 1000ull;
  uint32_t spins = 0;
  while (ld_acquire_cta_shared(verified) <= tl) {
    ++spins;
    if (limit_us == 0) { if (spins > SPIN_LIMIT || ((spins & 1023u) == 0 && *abort_flag)) return false; }
    else if ((spins & 1023u) == 0 && (*abort_flag || globaltimer_ns() - t0 > budget)) return false;
  }
  waited_ns += globaltimer_ns() - t0;
  return true;
}

}  // namespace mtb
