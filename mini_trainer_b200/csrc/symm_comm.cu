// NVLink / NVSwitch data path of the sharding engine over symmetric memory: every rank maps every
// peer's arena, and these kernels move parameter shards and gradients with plain peer loads and
// stores. No NCCL call is involved.
//
//   all-gather       pull: each rank copies every peer's parameter shard into its own full buffer.
//                    Shards only change in the optimizer step, which is followed by a cross-rank
//                    barrier, so pulling needs no per-transfer handshake.
//   reduce-scatter   pull + reduce: each rank reads ITS slice of every peer's gradient buffer, sums
//                    in fp32 and adds into its fp32 accumulator shard (optionally also the sum of
//                    squares of the result, for the gradient norm). A peer's buffer is read only
//                    after that peer signalled "complete" for the matching epoch; when the reader
//                    is done it signals "consumed" so the owner may overwrite the buffer.
//
// Flags are 32-bit epochs in the owner's arena, written by peers with system-scope release
// stores and polled with acquire loads. Every poll loop is bounded (a time limit on the global timer
// plus a poll count): when it runs out, the kernel
// records {code, peer} in the status word, skips its transfers and returns, so a missing peer ends
// in a host-side error instead of a hung GPU.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "flags.cuh"
#include "ptx.cuh"

namespace mtb {

constexpr int MAX_RANKS = 16;

struct PeerTable {
  uint64_t base[MAX_RANKS];   // device address of every rank's arena, as mapped into this process
};

// ---------------------------------------------------------------------------------- all-gather
// dst[p * shard_bytes + i] = arena_p[src_off + i] for every rank p; 16-byte accesses.
// Only 16-byte vectors [vec_lo, vec_hi) of the full buffer are copied (the whole buffer by default).
__global__ void __launch_bounds__(1024) symm_allgather_kernel(PeerTable peers, unsigned long long src_off, unsigned long long shard_bytes,
                                                             uint8_t* __restrict__ dst, int world, unsigned long long vec_lo,
                                                             unsigned long long vec_hi) {
  // Block b copies from peer (b % world); the blocks of one peer stride over that peer's part of
  // [vec_lo, vec_hi). No per-vector index arithmetic beyond an add: four independent loads in flight.
  const unsigned long long vec_per = shard_bytes >> 4;
  const int p = blockIdx.x % world;
  const unsigned long long sub = blockIdx.x / world, nsub = gridDim.x / world;
  const unsigned long long lo = max(vec_lo, static_cast<unsigned long long>(p) * vec_per);
  const unsigned long long hi = min(vec_hi, static_cast<unsigned long long>(p + 1) * vec_per);
  if (sub >= nsub || lo >= hi) return;
  const uint4* __restrict__ src = reinterpret_cast<const uint4*>(peers.base[p] + src_off) - static_cast<unsigned long long>(p) * vec_per;
  uint4* __restrict__ out = reinterpret_cast<uint4*>(dst);
  const unsigned long long stride = nsub * blockDim.x;
  unsigned long long i = lo + sub * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < hi; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < 4; ++u) out[i + u * stride] = v[u];
  }
  for (; i < hi; i += stride) out[i] = src[i];
}

// ---------------------------------------------------------------------------------- pull from one peer
// dst[0 : nvec] = arena_peer[src_off : ...] in 16-byte vectors (peer loads). The caller orders it after
// the owner's writes with a barrier.
__global__ void __launch_bounds__(512) symm_pull_kernel(unsigned long long src, uint4* __restrict__ dst, unsigned long long nvec) {
  const uint4* __restrict__ s = reinterpret_cast<const uint4*>(src);
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
  unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = s[i + u * stride];
#pragma unroll
    for (int u = 0; u < 4; ++u) dst[i + u * stride] = v[u];
  }
  for (; i < nvec; i += stride) dst[i] = s[i];
}

// ---------------------------------------------------------------------------------- signalling
// Writes `epoch` into slot [flag_off + 4 * rank] of every peer's arena (one thread per peer).
__global__ void symm_signal_kernel(PeerTable peers, unsigned long long flag_off, int rank, int world, uint32_t epoch) {
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(peers.base[p] + flag_off) + rank, epoch);
  }
}

// Waits until every peer's slot in MY flag row reached `epoch`. On expiry: status = code | peer << 8.
__global__ void symm_wait_kernel(const uint32_t* __restrict__ my_flags, int world, uint32_t epoch, uint32_t limit, int code, int* status) {
  const int p = threadIdx.x;
  if (p < world && !wait_flag(my_flags + p, epoch, limit)) atomicExch(status, code | (p << 8));
}

// ---------------------------------------------------------------------------------- reduce-scatter
// acc[i] (+)= sum_p bf16 grad_p[start + i] for i < n; optional sumsq of the result. `start` is where
// this rank's part of the region being reduced begins inside every rank's gradient buffer (the whole
// slice of the rank, or its intersection with one tensor region when the reduction follows backward
// tensor by tensor). n may be 0 (the region does not touch this rank's slice): nothing is read, but the
// kernel still takes part in the handshake. After all blocks have read, the last one signals
// "consumed" (epoch) to every peer.
template <int MAXW>   // compile-time bound on the rank count keeps the per-peer vectors in registers
__global__ void __launch_bounds__(512) symm_reduce_scatter_kernel(PeerTable peers, unsigned long long grad_off, long long start, long long n,
                                                                 float* __restrict__ acc, int accumulate, float* __restrict__ sumsq,
                                                                 const uint32_t* __restrict__ ready_flags, unsigned long long consumed_off,
                                                                 uint32_t epoch, uint32_t limit, int rank, int world,
                                                                 unsigned int* __restrict__ block_counter, int* status) {
  __shared__ int ok_s;
  __shared__ float red[32];
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (n > 0 && threadIdx.x < world && !wait_flag(ready_flags + threadIdx.x, epoch, limit)) {
    ok_s = 0;
    atomicExch(status, 41 | (threadIdx.x << 8));
  }
  __syncthreads();
  float ss = 0.f;
  if (ok_s) {
    const long long nvec = n >> 3;
    const unsigned long long slice_off = grad_off + static_cast<unsigned long long>(start) * 2;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    // two independent vectors per thread and iteration: 2 x world peer loads in flight
    for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < nvec; i0 += 2 * stride) {
      const long long idx[2] = {i0, i0 + stride};
      uint4 v[2][MAXW];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (idx[u] < nvec) {
#pragma unroll
          for (int p = 0; p < MAXW; ++p)
            if (p < world) v[u][p] = *(reinterpret_cast<const uint4*>(peers.base[p] + slice_off) + idx[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (idx[u] >= nvec) continue;
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int p = 0; p < MAXW; ++p) {
          if (p < world) {
            const float2 a = unpack_bf16(v[u][p].x), b = unpack_bf16(v[u][p].y), c = unpack_bf16(v[u][p].z), d = unpack_bf16(v[u][p].w);
            f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y; f[4] += c.x; f[5] += c.y; f[6] += d.x; f[7] += d.y;
          }
        }
        float4* dst = reinterpret_cast<float4*>(acc) + 2 * idx[u];
        if (accumulate) {
          const float4 a = dst[0], b = dst[1];
          f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w; f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
        }
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
        if (sumsq != nullptr) {
#pragma unroll
          for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
        }
      }
    }
  }
  if (sumsq != nullptr) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      t = warp_sum(t);
      if (threadIdx.x == 0) atomicAdd(sumsq, t);
    }
  }
  // last block out tells every peer that its buffer has been consumed by this rank
  __threadfence();
  __syncthreads();
  __shared__ int last_s;
  if (threadIdx.x == 0) last_s = (atomicAdd(block_counter, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last_s) {
    if (threadIdx.x == 0) *block_counter = 0;
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(peers.base[threadIdx.x] + consumed_off) + rank, epoch);
    }
  }
}

// ---------------------------------------------------------------------------------- reduce-scatter through NVSwitch
// Same contract and handshake as symm_reduce_scatter_kernel, but the sum over ranks is formed INSIDE
// the switch: one multimem.ld_reduce on the arena's multicast address returns, for 8 consecutive bf16
// gradients, the sum of all ranks' copies (accumulated in fp32 by the switch, delivered as bf16), so a
// rank receives 1/world of the bytes the peer-load version pulls. Only usable when the arena is bound
// to a multicast object (opt-in: a rank that dies while bound can fault its peers' GPUs).
__global__ void __launch_bounds__(512) symm_reduce_scatter_nvls_kernel(unsigned long long mc_base, PeerTable peers, unsigned long long grad_off,
                                                                      long long start, long long n, float* __restrict__ acc, int accumulate,
                                                                      float* __restrict__ sumsq, const uint32_t* __restrict__ ready_flags,
                                                                      unsigned long long consumed_off, uint32_t epoch, uint32_t limit, int rank,
                                                                      int world, unsigned int* __restrict__ block_counter, int* status) {
  __shared__ int ok_s;
  __shared__ float red[32];
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (n > 0 && threadIdx.x < world && !wait_flag(ready_flags + threadIdx.x, epoch, limit)) {
    ok_s = 0;
    atomicExch(status, 45 | (threadIdx.x << 8));
  }
  __syncthreads();
  float ss = 0.f;
  if (ok_s) {
    const long long nvec = n >> 3;
    const unsigned long long src = mc_base + grad_off + static_cast<unsigned long long>(start) * 2;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < nvec; i0 += 4 * stride) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec)
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(src + static_cast<unsigned long long>(i) * 16) : "memory");
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long i = i0 + u * stride;
        if (i >= nvec) continue;
        const float2 a = unpack_bf16(v[u].x), b = unpack_bf16(v[u].y), c = unpack_bf16(v[u].z), d = unpack_bf16(v[u].w);
        float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
        float4* dst = reinterpret_cast<float4*>(acc) + 2 * i;
        if (accumulate) {
          const float4 p0 = dst[0], p1 = dst[1];
          f[0] += p0.x; f[1] += p0.y; f[2] += p0.z; f[3] += p0.w; f[4] += p1.x; f[5] += p1.y; f[6] += p1.z; f[7] += p1.w;
        }
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
        if (sumsq != nullptr) {
#pragma unroll
          for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
        }
      }
    }
  }
  if (sumsq != nullptr) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      t = warp_sum(t);
      if (threadIdx.x == 0) atomicAdd(sumsq, t);
    }
  }
  __threadfence();
  __syncthreads();
  __shared__ int last_s;
  if (threadIdx.x == 0) last_s = (atomicAdd(block_counter, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last_s) {
    if (threadIdx.x == 0) *block_counter = 0;
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(peers.base[threadIdx.x] + consumed_off) + rank, epoch);
    }
  }
}

// ---------------------------------------------------------------------------------- scalar all-reduce
// Every rank deposits its value in slot [rank] of every peer's value row, then sums the row it
// received in rank order (so all ranks get the bitwise-same result).
__global__ void symm_allreduce_scalar_kernel(PeerTable peers, unsigned long long vals_off, unsigned long long flag_off,
                                             const uint32_t* __restrict__ my_vals, const uint32_t* __restrict__ my_flags,
                                             uint32_t epoch, uint32_t limit, float* __restrict__ inout, int rank, int world, int* status) {
  __shared__ int ok_s;
  const int p = threadIdx.x;
  if (p == 0) ok_s = 1;
  __syncthreads();
  if (p < world) {
    const float v = *inout;
    *(reinterpret_cast<float*>(peers.base[p] + vals_off) + rank) = v;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(peers.base[p] + flag_off) + rank, epoch);
    if (!wait_flag(my_flags + p, epoch, limit)) { ok_s = 0; atomicExch(status, 44 | (p << 8)); }
  }
  __syncthreads();
  if (p == 0 && ok_s) {
    float s = 0.f;
    for (int q = 0; q < world; ++q) s += __uint_as_float(ld_acquire_sys(my_vals + q));
    *inout = s;
  }
}

static inline PeerTable make_table(const unsigned long long* bases, int world) {
  PeerTable t;
  for (int i = 0; i < MAX_RANKS; ++i) t.base[i] = i < world ? bases[i] : 0;
  return t;
}

}  // namespace mtb

using namespace mtb;

extern "C" {

// bases: host array of `world` arena addresses. Offsets are byte offsets inside the arena.
// byte_lo/byte_hi (multiples of 16) restrict the copy to that range of the full buffer; byte_hi = 0 means everything.
int mtb200_symm_allgather(const unsigned long long* bases, int world, unsigned long long src_off, unsigned long long shard_bytes,
                          void* dst, unsigned long long byte_lo, unsigned long long byte_hi, int blocks, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS || shard_bytes % 16 || src_off % 16 || byte_lo % 16 || byte_hi % 16) return -10;
  if (byte_hi == 0) byte_hi = shard_bytes * world;
  if (byte_hi > shard_bytes * world || byte_lo > byte_hi) return -10;
  if (blocks < world) blocks = world;
  blocks -= blocks % world;   // the same number of blocks per peer
  symm_allgather_kernel<<<blocks, 1024, 0, st>>>(make_table(bases, world), src_off, shard_bytes, reinterpret_cast<uint8_t*>(dst), world,
                                                 byte_lo >> 4, byte_hi >> 4);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Copies `bytes` (a multiple of 16) from byte offset src_off of rank `peer`'s arena to local memory.
int mtb200_symm_pull(const unsigned long long* bases, int world, int peer, unsigned long long src_off, void* dst,
                     unsigned long long bytes, int blocks, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS || peer < 0 || peer >= world || src_off % 16 || bytes % 16 ||
      (reinterpret_cast<uintptr_t>(dst) & 15)) return -10;
  if (bytes == 0) return 0;
  const unsigned long long nvec = bytes >> 4;
  if (blocks < 1) blocks = 1;
  if (static_cast<unsigned long long>(blocks) > (nvec + 511) / 512) blocks = static_cast<int>((nvec + 511) / 512);
  symm_pull_kernel<<<blocks, 512, 0, st>>>(bases[peer] + src_off, reinterpret_cast<uint4*>(dst), nvec);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int mtb200_symm_signal(const unsigned long long* bases, int world, int rank, unsigned long long flag_off, unsigned int epoch, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS) return -10;
  symm_signal_kernel<<<1, 32, 0, st>>>(make_table(bases, world), flag_off, rank, world, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int mtb200_symm_wait(const void* my_flags, int world, unsigned int epoch, unsigned int limit, int code, int* status, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS) return -10;
  symm_wait_kernel<<<1, 32, 0, st>>>(reinterpret_cast<const uint32_t*>(my_flags), world, epoch, limit ? limit : FLAG_SPIN_LIMIT, code, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int mtb200_symm_reduce_scatter(const unsigned long long* bases, int world, int rank, unsigned long long grad_off, long long start,
                               long long n, float* acc, int accumulate, float* sumsq, const void* ready_flags,
                               unsigned long long consumed_off, unsigned int epoch, unsigned int limit, unsigned int* block_counter,
                               int* status, int blocks, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS || n < 0 || n % 8 || start % 8 || grad_off % 16) return -10;
  if (n == 0) blocks = 1;
  else if (blocks > (n / 8 + 511) / 512) blocks = static_cast<int>((n / 8 + 511) / 512);
#define MTB_RS(W)                                                                                                       \
  symm_reduce_scatter_kernel<W><<<blocks, 512, 0, st>>>(make_table(bases, world), grad_off, start, n, acc, accumulate, sumsq, \
                                                        reinterpret_cast<const uint32_t*>(ready_flags), consumed_off, epoch, \
                                                        limit ? limit : FLAG_SPIN_LIMIT, rank, world, block_counter, status)
  if (world <= 2) MTB_RS(2); else if (world <= 4) MTB_RS(4); else if (world <= 8) MTB_RS(8); else MTB_RS(16);
#undef MTB_RS
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// NVSwitch (multimem) form of mtb200_symm_reduce_scatter. mc_base: multicast address of the arena.
int mtb200_symm_reduce_scatter_nvls(unsigned long long mc_base, const unsigned long long* bases, int world, int rank,
                                    unsigned long long grad_off, long long start, long long n, float* acc, int accumulate, float* sumsq,
                                    const void* ready_flags, unsigned long long consumed_off, unsigned int epoch, unsigned int limit,
                                    unsigned int* block_counter, int* status, int blocks, cudaStream_t st) {
  if (mc_base == 0 || world < 1 || world > MAX_RANKS || n < 0 || n % 8 || start % 8 || grad_off % 16) return -10;
  if (n == 0) blocks = 1;
  else if (blocks > (n / 8 + 511) / 512) blocks = static_cast<int>((n / 8 + 511) / 512);
  symm_reduce_scatter_nvls_kernel<<<blocks, 512, 0, st>>>(mc_base, make_table(bases, world), grad_off, start, n, acc, accumulate, sumsq,
                                                          reinterpret_cast<const uint32_t*>(ready_flags), consumed_off, epoch,
                                                          limit ? limit : FLAG_SPIN_LIMIT, rank, world, block_counter, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int mtb200_symm_allreduce_scalar(const unsigned long long* bases, int world, int rank, unsigned long long vals_off,
                                 unsigned long long flag_off, const void* my_vals, const void* my_flags, unsigned int epoch,
                                 unsigned int limit, float* inout, int* status, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS) return -10;
  symm_allreduce_scalar_kernel<<<1, 32, 0, st>>>(make_table(bases, world), vals_off, flag_off, reinterpret_cast<const uint32_t*>(my_vals),
                                                 reinterpret_cast<const uint32_t*>(my_flags), epoch, limit ? limit : FLAG_SPIN_LIMIT, inout,
                                                 rank, world, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
