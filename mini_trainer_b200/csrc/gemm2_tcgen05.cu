// Two-CTA variant of the persistent bf16 GEMM: a cluster of two CTAs (two SMs) computes one
// 256 x 256 output tile with tcgen05.mma.cta_group::2. Each CTA stages its own 128 rows of A and
// HALF of the B tile (128 of the 256 N rows/columns), so per multiply the tensor core of each SM
// reads 8 KB of operands from shared memory instead of 12 KB, and the L2 -> SM traffic of B halves.
// That operand path, not the MMA itself, is what limits the one-CTA 128 x 256 kernel.
//
// Protocol (barriers live at the same shared-memory offsets in both CTAs):
//   full[s]    CTA 0 only. CTA 0's producer arms it with the bytes of BOTH CTAs; both producers'
//              TMA loads (cp.async.bulk.tensor ... .cta_group::2, no multicast) complete on it.
//   empty[s]   both CTAs; arrived by the leader's tcgen05.commit, multicast to the pair.
//   tfull[a]   both CTAs; accumulator `a` (128 lanes x 256 columns per CTA) is complete.
//   tempty[a]  CTA 0 only; the 8 epilogue warps of the pair arrive (CTA 1 remotely).
// Only CTA 0's MMA thread issues tcgen05.mma; every wait is bounded as in the one-CTA kernel.
// The two CTAs synchronise with barrier.cluster once after set-up and once before teardown.
//
// GATHER = true is the fused all-gather variant (see gather.cuh): both CTAs of a pair carry eight
// gather warps and a flag checker; each CTA's checker watches the chunks under ITS half of the B
// tile (128 weight rows, one contiguous byte range) and only that CTA's producer waits for them.
// No load in this file is multicast: every CTA issues its own TMA loads from local memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gather.cuh"
#include "ptx.cuh"

namespace mtb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

namespace g2 {

constexpr int BM = 128;            // rows of A / D per CTA (256 per pair)
constexpr int BN = 256;            // columns per pair; each CTA stages BN/2 of them
constexpr int BNH = BN / 2;
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;     // 16 KB
constexpr int B_BYTES = BNH * BK * 2;    // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int GROUP_M = 8;               // band of 8 pair-tiles = 2048 rows
constexpr int GATHER_GROUP_N = 4;        // column-tiles per band in the all-gather variant
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;   // clears the CTA-rank bit of a shared::cluster address -> CTA 0

struct Params {
  int M, N, K;
  void* D;
  long long ldd;
  const void* R;
  long long ldr;
  const __nv_bfloat16* bias;
  int* status;
  int num_pairs;
  float alpha;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t bar_addr_cta0, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_addr_cta0), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in BOTH CTAs once the leader's MMAs are done.
__device__ __forceinline__ void umma2_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cta0(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & PEER_MASK) : "memory");
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool GATHER = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GATHER ? THREADS + GATHER_EXTRA_THREADS : THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, Params p,
             const __grid_constant__ GatherParams g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* verified = tmem_slot + 2;      // gather variant: tiles whose chunks under this CTA's B half have arrived
  uint32_t* ticket_slot = tmem_slot + 3;   // gather variant: broadcast of the chunk ticket among the gather warps

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM), tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 8); }
    *abort_flag = 0;
    *verified = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();          // the partner's barriers are initialised before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coords = [&](int t, int& tm, int& tn) {
    if constexpr (GATHER) {   // bands of column-tiles: the weight is consumed front to back at an even rate
      const int band = t / (GATHER_GROUP_N * tiles_m);
      const int first_n = band * GATHER_GROUP_N;
      const int cols = min(GATHER_GROUP_N, tiles_n - first_n);
      const int local = t - band * GATHER_GROUP_N * tiles_m;
      tn = first_n + local % cols;
      tm = local / cols;
      return;
    }
    const int band = t / (GROUP_M * tiles_n);
    const int first_m = band * GROUP_M;
    const int rows = min(GROUP_M, tiles_m - first_m);
    const int local = t - band * GROUP_M * tiles_n;
    tm = first_m + local % rows;
    tn = local / rows;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      uint32_t it = 0, tl = 0;
      unsigned long long waited_ns = 0;
      for (int t = pair; t < num_tiles; t += p.num_pairs) {
        int tm, tn;
        tile_coords(t, tm, tn);
        const int row0 = tm * 2 * BM + rank * BM;        // this CTA's rows of A
        const int col0 = tn * BN + rank * BNH;           // this CTA's half of the B tile
        if (GATHER) {
          if (!wait_verified(verified, tl, abort_flag, waited_ns)) { *abort_flag = 1; atomicExch(p.status, 55); goto done; }
          asm volatile("fence.proxy.async;" ::: "memory");   // peer data was written with ordinary stores, TMA reads it
          ++tl;
        }
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) { atomicExch(p.status, 51); goto done; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t fb = smem_u32(&full_bar[s]) & PEER_MASK;   // CTA 0's barrier
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tmap_a, fb, row0 + j * 64, kb * BK);
          } else {
            tma_load_2d_pair(sa, &tmap_a, fb, kb * BK, row0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tmap_b, fb, col0 + j * 64, kb * BK);
          } else {
            tma_load_2d_pair(sb, &tmap_b, fb, kb * BK, col0);
          }
        }
      }
      if (GATHER && g.wait_ns != nullptr) {
        atomicAdd(g.wait_ns, waited_ns);
        atomicAdd(g.wait_ns + 1, 1ull);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      uint32_t it = 0, tl = 0;
      for (int t = pair; t < num_tiles; t += p.num_pairs, ++tl) {
        const int acc = tl & 1;
        const uint32_t aph = (tl >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], aph ^ 1, abort_flag)) { atomicExch(p.status, 52); goto done; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag)) { atomicExch(p.status, 53); goto done; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            umma2_bf16(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma2_commit_pair(&empty_bar[s]);
        }
        umma2_commit_pair(&tfull_bar[acc]);
      }
    }
  } else if (GATHER && warp == 6 + GATHER_THREADS / 32) {
    // ------------------------------------------------------------------ flag checker (warp 14, both CTAs)
    uint32_t tl = 0;
    for (int t = pair; t < num_tiles; t += p.num_pairs, ++tl) {
      int tm, tn;
      tile_coords(t, tm, tn);
      const int col0 = tn * BN + rank * BNH;
      bool ok = true;
      if (col0 < p.N) {   // rows [col0, col0 + BNH) of the K-major weight: one contiguous byte range
        const unsigned long long lo = g.b_byte_off + static_cast<unsigned long long>(col0) * p.K * 2;
        const int rows = min(BNH, p.N - col0);
        ok = wait_chunks(g, lo, lo + static_cast<unsigned long long>(rows) * p.K * 2 - 1, lane, abort_flag);
      }
      __syncwarp();
      if (!ok) {
        if (lane == 0) { *abort_flag = 1; atomicExch(p.status, 55); }
        break;
      }
      if (lane == 0) st_release_cta_shared(verified, tl + 1);
    }
  } else if (GATHER && warp >= 6) {
    // ------------------------------------------------------------------ gather warps (6..13, both CTAs)
    gather_chunks(g, threadIdx.x - THREADS, ticket_slot);
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    uint32_t tl = 0;
    for (int t = pair; t < num_tiles; t += p.num_pairs, ++tl) {
      int tm, tn;
      tile_coords(t, tm, tn);
      const int acc = tl & 1;
      const uint32_t aph = (tl >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], aph, abort_flag)) { atomicExch(p.status, 54); goto done; }
      tc_fence_after();
      const int row = tm * 2 * BM + rank * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.N) break;
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
        if (row_ok) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * p.alpha;
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                const uint4 b = *reinterpret_cast<const uint4*>(p.bias + col0 + j);
                const float2 b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y), b2 = unpack_bf16(b.z), b3 = unpack_bf16(b.w);
                f[j] += b0.x; f[j + 1] += b0.y; f[j + 2] += b1.x; f[j + 3] += b1.y;
                f[j + 4] += b2.x; f[j + 5] += b2.y; f[j + 6] += b3.x; f[j + 7] += b3.y;
              }
            }
          }
          if (OUT_F32) {
            float* dptr = reinterpret_cast<float*>(p.D) + static_cast<long long>(row) * p.ldd + col0;
            const float* rptr = p.R ? reinterpret_cast<const float*>(p.R) + static_cast<long long>(row) * p.ldr + col0 : nullptr;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col0 + j < p.N) {
                float4 o = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
                if (rptr) { const float4 r = *reinterpret_cast<const float4*>(rptr + j); o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w; }
                *reinterpret_cast<float4*>(dptr + j) = o;
              }
            }
          } else {
            __nv_bfloat16* dptr = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(row) * p.ldd + col0;
            const __nv_bfloat16* rptr = p.R ? reinterpret_cast<const __nv_bfloat16*>(p.R) + static_cast<long long>(row) * p.ldr + col0 : nullptr;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                if (rptr) {
                  const uint4 r = *reinterpret_cast<const uint4*>(rptr + j);
                  const float2 r0 = unpack_bf16(r.x), r1 = unpack_bf16(r.y), r2 = unpack_bf16(r.z), r3 = unpack_bf16(r.w);
                  f[j] += r0.x; f[j + 1] += r0.y; f[j + 2] += r1.x; f[j + 3] += r1.y;
                  f[j + 4] += r2.x; f[j + 5] += r2.y; f[j + 6] += r3.x; f[j + 7] += r3.y;
                }
                uint4 o;
                o.x = pack_bf16(f[j], f[j + 1]); o.y = pack_bf16(f[j + 2], f[j + 3]);
                o.z = pack_bf16(f[j + 4], f[j + 5]); o.w = pack_bf16(f[j + 6], f[j + 7]);
                *reinterpret_cast<uint4*>(dptr + j) = o;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cta0(&tempty_bar[acc]);
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  cluster_sync();          // nobody tears down while the partner may still signal or read
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

static int g_pairs[2] = {-1, -1};   // clusters of two that can be co-resident (0: unsupported), plain / gather variant

template <bool A_MN, bool B_MN, bool OUT_F32, bool GATHER = false>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, Params p, cudaStream_t stream, const GatherParams* gp = nullptr) {
  auto kern = gemm2_kernel<A_MN, B_MN, OUT_F32, GATHER>;
  constexpr int threads = GATHER ? THREADS + GATHER_EXTRA_THREADS : THREADS;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -4;
    configured = true;
  }
  int& pairs = g_pairs[GATHER ? 1 : 0];
  if (pairs < 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    pairs = n;
  }
  if (pairs <= 0) return -6;
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN);
  // the gathering variant always uses every pair: its extra warps carry the transfer
  p.num_pairs = (GATHER || tiles >= pairs) ? pairs : tiles;
  static const GatherParams none{};
  kern<<<2 * p.num_pairs, threads, SMEM, stream>>>(ta, tb, p, gp ? *gp : none);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Fused all-gather + GEMM on CTA pairs; called by mtb200_gemm_bf16_allgather.
int launch_gather(const void* A, long long lda, void* D, long long ldd, const void* bias, int M, int N, int K,
                  const void* w, int* status, const GatherParams& g, cudaStream_t stream) {
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, w, K, N, K, BK, BNH);
  if (rc) return rc - 10;
  Params p{M, N, K, D, ldd, nullptr, 0, reinterpret_cast<const __nv_bfloat16*>(bias), status, 0, 1.0f};
  return launch<false, false, false, true>(ta, tb, p, stream, &g);
}

}  // namespace g2
}  // namespace mtb

extern "C" {

// Same contract as mtb200_gemm_bf16, computed by CTA pairs (256 x 256 tiles). Returns -6 when
// clusters of two cannot be scheduled on this device; callers then use the one-CTA kernel.
int mtb200_gemm2_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* D,
                      long long ldd, int out_f32, const void* R, long long ldr, const void* bias, int M, int N, int K,
                      float alpha, int* status, cudaStream_t stream) {
  using namespace mtb;
  using namespace mtb::g2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (N % 8 || ldd % 8 || (R && ldr % 8)) return -10;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_tmap_2d_bf16(&ta, A, M, K, lda, 64, 64);
  else rc = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, 64);
  else rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, BNH);
  if (rc) return rc - 10;
  Params p{M, N, K, D, ldd, R, ldr, reinterpret_cast<const __nv_bfloat16*>(bias), status, 0, alpha};
  const int sel = (a_mn ? 4 : 0) | (b_mn ? 2 : 0) | (out_f32 ? 1 : 0);
  switch (sel) {
    case 0: return launch<false, false, false>(ta, tb, p, stream);
    case 1: return launch<false, false, true>(ta, tb, p, stream);
    case 2: return launch<false, true, false>(ta, tb, p, stream);
    case 3: return launch<false, true, true>(ta, tb, p, stream);
    case 4: return launch<true, false, false>(ta, tb, p, stream);
    case 5: return launch<true, false, true>(ta, tb, p, stream);
    case 6: return launch<true, true, false>(ta, tb, p, stream);
    default: return launch<true, true, true>(ta, tb, p, stream);
  }
}

}  // extern "C"
