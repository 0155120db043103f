// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory ->
// tcgen05.mma with the fp32 accumulator in tensor memory -> tcgen05.ld epilogue.
//
//   D[M, N] = A * B (+ bias[N]) (+ R[M, N])        bf16 inputs, fp32 accumulate, bf16 or fp32 out
//
// A is an "M x K" operand and B an "N x K" operand; each may be stored K-major (row-major
// [rows, K]) or MN-major (row-major [K, rows]), which covers the three products of a linear layer
// without any transposed copies:
//   forward  Y[T,N]  = X[T,K]  * W[N,K]^T   A K-major,  B K-major
//   dgrad    dX[T,K] = dY[T,N] * W[N,K]     A K-major,  B MN-major (W read as [red=N, out=K])
//   wgrad    dW[N,K] = dY[T,N]^T * X[T,K]   A MN-major, B MN-major (both read as [red=T, .])
//
// CTA layout (192 threads, one CTA per SM, grid = min(tiles, SMs)):
//   warp 0     TMA producer: fills a STAGES-deep ring of {A 128x64, B 256x64} tiles
//   warp 1     allocates 512 TMEM columns (two 128x256 fp32 accumulators) and issues the MMAs
//   warps 2-5  epilogue: each reads its 32-lane quarter of the accumulator, adds bias / residual,
//              converts and stores; runs concurrently with the next tile's MMAs (double buffer)
// Tiles are visited in bands of GROUP_M row-tiles so the A band stays in L2 while B streams.
//
// Out-of-range rows/columns/K are zero-filled by TMA and masked in the epilogue, so M, N and K
// need no padding (N and the leading dimensions must be multiples of 8 elements: TMA strides
// are multiples of 16 bytes).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "gather.cuh"
#include "ptx.cuh"

namespace mtb {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_TILE_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_TILE_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 16;
constexpr int GATHER_GROUP_N = 4;   // column-tiles per band in the all-gather variant
constexpr int GEMM_SMEM = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct GemmParams {
  int M, N, K;
  void* D;
  long long ldd;
  const void* R;          // optional residual / accumulate source, same dtype as D
  long long ldr;
  const __nv_bfloat16* bias;  // optional, [N]
  int* status;            // device word; set non-zero when a bounded wait expired
  float alpha;            // the product is multiplied by alpha before bias and residual are added
  int group_m;            // row-tiles per band of the tile order
  unsigned wait_hint_ns;  // suspend-time hint of the epilogue's and the MMA thread's long waits (0: plain polling)
  unsigned wait_limit_us; // > 0: every pipeline wait is bounded by this time instead of a poll count (fused reduce + GEMM)
};

// The fused all-gather variant (GATHER = true) adds the gather warps and the flag checker of gather.cuh;
// its tiles are visited in bands of GATHER_GROUP_N column-tiles.
// REDUCE (with GATHER): the gathered operand is A, and it is the SUM over ranks of a region of their gradient
// buffers (reduce_chunks in gather.cuh): the gradient reduce-scatter with ownership by tensor, fused into the GEMM
// that consumes the reduced gradient (OSFT factor gradients).
template <bool A_MN, bool B_MN, bool OUT_F32, bool GATHER = false, bool REDUCE = false>
__global__ void __launch_bounds__(GATHER ? GEMM_THREADS + GATHER_EXTRA_THREADS : GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmParams p,
            const __grid_constant__ GatherParams g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;   // [2] accumulator ready for the epilogue
  uint64_t* tempty_bar = tfull_bar + 2;       // [2] accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* verified = tmem_slot + 2;   // gather variant: tiles of this CTA whose weight chunks have all arrived
  uint32_t* ticket_slot = tmem_slot + 3;   // gather variant: broadcast of the chunk ticket among the gather warps

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 4); }
    *abort_flag = 0;
    *verified = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coords = [&](int t, int& tm, int& tn) {
    if constexpr (GATHER && !REDUCE) {
      // Bands of GROUP_N column-tiles, all row-tiles inside a band: the weight is consumed front to
      // back at an even rate over the whole launch (a band of row-tiles would need the ENTIRE weight
      // within its first band, i.e. within the first few waves, faster than the links deliver it).
      const int band = t / (GATHER_GROUP_N * tiles_m);
      const int first_n = band * GATHER_GROUP_N;
      const int cols = min(GATHER_GROUP_N, tiles_n - first_n);
      const int local = t - band * GATHER_GROUP_N * tiles_m;
      tn = first_n + local % cols;
      tm = local / cols;
      return;
    }
    const int band = t / (p.group_m * tiles_n);
    const int first_m = band * p.group_m;
    const int rows = min(p.group_m, tiles_m - first_m);
    const int local = t - band * p.group_m * tiles_n;
    tm = first_m + local % rows;
    tn = local / rows;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0, tl = 0;
      unsigned long long waited_ns = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, tm, tn);
        if (GATHER) {
          // the checker warp has seen the flags of every chunk under this tile's B rows
          if (!wait_verified(verified, tl, abort_flag, waited_ns, p.wait_limit_us)) { *abort_flag = 1; atomicExch(p.status, 5); goto done; }
          asm volatile("fence.proxy.async;" ::: "memory");   // peer data was written with ordinary stores, TMA reads it
          ++tl;
        }
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, 0, p.wait_limit_us)) { atomicExch(p.status, 1); goto done; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_TILE_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tmap_a, &full_bar[s], tm * BM + j * 64, kb * BK);
          } else {
            tma_load_2d(sa, &tmap_a, &full_bar[s], kb * BK, tm * BM);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[s], tn * BN + j * 64, kb * BK);
          } else {
            tma_load_2d(sb, &tmap_b, &full_bar[s], kb * BK, tn * BN);
          }
        }
      }
      if (GATHER && g.wait_ns != nullptr) {   // exposed-communication accounting: how long this producer starved
        atomicAdd(g.wait_ns, waited_ns);
        atomicAdd(g.wait_ns + 1, 1ull);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t it = 0, tl = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tl) {
        const int acc = tl & 1;
        const uint32_t aph = (tl >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], aph ^ 1, abort_flag, p.wait_hint_ns, p.wait_limit_us)) { atomicExch(p.status, 2); goto done; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, 0, p.wait_limit_us)) { atomicExch(p.status, 3); goto done; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[s]);   // frees the stage when these MMAs have read it
        }
        umma_commit(&tfull_bar[acc]);   // accumulator complete
      }
    }
  } else if (GATHER && warp == 6 + GATHER_THREADS / 32) {
    // ------------------------------------------------------------------ flag checker (warp 14)
    // Runs ahead of the TMA producer, so the producer thread never waits on a chain of dependent global loads.
    uint32_t tl = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tl) {
      int tm, tn;
      tile_coords(t, tm, tn);
      // rows [tn*BN, tn*BN+BN) of the K-major weight (reduce mode: rows [tm*BM, tm*BM+BM) of the K-major A operand)
      // are one contiguous byte range of the gathered buffer
      const unsigned long long lo = g.b_byte_off + static_cast<unsigned long long>(REDUCE ? tm * BM : tn * BN) * p.K * 2;
      const int rows = REDUCE ? min(BM, p.M - tm * BM) : min(BN, p.N - tn * BN);
      const unsigned long long hi = lo + static_cast<unsigned long long>(rows) * p.K * 2 - 1;
      const bool ok = wait_chunks(g, lo, hi, lane, abort_flag, p.wait_limit_us);
      __syncwarp();
      if (!ok) {
        if (lane == 0) { *abort_flag = 1; atomicExch(p.status, 5); }
        break;
      }
      if (lane == 0) st_release_cta_shared(verified, tl + 1);
    }
  } else if (GATHER && warp >= 6) {
    // ------------------------------------------------------------------ gather warps (6..13)
    if constexpr (REDUCE) reduce_chunks<8>(g, threadIdx.x - GEMM_THREADS, ticket_slot);
    else gather_chunks(g, threadIdx.x - GEMM_THREADS, ticket_slot);
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t tl = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tl) {
      int tm, tn;
      tile_coords(t, tm, tn);
      const int acc = tl & 1;
      const uint32_t aph = (tl >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], aph, abort_flag, p.wait_hint_ns, p.wait_limit_us)) { atomicExch(p.status, 4); goto done; }
      tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
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
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
int make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_inner, uint32_t box_outer);
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D bf16 tensor map over a row-major [outer, inner] matrix with leading dimension `ld`.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return -2;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// Same for an fp32 matrix (box_inner * 4 bytes must not exceed the 128-byte swizzle span).
int make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 4) % 16 || box_inner * 4 > 128) return -2;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 4};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

static int g_num_sms = 0;

// Tuning knobs read once from the environment (experiments; the defaults are what ships).
static int tune_group_m() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("MTB200_GEMM_GROUP_M"); v = e ? atoi(e) : GROUP_M; if (v < 1) v = GROUP_M; }
  return v;
}
static unsigned tune_wait_hint() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("MTB200_GEMM_WAIT_HINT_NS"); v = e ? atoi(e) : 0; if (v < 0) v = 0; }
  return static_cast<unsigned>(v);
}

namespace g2 {
int launch_gather(const void* A, long long lda, void* D, long long ldd, const void* bias, int M, int N, int K,
                  const void* w, int* status, const GatherParams& g, cudaStream_t stream);
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool GATHER = false, bool REDUCE = false>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream,
                  const GatherParams* gp = nullptr) {
  static bool configured = false;
  auto kern = gemm_kernel<A_MN, B_MN, OUT_F32, GATHER, REDUCE>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM) != cudaSuccess) return -4;
    configured = true;
  }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  // the gathering variant always uses every SM: its extra warps carry the transfer
  const int grid = (GATHER || tiles >= g_num_sms) ? g_num_sms : tiles;
  static const GatherParams none{};
  kern<<<grid, GATHER ? GEMM_THREADS + GATHER_EXTRA_THREADS : GEMM_THREADS, GEMM_SMEM, stream>>>(ta, tb, p, gp ? *gp : none);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace mtb

extern "C" {

// D[M,N] = alpha * op(A) * op(B) (+bias) (+R).
//   a_mn = 0: A is row-major [M, K] (lda >= K);  a_mn = 1: A is row-major [K, M] (lda >= M)
//   b_mn = 0: B is row-major [N, K] (ldb >= K);  b_mn = 1: B is row-major [K, N] (ldb >= N)
//   out_f32: D and R are fp32, else bf16. R may alias D (accumulate). bias is bf16 [N] or null.
// Returns 0 on success, a negative code on invalid arguments or launch failure.
int mtb200_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* D,
                     long long ldd, int out_f32, const void* R, long long ldr, const void* bias, int M, int N, int K,
                     float alpha, int* status, cudaStream_t stream) {
  using namespace mtb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (N % 8 || ldd % 8 || (R && ldr % 8)) return -10;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_tmap_2d_bf16(&ta, A, M, K, lda, 64, 64);
  else rc = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, 64);
  else rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, BN);
  if (rc) return rc - 10;
  GemmParams p{M, N, K, D, ldd, R, ldr, reinterpret_cast<const __nv_bfloat16*>(bias), status, alpha, tune_group_m(), tune_wait_hint(), 0u};
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

// Fused all-gather + GEMM:  D[M,N] = A[M,K] * W[N,K]^T (+bias) with W living in `full`, the local
// full parameter buffer of a sharded group that this same launch fills from the peers' shards.
//   bases/world       arena address of every rank; shard_off/shard_bytes locate the group's shard
//   full              local destination (world * shard_bytes); w_byte_off = offset of W inside it
//   flags/epoch       per-chunk (128 KB) completion words; a chunk is ready when its word == epoch
//   chunk_lo/chunk_hi chunks gathered by this launch (others must already carry `epoch`)
//   ticket            device word used to hand chunks out to whichever CTAs are resident (zeroed here)
//   wait_ns           optional device [2] counters: producer wait time summed over CTAs, CTA count
//   two_cta           run on CTA pairs (cta_group::2, 256 x 256 tiles) when the device can schedule them
// bias, if given, must lie in an already gathered part of `full` (or elsewhere).
int mtb200_gemm_bf16_allgather(const void* A, long long lda, void* D, long long ldd, const void* bias, int M, int N, int K,
                               const unsigned long long* bases, int world, unsigned long long shard_off,
                               unsigned long long shard_bytes, void* full, unsigned long long w_byte_off, unsigned int* flags,
                               unsigned int epoch, int chunk_lo, int chunk_hi, unsigned int* ticket, unsigned long long* wait_ns,
                               int two_cta, int* status, cudaStream_t stream) {
  using namespace mtb;
  if (M <= 0 || N <= 0 || K <= 0) return -10;
  if (N % 8 || ldd % 8 || K % 8 || world < 1 || world > GATHER_MAX_RANKS || shard_bytes % 16 || w_byte_off % 16) return -10;
  if (world > 1 && shard_bytes < static_cast<unsigned long long>(GATHER_CHUNK_BYTES)) return -11;   // a chunk may straddle one shard boundary at most
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, reinterpret_cast<const unsigned char*>(full) + w_byte_off, K, N, K, BK, BN);
  if (rc) return rc - 10;
  GemmParams p{M, N, K, D, ldd, nullptr, 0, reinterpret_cast<const __nv_bfloat16*>(bias), status, 1.0f, tune_group_m(), tune_wait_hint(), 0u};
  GatherParams g{};
  for (int i = 0; i < world; ++i) g.peer_base[i] = bases[i];
  g.shard_off = shard_off; g.shard_bytes = shard_bytes; g.dst = reinterpret_cast<unsigned char*>(full);
  g.flags = flags; g.epoch = epoch; g.world = world; g.chunk_lo = chunk_lo; g.chunk_hi = chunk_hi;
  g.ticket = ticket; g.wait_ns = wait_ns;
  g.b_byte_off = w_byte_off;
  int first = static_cast<int>(w_byte_off / GATHER_CHUNK_BYTES);
  g.chunk_first = first < chunk_lo ? chunk_lo : (first >= chunk_hi ? chunk_lo : first);
  if (ticket == nullptr) return -10;
  if (cudaMemsetAsync(ticket, 0, sizeof(unsigned int), stream) != cudaSuccess) return -5;   // chunk tickets start at 0 in every launch
  if (two_cta) {
    rc = g2::launch_gather(A, lda, D, ldd, bias, M, N, K, reinterpret_cast<const unsigned char*>(full) + w_byte_off, status, g, stream);
    if (rc != -6) return rc;   // -6: CTA pairs cannot be scheduled here; fall through to the one-CTA kernel
  }
  return launch<false, false, false, true>(ta, tb, p, stream, &g);
}

// Fused gradient reduce + GEMM:  D[M,N] (fp32) = (sum over ranks of G_r)[M,K] * B[N,K]^T (+ R), where G_r is the region
// [src_off, src_off + M*K*2) of rank r's arena (a tensor of its block gradient buffer). Gather warps pull the region from
// every rank, sum in fp32 and write bf16 into `dst` (local, M*K elements), which the TMA producer reads as the A operand as
// its chunks complete. Handshake of the reduce-scatter: waits for every rank's ready epoch, signals consumed when done.
//   flags/epoch   per-chunk completion words of dst;  ticket, done: device words, zeroed here
//   ready_flags   local row of ready epochs;  consumed_off: byte offset of the consumed row in every arena
int mtb200_gemm_bf16_reduce_a(void* dst, const void* B, long long ldb, float* D, long long ldd, const float* R, long long ldr,
                              int M, int N, int K, const unsigned long long* bases, int world, int rank,
                              unsigned long long src_off, unsigned int* flags, unsigned int epoch, unsigned int* ticket,
                              unsigned int* done, const void* ready_flags, unsigned long long consumed_off, unsigned int rs_epoch,
                              unsigned int limit_us, int* status, cudaStream_t stream) {
  using namespace mtb;
  if (M <= 0 || N <= 0 || K <= 0) return -10;
  if (N % 8 || ldd % 8 || K % 8 || (R && ldr % 8) || world < 1 || world > 8 || src_off % 16 || ticket == nullptr || done == nullptr) return -10;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, dst, K, M, K, BK, BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, BN);
  if (rc) return rc - 10;
  // every pipeline wait sits out the peers' skew: a little longer than the bound of the ready-flag wait itself
  const unsigned lim = limit_us ? limit_us : FLAG_SPIN_LIMIT;
  GemmParams p{M, N, K, D, ldd, R, ldr, nullptr, status, 1.0f, tune_group_m(), tune_wait_hint(), lim + lim / 2 + 10000000u};
  GatherParams g{};
  for (int i = 0; i < world; ++i) g.peer_base[i] = bases[i];
  g.dst = reinterpret_cast<unsigned char*>(dst);
  g.total_bytes = static_cast<unsigned long long>(M) * K * 2;
  g.flags = flags; g.epoch = epoch; g.world = world; g.rank = rank;
  g.chunk_lo = 0; g.chunk_hi = static_cast<int>((g.total_bytes + GATHER_CHUNK_BYTES - 1) / GATHER_CHUNK_BYTES);
  g.chunk_first = 0; g.b_byte_off = 0;
  g.ticket = ticket; g.done = done; g.wait_ns = nullptr;
  g.src_off = src_off; g.ready_flags = reinterpret_cast<const unsigned int*>(ready_flags); g.consumed_off = consumed_off;
  g.rs_epoch = rs_epoch; g.limit_us = limit_us ? limit_us : FLAG_SPIN_LIMIT; g.status = status;
  if (cudaMemsetAsync(ticket, 0, sizeof(unsigned int), stream) != cudaSuccess) return -5;
  if (cudaMemsetAsync(done, 0, sizeof(unsigned int), stream) != cudaSuccess) return -5;
  return launch<false, false, true, true, true>(ta, tb, p, stream, &g);
}

}  // extern "C"
