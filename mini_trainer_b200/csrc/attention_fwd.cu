// Varlen causal GQA attention forward for sm_100a.
//
// One CTA handles one (sequence, 128-row query block, query head). Q, K and V are read straight
// out of the fused qkv activation [T, (Hq + 2 Hkv) * D] through ONE tensor map (128B swizzle):
//   S = Q K^T      tcgen05.mma, M=128 queries, N=128 keys, K=D      (accumulator in TMEM, 2 buffers)
//   P = softmax    8 warps, two threads per query row, read S from TMEM, write bf16 P to smem (2 buffers)
//   O += P V       tcgen05.mma, M=128, N=D, K=2 x 64 keys            (two accumulators in TMEM)
// Roles: warp 0 = TMA (K/V double-buffered), warp 1 = MMA issue, warps 2-9 = softmax + epilogue
// (two threads per query row, each owning 64 of the 128 key columns of a tile).
// S (TMEM) and P (smem) are double-buffered: Q K^T of tile j+1 and P V of tile j-1 both run under the
// softmax of tile j, so the softmax warps never wait for the tensor core except to rescale O.
//
// The two threads of a query row never talk to each other inside the key loop: each keeps its own
// online-softmax state (reference maximum, row sum) for its 64 key columns of every tile, and P V is
// issued as two half-K MMAs into two O accumulators in tensor memory (O_a: key columns 0-63 of each
// tile, O_b: 64-127). The halves are merged once, in the epilogue, like a split-K softmax:
//   m = max(m_a, m_b), O = (O_a 2^(m_a-m) + O_b 2^(m_b-m)) / (l_a 2^(m_a-m) + l_b 2^(m_b-m)).
// (Exchanging the half-row maxima through shared memory and a barrier on every tile cost about a
// fifth of the softmax time.) A state only rescales its accumulator when its running maximum grew
// by more than 2^8 (exact: the final merge uses the same references), so the TMEM round trip for the
// rescale is rare. Only the last key tile of a query block touches the causal diagonal and is masked.
//
// Masked scores are -inf. The exponentials that run on the special-function unit turn them into exact zeros;
// the quarter that runs on the FMA pipe (ex2_fma2) clamps its argument at -126 and returns about 1e-38 instead, so
// on the diagonal tile one masked key in four adds a term of that size to a row sum that is at least 1 (the row's
// maximum contributes exp2(0)) and a bf16 zero to P: below fp32 resolution, no effect on out or lse.
//
// Outputs: out [T, Hq*D] bf16 and lse [Hq, T] fp32 (natural log, scaled scores), as needed by
// the backward. Sequence boundaries come from a host-built work table (seq_start, seq_len, q0),
// so there is no device-side search in cu_seqlens.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace mtb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

constexpr int ATT_BM = 128, ATT_BN = 128;
constexpr int ATT_THREADS = 320;   // TMA warp, MMA warp, 8 softmax warps (two threads per query row)

template <int D>
struct AttFwdSmem {
  static constexpr int Q_BYTES = ATT_BM * D * 2;
  static constexpr int KV_BYTES = ATT_BN * D * 2;
  static constexpr int P_BYTES = ATT_BM * ATT_BN * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;        // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;   // 2 stages
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;   // 2 buffers
  static constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
  static constexpr int OFF_MX = OFF_BAR + 256;          // float [reference maximum, row sum][2 halves][128 rows], epilogue only
  // No alignment slack: with D = 128 the tiles fill 224 KB of the 227 KB a CTA can have. The kernel
  // checks that the dynamic shared memory window starts on a 1024-byte boundary (swizzle atom).
  static constexpr int TOTAL = OFF_MX + 2 * 2 * 128 * 4;
};

struct AttFwdParams {
  __nv_bfloat16* out;
  long long ldo;
  float* lse;
  const int* plan;   // [n_items, 3] = seq_start, seq_len, q0
  int T, Hq, Hkv;
  float scale;
  int* status;
};

// PT: P stays in tensor memory. The softmax threads write bf16 P over the S columns they just read
// (tcgen05.st; keys 0-63 of a tile into columns 0-31 of its S buffer, keys 64-127 into columns 64-95, so a
// thread only ever overwrites S columns that it owns) and P V is issued with the A operand in tensor memory.
// No P tile in shared memory: no st.shared / proxy fence in the softmax loop, no shared-memory reads of P by
// the tensor core. Q K^T of tile j+2 overwrites the buffer after P V of tile j in the tensor pipe's issue order.
template <int D, int POLY, bool PT>   // every POLY-th exponential pair runs on the FMA pipe instead of the special-function unit
__global__ void __launch_bounds__(ATT_THREADS, 1) attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap, AttFwdParams p) {
  using L = AttFwdSmem<D>;
  constexpr int KB = D / 64;  // 64-element (128 B) column blocks of a D-wide row
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {   // uniform over the CTA: nothing has been allocated or armed yet
    if (threadIdx.x == 0) atomicExch(p.status, 10);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* v_full = bars + 3;        // 2
  uint64_t* k_empty = bars + 5;       // 2: Q K^T of the tile in this stage has completed
  uint64_t* v_empty = bars + 7;       // 2: P V of the tile in this stage has completed
  uint64_t* s_full = bars + 9;        // 2
  uint64_t* p_ready = bars + 11;      // 2: P buffer written and S buffer consumed (8 arrivals)
  uint64_t* p_empty = bars + 13;      // 2: P V of the tile in this P buffer has completed
  uint64_t* mx_bar = bars + 15;       // 1: epilogue, the two threads of every row have published their softmax state
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x / p.Hq, h = blockIdx.x % p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int seq_start = p.plan[item * 3 + 0], seq_len = p.plan[item * 3 + 1], q0 = p.plan[item * 3 + 2];
  const int n_tiles = q0 / ATT_BN + 1;
  // bounds check of the host-built work item (uniform over the CTA; nothing allocated or armed yet):
  // a row that does not lie inside the packed batch is reported, not dereferenced
  if (seq_start < 0 || seq_len <= 0 || q0 < 0 || q0 >= seq_len || static_cast<long long>(seq_start) + seq_len > p.T) {
    if (threadIdx.x == 0) atomicExch(p.status, 61);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 8); mbar_init(&p_empty[i], 1);
    }
    mbar_init(mx_bar, 8);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s0 = tmem_base, tmem_oa = tmem_base + 256, tmem_ob = tmem_base + 384;

  if (warp == 0) {
    if (elect_one()) {
      mbar_arrive_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) tma_load_2d(smem + L::OFF_Q + kb * 16384, &tmap, q_full, h * D + kb * 64, seq_start + q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&k_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) { atomicExch(p.status, 11); goto done; }
        const int row = seq_start + j * ATT_BN;
        mbar_arrive_expect_tx(&k_full[s], L::KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(smem + L::OFF_K + s * L::KV_BYTES + kb * 16384, &tmap, &k_full[s], (p.Hq + hk) * D + kb * 64, row);
        if (!mbar_wait(&v_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) { atomicExch(p.status, 11); goto done; }
        mbar_arrive_expect_tx(&v_full[s], L::KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(smem + L::OFF_V + s * L::KV_BYTES + kb * 16384, &tmap, &v_full[s], (p.Hq + p.Hkv + hk) * D + kb * 64, row);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(ATT_BM, ATT_BN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(ATT_BM, D, false, true);
      const uint32_t sq = smem_u32(smem + L::OFF_Q), sp = smem_u32(smem + L::OFF_P);
      // descriptors of tiles at fixed addresses are built once; a k-step is one 64-bit add
      const uint64_t dQ = make_smem_desc(sq, 16, 1024);
      const uint64_t dK0 = make_smem_desc(smem_u32(smem + L::OFF_K), 16, 1024);
      const uint64_t dV0 = make_smem_desc(smem_u32(smem + L::OFF_V), 16384, 1024);
      const uint64_t dP0 = make_smem_desc(sp, 16, 1024);
      auto kstep = [](int k) { return static_cast<uint64_t>((k >> 2) * 1024 + (k & 3) * 2); };
      auto issue_qk = [&](int j) {
        const uint64_t dK = dK0 + static_cast<uint64_t>((j & 1) * (L::KV_BYTES >> 4));
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem_s0 + (j & 1) * ATT_BN, dQ + kstep(k), dK + kstep(k), idesc_qk, k != 0);
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_empty[j & 1]);
      };
      if (!mbar_wait(q_full, 0, abort_flag)) { atomicExch(p.status, 12); goto done; }
      for (int j = 0; j < 2 && j < n_tiles; ++j) {
        if (!mbar_wait(&k_full[j], 0, abort_flag)) { atomicExch(p.status, 13); goto done; }
        tc_fence_after();
        issue_qk(j);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&p_ready[b], ph, abort_flag)) { atomicExch(p.status, 15); goto done; }
        if (!mbar_wait(&v_full[b], ph, abort_flag)) { atomicExch(p.status, 16); goto done; }
        tc_fence_after();
        const uint64_t dV = dV0 + static_cast<uint64_t>(b * (L::KV_BYTES >> 4));
        const uint64_t dP = dP0 + static_cast<uint64_t>(b * (L::P_BYTES >> 4));
#pragma unroll
        for (int k = 0; k < ATT_BN / 16; ++k) {   // key columns 0-63 accumulate into O_a, 64-127 into O_b
          constexpr int KH = ATT_BN / 32;
          if constexpr (PT) {
            // 16 keys = 8 packed columns; the two halves of P sit at columns 0 and 64 of the S buffer
            const uint32_t pa = tmem_s0 + b * ATT_BN + (k < KH ? k * 8 : 64 + (k - KH) * 8);
            umma_bf16_ts(k < KH ? tmem_oa : tmem_ob, pa, dV + static_cast<uint64_t>(k * 128), idesc_pv,
                         j != 0 || (k != 0 && k != KH));
          } else {
            umma_bf16(k < KH ? tmem_oa : tmem_ob, dP + kstep(k), dV + static_cast<uint64_t>(k * 128), idesc_pv,
                      j != 0 || (k != 0 && k != KH));
          }
        }
        umma_commit(&v_empty[b]);
        umma_commit(&p_empty[b]);
        if (j + 2 < n_tiles) {   // S buffer b was consumed by the softmax of tile j: refill it with tile j+2
          if (!mbar_wait(&k_full[b], ((j + 2) >> 1) & 1, abort_flag)) { atomicExch(p.status, 14); goto done; }
          tc_fence_after();
          issue_qk(j + 2);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue
    const int q = warp & 3;                   // TMEM lane quarter
    const int half = (warp - 2) >> 2;         // which 64 key columns / which half of the O columns
    const int r = q * 32 + lane;              // row inside the query block
    const int qpos = q0 + r;                  // position inside the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;       // state of THIS thread's 64 key columns per tile
    uint8_t* sp = smem + L::OFF_P;
    float* mx = reinterpret_cast<float*>(smem + L::OFF_MX);
    const uint32_t tmem_own = (half == 0 ? tmem_oa : tmem_ob) + lane_addr;
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag)) { atomicExch(p.status, 17); goto done; }
      tc_fence_after();
      const uint32_t ts = tmem_s0 + (j & 1) * ATT_BN + lane_addr;
      const bool diag = (j == n_tiles - 1);
      const int kbase = j * ATT_BN;
      // S is read from tensor memory once: this thread's 64 columns stay in registers for both the
      // maximum and the exponentials. Only the last tile touches the causal diagonal.
      uint32_t sv[2][32];
      tmem_ld_32x32(ts + (half * 2) * 32, sv[0]);
      tmem_ld_32x32(ts + (half * 2 + 1) * 32, sv[1]);
      tmem_ld_wait();
      if (diag) {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kbase + (half * 2 + cc) * 32 + i > qpos) sv[cc][i] = 0xff800000u;   // -inf
      }
      float mt = -INFINITY;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc)
#pragma unroll
        for (int i = 0; i < 32; i += 2) mt = fmax3(mt, __uint_as_float(sv[cc][i]), __uint_as_float(sv[cc][i + 1]));
      float factor = 1.f;
      bool rescale = false;
      if (mt > m_ref && (mt - m_ref) * sl2 > 8.f) {   // includes the first unmasked tile (m_ref = -inf)
        factor = (m_ref == -INFINITY) ? 0.f : ex2_mufu((m_ref - mt) * sl2);
        rescale = (j > 0) && (m_ref != -INFINITY);    // nothing but zeros was accumulated before the first maximum
        m_ref = mt;
        l *= factor;
      }
      if (!PT && j >= 2) {   // the shared-memory P buffer of this tile must have been read by P V of tile j-2
        if (!mbar_wait(&p_empty[j & 1], ((j - 2) >> 1) & 1, abort_flag)) { atomicExch(p.status, 18); goto done; }
      }
      if (j > 0) {
        if (__any_sync(0xffffffffu, rescale)) {   // this half's O must be complete through tile j-1 before it is rescaled
          if (!mbar_wait(&p_empty[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) { atomicExch(p.status, 18); goto done; }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_own + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * factor);
            tmem_st_32x32(tmem_own + c * 32, v);
          }
          tmem_st_wait();
        }
      }
      // probabilities -> bf16 P in shared memory (K-major, 128B swizzle), row sums; exp2(-inf) = 0 masks.
      // A state that has seen only masked entries so far (m_ref = -inf) writes zeros.
      const float mo = (m_ref == -INFINITY) ? 0.f : m_ref * sl2;
      const float2 sl2v = make_float2(sl2, sl2), nmo = make_float2(-mo, -mo);
      float2 l2 = make_float2(0.f, 0.f);   // this tile's row sum, two lanes of packed adds
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint8_t* rowp = sp + (j & 1) * L::P_BYTES + (c >> 1) * 16384 + r * 128;
        uint32_t pk[16];   // PT: the 32 probabilities of this chunk as 16 packed bf16 pairs
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float2 e[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // scale and shift two scores with one packed FMA; of every POLY pairs one runs its exponentials on the FMA pipe
            const float2 x = ffma2(make_float2(__uint_as_float(sv[cc][g * 8 + 2 * i]), __uint_as_float(sv[cc][g * 8 + 2 * i + 1])), sl2v, nmo);
            e[i] = (i % POLY == POLY - 1) ? ex2_fma2(x) : make_float2(ex2_mufu(x.x), ex2_mufu(x.y));
            l2 = fadd2(l2, e[i]);
          }
          if constexpr (PT) {
#pragma unroll
            for (int i = 0; i < 4; ++i) pk[g * 4 + i] = pack_bf16(e[i].x, e[i].y);
          } else {
            const int chunk = (c & 1) * 4 + g;
            uint4 o;
            o.x = pack_bf16(e[0].x, e[0].y); o.y = pack_bf16(e[1].x, e[1].y); o.z = pack_bf16(e[2].x, e[2].y); o.w = pack_bf16(e[3].x, e[3].y);
            *reinterpret_cast<uint4*>(rowp + ((chunk ^ (r & 7)) << 4)) = o;
          }
        }
        if constexpr (PT) tmem_st_32x16(ts + half * 64 + cc * 16, pk);   // keys (half*64 + cc*32 ..+32) -> 16 packed columns
      }
      if constexpr (PT) tmem_st_wait();
      l += l2.x + l2.y;
      if constexpr (!PT) fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[j & 1]);
    }
    // epilogue: merge the two half-row states, O -> out, lse
    if (!mbar_wait(&p_empty[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort_flag)) { atomicExch(p.status, 19); goto done; }
    tc_fence_after();
    mx[half * 128 + r] = m_ref;
    mx[256 + half * 128 + r] = l;
    __syncwarp();
    if (lane == 0) mbar_arrive(mx_bar);
    if (!mbar_wait(mx_bar, 0, abort_flag)) { atomicExch(p.status, 20); goto done; }   // bounded, unlike bar.sync
    const float m_a = mx[r], m_b = mx[128 + r], l_a = mx[256 + r], l_b = mx[384 + r];
    const float m_all = fmaxf(m_a, m_b);   // finite: the diagonal entry of every row is unmasked
    const float f_a = (m_a == -INFINITY) ? 0.f : ex2_mufu((m_a - m_all) * sl2);
    const float f_b = (m_b == -INFINITY) ? 0.f : ex2_mufu((m_b - m_all) * sl2);
    const float l_all = l_a * f_a + l_b * f_b;
    const bool ok = qpos < seq_len;
    const float inv = 1.f / l_all;
    const float w_a = f_a * inv, w_b = f_b * inv;
    const long long tok = static_cast<long long>(seq_start) + qpos;
    __nv_bfloat16* orow = p.out + tok * p.ldo + h * D;
#pragma unroll 1
    for (int cc = 0; cc < D / 64; ++cc) {
      const int c = half * (D / 64) + cc;     // this thread writes half of the D columns of its row
      uint32_t va[32], vb[32];
      tmem_ld_32x32(tmem_oa + lane_addr + c * 32, va);
      tmem_ld_32x32(tmem_ob + lane_addr + c * 32, vb);
      tmem_ld_wait();
      if (ok) {
        float f[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          // an accumulator whose half never saw an unmasked entry holds zeros; w = 0 also covers its garbage-free case
          f[i] = __uint_as_float(va[i]) * w_a + __uint_as_float(vb[i]) * w_b;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack_bf16(f[g * 8 + 0], f[g * 8 + 1]);
          o.y = pack_bf16(f[g * 8 + 2], f[g * 8 + 3]);
          o.z = pack_bf16(f[g * 8 + 4], f[g * 8 + 5]);
          o.w = pack_bf16(f[g * 8 + 6], f[g * 8 + 7]);
          *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
        }
      }
    }
    if (ok && half == 0) p.lse[static_cast<long long>(h) * p.T + tok] = m_all * p.scale + logf(l_all);
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D, int POLY, bool PT>
static int launch_fwd(const CUtensorMap& tm, const AttFwdParams& p, int n_items, cudaStream_t st) {
  static bool configured = false;
  auto kern = attn_fwd_kernel<D, POLY, PT>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttFwdSmem<D>::TOTAL) != cudaSuccess) return -4;
    configured = true;
  }
  kern<<<n_items * p.Hq, ATT_THREADS, AttFwdSmem<D>::TOTAL, st>>>(tm, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace mtb

extern "C" int mtb200_attn_fwd(const void* qkv, long long ld, void* out, long long ldo, float* lse, const int* plan, int n_items,
                               int T, int Hq, int Hkv, int D, int reserved, float scale, int* status, cudaStream_t st) {
  using namespace mtb;
  if (n_items <= 0 || T <= 0) return 0;
  if ((D != 64 && D != 128) || Hq % Hkv || ld % 8 || ldo % 8) return -10;
  CUtensorMap tm;
  const int rc = make_tmap_2d_bf16(&tm, qkv, static_cast<uint64_t>(ld), static_cast<uint64_t>(T), static_cast<uint64_t>(ld), 64, 128);
  if (rc) return rc;
  AttFwdParams p{reinterpret_cast<__nv_bfloat16*>(out), ldo, lse, plan, T, Hq, Hkv, scale, status};
  // a quarter of the exponentials on the FMA pipe: 1011 vs 972 TFLOP/s (2 x 16384 tokens); half of them: no gain
  // reserved bit 0: P through a shared-memory tile (the earlier form, kept for A/B timing) instead of tensor memory
  if (reserved & 1) return D == 128 ? launch_fwd<128, 4, false>(tm, p, n_items, st) : launch_fwd<64, 4, false>(tm, p, n_items, st);
  // one exponential pair in four on the FMA pipe; one in two and one in eight measured the same within the spread
  return D == 128 ? launch_fwd<128, 4, true>(tm, p, n_items, st) : launch_fwd<64, 4, true>(tm, p, n_items, st);
}
