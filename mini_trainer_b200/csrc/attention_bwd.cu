// Varlen causal GQA attention backward for sm_100a.
//
// One CTA owns one (sequence, 128-key block, kv head): K and V of that block stay in shared memory
// and dK, dV accumulate in tensor memory over every query head of the GQA group and every query
// block at or below the causal diagonal, so they are written once, without atomics. Per
// (query head, query block) the CTA runs five tcgen05 GEMMs:
//   S  = Q K^T            dP = dO V^T                      (TMEM, 128 columns each)
//   P  = exp(S*scale - lse), dS = P * (dP - delta) * scale  (4 warps; bf16 P and dS to smem)
//   dQ = dS K  (into S's TMEM columns)   dV += P^T dO   dK += dS^T Q
// dQ tiles (several key blocks contribute to one query block) are staged in shared memory and added
// into an fp32 [T, Hq*D] accumulator with TMA tensor reduces (cp.reduce.async.bulk.tensor .add, one
// 32-column x 128-row box each, 128B-swizzled so the staging stores are free of bank conflicts); a
// small kernel rounds the accumulator to bf16 afterwards. The first half of the D columns is staged
// in the P tile (idle once the MMAs have read it), the second half in a buffer of its own, and a
// separate warp issues the reduces: those of the P tile first and alone, so that the next softmax, which
// has to overwrite P, waits for half of the read-out only, and never for the thread that issued it.
// P and dS are stored once as [query, key] 128B-swizzled tiles and read both K-major (for dQ) and
// MN-major (for dV / dK), so no transposes are materialised.
//
// Rows past the end of the sequence (queries or keys) are masked to zero contribution.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace mtb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
int make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_inner, uint32_t box_outer);

constexpr int AB_B = 128;          // block edge (queries and keys)
constexpr int AB_THREADS = 352;     // TMA warp, MMA warp, 8 softmax warps (two threads per query row), dQ reduce warp

// Phase timestamps for kernel development. They exist only in a library built with
// -DMTB200_ATTN_BWD_TIMESTAMPS (the shipped build has neither the buffer nor the stores): per
// iteration of CTA 0, 4 clock64 values from the MMA thread (start, S/dP issued, P/dS seen, late MMAs
// issued) and 5 from one softmax thread (S/dP seen, P/dS computed, P tile free, dQ complete, dQ
// staged), read back with mtb200_attn_bwd_debug_read.
#ifdef MTB200_ATTN_BWD_TIMESTAMPS
constexpr int DBG_ITERS = 256;
__device__ long long g_attn_bwd_dbg[DBG_ITERS * 9];
#define MTB_STAMP(cond, it, slot) do { if ((cond) && (it) < DBG_ITERS) g_attn_bwd_dbg[(it) * 9 + (slot)] = clock64(); } while (0)
#else
#define MTB_STAMP(cond, it, slot) do { } while (0)
#endif

template <int D>
struct AttBwdSmem {
  static constexpr int TILE = AB_B * D * 2;         // a [128, D] bf16 tile
  static constexpr int PT = AB_B * AB_B * 2;        // a [128, 128] bf16 tile
  static constexpr int OFF_K = 0, OFF_V = TILE, OFF_Q = 2 * TILE, OFF_DO = 3 * TILE;
  static constexpr int OFF_P = 4 * TILE, OFF_DS = OFF_P + PT;
  static constexpr int OFF_ST2 = OFF_DS + PT;       // staging of the second half of a dQ tile: D/64 boxes of [128 rows x 128 B]
  static constexpr int ST2 = (D / 64) * 16384;
  static constexpr int OFF_BAR = OFF_ST2 + ST2;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

struct AttBwdParams {
  __nv_bfloat16* dqkv;
  long long ldq;
  const float* lse;
  const float* delta;
  float* dq_acc;        // [T, Hq*D] fp32, zero-initialised
  const int* plan;      // [n_items, 3] = seq_start, seq_len, k0
  int T, Hq, Hkv;
  float scale;
  int* status;
};

template <int D>
__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_dq, AttBwdParams p) {
  using L = AttBwdSmem<D>;
  constexpr int KB = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* kv_full = bars;        // K and V resident
  uint64_t* qdo_full = bars + 1;   // [2] Q_i landed / dO_i landed (at bars + 1 and bars + 9)
  uint64_t* sdp_full = bars + 2;   // S and dP complete
  uint64_t* pds_ready = bars + 3;  // P and dS written (4 arrivals)
  uint64_t* stage_full = bars + 4; // dQ tile copied from TMEM to the smem staging area (8 arrivals)
  uint64_t* mma_done = bars + 5;   // dV, dK, dQ complete: Q, dO, P, dS reusable, dQ readable
  uint64_t* dq_read = bars + 6;    // dQ tile drained from TMEM (8 arrivals): S columns reusable
  uint64_t* stage_free = bars + 7; // the tensor reduces have read the dQ half staged in the P tile: P writable
  uint64_t* q_free = bars + 8;     // dK has read Q: the next Q tile may be loaded while dV and dQ still run
  uint64_t* do_full = bars + 9;    // dO_i landed
  uint64_t* do_free = bars + 10;   // dV has read dO: the next dO tile may be loaded while dQ still runs
  uint64_t* st2_free = bars + 11;  // the tensor reduces have read the second staging buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x / p.Hkv, hk = blockIdx.x % p.Hkv;
  const int G = p.Hq / p.Hkv;
  const int seq_start = p.plan[item * 3 + 0], seq_len = p.plan[item * 3 + 1], k0 = p.plan[item * 3 + 2];
  const int jblk = k0 / AB_B;
  const int nq = (seq_len + AB_B - 1) / AB_B;      // query blocks of the sequence
  const int per_head = nq - jblk;                  // query blocks at or below the diagonal
  const int n_iters = G * per_head;
  // bounds check of the host-built work item (uniform over the CTA; nothing allocated or armed yet)
  if (seq_start < 0 || seq_len <= 0 || k0 < 0 || k0 >= seq_len || static_cast<long long>(seq_start) + seq_len > p.T) {
    if (threadIdx.x == 0) atomicExch(p.status, 61);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(qdo_full, 1); mbar_init(sdp_full, 1); mbar_init(pds_ready, 8);
    mbar_init(stage_full, 8); mbar_init(mma_done, 1); mbar_init(dq_read, 8); mbar_init(stage_free, 1);
    mbar_init(q_free, 1); mbar_init(do_full, 1); mbar_init(do_free, 1); mbar_init(st2_free, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_qkv);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_dq);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 256 + D;

  if (warp == 0) {
    if (elect_one()) {
      mbar_arrive_expect_tx(kv_full, 2 * L::TILE);
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) {
        tma_load_2d(smem + L::OFF_K + kb * 16384, &tm_qkv, kv_full, (p.Hq + hk) * D + kb * 64, seq_start + k0);
        tma_load_2d(smem + L::OFF_V + kb * 16384, &tm_qkv, kv_full, (p.Hq + p.Hkv + hk) * D + kb * 64, seq_start + k0);
      }
      for (int it = 0; it < n_iters; ++it) {
        const int h = hk * G + it / per_head, i = jblk + it % per_head;
        // Q is released first (after dK), dO second (after dV): both loads overlap the tail of the MMAs
        if (it > 0 && !mbar_wait(q_free, (it - 1) & 1, abort_flag)) { atomicExch(p.status, 21); goto done; }
        mbar_arrive_expect_tx(qdo_full, L::TILE);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(smem + L::OFF_Q + kb * 16384, &tm_qkv, qdo_full, h * D + kb * 64, seq_start + i * AB_B);
        if (it > 0 && !mbar_wait(do_free, (it - 1) & 1, abort_flag)) { atomicExch(p.status, 21); goto done; }
        mbar_arrive_expect_tx(do_full, L::TILE);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(smem + L::OFF_DO + kb * 16384, &tm_do, do_full, h * D + kb * 64, seq_start + i * AB_B);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t id_nt = make_idesc_bf16(AB_B, AB_B, false, false);   // S, dP
      constexpr uint32_t id_dq = make_idesc_bf16(AB_B, D, false, true);       // dQ = dS K
      constexpr uint32_t id_tn = make_idesc_bf16(AB_B, D, true, true);        // dV, dK
      const uint32_t sk = smem_u32(smem + L::OFF_K), sv = smem_u32(smem + L::OFF_V), sq = smem_u32(smem + L::OFF_Q);
      const uint32_t sdo = smem_u32(smem + L::OFF_DO), spp = smem_u32(smem + L::OFF_P), sds = smem_u32(smem + L::OFF_DS);
      // every tile lives at a fixed shared-memory address, so the descriptors are built once; inside
      // the loop a k-step is one 64-bit add (start-address field, in 16-byte units)
      const uint64_t dQk = make_smem_desc(sq, 16, 1024), dKk = make_smem_desc(sk, 16, 1024);
      const uint64_t dDOk = make_smem_desc(sdo, 16, 1024), dVk = make_smem_desc(sv, 16, 1024);
      const uint64_t dDSk = make_smem_desc(sds, 16, 1024);
      const uint64_t dDSm = make_smem_desc(sds, 16384, 1024), dPm = make_smem_desc(spp, 16384, 1024);
      const uint64_t dQm = make_smem_desc(sq, 16384, 1024), dDOm = make_smem_desc(sdo, 16384, 1024);
      const uint64_t dKm = make_smem_desc(sk, 16384, 1024);
      auto kstep = [](int k) { return static_cast<uint64_t>((k >> 2) * 1024 + (k & 3) * 2); };   // K-major: 32 B per step, 16 KB per 64
      auto mstep = [](int k) { return static_cast<uint64_t>(k * 128); };                           // MN-major: 2048 B per step
      if (!mbar_wait(kv_full, 0, abort_flag)) { atomicExch(p.status, 22); goto done; }
      for (int it = 0; it < n_iters; ++it) {
        if (!mbar_wait(qdo_full, it & 1, abort_flag)) { atomicExch(p.status, 23); goto done; }
        if (it > 0 && !mbar_wait(dq_read, (it - 1) & 1, abort_flag)) { atomicExch(p.status, 24); goto done; }
        tc_fence_after();
        MTB_STAMP(blockIdx.x == 0, it, 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          umma_bf16(t_s, dQk + kstep(k), dKk + kstep(k), id_nt, k != 0);
        }
        if (!mbar_wait(do_full, it & 1, abort_flag)) { atomicExch(p.status, 23); goto done; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          umma_bf16(t_dp, dDOk + kstep(k), dVk + kstep(k), id_nt, k != 0);
        }
        umma_commit(sdp_full);
        MTB_STAMP(blockIdx.x == 0, it, 1);
        if (!mbar_wait(pds_ready, it & 1, abort_flag)) { atomicExch(p.status, 25); goto done; }
        tc_fence_after();
        MTB_STAMP(blockIdx.x == 0, it, 2);
        // dK += dS^T Q, then dV += P^T dO  (A = [query, key] tile read MN-major, B = [query, D] tile read MN-major)
#pragma unroll
        for (int k = 0; k < AB_B / 16; ++k)
          umma_bf16(t_dk, dDSm + mstep(k), dQm + mstep(k), id_tn, (it | k) != 0);
        umma_commit(q_free);
#pragma unroll
        for (int k = 0; k < AB_B / 16; ++k)
          umma_bf16(t_dv, dPm + mstep(k), dDOm + mstep(k), id_tn, (it | k) != 0);
        umma_commit(do_free);
        // dQ = dS K  (A K-major over keys, B = K tile read MN-major), into the columns S occupied
#pragma unroll
        for (int k = 0; k < AB_B / 16; ++k)
          umma_bf16(t_s, dDSk + kstep(k), dKm + mstep(k), id_dq, k != 0);
        umma_commit(mma_done);
        MTB_STAMP(blockIdx.x == 0, it, 3);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ dQ reduce warp
    if (elect_one()) {
      uint8_t* stage_a = smem + L::OFF_P;     // boxes 0 .. D/64-1
      uint8_t* stage_b = smem + L::OFF_ST2;   // boxes D/64 .. D/32-1
      for (int it = 0; it < n_iters; ++it) {
        const int h = hk * G + it / per_head, i = jblk + it % per_head;
        if (!mbar_wait(stage_full, it & 1, abort_flag)) { atomicExch(p.status, 30); goto done; }
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                       ::"l"(reinterpret_cast<uint64_t>(&tm_dq)), "r"(smem_u32(stage_a + c * 16384)), "r"(h * D + c * 32),
                         "r"(seq_start + i * AB_B) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        // The second half is only issued once the P tile has been read: boxes in flight together share
        // the read-out bandwidth, and the next softmax is waiting for the P tile alone.
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        mbar_arrive(stage_free);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                       ::"l"(reinterpret_cast<uint64_t>(&tm_dq)), "r"(smem_u32(stage_b + c * 16384)), "r"(h * D + (D / 64 + c) * 32),
                         "r"(seq_start + i * AB_B) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        mbar_arrive(st2_free);
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every add has been performed before the CTA exits
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;      // which 64 key columns (softmax) / which half of the D columns (drains)
    const int r = q * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    const int HqD = p.Hq * D;
    for (int it = 0; it < n_iters; ++it) {
      const int h = hk * G + it / per_head, i = jblk + it % per_head;
      const int qpos = i * AB_B + r;
      const bool qok = qpos < seq_len;
      const long long tok = static_cast<long long>(seq_start) + qpos;
      const float lse2 = qok ? p.lse[static_cast<long long>(h) * p.T + tok] * 1.4426950408889634f : 0.f;
      const float delta = qok ? p.delta[static_cast<long long>(h) * p.T + tok] : 0.f;
      if (!mbar_wait(sdp_full, it & 1, abort_flag)) { atomicExch(p.status, 26); goto done; }
      tc_fence_after();
      MTB_STAMP(blockIdx.x == 0 && threadIdx.x == 64, it, 4);
      const bool need_mask = (i == jblk) || (k0 + AB_B > seq_len) || (i * AB_B + AB_B > seq_len);
      // this thread's 64 columns of S and dP are fetched with all four loads in flight
      uint32_t sv_[2][32], dv_[2][32];
      tmem_ld_32x32(t_s + lane_addr + (half * 2) * 32, sv_[0]);
      tmem_ld_32x32(t_dp + lane_addr + (half * 2) * 32, dv_[0]);
      tmem_ld_32x32(t_s + lane_addr + (half * 2 + 1) * 32, sv_[1]);
      tmem_ld_32x32(t_dp + lane_addr + (half * 2 + 1) * 32, dv_[1]);
      tmem_ld_wait();
      if (need_mask) {   // diagonal block, last key block or last query block: out-of-range entries get P = 0
#pragma unroll
        for (int cc = 0; cc < 2; ++cc)
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            const int kpos = k0 + (half * 2 + cc) * 32 + x;
            if (!qok || kpos > qpos || kpos >= seq_len) sv_[cc][x] = 0xff800000u;   // exp2(-inf) = 0
          }
      }
      // The P tile still holds half of the previous dQ tile until its reduces have read it. The first 32
      // columns are computed before that wait; their stores then overlap the math of the other 32.
      uint32_t pk[2][16], dk[2][16];
      const float2 sl2v = make_float2(sl2, sl2), nlse = make_float2(-lse2, -lse2);
      const float2 scv = make_float2(p.scale, p.scale), nds = make_float2(-delta * p.scale, -delta * p.scale);
      auto compute = [&](int cc) {
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          // packed fp32 pairs: one FMA scales and shifts two scores, one FMA forms (dP - delta) * scale for both
          const float2 a = ffma2(make_float2(__uint_as_float(sv_[cc][x]), __uint_as_float(sv_[cc][x + 1])), sl2v, nlse);
          // a quarter of the exponentials runs on the FMA pipe: the special-function unit bounds this phase
          const float2 pr = make_float2(ex2_mufu(a.x), (x & 2) ? ex2_fma(a.y) : ex2_mufu(a.y));
          const float2 dd = ffma2(make_float2(__uint_as_float(dv_[cc][x]), __uint_as_float(dv_[cc][x + 1])), scv, nds);
          const float2 ds = fmul2(pr, dd);
          pk[cc][x >> 1] = pack_bf16(pr.x, pr.y);
          dk[cc][x >> 1] = pack_bf16(ds.x, ds.y);
        }
      };
      auto store = [&](int cc) {
        const int c = half * 2 + cc;
        const int rowoff = (c >> 1) * 16384 + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = (((c & 1) * 4 + g) ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(smem + L::OFF_P + rowoff + chunk) = make_uint4(pk[cc][g * 4], pk[cc][g * 4 + 1], pk[cc][g * 4 + 2], pk[cc][g * 4 + 3]);
          *reinterpret_cast<uint4*>(smem + L::OFF_DS + rowoff + chunk) = make_uint4(dk[cc][g * 4], dk[cc][g * 4 + 1], dk[cc][g * 4 + 2], dk[cc][g * 4 + 3]);
        }
      };
      compute(0);
      MTB_STAMP(blockIdx.x == 0 && threadIdx.x == 64, it, 5);
      if (it > 0 && !mbar_wait(stage_free, (it - 1) & 1, abort_flag)) { atomicExch(p.status, 27); goto done; }
      MTB_STAMP(blockIdx.x == 0 && threadIdx.x == 64, it, 6);
      store(0);
      compute(1);
      store(1);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready);
      // drain dQ: TMEM -> fp32 staging (128B-swizzled boxes); the reduce warp adds the boxes into global memory
      if (!mbar_wait(mma_done, it & 1, abort_flag)) { atomicExch(p.status, 28); goto done; }
      if (half == 1 && it > 0 && !mbar_wait(st2_free, (it - 1) & 1, abort_flag)) { atomicExch(p.status, 31); goto done; }
      tc_fence_after();
      MTB_STAMP(blockIdx.x == 0 && threadIdx.x == 64, it, 7);
      uint8_t* stage = half == 0 ? smem + L::OFF_P : smem + L::OFF_ST2;
      // both loads in flight; the S columns are released as soon as the tile is in registers, so the
      // next S = Q K^T runs under the staging stores
      uint32_t v[D / 64][32];
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) tmem_ld_32x32(t_s + lane_addr + (half * (D / 64) + cc) * 32, v[cc]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_read);
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        uint8_t* rowp = stage + cc * 16384 + r * 128;
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<uint4*>(rowp + ((g ^ (r & 7)) << 4)) = make_uint4(v[cc][g * 4], v[cc][g * 4 + 1], v[cc][g * 4 + 2], v[cc][g * 4 + 3]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(stage_full);
      MTB_STAMP(blockIdx.x == 0 && threadIdx.x == 64, it, 8);
    }
    // epilogue: dK, dV (rows = keys)
    if (n_iters > 0) {
      if (!mbar_wait(mma_done, (n_iters - 1) & 1, abort_flag)) { atomicExch(p.status, 29); goto done; }
      tc_fence_after();
      const int kpos = k0 + r;
      const bool ok = kpos < seq_len;
      __nv_bfloat16* rowp = p.dqkv + (static_cast<long long>(seq_start) + kpos) * p.ldq;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = (which == 0 ? t_dk : t_dv) + lane_addr;
        __nv_bfloat16* o = rowp + (which == 0 ? (p.Hq + hk) * D : (p.Hq + p.Hkv + hk) * D);
#pragma unroll 1
        for (int cc = 0; cc < D / 64; ++cc) {
          const int c = half * (D / 64) + cc;
          uint32_t v[32];
          tmem_ld_32x32(src + c * 32, v);
          tmem_ld_wait();
          if (ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
              *reinterpret_cast<uint4*>(o + c * 32 + g * 8) =
                  make_uint4(pack_bf16(__uint_as_float(v[g * 8]), __uint_as_float(v[g * 8 + 1])),
                             pack_bf16(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3])),
                             pack_bf16(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5])),
                             pack_bf16(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7])));
          }
        }
      }
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

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h).
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long ldo, const __nv_bfloat16* __restrict__ dout,
                                                        long long lddo, float* __restrict__ delta, int T, int Hq, int D) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(T) * Hq) return;
  const int t = static_cast<int>(w / Hq), h = static_cast<int>(w % Hq);
  const __nv_bfloat16* a = o + static_cast<long long>(t) * ldo + h * D;
  const __nv_bfloat16* b = dout + static_cast<long long>(t) * lddo + h * D;
  float s = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + c));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + c));
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

// dqkv[t, 0:Hq*D] = bf16(dq_acc[t, :])
__global__ void __launch_bounds__(256) attn_dq_store_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv, long long ldq,
                                                           long long T, int HqD) {
  // grid = (tokens, column blocks): no 64-bit division per thread
  const long long t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= HqD) return;
  const float4 a = *reinterpret_cast<const float4*>(acc + t * HqD + c), b = *reinterpret_cast<const float4*>(acc + t * HqD + c + 4);
  *reinterpret_cast<uint4*>(dqkv + t * ldq + c) =
      make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
}

template <int D>
static int launch_bwd(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const AttBwdParams& p, int n_items, cudaStream_t st) {
  static bool configured = false;
  auto kern = attn_bwd_kernel<D>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttBwdSmem<D>::TOTAL) != cudaSuccess) return -4;
    configured = true;
  }
  kern<<<n_items * p.Hkv, AB_THREADS, AttBwdSmem<D>::TOTAL, st>>>(a, b, c, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace mtb

// plan: key-block work table [n_items, 3] = (seq_start, seq_len, k0), most work first.
// dq_acc: zero-initialised fp32 [T, Hq*D] scratch; delta: fp32 [Hq, T] scratch.
extern "C" int mtb200_attn_bwd(const void* qkv, long long ld, const void* out, long long ldo, const void* dout, long long lddo,
                               void* dqkv, long long ldq, const float* lse, float* delta, float* dq_acc, const int* plan,
                               int n_items, int T, int Hq, int Hkv, int D, int reserved, float scale, int* status, cudaStream_t st) {
  using namespace mtb;
  if (n_items <= 0 || T <= 0) return 0;
  if ((D != 64 && D != 128) || Hq % Hkv || ld % 8 || ldo % 8 || lddo % 8 || ldq % 8) return -10;
  CUtensorMap tq, tdo, tdq;
  int rc = make_tmap_2d_bf16(&tq, qkv, static_cast<uint64_t>(ld), static_cast<uint64_t>(T), static_cast<uint64_t>(ld), 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tdo, dout, static_cast<uint64_t>(Hq) * D, static_cast<uint64_t>(T), static_cast<uint64_t>(lddo), 64, 128);
  if (rc) return rc - 10;
  rc = make_tmap_2d_f32(&tdq, dq_acc, static_cast<uint64_t>(Hq) * D, static_cast<uint64_t>(T), static_cast<uint64_t>(Hq) * D, 32, 128);
  if (rc) return rc - 20;
  const long long warps = static_cast<long long>(T) * Hq;
  attn_delta_kernel<<<static_cast<int>((warps * 32 + 255) / 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(out), ldo, reinterpret_cast<const __nv_bfloat16*>(dout), lddo, delta, T, Hq, D);
  (void)reserved;
  AttBwdParams p{reinterpret_cast<__nv_bfloat16*>(dqkv), ldq, lse, delta, dq_acc, plan, T, Hq, Hkv, scale, status};
  rc = D == 128 ? launch_bwd<128>(tq, tdo, tdq, p, n_items, st) : launch_bwd<64>(tq, tdo, tdq, p, n_items, st);
  if (rc) return rc;
  attn_dq_store_kernel<<<dim3(static_cast<unsigned>(T), (Hq * D / 8 + 255) / 256), 256, 0, st>>>(dq_acc, reinterpret_cast<__nv_bfloat16*>(dqkv), ldq, T, Hq * D);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

#ifdef MTB200_ATTN_BWD_TIMESTAMPS
// Copies the phase timestamps recorded by the last launch to the host (development builds only).
extern "C" int mtb200_attn_bwd_debug_read(long long* out, int n) {
  if (n > mtb::DBG_ITERS * 9) n = mtb::DBG_ITERS * 9;
  return cudaMemcpyFromSymbol(out, mtb::g_attn_bwd_dbg, sizeof(long long) * n) == cudaSuccess ? 0 : -1;
}
#endif
