// Bandwidth-bound kernels: RMSNorm (+residual gradient), RoPE, SwiGLU, embedding gather,
// cross-entropy over a logits chunk, column sums (bias gradient), gradient accumulation,
// sum of squares and the fused AdamW update. All use 128-bit accesses, fp32 math and bf16 storage.
//
// These replace what the reference gets from Liger's Triton kernels (rms_norm, rope, swiglu,
// cross_entropy) and ATen foreach ops (clip, AdamW).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace mtb {

constexpr int EW_THREADS = 256;

struct bf16x8 {
  uint4 u;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { u = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = u; }
  __device__ __forceinline__ void to_float(float (&f)[8]) const {
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  __device__ __forceinline__ void from_float(const float (&f)[8]) {
    u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]); u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
  }
};

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (w == 0) t = warp_sum(t);
  if (threadIdx.x == 0) red[0] = t;
  __syncthreads();
  return red[0];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : -INFINITY;
  if (w == 0) t = warp_max(t);
  if (threadIdx.x == 0) red[0] = t;
  __syncthreads();
  return red[0];
}

// ------------------------------------------------------------------------------ RMSNorm fwd
// y = bf16(x * rstd) * w ; rstd saved. A row is read ONCE: a group of LANES threads (one to eight
// warps) holds it in registers, VPT 8-wide vectors per thread with all loads issued before the first
// use, and a 256-thread block works on 256 / LANES rows at a time. One block-wide barrier per row set
// (none when a row fits one warp).
template <int VPT>
__global__ void __launch_bounds__(EW_THREADS) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                                __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                                                                float eps, int T, int H, int lanes) {
  __shared__ float red[EW_THREADS / 32];
  const int rows_per_block = EW_THREADS / lanes;
  const int sub = threadIdx.x / lanes, l = threadIdx.x % lanes;
  const long long row = static_cast<long long>(blockIdx.x) * rows_per_block + sub;
  const bool row_ok = row < T;
  const __nv_bfloat16* xr = x + row * H;
  bf16x8 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = (l + k * lanes) * 8;
    if (row_ok && c < H) v[k].load(xr + c); else v[k].u = make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    float f[8]; v[k].to_float(f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  if (lanes > 32) {   // uniform over the block
    const int wid = threadIdx.x >> 5, wpr = lanes >> 5;
    if ((threadIdx.x & 31) == 0) red[wid] = ss;
    __syncthreads();
    ss = 0.f;
    for (int k = 0; k < wpr; ++k) ss += red[sub * wpr + k];
  }
  if (!row_ok) return;
  const float rstd = rsqrtf(ss / H + eps);
  if (l == 0) rstd_out[row] = rstd;
  __nv_bfloat16* yr = y + row * H;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = (l + k * lanes) * 8;
    if (c < H) {
      bf16x8 wv; wv.load(w + c);
      float f[8], g[8]; v[k].to_float(f); wv.to_float(g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] * rstd)) * g[i];
      bf16x8 o; o.from_float(f); o.store(yr + c);
    }
  }
}

// ------------------------------------------------------------------------------ RMSNorm bwd
// dx = rstd * (g - xhat * mean(g * xhat)) (+ add_to), g = dy * w, xhat = x * rstd
// dw partial per block in fp32: dwp[block, H] += dy * bf16(xhat). Persistent blocks loop over rows.
// Wide rows use 512 threads with one or two vectors each: half the registers per thread of the 256-thread
// form, so twice the warps stay resident and more loads are in flight around the per-row reduction.
template <int VPT, int THREADS>  // 8-wide vectors per thread; H <= VPT * 8 * THREADS
__global__ void __launch_bounds__(THREADS) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ w,
                                                                const __nv_bfloat16* __restrict__ add_to, __nv_bfloat16* __restrict__ dx,
                                                                float* __restrict__ dwp, int T, int H) {
  __shared__ float red[32];
  float dwacc[VPT][8];
  float wreg[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int c = (threadIdx.x + v * THREADS) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) { dwacc[v][i] = 0.f; wreg[v][i] = 0.f; }
    if (c < H) { bf16x8 wv; wv.load(w + c); wv.to_float(wreg[v]); }
  }
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float g[VPT][8], xh[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = (threadIdx.x + v * THREADS) * 8;
      if (c < H) {
        bf16x8 a, b; a.load(dy + row * H + c); b.load(x + row * H + c);
        float fa[8], fb[8]; a.to_float(fa); b.to_float(fb);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[v][i] = fb[i] * rstd;
          g[v][i] = fa[i] * wreg[v][i];
          dot += g[v][i] * xh[v][i];
          dwacc[v][i] += fa[i] * __bfloat162float(__float2bfloat16(xh[v][i]));
        }
      }
    }
    dot = block_sum(dot, red) / H;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = (threadIdx.x + v * THREADS) * 8;
      if (c < H) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (g[v][i] - xh[v][i] * dot);
        if (add_to != nullptr) {
          bf16x8 r; r.load(add_to + row * H + c);
          float fr[8]; r.to_float(fr);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += fr[i];
        }
        bf16x8 ov; ov.from_float(o); ov.store(dx + row * H + c);
      }
    }
  }
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int c = (threadIdx.x + v * THREADS) * 8;
    if (c < H) {
      float* dst = dwp + static_cast<long long>(blockIdx.x) * H + c;
      *reinterpret_cast<float4*>(dst) = make_float4(dwacc[v][0], dwacc[v][1], dwacc[v][2], dwacc[v][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[v][4], dwacc[v][5], dwacc[v][6], dwacc[v][7]);
    }
  }
}

// out[c] = bf16(sum_r part[r, c]); one thread per column, coalesced across threads.
__global__ void reduce_rows_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int R, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int r = 0; r < R; ++r) s += part[static_cast<long long>(r) * C + c];
  out[c] = __float2bfloat16(s);
}

// Same for rows that hold two vectors of D columns each, delivered to two outputs.
__global__ void reduce_rows_pair_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out_a, __nv_bfloat16* __restrict__ out_b,
                                        int R, int D) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= 2 * D) return;
  float s = 0.f;
  for (int r = 0; r < R; ++r) s += part[static_cast<long long>(r) * 2 * D + c];
  if (c < D) out_a[c] = __float2bfloat16(s); else out_b[c - D] = __float2bfloat16(s);
}

// ------------------------------------------------------------------------------ LayerNorm (Starcoder2)
// y = ((x - mean) * rstd) * w + b, statistics in fp32 over the row held in registers (two-pass: the mean first, then
// the centred sum of squares), mean and rstd saved. One 256-thread block per row, VPT 8-wide vectors per thread.
template <int VPT>
__global__ void __launch_bounds__(EW_THREADS) layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                                  const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                                  float* __restrict__ mean_out, float* __restrict__ rstd_out, float eps, int H) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  float f[VPT][8];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = (threadIdx.x + k * EW_THREADS) * 8;
    if (c < H) {
      bf16x8 v; v.load(xr + c); v.to_float(f[k]);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += f[k][i];
    }
  }
  const float mean = block_sum(s, red) / H;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = (threadIdx.x + k * EW_THREADS) * 8;
    if (c < H) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { f[k][i] -= mean; ss += f[k][i] * f[k][i]; }
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / H + eps);
  if (threadIdx.x == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = (threadIdx.x + k * EW_THREADS) * 8;
    if (c < H) {
      bf16x8 wv, bv; wv.load(w + c); bv.load(b + c);
      float fw[8], fb[8], o[8]; wv.to_float(fw); bv.to_float(fb);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = f[k][i] * rstd * fw[i] + fb[i];
      bf16x8 ov; ov.from_float(o); ov.store(y + row * H + c);
    }
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) (+ add_to), g = dy * w, xhat = (x - mean) * rstd.
// Partials per block in fp32: dwp[block, 0, :] += dy * xhat, dwp[block, 1, :] += dy (the bias gradient); summed over
// blocks by reduce_rows_pair_kernel. Persistent blocks loop over rows.
template <int VPT>
__global__ void __launch_bounds__(EW_THREADS) layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                  const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                                                  const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ add_to,
                                                                  __nv_bfloat16* __restrict__ dx, float* __restrict__ dwp, int T, int H) {
  __shared__ float red[32];
  float dwacc[VPT][8], dbacc[VPT][8], wreg[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int c = (threadIdx.x + v * EW_THREADS) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) { dwacc[v][i] = 0.f; dbacc[v][i] = 0.f; wreg[v][i] = 0.f; }
    if (c < H) { bf16x8 wv; wv.load(w + c); wv.to_float(wreg[v]); }
  }
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    float g[VPT][8], xh[VPT][8];
    float d1 = 0.f, d2 = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = (threadIdx.x + v * EW_THREADS) * 8;
      if (c < H) {
        bf16x8 a, b; a.load(dy + row * H + c); b.load(x + row * H + c);
        float fa[8], fb[8]; a.to_float(fa); b.to_float(fb);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[v][i] = (fb[i] - mean) * rstd;
          g[v][i] = fa[i] * wreg[v][i];
          d1 += g[v][i];
          d2 += g[v][i] * xh[v][i];
          dwacc[v][i] += fa[i] * xh[v][i];
          dbacc[v][i] += fa[i];
        }
      }
    }
    d1 = block_sum(d1, red) / H;
    d2 = block_sum(d2, red) / H;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = (threadIdx.x + v * EW_THREADS) * 8;
      if (c < H) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (g[v][i] - d1 - xh[v][i] * d2);
        if (add_to != nullptr) {
          bf16x8 r; r.load(add_to + row * H + c);
          float fr[8]; r.to_float(fr);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += fr[i];
        }
        bf16x8 ov; ov.from_float(o); ov.store(dx + row * H + c);
      }
    }
  }
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int c = (threadIdx.x + v * EW_THREADS) * 8;
    if (c < H) {
      float* dst = dwp + static_cast<long long>(blockIdx.x) * 2 * H + c;
      *reinterpret_cast<float4*>(dst) = make_float4(dwacc[v][0], dwacc[v][1], dwacc[v][2], dwacc[v][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[v][4], dwacc[v][5], dwacc[v][6], dwacc[v][7]);
      *reinterpret_cast<float4*>(dst + H) = make_float4(dbacc[v][0], dbacc[v][1], dbacc[v][2], dbacc[v][3]);
      *reinterpret_cast<float4*>(dst + H + 4) = make_float4(dbacc[v][4], dbacc[v][5], dbacc[v][6], dbacc[v][7]);
    }
  }
}

// ------------------------------------------------------------------------------ RoPE
// In place on the first n_heads (q then k) heads of each row of qkv[T, ld]. Rotate-half
// convention: (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin), angle = fp32(pos) * inv_freq[i]
// (the fp32 product and fp32 sine / cosine that the Hugging Face rotary embedding computes).
// A thread owns 8 frequencies of one token for ROPE_HPT consecutive heads (grid.y = head groups):
// all of its loads are issued before the first store, so a thread keeps 2 * ROPE_HPT 16-byte loads in flight.
constexpr int ROPE_HPT = 4;
__global__ void __launch_bounds__(EW_THREADS) rope_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                                                         const float* __restrict__ inv_freq, int T, long long ld,
                                                         int n_heads, int D, float sign) {
  const int half = D >> 1;
  const int vec_per_tok = half >> 3;  // 8 frequencies per thread
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<long long>(T) * vec_per_tok) return;
  const int t = static_cast<int>(gid / vec_per_tok);
  const int i0 = static_cast<int>(gid % vec_per_tok) * 8;
  const int h0 = blockIdx.y * ROPE_HPT;
  __nv_bfloat16* row = qkv + static_cast<long long>(t) * ld;
  bf16x8 a[ROPE_HPT], b[ROPE_HPT];
#pragma unroll
  for (int j = 0; j < ROPE_HPT; ++j) {
    if (h0 + j < n_heads) { a[j].load(row + (h0 + j) * D + i0); b[j].load(row + (h0 + j) * D + i0 + half); }
  }
  const float p = static_cast<float>(pos[t]);
  float cs[8], sn[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    sincosf(p * inv_freq[i0 + i], &sn[i], &cs[i]);
    sn[i] *= sign;
  }
#pragma unroll
  for (int j = 0; j < ROPE_HPT; ++j) {
    if (h0 + j < n_heads) {
      float x1[8], x2[8], o1[8], o2[8]; a[j].to_float(x1); b[j].to_float(x2);
#pragma unroll
      for (int i = 0; i < 8; ++i) { o1[i] = x1[i] * cs[i] - x2[i] * sn[i]; o2[i] = x2[i] * cs[i] + x1[i] * sn[i]; }
      a[j].from_float(o1); b[j].from_float(o2);
      a[j].store(row + (h0 + j) * D + i0); b[j].store(row + (h0 + j) * D + i0 + half);
    }
  }
}

// ------------------------------------------------------------------------------ per-head RMSNorm (q_norm / k_norm)
// Qwen3 normalises every q and k head over head_dim before the rotary embedding, with one weight vector for all q
// heads and one for all k heads. In place on the first n_heads (q then k) heads of each row of qkv[T, ld]: one warp per
// (token, head), a lane holds EPL = head_dim / 32 consecutive elements, the sum of squares is a shuffle reduction.
// y = bf16(x * rstd) * w, rstd[token * n_heads + head] saved.
template <int EPL>
struct HeadVec {
  uint32_t raw[EPL / 2];
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    if constexpr (EPL == 8) { const uint4 v = *reinterpret_cast<const uint4*>(p); raw[0] = v.x; raw[1] = v.y; raw[2] = v.z; raw[3] = v.w; }
    else if constexpr (EPL == 4) { const uint2 v = *reinterpret_cast<const uint2*>(p); raw[0] = v.x; raw[1] = v.y; }
    else { raw[0] = *reinterpret_cast<const uint32_t*>(p); }
  }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const {
    if constexpr (EPL == 8) *reinterpret_cast<uint4*>(p) = make_uint4(raw[0], raw[1], raw[2], raw[3]);
    else if constexpr (EPL == 4) *reinterpret_cast<uint2*>(p) = make_uint2(raw[0], raw[1]);
    else *reinterpret_cast<uint32_t*>(p) = raw[0];
  }
  __device__ __forceinline__ void to_float(float (&f)[EPL]) const {
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) { const float2 a = unpack_bf16(raw[i]); f[2 * i] = a.x; f[2 * i + 1] = a.y; }
  }
  __device__ __forceinline__ void from_float(const float (&f)[EPL]) {
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) raw[i] = pack_bf16(f[2 * i], f[2 * i + 1]);
  }
};

template <int EPL>
__global__ void __launch_bounds__(EW_THREADS) head_rmsnorm_fwd_kernel(__nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
                                                                     const __nv_bfloat16* __restrict__ wk, float* __restrict__ rstd_out,
                                                                     float eps, long long n_rows, long long ld, int n_q, int n_heads) {
  constexpr int D = EPL * 32;
  const long long r = static_cast<long long>(blockIdx.x) * (EW_THREADS / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= n_rows) return;   // whole warps leave together
  const long long t = r / n_heads;
  const int h = static_cast<int>(r - t * n_heads);
  __nv_bfloat16* p = qkv + t * ld + static_cast<long long>(h) * D + lane * EPL;
  HeadVec<EPL> xv, wv;
  xv.load(p);
  wv.load((h < n_q ? wq : wk) + lane * EPL);
  float f[EPL], g[EPL];
  xv.to_float(f); wv.to_float(g);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) ss += f[i] * f[i];
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / D + eps);
  if (lane == 0) rstd_out[r] = rstd;
#pragma unroll
  for (int i = 0; i < EPL; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] * rstd)) * g[i];
  xv.from_float(f);
  xv.store(p);
}

// Backward, in place on dqkv (gradient of the normalised heads in, gradient of the projection output out):
// dx = rstd * (g - xhat * mean(g * xhat)), g = dy * w, xhat = x * rstd with x the heads BEFORE the norm (pre[T, ld_pre],
// q then k heads). Weight gradients: dwp[block, 2, D] += dy * bf16(xhat) per block in fp32 (q heads in row 0, k heads in
// row 1), summed over blocks by reduce_rows_kernel: no atomics. Persistent warps loop over (token, head) rows; a lane
// keeps the same columns throughout, so its partial sums stay in registers.
template <int EPL>
__global__ void __launch_bounds__(EW_THREADS) head_rmsnorm_bwd_kernel(__nv_bfloat16* __restrict__ dqkv, const __nv_bfloat16* __restrict__ pre,
                                                                     const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ wq,
                                                                     const __nv_bfloat16* __restrict__ wk, float* __restrict__ dwp,
                                                                     long long n_rows, long long ld, long long ld_pre, int n_q, int n_heads) {
  constexpr int D = EPL * 32;
  constexpr int WARPS = EW_THREADS / 32;
  __shared__ float sm[WARPS][2][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float wqf[EPL], wkf[EPL], accq[EPL], acck[EPL];
  {
    HeadVec<EPL> a, b;
    a.load(wq + lane * EPL); b.load(wk + lane * EPL);
    a.to_float(wqf); b.to_float(wkf);
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i) { accq[i] = 0.f; acck[i] = 0.f; }
  const long long stride = static_cast<long long>(gridDim.x) * WARPS;
  for (long long r = static_cast<long long>(blockIdx.x) * WARPS + warp; r < n_rows; r += stride) {
    const long long t = r / n_heads;
    const int h = static_cast<int>(r - t * n_heads);
    const bool is_q = h < n_q;
    __nv_bfloat16* gp = dqkv + t * ld + static_cast<long long>(h) * D + lane * EPL;
    HeadVec<EPL> gv, xv;
    gv.load(gp);
    xv.load(pre + t * ld_pre + static_cast<long long>(h) * D + lane * EPL);
    const float rstd = rstd_in[r];
    float dy[EPL], x[EPL], g[EPL], xh[EPL];
    gv.to_float(dy); xv.to_float(x);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      xh[i] = x[i] * rstd;
      g[i] = dy[i] * (is_q ? wqf[i] : wkf[i]);
      dot += g[i] * xh[i];
      const float c = dy[i] * __bfloat162float(__float2bfloat16(xh[i]));
      if (is_q) accq[i] += c; else acck[i] += c;
    }
    dot = warp_sum(dot) / D;
#pragma unroll
    for (int i = 0; i < EPL; ++i) g[i] = rstd * (g[i] - xh[i] * dot);
    gv.from_float(g);
    gv.store(gp);
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i) { sm[warp][0][lane * EPL + i] = accq[i]; sm[warp][1][lane * EPL + i] = acck[i]; }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * D; c += EW_THREADS) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) s += sm[w][c / D][c % D];
    dwp[static_cast<long long>(blockIdx.x) * 2 * D + c] = s;
  }
}

// ------------------------------------------------------------------------------ gated MLP activations
// act(gate) * up over gu = [gate | up]. ACT 0: SiLU (SwiGLU: Llama, Qwen, Mistral, Granite, Mixtral, Phi-3);
// ACT 1: tanh-approximated GELU (GeGLU: Gemma's gelu_pytorch_tanh).
template <int ACT>
__device__ __forceinline__ float glu_act(float g) {
  if constexpr (ACT == 0) {
    return __fdividef(g, 1.f + __expf(-g));
  } else {
    const float th = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
    return 0.5f * g * (1.f + th);
  }
}
// d act(g) / d g
template <int ACT>
__device__ __forceinline__ float glu_act_grad(float g) {
  if constexpr (ACT == 0) {
    const float sig = __fdividef(1.f, 1.f + __expf(-g));
    return sig * (1.f + g * (1.f - sig));
  } else {
    const float th = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
    return 0.5f * (1.f + th) + 0.5f * g * (1.f - th * th) * 0.7978845608028654f * (1.f + 0.134145f * g * g);
  }
}

template <int ACT>
__global__ void __launch_bounds__(EW_THREADS) swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                                                               long long T, int F) {
  // grid = (tokens, column blocks): no 64-bit division per thread
  const long long t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= F) return;
  bf16x8 g, u; g.load(gu + t * 2 * F + c); u.load(gu + t * 2 * F + F + c);
  float fg[8], fu[8], o[8]; g.to_float(fg); u.to_float(fu);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = glu_act<ACT>(fg[i]) * fu[i];
  g.from_float(o); g.store(act + t * F + c);
}

// WITH_ACT: the forward output act(gate) * up is also produced, written over dact (each thread reads its
// dact vector before it stores there), for a backward that did not keep it: one pass over gate/up
// instead of a forward kernel plus this one.
template <bool WITH_ACT, int ACT>
__global__ void __launch_bounds__(EW_THREADS) swiglu_bwd_kernel(__nv_bfloat16* dact, const __nv_bfloat16* __restrict__ gu,
                                                               __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  // grid = (tokens, column blocks): no 64-bit division per thread
  const long long t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= F) return;
  bf16x8 g, u, d; g.load(gu + t * 2 * F + c); u.load(gu + t * 2 * F + F + c); d.load(dact + t * F + c);
  float fg[8], fu[8], fd[8], og[8], ou[8]; g.to_float(fg); u.to_float(fu); d.to_float(fd);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if constexpr (ACT == 0) {
      const float sig = __fdividef(1.f, 1.f + __expf(-fg[i]));
      og[i] = fd[i] * fu[i] * sig * (1.f + fg[i] * (1.f - sig));
      ou[i] = fd[i] * fg[i] * sig;
    } else {
      og[i] = fd[i] * fu[i] * glu_act_grad<ACT>(fg[i]);
      ou[i] = fd[i] * glu_act<ACT>(fg[i]);
    }
  }
  if (WITH_ACT) {
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = glu_act<ACT>(fg[i]) * fu[i];   // same expression as the forward kernel
    d.from_float(o); d.store(dact + t * F + c);
  }
  g.from_float(og); u.from_float(ou);
  g.store(dgu + t * 2 * F + c); u.store(dgu + t * 2 * F + F + c);
}

// Plain (not gated) activation over n elements, forward and backward: Starcoder2's MLP is c_proj(gelu(c_fc(x))).
template <int ACT>
__global__ void __launch_bounds__(EW_THREADS) act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  const long long i0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i0 >= n) return;
  bf16x8 v; v.load(x + i0);
  float f[8]; v.to_float(f);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = glu_act<ACT>(f[i]);
  v.from_float(f); v.store(y + i0);
}
template <int ACT>
__global__ void __launch_bounds__(EW_THREADS) act_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                            __nv_bfloat16* __restrict__ dx, long long n) {
  const long long i0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i0 >= n) return;
  bf16x8 v, d; v.load(x + i0); d.load(dy + i0);
  float f[8], g[8]; v.to_float(f); d.to_float(g);
#pragma unroll
  for (int i = 0; i < 8; ++i) g[i] *= glu_act_grad<ACT>(f[i]);
  d.from_float(g); d.store(dx + i0);
}

// ------------------------------------------------------------------------------ embedding
// An id outside [0, V) (a tokenizer larger than the embedding table) is not dereferenced: the row is zero-filled
// and code 60 is recorded in the status word, which the host turns into an exception.
__global__ void __launch_bounds__(128) embedding_fwd_kernel(const __nv_bfloat16* __restrict__ w, const long long* __restrict__ ids,
                                                           __nv_bfloat16* __restrict__ out, int H, int V, int* status) {
  const long long t = blockIdx.x;
  const long long id = ids[t];
  __nv_bfloat16* dst = out + t * H;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 60);
    for (int c = threadIdx.x * 8; c < H; c += 128 * 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const __nv_bfloat16* src = w + id * H;
  for (int c = threadIdx.x * 8; c < H; c += 128 * 8) *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
}

// dW[id, :] += sum over the tokens t with ids[t] == id of dx[t, :], deterministic: the token ids arrive
// sorted (stable, so equal ids keep their token order) with the permutation that sorted them. The block
// at the first position of each run of equal ids sums the run's rows in fp32, in that fixed order, adds
// what dW already holds (the LM-head gradient when the embeddings are tied) and rounds once. The other
// blocks of the run exit at once. No atomics, so the result does not depend on scheduling.
__global__ void __launch_bounds__(128) embedding_bwd_kernel(__nv_bfloat16* __restrict__ dw, const long long* __restrict__ sorted_ids,
                                                           const long long* __restrict__ order, const __nv_bfloat16* __restrict__ dx,
                                                           int T, int H, int V, int* status) {
  const int j = blockIdx.x;
  const long long id = sorted_ids[j];
  if (j > 0 && sorted_ids[j - 1] == id) return;
  if (id < 0 || id >= V) {   // skipped and reported, never dereferenced
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 60);
    return;
  }
  __nv_bfloat16* dst = dw + id * H;
  for (int c = threadIdx.x * 8; c < H; c += 128 * 8) {
    float acc[8];
    {
      const uint4 v = *reinterpret_cast<const uint4*>(dst + c);
      const float2 a0 = unpack_bf16(v.x), a1 = unpack_bf16(v.y), a2 = unpack_bf16(v.z), a3 = unpack_bf16(v.w);
      acc[0] = a0.x; acc[1] = a0.y; acc[2] = a1.x; acc[3] = a1.y; acc[4] = a2.x; acc[5] = a2.y; acc[6] = a3.x; acc[7] = a3.y;
    }
    for (int k = j; k < T && sorted_ids[k] == id; ++k) {
      const uint4 v = *reinterpret_cast<const uint4*>(dx + order[k] * H + c);
      const float2 a0 = unpack_bf16(v.x), a1 = unpack_bf16(v.y), a2 = unpack_bf16(v.z), a3 = unpack_bf16(v.w);
      acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y; acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
    }
    *reinterpret_cast<uint4*>(dst + c) = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

// ------------------------------------------------------------------------------ cross-entropy
// One block per row of a logits chunk ([R, V] fp32 or bf16, leading dimension ld). Pass 1: online
// max / sum-exp. Pass 2: dlogits = (softmax - onehot) * scale in bf16. Rows whose target is
// ignore_index get zero loss and zero gradient. With bf16 logits the gradient may be written over
// the logits (dlogits == logits): a thread reads a vector of the row before it overwrites the same
// vector, and pass 2 starts after the block-wide reductions that end pass 1.
template <typename LogitT>
__device__ __forceinline__ void load8(const LogitT* p, float (&f)[8]) {
  if constexpr (sizeof(LogitT) == 2) { bf16x8 v; v.load(reinterpret_cast<const __nv_bfloat16*>(p)); v.to_float(f); }
  else {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
}

template <typename LogitT>
__global__ void __launch_bounds__(1024) ce_fwd_bwd_kernel(const LogitT* logits, long long ld, const long long* __restrict__ targets,
                                                         float* __restrict__ loss, __nv_bfloat16* dlogits, long long ldd,
                                                         int V, float grad_scale, long long ignore_index) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const LogitT* lr = logits + row * ld;
  __nv_bfloat16* dr = dlogits + row * ldd;
  const long long tgt = targets[row];
  if (tgt == ignore_index) {
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) *reinterpret_cast<uint4*>(dr + c) = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) loss[row] = 0.f;
    return;
  }
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    float v[8];
    load8(lr + c, v);
    float mx = v[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, v[i]);
    if (mx > m) { s *= __expf(m - mx); m = mx; }
#pragma unroll
    for (int i = 0; i < 8; ++i) s += __expf(v[i] - m);
  }
  const float gm = block_max(m, red);
  s *= __expf(m - gm);
  const float gs = block_sum(s, red);
  const float lse = gm + logf(gs);
  if (threadIdx.x == 0) {
    float t;
    if constexpr (sizeof(LogitT) == 2) t = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(lr)[tgt]); else t = lr[tgt];
    loss[row] = lse - t;
  }
  __syncthreads();   // the target logit has been read before any thread overwrites the row
  const float inv = grad_scale / gs;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    float o[8];
    load8(lr + c, o);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = __expf(o[i] - gm) * inv;
    if (tgt >= c && tgt < c + 8) o[tgt - c] -= grad_scale;
    bf16x8 ov; ov.from_float(o); ov.store(dr + c);
  }
}

// ------------------------------------------------------------------------------ column sums (bias grad)
// part[split, c] = sum over this split's rows of x[r, c]; then reduce_rows_kernel.
__global__ void __launch_bounds__(256) colsum_partial_kernel(const __nv_bfloat16* __restrict__ x, long long ld, float* __restrict__ part,
                                                            int T, int N) {
  __shared__ float sm[8][64];
  const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
  const int c = blockIdx.x * 64 + lane * 2;
  const int rows_per = (T + gridDim.y - 1) / gridDim.y;
  const int r0 = blockIdx.y * rows_per, r1 = min(T, r0 + rows_per);
  float a = 0.f, b = 0.f;
  if (c < N) {
    for (int r = r0 + wy; r < r1; r += 8) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + static_cast<long long>(r) * ld + c));
      a += v.x; b += v.y;
    }
  }
  sm[wy][lane * 2] = a; sm[wy][lane * 2 + 1] = b;
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += sm[i][threadIdx.x];
    const int cc = blockIdx.x * 64 + threadIdx.x;
    if (cc < N) part[static_cast<long long>(blockIdx.y) * N + cc] = s;
  }
}

// ------------------------------------------------------------------------------ optimizer-side
// acc = (accumulate ? acc : 0) + src   (fp32 accumulator, bf16 or fp32 source)
template <typename SrcT>
__global__ void __launch_bounds__(EW_THREADS) accumulate_kernel(float* __restrict__ acc, const SrcT* __restrict__ src, long long n, int accumulate) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  float f[8];
  if constexpr (sizeof(SrcT) == 2) { bf16x8 v; v.load(reinterpret_cast<const __nv_bfloat16*>(src) + i); v.to_float(f); }
  else {
    const float4 a = *reinterpret_cast<const float4*>(src + i), b = *reinterpret_cast<const float4*>(src + i + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  float4* d = reinterpret_cast<float4*>(acc + i);
  if (accumulate) {
    const float4 a = d[0], b = d[1];
    f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w; f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
  }
  d[0] = make_float4(f[0], f[1], f[2], f[3]);
  d[1] = make_float4(f[4], f[5], f[6], f[7]);
}

// dst(bf16) = (accumulate ? dst : 0) + src(fp32)
__global__ void __launch_bounds__(EW_THREADS) f32_to_bf16_kernel(__nv_bfloat16* __restrict__ dst, const float* __restrict__ src, long long n, int accumulate) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  const float4 a = *reinterpret_cast<const float4*>(src + i), b = *reinterpret_cast<const float4*>(src + i + 4);
  float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  if (accumulate) {
    bf16x8 v; v.load(dst + i); float g[8]; v.to_float(g);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] += g[k];
  }
  bf16x8 o; o.from_float(f); o.store(dst + i);
}

// out[0] += sum(x^2): per-block partial sums combined with one atomic per block.
__global__ void __launch_bounds__(EW_THREADS) sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// Fused AdamW on a shard: g = grad * coef[0]; moments in fp32 or bf16; master fp32; bf16 working copy refreshed.
template <typename StateT>
__global__ void __launch_bounds__(EW_THREADS) adamw_kernel(float* __restrict__ master, StateT* __restrict__ m, StateT* __restrict__ v,
                                                          const float* __restrict__ grad, __nv_bfloat16* __restrict__ param,
                                                          long long n, float lr, float beta1, float beta2, float eps, float wd,
                                                          float inv_bc1, float inv_sqrt_bc2, const float* __restrict__ coef) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  const float c = coef[0];
  const float4 g4 = *reinterpret_cast<const float4*>(grad + i);
  float4 w4 = *reinterpret_cast<float4*>(master + i);
  float g[4] = {g4.x * c, g4.y * c, g4.z * c, g4.w * c};
  float w[4] = {w4.x, w4.y, w4.z, w4.w};
  float mm[4], vv[4];
  if constexpr (sizeof(StateT) == 4) {
    const float4 a = *reinterpret_cast<const float4*>(m + i), b = *reinterpret_cast<const float4*>(v + i);
    mm[0] = a.x; mm[1] = a.y; mm[2] = a.z; mm[3] = a.w; vv[0] = b.x; vv[1] = b.y; vv[2] = b.z; vv[3] = b.w;
  } else {
    const uint2 a = *reinterpret_cast<const uint2*>(m + i), b = *reinterpret_cast<const uint2*>(v + i);
    float2 t;
    t = unpack_bf16(a.x); mm[0] = t.x; mm[1] = t.y; t = unpack_bf16(a.y); mm[2] = t.x; mm[3] = t.y;
    t = unpack_bf16(b.x); vv[0] = t.x; vv[1] = t.y; t = unpack_bf16(b.y); vv[2] = t.x; vv[3] = t.y;
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    w[k] *= (1.f - lr * wd);
    mm[k] = beta1 * mm[k] + (1.f - beta1) * g[k];
    vv[k] = beta2 * vv[k] + (1.f - beta2) * g[k] * g[k];
    const float denom = sqrtf(vv[k]) * inv_sqrt_bc2 + eps;
    w[k] -= lr * inv_bc1 * mm[k] / denom;
  }
  *reinterpret_cast<float4*>(master + i) = make_float4(w[0], w[1], w[2], w[3]);
  if constexpr (sizeof(StateT) == 4) {
    *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
  } else {
    *reinterpret_cast<uint2*>(m + i) = make_uint2(pack_bf16(mm[0], mm[1]), pack_bf16(mm[2], mm[3]));
    *reinterpret_cast<uint2*>(v + i) = make_uint2(pack_bf16(vv[0], vv[1]), pack_bf16(vv[2], vv[3]));
  }
  *reinterpret_cast<uint2*>(param + i) = make_uint2(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]));
}

static inline int cdiv(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }
static inline int launch_ok() { return cudaGetLastError() == cudaSuccess ? 0 : -5; }
static int num_sms() {
  static int n = 0;
  if (n == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev); }
  return n;
}

}  // namespace mtb

using namespace mtb;
typedef __nv_bfloat16 bf16;

extern "C" {

int mtb200_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, float eps, int T, int H, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 || H > 8 * 8 * EW_THREADS) return -10;
  // about four vectors per thread; a row is held by 32 .. 256 threads (a power of two)
  const int vecs = H / 8;
  int lanes = 32;
  while (lanes < EW_THREADS && lanes * 4 < vecs) lanes *= 2;
  const int vpt = cdiv(vecs, lanes);
  const int blocks = cdiv(T, EW_THREADS / lanes);
#define RF(V) rmsnorm_fwd_kernel<V><<<blocks, EW_THREADS, 0, st>>>((const bf16*)x, (const bf16*)w, (bf16*)y, rstd, eps, T, H, lanes)
  if (vpt <= 1) RF(1); else if (vpt <= 2) RF(2); else if (vpt <= 4) RF(4); else RF(8);
#undef RF
  return launch_ok();
}

// Number of row-partials the backward writes (rows of the dw_partial scratch, [blocks, H] fp32).
int mtb200_rmsnorm_bwd_blocks(int T) { const int b = num_sms() * 2; return T < b ? (T > 0 ? T : 1) : b; }

int mtb200_rmsnorm_bwd(const void* dy, const void* x, const float* rstd, const void* w, const void* add_to, void* dx,
                       float* dw_partial, void* dw_out, int T, int H, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 || H > 4 * 8 * 512) return -10;
  const int blocks = mtb200_rmsnorm_bwd_blocks(T);
#define RB(V, TH) rmsnorm_bwd_kernel<V, TH><<<blocks, TH, 0, st>>>((const bf16*)dy, (const bf16*)x, rstd, (const bf16*)w, (const bf16*)add_to, (bf16*)dx, dw_partial, T, H)
  if (H <= 8 * EW_THREADS) RB(1, EW_THREADS);
  else {
    const int vpt = cdiv(H, 8 * 512);
    if (vpt <= 1) RB(1, 512); else if (vpt == 2) RB(2, 512); else if (vpt == 3) RB(3, 512); else RB(4, 512);
  }
#undef RB
  reduce_rows_kernel<<<cdiv(H, 256), 256, 0, st>>>(dw_partial, (bf16*)dw_out, blocks, H);
  return launch_ok();
}

// LayerNorm with bias over rows of H <= 8192 elements; mean / rstd: [T] fp32 each.
int mtb200_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, float eps, int T, int H,
                         cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 || H > 4 * 8 * EW_THREADS) return -10;
  const int vpt = cdiv(H, 8 * EW_THREADS);
#define LF(V) layernorm_fwd_kernel<V><<<T, EW_THREADS, 0, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)b, (bf16*)y, mean, rstd, eps, H)
  if (vpt <= 1) LF(1); else if (vpt == 2) LF(2); else if (vpt == 3) LF(3); else LF(4);
#undef LF
  return launch_ok();
}

// dw_partial: [mtb200_rmsnorm_bwd_blocks(T), 2, H] fp32 scratch; dw_out / db_out: [H] bf16 each.
int mtb200_layernorm_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* w, const void* add_to, void* dx,
                         float* dw_partial, void* dw_out, void* db_out, int T, int H, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 || H > 4 * 8 * EW_THREADS) return -10;
  const int blocks = mtb200_rmsnorm_bwd_blocks(T);
  const int vpt = cdiv(H, 8 * EW_THREADS);
#define LB(V) layernorm_bwd_kernel<V><<<blocks, EW_THREADS, 0, st>>>((const bf16*)dy, (const bf16*)x, mean, rstd, (const bf16*)w, (const bf16*)add_to, (bf16*)dx, dw_partial, T, H)
  if (vpt <= 1) LB(1); else if (vpt == 2) LB(2); else if (vpt == 3) LB(3); else LB(4);
#undef LB
  reduce_rows_pair_kernel<<<cdiv(2 * H, 256), 256, 0, st>>>(dw_partial, (bf16*)dw_out, (bf16*)db_out, blocks, H);
  return launch_ok();
}

int mtb200_rope(void* qkv, const int* pos, const float* inv_freq, int T, long long ld, int n_heads, int D, int inverse, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D % 16 || ld % 8) return -10;
  const long long n = static_cast<long long>(T) * (D / 16);
  rope_kernel<<<dim3(cdiv(n, EW_THREADS), cdiv(n_heads, ROPE_HPT)), EW_THREADS, 0, st>>>((bf16*)qkv, pos, inv_freq, T, ld, n_heads, D,
                                                                                        inverse ? -1.f : 1.f);
  return launch_ok();
}

// Per-head RMSNorm of the q and k heads (n_q then n_heads - n_q) of qkv[T, ld], in place; rstd: [T * n_heads] fp32.
int mtb200_head_rmsnorm_fwd(void* qkv, const void* wq, const void* wk, float* rstd, float eps, int T, long long ld, int n_q, int n_heads,
                            int D, cudaStream_t st) {
  if (T <= 0 || n_heads <= 0) return 0;
  if ((D != 64 && D != 128 && D != 256) || ld % 8 || n_q < 0 || n_q > n_heads) return -10;
  const long long n_rows = static_cast<long long>(T) * n_heads;
  const unsigned blocks = static_cast<unsigned>(cdiv(n_rows, EW_THREADS / 32));
#define HF(E) head_rmsnorm_fwd_kernel<E><<<blocks, EW_THREADS, 0, st>>>((bf16*)qkv, (const bf16*)wq, (const bf16*)wk, rstd, eps, n_rows, ld, n_q, n_heads)
  if (D == 64) HF(2); else if (D == 128) HF(4); else HF(8);
#undef HF
  return launch_ok();
}

// Rows of the dw_partial scratch ([blocks, 2, D] fp32) the backward writes.
int mtb200_head_rmsnorm_bwd_blocks(int T, int n_heads) {
  const long long rows = static_cast<long long>(T) * n_heads;
  const long long want = cdiv(rows, EW_THREADS / 32);
  const long long cap = num_sms() * 4;
  return static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
}

// dqkv (q and k heads) in place; pre: the heads before the norm, [T, ld_pre]; dwq_out / dwk_out: [D] bf16 each.
int mtb200_head_rmsnorm_bwd(void* dqkv, const void* pre, const float* rstd, const void* wq, const void* wk, float* dw_partial,
                            void* dwq_out, void* dwk_out, int T, long long ld, long long ld_pre, int n_q, int n_heads, int D,
                            cudaStream_t st) {
  if (T <= 0 || n_heads <= 0) return 0;
  if ((D != 64 && D != 128 && D != 256) || ld % 8 || ld_pre % 8 || n_q < 0 || n_q > n_heads) return -10;
  const long long n_rows = static_cast<long long>(T) * n_heads;
  const int blocks = mtb200_head_rmsnorm_bwd_blocks(T, n_heads);
#define HB(E) head_rmsnorm_bwd_kernel<E><<<blocks, EW_THREADS, 0, st>>>((bf16*)dqkv, (const bf16*)pre, rstd, (const bf16*)wq, (const bf16*)wk, dw_partial, n_rows, ld, ld_pre, n_q, n_heads)
  if (D == 64) HB(2); else if (D == 128) HB(4); else HB(8);
#undef HB
  // partial rows are [2, D]: columns 0..D-1 belong to the q weight, D..2D-1 to the k weight
  reduce_rows_pair_kernel<<<cdiv(2 * D, 256), 256, 0, st>>>(dw_partial, (bf16*)dwq_out, (bf16*)dwk_out, blocks, D);
  return launch_ok();
}

int mtb200_swiglu_fwd(const void* gu, void* act, long long T, int F, cudaStream_t st) {
  if (T <= 0) return 0;
  if (F % 8) return -10;
  swiglu_fwd_kernel<0><<<dim3(static_cast<unsigned>(T), cdiv(F / 8, EW_THREADS)), EW_THREADS, 0, st>>>((const bf16*)gu, (bf16*)act, T, F);
  return launch_ok();
}

int mtb200_swiglu_bwd(const void* dact, const void* gu, void* dgu, long long T, int F, cudaStream_t st) {
  if (T <= 0) return 0;
  if (F % 8) return -10;
  swiglu_bwd_kernel<false, 0><<<dim3(static_cast<unsigned>(T), cdiv(F / 8, EW_THREADS)), EW_THREADS, 0, st>>>((bf16*)const_cast<void*>(dact), (const bf16*)gu, (bf16*)dgu, T, F);
  return launch_ok();
}

// Same, and dact_inout is overwritten with the forward output silu(gate) * up.
int mtb200_swiglu_bwd_act(void* dact_inout, const void* gu, void* dgu, long long T, int F, cudaStream_t st) {
  if (T <= 0) return 0;
  if (F % 8) return -10;
  swiglu_bwd_kernel<true, 0><<<dim3(static_cast<unsigned>(T), cdiv(F / 8, EW_THREADS)), EW_THREADS, 0, st>>>((bf16*)dact_inout, (const bf16*)gu, (bf16*)dgu, T, F);
  return launch_ok();
}

// GeGLU (tanh-approximated GELU on the gate): same three entry points as SwiGLU.
int mtb200_geglu_fwd(const void* gu, void* act, long long T, int F, cudaStream_t st) {
  if (T <= 0) return 0;
  if (F % 8) return -10;
  swiglu_fwd_kernel<1><<<dim3(static_cast<unsigned>(T), cdiv(F / 8, EW_THREADS)), EW_THREADS, 0, st>>>((const bf16*)gu, (bf16*)act, T, F);
  return launch_ok();
}
int mtb200_geglu_bwd(const void* dact, const void* gu, void* dgu, long long T, int F, cudaStream_t st) {
  if (T <= 0) return 0;
  if (F % 8) return -10;
  swiglu_bwd_kernel<false, 1><<<dim3(static_cast<unsigned>(T), cdiv(F / 8, EW_THREADS)), EW_THREADS, 0, st>>>((bf16*)const_cast<void*>(dact), (const bf16*)gu, (bf16*)dgu, T, F);
  return launch_ok();
}
int mtb200_geglu_bwd_act(void* dact_inout, const void* gu, void* dgu, long long T, int F, cudaStream_t st) {
  if (T <= 0) return 0;
  if (F % 8) return -10;
  swiglu_bwd_kernel<true, 1><<<dim3(static_cast<unsigned>(T), cdiv(F / 8, EW_THREADS)), EW_THREADS, 0, st>>>((bf16*)dact_inout, (const bf16*)gu, (bf16*)dgu, T, F);
  return launch_ok();
}

// y = gelu_tanh(x) over n elements; dx = dy * gelu_tanh'(x) (dx may be dy).
int mtb200_gelu_fwd(const void* x, void* y, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return -10;
  act_fwd_kernel<1><<<static_cast<unsigned>(cdiv(n / 8, EW_THREADS)), EW_THREADS, 0, st>>>((const bf16*)x, (bf16*)y, n);
  return launch_ok();
}
int mtb200_gelu_bwd(const void* dy, const void* x, void* dx, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return -10;
  act_bwd_kernel<1><<<static_cast<unsigned>(cdiv(n / 8, EW_THREADS)), EW_THREADS, 0, st>>>((const bf16*)dy, (const bf16*)x, (bf16*)dx, n);
  return launch_ok();
}

int mtb200_embedding_fwd(const void* w, const long long* ids, void* out, int T, int H, int V, int* status, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  embedding_fwd_kernel<<<T, 128, 0, st>>>((const bf16*)w, ids, (bf16*)out, H, V, status);
  return launch_ok();
}

int mtb200_embedding_bwd(void* dw, const long long* sorted_ids, const long long* order, const void* dx, int T, int H, int V,
                         int* status, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  embedding_bwd_kernel<<<T, 128, 0, st>>>((bf16*)dw, sorted_ids, order, (const bf16*)dx, T, H, V, status);
  return launch_ok();
}

// logits: [R, V] fp32, or bf16 when logits_bf16 (dlogits may then be the same buffer).
int mtb200_ce_fwd_bwd(const void* logits, long long ld, int logits_bf16, const long long* targets, float* loss, void* dlogits,
                      long long ldd, int R, int V, float grad_scale, long long ignore_index, cudaStream_t st) {
  if (R <= 0) return 0;
  if (V % 8 || ld % 8 || ldd % 8) return -10;
  if (logits_bf16) ce_fwd_bwd_kernel<bf16><<<R, 1024, 0, st>>>((const bf16*)logits, ld, targets, loss, (bf16*)dlogits, ldd, V, grad_scale, ignore_index);
  else ce_fwd_bwd_kernel<float><<<R, 1024, 0, st>>>((const float*)logits, ld, targets, loss, (bf16*)dlogits, ldd, V, grad_scale, ignore_index);
  return launch_ok();
}

// out[N] (bf16) = column sums of x[T, N]. scratch: fp32 [32, N].
int mtb200_colsum(const void* x, long long ld, void* out, float* scratch, int T, int N, cudaStream_t st) {
  if (T <= 0 || N <= 0) return 0;
  if (N % 2) return -10;
  const int splits = T < 32 ? 1 : 32;
  colsum_partial_kernel<<<dim3(cdiv(N, 64), splits), 256, 0, st>>>((const bf16*)x, ld, scratch, T, N);
  reduce_rows_kernel<<<cdiv(N, 256), 256, 0, st>>>(scratch, (bf16*)out, splits, N);
  return launch_ok();
}

int mtb200_accumulate(float* acc, const void* src, long long n, int src_is_f32, int accumulate, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return -10;
  if (src_is_f32) accumulate_kernel<float><<<cdiv(n / 8, EW_THREADS), EW_THREADS, 0, st>>>(acc, (const float*)src, n, accumulate);
  else accumulate_kernel<bf16><<<cdiv(n / 8, EW_THREADS), EW_THREADS, 0, st>>>(acc, (const bf16*)src, n, accumulate);
  return launch_ok();
}

int mtb200_f32_to_bf16(void* dst, const float* src, long long n, int accumulate, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return -10;
  f32_to_bf16_kernel<<<cdiv(n / 8, EW_THREADS), EW_THREADS, 0, st>>>((bf16*)dst, src, n, accumulate);
  return launch_ok();
}

int mtb200_sumsq(const float* x, long long n, float* out, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 4) return -10;
  const int blocks = static_cast<int>(min(static_cast<long long>(num_sms() * 8), (n / 4 + EW_THREADS - 1) / EW_THREADS));
  sumsq_kernel<<<blocks, EW_THREADS, 0, st>>>(x, n, out);
  return launch_ok();
}

int mtb200_adamw(float* master, void* m, void* v, int state_is_f32, const float* grad, void* param, long long n, float lr,
                 float beta1, float beta2, float eps, float wd, int step, const float* coef, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 4) return -10;
  const float inv_bc1 = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  const float inv_sqrt_bc2 = 1.f / sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  const int blocks = cdiv(n / 4, EW_THREADS);
  if (state_is_f32)
    adamw_kernel<float><<<blocks, EW_THREADS, 0, st>>>(master, (float*)m, (float*)v, grad, (bf16*)param, n, lr, beta1, beta2, eps, wd, inv_bc1, inv_sqrt_bc2, coef);
  else
    adamw_kernel<bf16><<<blocks, EW_THREADS, 0, st>>>(master, (bf16*)m, (bf16*)v, grad, (bf16*)param, n, lr, beta1, beta2, eps, wd, inv_bc1, inv_sqrt_bc2, coef);
  return launch_ok();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Allocation-free variant of mtb200_colsum (declared in mtb200_noalloc.h).
//
// For callers that cannot allocate device memory when they need the kernel: the fp32 partial-sum
// workspace lives in a file-scope device array. In host code the array's name is only a handle,
// never a pointer a kernel could dereference, so its device address is looked up once per device
// with cudaGetSymbolAddress and that address is what the kernels receive.
// ------------------------------------------------------------------------------------------
#include "mtb200_noalloc.h"

static __device__ __align__(256) float g_colsum_noalloc_ws[32 * MTB200_COLSUM_NOALLOC_MAX_N];

namespace {
constexpr int kMaxDevices = 64;
float* g_colsum_ws_addr[kMaxDevices] = {nullptr};

// Device address of the workspace on the current device (looked up on first use per device).
float* colsum_noalloc_workspace() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_colsum_ws_addr[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_colsum_noalloc_ws) != cudaSuccess) return nullptr;
    g_colsum_ws_addr[dev] = ptr;
  }
  return g_colsum_ws_addr[dev];
}
}  // namespace

extern "C" int mtb200_colsum_noalloc(const void* x, long long ld, void* out, int T, int N, cudaStream_t st) {
  if (T <= 0 || N <= 0) return 0;
  if (N % 2 || ld < N) return -10;
  if (N > MTB200_COLSUM_NOALLOC_MAX_N) return -11;   // beyond the built-in workspace
  float* ws = colsum_noalloc_workspace();
  if (ws == nullptr) return -12;
  // Every element of ws[0 : splits * N] that the second kernel reads is written by the first one,
  // so nothing left over from an earlier call can reach the result and no clearing pass is needed.
  const int splits = T < 32 ? 1 : 32;
  colsum_partial_kernel<<<dim3(cdiv(N, 64), splits), 256, 0, st>>>((const bf16*)x, ld, ws, T, N);
  reduce_rows_kernel<<<cdiv(N, 256), 256, 0, st>>>(ws, (bf16*)out, splits, N);
  return launch_ok();
}

