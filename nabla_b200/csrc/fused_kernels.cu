// Memory-bound fused kernels for sm_100a: LayerNorm fwd/bwd, softmax / log-softmax,
// cross-entropy fwd/bwd, AdamW / SGD steps, embedding gather / scatter-add, activation
// backward, column sums (bias gradients), casts, Philox RNG, dropout, NF4 dequantisation,
// pooling and a direct NHWC convolution for small channel counts.
//
// These replace compositions of primitive ops in the reference:
//   layer_norm         nabla/nn/functional/layers.py:38-56   (9 primitive ops)
//   cross_entropy      nabla/nn/functional/losses.py:20-44   (logsoftmax, one-hot mul, sum)
//   adamw_step         nabla/nn/optim/functional.py:116-162  (~15 primitive ops per leaf)
//   embedding          nabla/nn/functional/layers.py:84-98 + nabla/ops/view/indexing.py
//   dequantize_nf4     nabla/nn/finetune/qlora.py:77-98
//   pooling            nabla/ops/pooling.py:53-137 (python loop of slices)
// All of them are bandwidth bound: 16-byte vector accesses, fp32 math, one pass over DRAM
// where the row fits in registers / L1.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "nb_debug.cuh"

namespace nbk {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16(v); }

// 16-byte vector of T
template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float* out) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::N; ++i) out[i] = to_f<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float* in) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::N; ++i) e[i] = from_f<T>(in[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int NW>
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < NW; ++i) r += sh[i];
  return r;
}
template <int NW>
__device__ __forceinline__ float block_max(float v, float* sh) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = -INFINITY;
#pragma unroll
  for (int i = 0; i < NW; ++i) r = fmaxf(r, sh[i]);
  return r;
}

// ============================================================== LayerNorm
template <typename T>
__device__ __forceinline__ void unpack_vec(const uint4& raw, float* out) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::N; ++i) out[i] = to_f<T>(e[i]);
}

// One warp per row. The row is read once and stays in registers in its packed 16-byte form
// (D <= 32 * VPL * Vec::N); it is unpacked for the mean, the variance and the output, which keeps
// the register count low enough for the number of rows in flight that a bandwidth-bound pass needs.
template <typename T, int VPL>
__global__ void __launch_bounds__(128, 8) layernorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                              const T* __restrict__ beta, T* __restrict__ y,
                                                              float* __restrict__ mean, float* __restrict__ rstd,
                                                              int rows, int D, float eps) {
  constexpr int V = Vec<T>::N;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + (size_t)row * D;
  uint4 raw[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * V;
    if (c < D) raw[i] = *reinterpret_cast<const uint4*>(xr + c);
  }
  // one pass over the registers for both moments (shifted by the row's first element so that the
  // E[x^2] - E[x]^2 form does not cancel for rows with a large common offset), one pair of warp
  // reductions issued back to back
  const float shift = __shfl_sync(0xffffffffu, to_f<T>(reinterpret_cast<const T*>(&raw[0])[0]), 0);
  float s = 0.f, q = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * V;
    if (c < D) {
      float v[V];
      unpack_vec<T>(raw[i], v);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float d = v[j] - shift;
        s += d;
        q = fmaf(d, d, q);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    q += __shfl_xor_sync(0xffffffffu, q, o);
  }
  const float ms = s / D;
  const float mu = ms + shift;
  const float rs = rsqrtf(fmaxf(q / D - ms * ms, 0.f) + eps);
  if (lane == 0) {
    if (mean) mean[row] = mu;
    if (rstd) rstd[row] = rs;
  }
  T* yr = y + (size_t)row * D;
  const float nmr = -mu * rs;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * V;
    if (c < D) {
      float g[V], b[V], o[V], v[V];
      unpack_vec<T>(raw[i], v);
      if (gamma) load_vec<T>(gamma + c, g);
      if (beta) load_vec<T>(beta + c, b);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float n = fmaf(v[j], rs, nmr);
        o[j] = gamma ? fmaf(n, g[j], beta ? b[j] : 0.f) : (n + (beta ? b[j] : 0.f));
      }
      store_vec<T>(yr + c, o);
    }
  }
}

// Backward, part 1: dx. One warp per row. The row's x and dy stay in registers in their packed
// 16-byte form (half the registers of keeping them as floats, so twice as many rows are in flight
// per SM for this bandwidth-bound pass) and are unpacked once for the two sums and once for dx.
template <typename T, int VPL>
__global__ void __launch_bounds__(128, 4) layernorm_bwd_dx_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                              const T* __restrict__ gamma, const float* __restrict__ mean,
                                                              const float* __restrict__ rstd, T* __restrict__ dx,
                                                              int rows, int D) {
  constexpr int V = Vec<T>::N;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + (size_t)row * D;
  const T* dyr = dy + (size_t)row * D;
  uint4 xraw[VPL], draw[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * V;
    if (c < D) {
      xraw[i] = *reinterpret_cast<const uint4*>(xr + c);
      draw[i] = *reinterpret_cast<const uint4*>(dyr + c);
    }
  }
  const float mu = mean[row], rs = rstd[row];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * V;
    if (c < D) {
      float xv[V], dv[V], gm[V];
      unpack_vec<T>(xraw[i], xv);
      unpack_vec<T>(draw[i], dv);
      if (gamma) load_vec<T>(gamma + c, gm);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float g = dv[j] * (gamma ? gm[j] : 1.f);
        s1 += g;
        s2 += g * (xv[j] - mu) * rs;
      }
    }
  }
  s1 = warp_sum(s1) / D;
  s2 = warp_sum(s2) / D;
  T* dxr = dx + (size_t)row * D;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * V;
    if (c < D) {
      float xv[V], dv[V], gm[V], o[V];
      unpack_vec<T>(xraw[i], xv);
      unpack_vec<T>(draw[i], dv);
      if (gamma) load_vec<T>(gamma + c, gm);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float g = dv[j] * (gamma ? gm[j] : 1.f);
        o[j] = (g - s1 - (xv[j] - mu) * rs * s2) * rs;
      }
      store_vec<T>(dxr + c, o);
    }
  }
}

// Backward in one pass (rows of up to 8 vectors per lane): a persistent grid of warps walks the rows,
// each warp computing dx of its row as above while it also adds the row's dy * xhat and dy into
// per-lane register accumulators for the columns it holds, so dy and x are read from DRAM once
// instead of twice. At the end the four warps of a block fold their accumulators through shared
// memory and the block writes one row of `partial` ([gridDim.x][2][D] fp32), which
// colsum_partials_kernel adds up into dgamma / dbeta.
// 16-byte vector <-> pairs of floats, for the packed two-wide fp32 instructions (fma.rn.f32x2).
template <typename T> __device__ __forceinline__ void unpack_pairs(const uint4& raw, float2* out);
template <> __device__ __forceinline__ void unpack_pairs<float>(const uint4& raw, float2* out) {
  out[0] = make_float2(__uint_as_float(raw.x), __uint_as_float(raw.y));
  out[1] = make_float2(__uint_as_float(raw.z), __uint_as_float(raw.w));
}
template <> __device__ __forceinline__ void unpack_pairs<bf16>(const uint4& raw, float2* out) {
  const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) out[k] = make_float2(__uint_as_float(w[k] << 16), __uint_as_float(w[k] & 0xffff0000u));
}
template <typename T> __device__ __forceinline__ uint4 pack_pairs(const float2* in);
template <> __device__ __forceinline__ uint4 pack_pairs<float>(const float2* in) {
  return make_uint4(__float_as_uint(in[0].x), __float_as_uint(in[0].y), __float_as_uint(in[1].x), __float_as_uint(in[1].y));
}
template <> __device__ __forceinline__ uint4 pack_pairs<bf16>(const float2* in) {
  unsigned w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    __nv_bfloat162 h = __float22bfloat162_rn(in[k]);
    w[k] = *reinterpret_cast<unsigned*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T, int VPL>
__global__ void __launch_bounds__(128, (VPL * Vec<T>::N >= 64 ? 2 : VPL * Vec<T>::N >= 32 ? 3 : 4))
    layernorm_bwd_fused_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                               const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                               float* __restrict__ partial, int rows, int D) {
  constexpr int V = Vec<T>::N, P = V / 2;
  __shared__ float sh[2][32 * V * VPL];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float2 ag[VPL][P], ab[VPL][P];
#pragma unroll
  for (int i = 0; i < VPL; ++i)
#pragma unroll
    for (int k = 0; k < P; ++k) { ag[i][k] = make_float2(0.f, 0.f); ab[i][k] = make_float2(0.f, 0.f); }
  for (int row = blockIdx.x * 4 + warp; row < rows; row += gridDim.x * 4) {
    const T* xr = x + (size_t)row * D;
    const T* dyr = dy + (size_t)row * D;
    uint4 xraw[VPL], draw[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = (i * 32 + lane) * V;
      if (c < D) {
        xraw[i] = *reinterpret_cast<const uint4*>(xr + c);
        draw[i] = *reinterpret_cast<const uint4*>(dyr + c);
      }
    }
    const float mu = mean[row], rs = rstd[row];
    const float2 rs2 = make_float2(rs, rs), nmr2 = make_float2(-mu * rs, -mu * rs);
    float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = (i * 32 + lane) * V;
      if (c < D) {
        float2 xv[P], dv[P], gm[P];
        unpack_pairs<T>(xraw[i], xv);
        unpack_pairs<T>(draw[i], dv);
        if (gamma) unpack_pairs<T>(*reinterpret_cast<const uint4*>(gamma + c), gm);
#pragma unroll
        for (int k = 0; k < P; ++k) {
          const float2 xh = __ffma2_rn(xv[k], rs2, nmr2);              // (x - mean) * rstd
          const float2 g = gamma ? __fmul2_rn(dv[k], gm[k]) : dv[k];
          s1 = __fadd2_rn(s1, g);
          s2 = __ffma2_rn(g, xh, s2);
          ag[i][k] = __ffma2_rn(dv[k], xh, ag[i][k]);
          ab[i][k] = __fadd2_rn(ab[i][k], dv[k]);
        }
      }
    }
    const float m1 = warp_sum(s1.x + s1.y) / D;
    const float m2 = warp_sum(s2.x + s2.y) / D;
    // dx = rstd * (g - m1 - xhat * m2) = g * rstd + (xhat * (-rstd * m2) + (-rstd * m1))
    const float2 a2 = make_float2(-rs * m2, -rs * m2), b2 = make_float2(-rs * m1, -rs * m1);
    T* dxr = dx + (size_t)row * D;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = (i * 32 + lane) * V;
      if (c < D) {
        float2 xv[P], dv[P], gm[P], o[P];
        unpack_pairs<T>(xraw[i], xv);
        unpack_pairs<T>(draw[i], dv);
        if (gamma) unpack_pairs<T>(*reinterpret_cast<const uint4*>(gamma + c), gm);
#pragma unroll
        for (int k = 0; k < P; ++k) {
          const float2 xh = __ffma2_rn(xv[k], rs2, nmr2);
          const float2 g = gamma ? __fmul2_rn(dv[k], gm[k]) : dv[k];
          o[k] = __ffma2_rn(g, rs2, __ffma2_rn(xh, a2, b2));
        }
        *reinterpret_cast<uint4*>(dxr + c) = pack_pairs<T>(o);
      }
    }
  }
  for (int w = 0; w < 4; ++w) {
    if (warp == w) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = (i * 32 + lane) * V;
        if (c < D) {
#pragma unroll
          for (int k = 0; k < P; ++k) {
            sh[0][c + 2 * k] = (w == 0 ? 0.f : sh[0][c + 2 * k]) + ag[i][k].x;
            sh[0][c + 2 * k + 1] = (w == 0 ? 0.f : sh[0][c + 2 * k + 1]) + ag[i][k].y;
            sh[1][c + 2 * k] = (w == 0 ? 0.f : sh[1][c + 2 * k]) + ab[i][k].x;
            sh[1][c + 2 * k + 1] = (w == 0 ? 0.f : sh[1][c + 2 * k + 1]) + ab[i][k].y;
          }
        }
      }
    }
    __syncthreads();
  }
  float* prow = partial + (size_t)blockIdx.x * 2 * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    prow[c] = sh[0][c];
    prow[D + c] = sh[1][c];
  }
}

// Backward, part 2 (rows wider than that): dgamma = sum_rows dy * xhat, dbeta = sum_rows dy. Block = 32*V columns x a
// slab of rows; 8 warps stride over the slab's rows with register accumulators; partial sums go
// to `partial` ([gridDim.y][2][D] fp32) and are folded by colsum_partials_kernel.
template <typename T>
__global__ void __launch_bounds__(256) layernorm_bwd_dgb_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                               const float* __restrict__ mean,
                                                               const float* __restrict__ rstd,
                                                               float* __restrict__ partial, int rows, int D,
                                                               int rows_per_block) {
  constexpr int V = Vec<T>::N;
  __shared__ float sh[2][8][32 * V];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * V;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float ag[V], ab[V];
#pragma unroll
  for (int j = 0; j < V; ++j) { ag[j] = 0.f; ab[j] = 0.f; }
  if (c < D) {
    for (int r = r0 + warp; r < r1; r += 8) {
      float xv[V], dv[V];
      load_vec<T>(x + (size_t)r * D + c, xv);
      load_vec<T>(dy + (size_t)r * D + c, dv);
      const float mu = mean[r], rs = rstd[r];
#pragma unroll
      for (int j = 0; j < V; ++j) {
        ag[j] += dv[j] * (xv[j] - mu) * rs;
        ab[j] += dv[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) { sh[0][warp][lane * V + j] = ag[j]; sh[1][warp][lane * V + j] = ab[j]; }
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * V; i += blockDim.x) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { a += sh[0][w][i]; b += sh[1][w][i]; }
    const int col = blockIdx.x * 32 * V + i;
    if (col < D) {
      partial[(size_t)blockIdx.y * 2 * D + col] = a;
      partial[(size_t)blockIdx.y * 2 * D + D + col] = b;
    }
  }
}

// out0[c] = sum_b partial[b][0][c], out1[c] = sum_b partial[b][1][c]  (two planes of width D per row
// of `partial`). A block covers 32 columns; its 8 warps take every 8th row, so a few hundred rows of
// partials are a few dozen dependent loads per thread instead of a few hundred.
template <typename T>
__global__ void __launch_bounds__(256) colsum_partials_kernel(const float* __restrict__ partial, T* __restrict__ out0,
                                                             T* __restrict__ out1, int nblocks, int D) {
  __shared__ float sh[2][8][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float a = 0.f, b = 0.f;
  if (c < D) {
    for (int i = w; i < nblocks; i += 8) {
      a += partial[(size_t)i * 2 * D + c];
      b += partial[(size_t)i * 2 * D + D + c];
    }
  }
  sh[0][w][lane] = a;
  sh[1][w][lane] = b;
  __syncthreads();
  if (w == 0 && c < D) {
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { sa += sh[0][k][lane]; sb += sh[1][k][lane]; }
    if (out0) out0[c] = from_f<T>(sa);
    if (out1) out1[c] = from_f<T>(sb);
  }
}

// ============================================================== column sum (bias gradient)
// x [rows][N] -> partial[gridDim.y][N] ; each block sums a slab of rows for 32*V columns.
template <typename T>
__global__ void __launch_bounds__(256) colsum_kernel(const T* __restrict__ x, float* __restrict__ partial, int rows,
                                                    int N, int rows_per_block) {
  constexpr int V = Vec<T>::N;
  __shared__ float sh[8][32 * V];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * V;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.f;
  if (c < N) {
    for (int r = r0 + warp; r < r1; r += 8) {
      float v[V];
      load_vec<T>(x + (size_t)r * N + c, v);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) sh[warp][lane * V + j] = acc[j];
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * V; i += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += sh[w][i];
    const int col = blockIdx.x * 32 * V + i;
    if (col < N) partial[(size_t)blockIdx.y * N + col] = s;
  }
}
template <typename T>
__global__ void colsum_final_kernel(const float* __restrict__ partial, T* __restrict__ out, int nparts, int N) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float s = 0.f;
  for (int i = 0; i < nparts; ++i) s += partial[(size_t)i * N + c];
  out[c] = from_f<T>(s);
}

// ============================================================== softmax / log-softmax (last dim)
template <typename T, bool LOG>
__global__ void __launch_bounds__(256) softmax_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int D) {
  __shared__ float sh[8];
  const int row = blockIdx.x;
  if (!NB_IN_BOUNDS(NB_SITE_ROW_INDEX, row, rows)) return;   // debug build: one block per row
  const T* xr = x + (size_t)row * D;
  T* yr = y + (size_t)row * D;
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    const float v = to_f<T>(xr[c]);
    if (v > m) { s = s * __expf(m - v); m = v; }
    s += __expf(v - m);
  }
  const float gm = block_max<8>(m, sh);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum<8>(s, sh);
  const float lse = gm + logf(gs);
  const float inv = 1.f / gs;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    const float v = to_f<T>(xr[c]);
    yr[c] = from_f<T>(LOG ? (v - lse) : __expf(v - gm) * inv);
  }
}

// ============================================================== cross entropy building blocks
// Per row: lse = logsumexp(logits_row); picked = logits_row[target] when 0 <= target < D else 0.
// A vocabulary shard passes targets shifted by its offset, so out-of-range simply means
// "another shard holds this class"; the caller combines shards with max/sum reductions.
template <typename T>
__global__ void __launch_bounds__(256) lse_pick_fwd_kernel(const T* __restrict__ logits,
                                                          const long long* __restrict__ tgt, float* __restrict__ lse_out,
                                                          float* __restrict__ picked, int rows, int D) {
  __shared__ float sh[8];
  const int row = blockIdx.x;
  if (!NB_IN_BOUNDS(NB_SITE_ROW_INDEX, row, rows)) return;   // debug build: one block per row
  const T* xr = logits + (size_t)row * D;
  float m = -INFINITY, s = 0.f;
  constexpr int V = Vec<T>::N;
  if ((D % V) == 0) {
    for (int c = threadIdx.x * V; c < D; c += blockDim.x * V) {
      float v[V];
      load_vec<T>(xr + c, v);
      float lm = v[0];
#pragma unroll
      for (int j = 1; j < V; ++j) lm = fmaxf(lm, v[j]);
      if (lm > m) { s = s * __expf(m - lm); m = lm; }
#pragma unroll
      for (int j = 0; j < V; ++j) s += __expf(v[j] - m);
    }
  } else {
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      const float v = to_f<T>(xr[c]);
      if (v > m) { s = s * __expf(m - v); m = v; }
      s += __expf(v - m);
    }
  }
  const float gm = block_max<8>(m, sh);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum<8>(s, sh);
  if (threadIdx.x == 0) {
    const long long t = tgt[row];
    lse_out[row] = gm + logf(gs);
    picked[row] = (t >= 0 && t < D) ? to_f<T>(xr[t]) : 0.f;
  }
}
// dlogits = exp(logits - lse) * g_lse[row] + onehot(target) * g_pick[row]
template <typename T>
__global__ void __launch_bounds__(256) lse_pick_bwd_kernel(const T* __restrict__ logits,
                                                          const long long* __restrict__ tgt,
                                                          const float* __restrict__ lse, const float* __restrict__ g_lse,
                                                          const float* __restrict__ g_pick, T* __restrict__ dlogits,
                                                          int rows, int D) {
  const int row = blockIdx.x;
  if (!NB_IN_BOUNDS(NB_SITE_ROW_INDEX, row, rows)) return;   // debug build: one block per row
  const T* xr = logits + (size_t)row * D;
  T* dr = dlogits + (size_t)row * D;
  const float l = lse[row];
  const long long t = tgt[row];
  const float gl = g_lse ? g_lse[row] : 0.f;
  const float gp = g_pick ? g_pick[row] : 0.f;
  constexpr int V = Vec<T>::N;
  if ((D % V) == 0) {
    for (int c = threadIdx.x * V; c < D; c += blockDim.x * V) {
      float v[V], o[V];
      load_vec<T>(xr + c, v);
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = __expf(v[j] - l) * gl + ((c + j) == t ? gp : 0.f);
      store_vec<T>(dr + c, o);
    }
  } else {
    for (int c = threadIdx.x; c < D; c += blockDim.x)
      dr[c] = from_f<T>(__expf(to_f<T>(xr[c]) - l) * gl + (c == t ? gp : 0.f));
  }
}

// ============================================================== optimizers
// AdamW with decoupled weight decay; P/G may be bf16 or fp32, moments fp32.
// step-dependent bias corrections are passed as bc1 = 1 - b1^t, bc2 = 1 - b2^t via device scalars
// when `hyper` is non-null: hyper = {lr, bc1, bc2, grad_scale}.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float* out);
template <>
__device__ __forceinline__ void load8<bf16>(const bf16* p, float* out) { load_vec<bf16>(p, out); }
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* out) {
  load_vec<float>(p, out);
  load_vec<float>(p + 4, out + 4);
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float* in);
template <>
__device__ __forceinline__ void store8<bf16>(bf16* p, const float* in) { store_vec<bf16>(p, in); }
template <>
__device__ __forceinline__ void store8<float>(float* p, const float* in) {
  store_vec<float>(p, in);
  store_vec<float>(p + 4, in + 4);
}

// 8 elements per thread with 16-byte accesses (all tensors come from the caching allocator and
// are at least 16-byte aligned); the ragged tail is handled element-wise.
template <typename TP, typename TG>
__global__ void __launch_bounds__(256) adamw_kernel(const TP* __restrict__ p, const TG* __restrict__ g,
                                                   const float* __restrict__ m, const float* __restrict__ v,
                                                   TP* __restrict__ p_out, float* __restrict__ m_out,
                                                   float* __restrict__ v_out, size_t n, float lr, float b1, float b2,
                                                   float eps, float wd, float bc1, float bc2, float grad_scale,
                                                   const float* __restrict__ hyper) {
  if (hyper) { lr = hyper[0]; bc1 = hyper[1]; bc2 = hyper[2]; grad_scale = hyper[3]; }
  const float ibc1 = 1.f / bc1, ibc2 = 1.f / bc2;
  const size_t i0 = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  const size_t stride = (size_t)gridDim.x * blockDim.x * 8;
  for (size_t i = i0; i < n; i += stride) {
    float pv[8], gv[8], mv[8], vv[8];
    const bool full = i + 8 <= n;
    if (full) {
      load8<TP>(p + i, pv);
      load8<TG>(g + i, gv);
      load8<float>(m + i, mv);
      load8<float>(v + i, vv);
    } else {
      for (int j = 0; j < 8; ++j) {
        const bool ok = i + j < n;
        pv[j] = ok ? to_f<TP>(p[i + j]) : 0.f;
        gv[j] = ok ? to_f<TG>(g[i + j]) : 0.f;
        mv[j] = ok ? m[i + j] : 0.f;
        vv[j] = ok ? v[i + j] : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gr = gv[j] * grad_scale;
      mv[j] = b1 * mv[j] + (1.f - b1) * gr;
      vv[j] = b2 * vv[j] + (1.f - b2) * gr * gr;
      const float upd = (mv[j] * ibc1) / (sqrtf(vv[j] * ibc2) + eps) + wd * pv[j];
      pv[j] -= lr * upd;
    }
    if (full) {
      store8<TP>(p_out + i, pv);
      store8<float>(m_out + i, mv);
      store8<float>(v_out + i, vv);
    } else {
      for (int j = 0; j < 8; ++j)
        if (i + j < n) {
          p_out[i + j] = from_f<TP>(pv[j]);
          m_out[i + j] = mv[j];
          v_out[i + j] = vv[j];
        }
    }
  }
}
template <typename TP, typename TG>
__global__ void __launch_bounds__(256) sgd_kernel(const TP* __restrict__ p, const TG* __restrict__ g,
                                                 const float* __restrict__ buf, TP* __restrict__ p_out,
                                                 float* __restrict__ buf_out, size_t n, float lr, float momentum,
                                                 float wd, float grad_scale) {
  const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t k = i0; k < n; k += stride) {
    const float pm = to_f<TP>(p[k]);
    float gr = to_f<TG>(g[k]) * grad_scale + wd * pm;
    if (buf) {
      gr = momentum * buf[k] + gr;
      buf_out[k] = gr;
    }
    p_out[k] = from_f<TP>(pm - lr * gr);
  }
}

// ============================================================== embedding
template <typename T>
__global__ void __launch_bounds__(128) embedding_gather_kernel(const T* __restrict__ table,
                                                              const long long* __restrict__ ids, T* __restrict__ out,
                                                              int n_ids, int D, int vocab) {
  constexpr int V = Vec<T>::N;
  const int i = blockIdx.x;
  if (!NB_IN_BOUNDS(NB_SITE_ROW_INDEX, i, n_ids)) return;   // debug build: one block per id
  long long id = ids[i];
  const bool ok = id >= 0 && id < vocab;
  const T* src = table + (size_t)(ok ? id : 0) * D;
  T* dst = out + (size_t)i * D;
  if ((D % V) == 0) {
    for (int c = threadIdx.x * V; c < D; c += blockDim.x * V) {
      uint4 raw = ok ? *reinterpret_cast<const uint4*>(src + c) : make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(dst + c) = raw;
    }
  } else {
    for (int c = threadIdx.x; c < D; c += blockDim.x) dst[c] = ok ? src[c] : from_f<T>(0.f);
  }
}
// acc[ids[i]] += upd[i]  (fp32 accumulation table)
template <typename T>
__global__ void __launch_bounds__(128) embedding_scatter_add_kernel(float* __restrict__ acc,
                                                                   const long long* __restrict__ ids,
                                                                   const T* __restrict__ upd, int n_ids, int D,
                                                                   int vocab) {
  const int i = blockIdx.x;
  if (!NB_IN_BOUNDS(NB_SITE_ROW_INDEX, i, n_ids)) return;   // debug build: one block per id
  const long long id = ids[i];
  if (id < 0 || id >= vocab) return;
  float* dst = acc + (size_t)id * D;
  const T* src = upd + (size_t)i * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) atomicAdd(dst + c, to_f<T>(src[c]));
}
// The same sum without atomics, for runs that must repeat bit for bit: the ids come sorted (stable,
// `perm[k]` = position of the k-th sorted id in the original order); the block at the head of each
// run of equal ids adds the run's rows in that order and writes base + sum.
template <typename T>
__global__ void __launch_bounds__(128) embedding_scatter_sorted_kernel(const long long* __restrict__ sorted_ids,
                                                                      const long long* __restrict__ perm,
                                                                      const T* __restrict__ upd, const T* __restrict__ base,
                                                                      T* __restrict__ out, int n_ids, int D, int vocab) {
  const int i = blockIdx.x;
  if (!NB_IN_BOUNDS(NB_SITE_ROW_INDEX, i, n_ids)) return;
  const long long id = sorted_ids[i];
  if (id < 0 || id >= vocab) return;
  if (i > 0 && sorted_ids[i - 1] == id) return;   // not the head of its run
  int end = i + 1;
  while (end < n_ids && sorted_ids[end] == id) ++end;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.f;
    for (int k = i; k < end; ++k) {
      const long long src = perm[k];
      if (!NB_IN_BOUNDS(NB_SITE_EMB_SCATTER_ID, src, n_ids)) continue;
      acc += to_f<T>(upd[(size_t)src * D + c]);
    }
    out[(size_t)id * D + c] = from_f<T>(to_f<T>(base[(size_t)id * D + c]) + acc);
  }
}
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n,
                                                  const TO* __restrict__ add_to) {
  const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t k = i0; k < n; k += stride) {
    float v = to_f<TI>(in[k]);
    if (add_to) v += to_f<TO>(add_to[k]);
    out[k] = from_f<TO>(v);
  }
}

// ============================================================== activations
__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
  return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float dgelu_f(float x) {
  return 0.5f * (1.f + erff(x * 0.70710678118654752f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}
__device__ __forceinline__ float dgelu_tanh_f(float x) {
  const float x2 = x * x, u = 0.7978845608028654f * (x + 0.044715f * x * x2), t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * x2);
}
// mode: 0 relu, 1 gelu(erf), 2 gelu(tanh), 3 silu ; bwd: out = dy * act'(z)
template <typename T, bool BWD>
__global__ void __launch_bounds__(256) act_kernel(const T* __restrict__ z, const T* __restrict__ dy, T* __restrict__ out,
                                                 size_t n, int mode) {
  constexpr int V = Vec<T>::N;
  const size_t i0 = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V;
  const size_t stride = (size_t)gridDim.x * blockDim.x * V;
  for (size_t i = i0; i < n; i += stride) {
    float zv[V], dv[V], o[V];
    if (i + V <= n) {
      load_vec<T>(z + i, zv);
      if (BWD) load_vec<T>(dy + i, dv);
    } else {
      for (int j = 0; j < V; ++j) {
        zv[j] = (i + j < n) ? to_f<T>(z[i + j]) : 0.f;
        dv[j] = (BWD && i + j < n) ? to_f<T>(dy[i + j]) : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float x = zv[j];
      float r;
      if (!BWD) {
        r = mode == 0 ? fmaxf(x, 0.f) : mode == 1 ? gelu_f(x) : mode == 2 ? gelu_tanh_f(x) : x / (1.f + __expf(-x));
      } else {
        float d;
        if (mode == 0) d = x > 0.f ? 1.f : 0.f;
        else if (mode == 1) d = dgelu_f(x);
        else if (mode == 2) d = dgelu_tanh_f(x);
        else { const float sg = 1.f / (1.f + __expf(-x)); d = sg * (1.f + x * (1.f - sg)); }
        r = dv[j] * d;
      }
      o[j] = r;
    }
    if (i + V <= n) store_vec<T>(out + i, o);
    else for (int j = 0; j < V; ++j) if (i + j < n) out[i + j] = from_f<T>(o[j]);
  }
}

// ============================================================== Philox4x32-10 RNG
struct Philox {
  uint32_t key[2];
  uint32_t ctr[4];
  __device__ Philox(uint64_t seed, uint64_t subseq, uint64_t offset) {
    key[0] = (uint32_t)seed; key[1] = (uint32_t)(seed >> 32);
    ctr[0] = (uint32_t)offset; ctr[1] = (uint32_t)(offset >> 32);
    ctr[2] = (uint32_t)subseq; ctr[3] = (uint32_t)(subseq >> 32);
  }
  __device__ uint4 next() {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3], k0 = key[0], k1 = key[1];
#pragma unroll
    for (int r = 0; r < 10; ++r) {
      const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
      const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
      const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
      c0 = n0; c1 = n1; c2 = n2; c3 = n3;
      k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    if (++ctr[0] == 0) ++ctr[1];
    return make_uint4(c0, c1, c2, c3);
  }
};
__device__ __forceinline__ float u01(uint32_t x) { return ((x >> 8) + 0.5f) * (1.0f / 16777216.0f); }

// Random streams. With `state` (device memory: [0] seed, [1] number of draws made so far on this
// device) the Philox key and offset come from there and `seed` is only a salt that tells the shards
// of one tensor apart; the launcher advances state[1] with a one-thread kernel afterwards. Because
// the kernel reads the state when it RUNS, a launch replayed from a CUDA graph draws fresh numbers
// every time (reference: the seed threaded graph-in -> graph-out, nabla/core/graph/engine.py:80-88).
__device__ __forceinline__ void rng_resolve(const unsigned long long* state, uint64_t& seed, uint64_t& offset) {
  if (state != nullptr) {
    seed = state[0] * 1000003ull + seed;
    offset = state[1] << 32;
  }
}
__global__ void rng_bump_kernel(unsigned long long* state) { state[1] += 1ull; }

// mode 0: uniform in [a, b); mode 1: gaussian mean a std b
template <typename T>
__global__ void __launch_bounds__(256) rng_kernel(T* __restrict__ out, size_t n, uint64_t seed, uint64_t offset,
                                                 int mode, float a, float b, const unsigned long long* state) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nthreads = (size_t)gridDim.x * blockDim.x;
  rng_resolve(state, seed, offset);
  Philox ph(seed, tid, offset);
  for (size_t i = tid * 4; i < n; i += nthreads * 4) {
    const uint4 r = ph.next();
    float f[4];
    if (mode == 0) {
      f[0] = a + (b - a) * u01(r.x); f[1] = a + (b - a) * u01(r.y);
      f[2] = a + (b - a) * u01(r.z); f[3] = a + (b - a) * u01(r.w);
    } else {
      const float r1 = sqrtf(-2.f * logf(u01(r.x))), t1 = 6.283185307179586f * u01(r.y);
      const float r2 = sqrtf(-2.f * logf(u01(r.z))), t2 = 6.283185307179586f * u01(r.w);
      f[0] = a + b * r1 * cosf(t1); f[1] = a + b * r1 * sinf(t1);
      f[2] = a + b * r2 * cosf(t2); f[3] = a + b * r2 * sinf(t2);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) if (i + j < n) out[i + j] = from_f<T>(f[j]);
  }
}
// y = x * mask / (1-p); mask (uint8) kept for the backward
template <typename T>
__global__ void __launch_bounds__(256) dropout_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                     uint8_t* __restrict__ mask, size_t n, float p, uint64_t seed,
                                                     uint64_t offset, const unsigned long long* state) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nthreads = (size_t)gridDim.x * blockDim.x;
  rng_resolve(state, seed, offset);
  Philox ph(seed, tid, offset);
  const float keep_scale = 1.f / (1.f - p);
  for (size_t i = tid * 4; i < n; i += nthreads * 4) {
    const uint4 r = ph.next();
    const float u[4] = {u01(r.x), u01(r.y), u01(r.z), u01(r.w)};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (i + j < n) {
        const bool keep = u[j] >= p;
        mask[i + j] = keep ? 1 : 0;
        y[i + j] = from_f<T>(keep ? to_f<T>(x[i + j]) * keep_scale : 0.f);
      }
    }
  }
}

// ============================================================== NF4 dequantisation
// packed: 2 codes per byte (high nibble first); absmax per block of `block` elements.
__constant__ float NF4_CODE[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                   -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                   0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f,
                                   0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f,
                                   0.7229568362236023f, 1.0f};
template <typename T>
__global__ void __launch_bounds__(256) nf4_dequant_kernel(const uint8_t* __restrict__ packed,
                                                         const float* __restrict__ absmax, T* __restrict__ out,
                                                         size_t n, int block) {
  const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t b = i0; b * 2 < n; b += stride) {
    const uint8_t byte = packed[b];
    const size_t e0 = b * 2;
    out[e0] = from_f<T>(NF4_CODE[byte >> 4] * absmax[e0 / block]);
    if (e0 + 1 < n) out[e0 + 1] = from_f<T>(NF4_CODE[byte & 15] * absmax[(e0 + 1) / block]);
  }
}

// One code per byte (the layout of the QLoRA weight dict: `indices` uint8 [padded_numel], `scales`
// fp32 per block) and the 16-entry codebook passed by the caller. 16 codes per thread: one 16-byte
// load of codes, the block scale read once per run of codes in the same block.
template <typename T>
__global__ void __launch_bounds__(256) nf4_dequant_codes_kernel(const uint8_t* __restrict__ codes,
                                                               const float* __restrict__ absmax,
                                                               const float* __restrict__ codebook, T* __restrict__ out,
                                                               size_t n, int block) {
  __shared__ float cb[16];
  if (threadIdx.x < 16) cb[threadIdx.x] = codebook[threadIdx.x];
  __syncthreads();
  const size_t stride = (size_t)gridDim.x * blockDim.x * 16;
  for (size_t i0 = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 16; i0 < n; i0 += stride) {
    uint8_t c[16];
    if (i0 + 16 <= n && (reinterpret_cast<uintptr_t>(codes + i0) & 15) == 0) {
      *reinterpret_cast<uint4*>(c) = *reinterpret_cast<const uint4*>(codes + i0);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) c[j] = i0 + j < n ? codes[i0 + j] : 0;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (i0 + j < n) out[i0 + j] = from_f<T>(cb[c[j] & 15] * absmax[(i0 + j) / block]);
  }
}

// ============================================================== pooling (NHWC)
// mode 0 avg, 1 max. Backward: avg spreads dy/(kh*kw); max routes to the first arg-max.
template <typename T>
__global__ void __launch_bounds__(256) pool2d_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int N, int H, int W,
                                                        int C, int OH, int OW, int kh, int kw, int sh, int sw, int ph,
                                                        int pw, int mode) {
  const size_t total = (size_t)N * OH * OW * C;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = i % C;
    size_t r = i / C;
    const int ow = r % OW; r /= OW;
    const int oh = r % OH;
    const int n = r / OH;
    float acc = mode == 0 ? 0.f : -INFINITY;
    for (int a = 0; a < kh; ++a)
      for (int b = 0; b < kw; ++b) {
        const int ih = oh * sh - ph + a, iw = ow * sw - pw + b;
        float v = mode == 0 ? 0.f : -INFINITY;
        if (ih >= 0 && ih < H && iw >= 0 && iw < W) v = to_f<T>(x[(((size_t)n * H + ih) * W + iw) * C + c]);
        acc = mode == 0 ? acc + v : fmaxf(acc, v);
      }
    y[i] = from_f<T>(mode == 0 ? acc / (kh * kw) : acc);
  }
}
// out[window] = t[first arg-max of x over the window] (0 for a window that lies in the padding): the
// forward-mode derivative of max pooling, and the transpose of its backward routing.
template <typename T>
__global__ void __launch_bounds__(256) pool2d_select_kernel(const T* __restrict__ x, const T* __restrict__ t,
                                                           T* __restrict__ y, int N, int H, int W, int C, int OH, int OW,
                                                           int kh, int kw, int sh, int sw, int ph, int pw) {
  const size_t total = (size_t)N * OH * OW * C;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = i % C;
    size_t r = i / C;
    const int ow = r % OW; r /= OW;
    const int oh = r % OH;
    const int n = r / OH;
    float best = -INFINITY;
    size_t at = 0;
    bool found = false;
    for (int a = 0; a < kh; ++a)
      for (int b = 0; b < kw; ++b) {
        const int ih = oh * sh - ph + a, iw = ow * sw - pw + b;
        if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
          const size_t off = (((size_t)n * H + ih) * W + iw) * C + c;
          const float v = to_f<T>(x[off]);
          if (v > best || !found) { best = v; at = off; found = true; }
        }
      }
    y[i] = found ? t[at] : from_f<T>(0.f);
  }
}

// Backward in gather form: one thread per input pixel sums over the windows that cover it (for max
// pooling it finds each window's first arg-max again and takes the gradient when that is this
// pixel). No atomics, so the result does not depend on the order in which blocks run, and dx needs
// no zero fill and no fp32 staging.
template <typename T>
__global__ void __launch_bounds__(256) pool2d_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                        T* __restrict__ dx, int N, int H, int W, int C, int OH,
                                                        int OW, int kh, int kw, int sh, int sw, int ph, int pw, int mode) {
  const size_t total = (size_t)N * H * W * C;
  const float inv = 1.f / (kh * kw);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = i % C;
    size_t r = i / C;
    const int iw = r % W; r /= W;
    const int ih = r % H;
    const int n = r / H;
    // windows (oh, ow) with oh*sh - ph <= ih < oh*sh - ph + kh, likewise for the width
    const int th = ih + ph - kh + 1, tw = iw + pw - kw + 1;
    const int oh_lo = th > 0 ? (th + sh - 1) / sh : 0, oh_hi = min(OH - 1, (ih + ph) / sh);
    const int ow_lo = tw > 0 ? (tw + sw - 1) / sw : 0, ow_hi = min(OW - 1, (iw + pw) / sw);
    float acc = 0.f;
    for (int oh = oh_lo; oh <= oh_hi; ++oh)
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        const size_t yo = (((size_t)n * OH + oh) * OW + ow) * C + c;
        if (!NB_IN_BOUNDS(NB_SITE_POOL_INPUT, yo, (size_t)N * OH * OW * C)) continue;
        const float g = to_f<T>(dy[yo]);
        if (mode == 0) {
          acc += g * inv;
        } else {
          float best = -INFINITY;
          int bh = -1, bw = -1;
          for (int a = 0; a < kh; ++a)
            for (int b = 0; b < kw; ++b) {
              const int jh = oh * sh - ph + a, jw = ow * sw - pw + b;
              if (jh >= 0 && jh < H && jw >= 0 && jw < W) {
                const float v = to_f<T>(x[(((size_t)n * H + jh) * W + jw) * C + c]);
                if (v > best) { best = v; bh = jh; bw = jw; }
              }
            }
          if (bh == ih && bw == iw) acc += g;
        }
      }
    dx[i] = from_f<T>(acc);
  }
}

// ============================================================== direct conv2d NHWC x RSCF (small C)
// y[n,oh,ow,f] = sum_{r,s,c} x[n, oh*sh - pt + r*dh, ow*sw - pl + s*dw, c] * w[r,s,c,f] (+ bias[f])
template <typename T>
__global__ void __launch_bounds__(128) conv2d_direct_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                           const T* __restrict__ bias, T* __restrict__ y, int N, int H,
                                                           int W, int C, int R, int S, int F, int OH, int OW, int sh,
                                                           int sw, int pt, int pl) {
  const size_t total = (size_t)N * OH * OW * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int f = i % F;
    size_t r_ = i / F;
    const int ow = r_ % OW; r_ /= OW;
    const int oh = r_ % OH;
    const int n = r_ / OH;
    float acc = bias ? to_f<T>(bias[f]) : 0.f;
    for (int r = 0; r < R; ++r) {
      const int ih = oh * sh - pt + r;
      if (ih < 0 || ih >= H) continue;
      for (int s = 0; s < S; ++s) {
        const int iw = ow * sw - pl + s;
        if (iw < 0 || iw >= W) continue;
        if (!NB_IN_BOUNDS(NB_SITE_CONV_INPUT, (((size_t)n * H + ih) * W + iw) * C, (size_t)N * H * W * C)) continue;
        const T* xp = x + (((size_t)n * H + ih) * W + iw) * C;
        const T* wp = w + ((size_t)(r * S + s) * C) * F + f;
        for (int c = 0; c < C; ++c) acc += to_f<T>(xp[c]) * to_f<T>(wp[(size_t)c * F]);
      }
    }
    y[i] = from_f<T>(acc);
  }
}

// Filter gradient of the direct convolution (small channel counts, fp32 or bf16):
//   dw[r,s,c,f] = sum_{n,oh,ow} x[n, oh*sh - pt + r, ow*sw - pl + s, c] * dy[n,oh,ow,f]
// One block per (r, s, c) and tile of 32 output channels. Lane = output channel (coalesced reads
// of dy, one broadcast read of x per position), the 8 warps split the N*OH*OW positions and are
// summed through shared memory: plain stores, no atomics, deterministic.
template <typename T>
__global__ void __launch_bounds__(256) conv2d_wgrad_direct_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                                 T* __restrict__ dw, int N, int H, int W, int C, int R,
                                                                 int S, int F, int OH, int OW, int sh, int sw, int pt,
                                                                 int pl) {
  __shared__ float part[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int f = blockIdx.y * 32 + lane;
  int rsc = blockIdx.x;
  const int c = rsc % C; rsc /= C;
  const int s = rsc % S;
  const int r = rsc / S;
  const long long positions = (long long)N * OH * OW;
  float acc = 0.f;
  for (long long p = warp; p < positions; p += 8) {
    const int ow = (int)(p % OW);
    long long q = p / OW;
    const int oh = (int)(q % OH);
    const int n = (int)(q / OH);
    const int ih = oh * sh - pt + r, iw = ow * sw - pl + s;
    if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
    const float xv = to_f<T>(x[(((size_t)n * H + ih) * W + iw) * C + c]);
    if (f < F) acc += xv * to_f<T>(dy[(size_t)p * F + f]);
  }
  part[warp][lane] = acc;
  __syncthreads();
  if (warp == 0 && f < F) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += part[i][lane];
    dw[((size_t)(r * S + s) * C + c) * F + f] = from_f<T>(t);
  }
}

// out[i] = sum_j part[j][i] for `slices` fp32 slices of n elements (n % 4 == 0): the second half of
// a split-K GEMM, whose partial products are written as fp32 by the tensor-core kernel.
template <typename T>
__global__ void __launch_bounds__(256) sum_slices_kernel(const float* __restrict__ part, T* __restrict__ out, size_t n,
                                                        int slices) {
  const size_t nv = n / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    float4 acc = reinterpret_cast<const float4*>(part)[i];
    for (int j = 1; j < slices; ++j) {
      const float4 v = reinterpret_cast<const float4*>(part + (size_t)j * n)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    out[4 * i] = from_f<T>(acc.x); out[4 * i + 1] = from_f<T>(acc.y);
    out[4 * i + 2] = from_f<T>(acc.z); out[4 * i + 3] = from_f<T>(acc.w);
  }
}

static inline int grid_for(size_t n, int per_block, int cap = 148 * 16) {
  size_t g = (n + per_block - 1) / per_block;
  if (g < 1) g = 1;
  return (int)(g > (size_t)cap ? cap : g);
}

}  // namespace nbk

using namespace nbk;
#define STREAM reinterpret_cast<cudaStream_t>(stream)
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : -1)

// dtype codes: 0 = fp32, 1 = bf16
extern "C" {

int nb_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int rows,
                     int D, float eps, int dtype, void* stream) {
  if (rows <= 0) return 0;
  const int V = dtype ? 8 : 4;
  if (D % V) return -2;
  const int vpl = (D / V + 31) / 32;
  dim3 grid((rows + 3) / 4), block(128);
#define LN_FWD(T, VPL) layernorm_fwd_kernel<T, VPL><<<grid, block, 0, STREAM>>>((const T*)x, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, D, eps)
  if (dtype) {
    if (vpl <= 1) LN_FWD(bf16, 1); else if (vpl <= 2) LN_FWD(bf16, 2); else if (vpl <= 4) LN_FWD(bf16, 4);
    else if (vpl <= 8) LN_FWD(bf16, 8); else if (vpl <= 16) LN_FWD(bf16, 16); else return -3;
  } else {
    if (vpl <= 1) LN_FWD(float, 1); else if (vpl <= 2) LN_FWD(float, 2); else if (vpl <= 4) LN_FWD(float, 4);
    else if (vpl <= 8) LN_FWD(float, 8); else if (vpl <= 16) LN_FWD(float, 16); else return -3;
  }
  return CHECK_LAUNCH();
}

// Number of rows of the `partial` scratch buffer (each 2*D floats) that nb_layernorm_bwd writes for
// this problem: the grid of the one-pass kernel when the row fits 8 vectors per lane, else the
// number of row slabs of the two-kernel path.
static int ln_bwd_vpl(int D, int dtype) { const int V = dtype ? 8 : 4; return (D / V + 31) / 32; }
static int g_ln_bwd_two_kernels = 0;
// 1: always take the two-kernel path (dx, then dgamma / dbeta), for comparisons.
void nb_layernorm_bwd_two_kernels(int on) { g_ln_bwd_two_kernels = on; }
int nb_layernorm_bwd_nblocks(int rows, int D, int dtype) {
  const int vpl = ln_bwd_vpl(D, dtype);
  if (vpl <= 8 && !g_ln_bwd_two_kernels) {
    const int V = dtype ? 8 : 4;
    const int cap = 148 * (vpl * V >= 64 ? 2 : vpl * V >= 32 ? 3 : 4);   // resident blocks of the kernel
    int nb = (rows + 3) / 4;
    if (nb > cap) nb = cap;
    return nb < 1 ? 1 : nb;
  }
  int nb = (rows + 255) / 256;
  if (nb > 128) nb = 128;
  return nb < 1 ? 1 : nb;
}

int nb_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                     void* dgamma, void* dbeta, float* partial, int rows, int D, int dtype, void* stream) {
  if (rows <= 0) return 0;
  const int V = dtype ? 8 : 4;
  if (D % V) return -2;
  const int vpl = ln_bwd_vpl(D, dtype);
  const int nb = nb_layernorm_bwd_nblocks(rows, D, dtype);
  const int rpb = (rows + nb - 1) / nb;
  dim3 grid_dx((rows + 3) / 4);
  dim3 grid_gb((D + 32 * V - 1) / (32 * V), nb);
#define LN_BWD1(T, VPL)                                                                                               \
  {                                                                                                                   \
    layernorm_bwd_fused_kernel<T, VPL><<<nb, 128, 0, STREAM>>>((const T*)dy, (const T*)x, (const T*)gamma, mean, rstd, \
                                                               (T*)dx, partial, rows, D);                            \
    colsum_partials_kernel<T><<<(D + 31) / 32, 256, 0, STREAM>>>(partial, (T*)dgamma, (T*)dbeta, nb, D);            \
  }
#define LN_BWD(T, VPL)                                                                                                \
  {                                                                                                                   \
    layernorm_bwd_dx_kernel<T, VPL><<<grid_dx, 128, 0, STREAM>>>((const T*)dy, (const T*)x, (const T*)gamma, mean,    \
                                                                  rstd, (T*)dx, rows, D);                            \
    layernorm_bwd_dgb_kernel<T><<<grid_gb, 256, 0, STREAM>>>((const T*)dy, (const T*)x, mean, rstd, partial, rows, D, \
                                                              rpb);                                                   \
    colsum_partials_kernel<T><<<(D + 31) / 32, 256, 0, STREAM>>>(partial, (T*)dgamma, (T*)dbeta, nb, D);            \
  }
  if (g_ln_bwd_two_kernels) {
    if (dtype) {
      if (vpl <= 1) LN_BWD(bf16, 1) else if (vpl <= 2) LN_BWD(bf16, 2) else if (vpl <= 4) LN_BWD(bf16, 4)
      else if (vpl <= 8) LN_BWD(bf16, 8) else if (vpl <= 16) LN_BWD(bf16, 16) else return -3;
    } else {
      if (vpl <= 1) LN_BWD(float, 1) else if (vpl <= 2) LN_BWD(float, 2) else if (vpl <= 4) LN_BWD(float, 4)
      else if (vpl <= 8) LN_BWD(float, 8) else if (vpl <= 16) LN_BWD(float, 16) else return -3;
    }
  } else if (dtype) {
    if (vpl <= 1) LN_BWD1(bf16, 1) else if (vpl <= 2) LN_BWD1(bf16, 2) else if (vpl <= 4) LN_BWD1(bf16, 4)
    else if (vpl <= 8) LN_BWD1(bf16, 8) else if (vpl <= 16) LN_BWD(bf16, 16) else return -3;
  } else {
    if (vpl <= 1) LN_BWD1(float, 1) else if (vpl <= 2) LN_BWD1(float, 2) else if (vpl <= 4) LN_BWD1(float, 4)
    else if (vpl <= 8) LN_BWD1(float, 8) else if (vpl <= 16) LN_BWD(float, 16) else return -3;
  }
  return CHECK_LAUNCH();
}

int nb_colsum_nparts(int rows) {
  int np = (rows + 511) / 512;
  if (np > 64) np = 64;
  return np < 1 ? 1 : np;
}
int nb_colsum(const void* x, void* out, float* partial, int rows, int N, int in_dtype, int out_dtype, void* stream) {
  const int V = in_dtype ? 8 : 4;
  if (N % V) return -2;
  const int np = nb_colsum_nparts(rows);
  const int rpb = (rows + np - 1) / np;
  dim3 grid((N + 32 * V - 1) / (32 * V), np);
  if (in_dtype) colsum_kernel<bf16><<<grid, 256, 0, STREAM>>>((const bf16*)x, partial, rows, N, rpb);
  else colsum_kernel<float><<<grid, 256, 0, STREAM>>>((const float*)x, partial, rows, N, rpb);
  if (out_dtype) colsum_final_kernel<bf16><<<(N + 255) / 256, 256, 0, STREAM>>>(partial, (bf16*)out, np, N);
  else colsum_final_kernel<float><<<(N + 255) / 256, 256, 0, STREAM>>>(partial, (float*)out, np, N);
  return CHECK_LAUNCH();
}

int nb_softmax(const void* x, void* y, int rows, int D, int log, int dtype, void* stream) {
  if (rows <= 0) return 0;
  if (dtype) {
    if (log) softmax_kernel<bf16, true><<<rows, 256, 0, STREAM>>>((const bf16*)x, (bf16*)y, rows, D);
    else softmax_kernel<bf16, false><<<rows, 256, 0, STREAM>>>((const bf16*)x, (bf16*)y, rows, D);
  } else {
    if (log) softmax_kernel<float, true><<<rows, 256, 0, STREAM>>>((const float*)x, (float*)y, rows, D);
    else softmax_kernel<float, false><<<rows, 256, 0, STREAM>>>((const float*)x, (float*)y, rows, D);
  }
  return CHECK_LAUNCH();
}

int nb_lse_pick_fwd(const void* logits, const long long* tgt, float* lse, float* picked, int rows, int D, int dtype,
                    void* stream) {
  if (rows <= 0) return 0;
  if (dtype) lse_pick_fwd_kernel<bf16><<<rows, 256, 0, STREAM>>>((const bf16*)logits, tgt, lse, picked, rows, D);
  else lse_pick_fwd_kernel<float><<<rows, 256, 0, STREAM>>>((const float*)logits, tgt, lse, picked, rows, D);
  return CHECK_LAUNCH();
}
int nb_lse_pick_bwd(const void* logits, const long long* tgt, const float* lse, const float* g_lse, const float* g_pick,
                    void* dlogits, int rows, int D, int dtype, void* stream) {
  if (rows <= 0) return 0;
  if (dtype)
    lse_pick_bwd_kernel<bf16><<<rows, 256, 0, STREAM>>>((const bf16*)logits, tgt, lse, g_lse, g_pick, (bf16*)dlogits, rows, D);
  else
    lse_pick_bwd_kernel<float><<<rows, 256, 0, STREAM>>>((const float*)logits, tgt, lse, g_lse, g_pick, (float*)dlogits, rows, D);
  return CHECK_LAUNCH();
}

int nb_adamw(const void* p, const void* g, const float* m, const float* v, void* p_out, float* m_out, float* v_out,
             long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
             const float* hyper, int p_dtype, int g_dtype, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for((size_t)n, 256 * 8, 148 * 8);
#define ADAMW(TP, TG) adamw_kernel<TP, TG><<<grid, 256, 0, STREAM>>>((const TP*)p, (const TG*)g, m, v, (TP*)p_out, m_out, v_out, (size_t)n, lr, b1, b2, eps, wd, bc1, bc2, grad_scale, hyper)
  if (p_dtype && g_dtype) ADAMW(bf16, bf16);
  else if (p_dtype) ADAMW(bf16, float);
  else if (g_dtype) ADAMW(float, bf16);
  else ADAMW(float, float);
  return CHECK_LAUNCH();
}
int nb_sgd(const void* p, const void* g, const float* buf, void* p_out, float* buf_out, long long n, float lr,
           float momentum, float wd, float grad_scale, int p_dtype, int g_dtype, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for((size_t)n, 256);
#define SGD(TP, TG) sgd_kernel<TP, TG><<<grid, 256, 0, STREAM>>>((const TP*)p, (const TG*)g, buf, (TP*)p_out, buf_out, (size_t)n, lr, momentum, wd, grad_scale)
  if (p_dtype && g_dtype) SGD(bf16, bf16);
  else if (p_dtype) SGD(bf16, float);
  else if (g_dtype) SGD(float, bf16);
  else SGD(float, float);
  return CHECK_LAUNCH();
}

int nb_embedding_gather(const void* table, const long long* ids, void* out, int n_ids, int D, int vocab, int dtype,
                        void* stream) {
  if (n_ids <= 0) return 0;
  if (dtype) embedding_gather_kernel<bf16><<<n_ids, 128, 0, STREAM>>>((const bf16*)table, ids, (bf16*)out, n_ids, D, vocab);
  else embedding_gather_kernel<float><<<n_ids, 128, 0, STREAM>>>((const float*)table, ids, (float*)out, n_ids, D, vocab);
  return CHECK_LAUNCH();
}
// acc (fp32, [vocab][D]) must be zeroed by the caller; out = base + acc, cast to dtype.
int nb_embedding_scatter_add(float* acc, const long long* ids, const void* upd, const void* base, void* out, int n_ids,
                             int D, int vocab, int dtype, void* stream) {
  if (n_ids > 0) {
    if (dtype) embedding_scatter_add_kernel<bf16><<<n_ids, 128, 0, STREAM>>>(acc, ids, (const bf16*)upd, n_ids, D, vocab);
    else embedding_scatter_add_kernel<float><<<n_ids, 128, 0, STREAM>>>(acc, ids, (const float*)upd, n_ids, D, vocab);
  }
  const size_t n = (size_t)vocab * D;
  const int grid = grid_for(n, 256);
  if (dtype) cast_kernel<float, bf16><<<grid, 256, 0, STREAM>>>(acc, (bf16*)out, n, (const bf16*)base);
  else cast_kernel<float, float><<<grid, 256, 0, STREAM>>>(acc, (float*)out, n, (const float*)base);
  return CHECK_LAUNCH();
}

// out = base + scatter_add(ids, upd) from stably sorted ids; `out` already holds a copy of `base`.
int nb_embedding_scatter_sorted(const long long* sorted_ids, const long long* perm, const void* upd, const void* base,
                                void* out, int n_ids, int D, int vocab, int dtype, void* stream) {
  if (n_ids <= 0) return 0;
  if (dtype) embedding_scatter_sorted_kernel<bf16><<<n_ids, 128, 0, STREAM>>>(sorted_ids, perm, (const bf16*)upd, (const bf16*)base, (bf16*)out, n_ids, D, vocab);
  else embedding_scatter_sorted_kernel<float><<<n_ids, 128, 0, STREAM>>>(sorted_ids, perm, (const float*)upd, (const float*)base, (float*)out, n_ids, D, vocab);
  return CHECK_LAUNCH();
}

int nb_cast(const void* in, void* out, long long n, int in_dtype, int out_dtype, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for((size_t)n, 256);
  if (in_dtype && !out_dtype) cast_kernel<bf16, float><<<grid, 256, 0, STREAM>>>((const bf16*)in, (float*)out, (size_t)n, nullptr);
  else if (!in_dtype && out_dtype) cast_kernel<float, bf16><<<grid, 256, 0, STREAM>>>((const float*)in, (bf16*)out, (size_t)n, nullptr);
  else return -2;
  return CHECK_LAUNCH();
}

int nb_activation(const void* z, const void* dy, void* out, long long n, int mode, int bwd, int dtype, void* stream) {
  if (n <= 0) return 0;
  const int V = dtype ? 8 : 4;
  const int grid = grid_for((size_t)n, 256 * V);
  if (dtype) {
    if (bwd) act_kernel<bf16, true><<<grid, 256, 0, STREAM>>>((const bf16*)z, (const bf16*)dy, (bf16*)out, (size_t)n, mode);
    else act_kernel<bf16, false><<<grid, 256, 0, STREAM>>>((const bf16*)z, nullptr, (bf16*)out, (size_t)n, mode);
  } else {
    if (bwd) act_kernel<float, true><<<grid, 256, 0, STREAM>>>((const float*)z, (const float*)dy, (float*)out, (size_t)n, mode);
    else act_kernel<float, false><<<grid, 256, 0, STREAM>>>((const float*)z, nullptr, (float*)out, (size_t)n, mode);
  }
  return CHECK_LAUNCH();
}

int nb_rng(void* out, long long n, unsigned long long seed, unsigned long long offset, int mode, float a, float b,
           int dtype, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for((size_t)n, 256 * 4, 148 * 8);
  if (dtype) rng_kernel<bf16><<<grid, 256, 0, STREAM>>>((bf16*)out, (size_t)n, seed, offset, mode, a, b, nullptr);
  else rng_kernel<float><<<grid, 256, 0, STREAM>>>((float*)out, (size_t)n, seed, offset, mode, a, b, nullptr);
  return CHECK_LAUNCH();
}
int nb_dropout(const void* x, void* y, unsigned char* mask, long long n, float p, unsigned long long seed,
               unsigned long long offset, int dtype, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for((size_t)n, 256 * 4, 148 * 8);
  if (dtype) dropout_kernel<bf16><<<grid, 256, 0, STREAM>>>((const bf16*)x, (bf16*)y, mask, (size_t)n, p, seed, offset, nullptr);
  else dropout_kernel<float><<<grid, 256, 0, STREAM>>>((const float*)x, (float*)y, mask, (size_t)n, p, seed, offset, nullptr);
  return CHECK_LAUNCH();
}
// Variants whose stream position lives on the device: `state` = [seed, draws so far] (two 64-bit
// words of device memory), `salt` distinguishes the shards of one tensor. The draw counter is
// advanced here, after the kernel, by a one-thread launch on the same stream.
int nb_rng_dev(void* out, long long n, unsigned long long* state, unsigned long long salt, int mode, float a, float b,
               int dtype, void* stream) {
  if (n > 0) {
    const int grid = grid_for((size_t)n, 256 * 4, 148 * 8);
    if (dtype) rng_kernel<bf16><<<grid, 256, 0, STREAM>>>((bf16*)out, (size_t)n, salt, 0, mode, a, b, state);
    else rng_kernel<float><<<grid, 256, 0, STREAM>>>((float*)out, (size_t)n, salt, 0, mode, a, b, state);
  }
  rng_bump_kernel<<<1, 1, 0, STREAM>>>(state);
  return CHECK_LAUNCH();
}
int nb_dropout_dev(const void* x, void* y, unsigned char* mask, long long n, float p, unsigned long long* state,
                   unsigned long long salt, int dtype, void* stream) {
  if (n > 0) {
    const int grid = grid_for((size_t)n, 256 * 4, 148 * 8);
    if (dtype) dropout_kernel<bf16><<<grid, 256, 0, STREAM>>>((const bf16*)x, (bf16*)y, mask, (size_t)n, p, salt, 0, state);
    else dropout_kernel<float><<<grid, 256, 0, STREAM>>>((const float*)x, (float*)y, mask, (size_t)n, p, salt, 0, state);
  }
  rng_bump_kernel<<<1, 1, 0, STREAM>>>(state);
  return CHECK_LAUNCH();
}

int nb_nf4_dequant(const unsigned char* packed, const float* absmax, void* out, long long n, int block, int dtype,
                   void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for((size_t)(n + 1) / 2, 256);
  if (dtype) nf4_dequant_kernel<bf16><<<grid, 256, 0, STREAM>>>(packed, absmax, (bf16*)out, (size_t)n, block);
  else nf4_dequant_kernel<float><<<grid, 256, 0, STREAM>>>(packed, absmax, (float*)out, (size_t)n, block);
  return CHECK_LAUNCH();
}

int nb_nf4_dequant_codes(const unsigned char* codes, const float* absmax, const float* codebook, void* out, long long n,
                         int block, int dtype, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for((size_t)(n + 15) / 16, 256);
  if (dtype) nf4_dequant_codes_kernel<bf16><<<grid, 256, 0, STREAM>>>(codes, absmax, codebook, (bf16*)out, (size_t)n, block);
  else nf4_dequant_codes_kernel<float><<<grid, 256, 0, STREAM>>>(codes, absmax, codebook, (float*)out, (size_t)n, block);
  return CHECK_LAUNCH();
}

int nb_pool2d_fwd(const void* x, void* y, int N, int H, int W, int C, int OH, int OW, int kh, int kw, int sh, int sw,
                  int ph, int pw, int mode, int dtype, void* stream) {
  const size_t total = (size_t)N * OH * OW * C;
  if (!total) return 0;
  const int grid = grid_for(total, 256);
  if (dtype) pool2d_fwd_kernel<bf16><<<grid, 256, 0, STREAM>>>((const bf16*)x, (bf16*)y, N, H, W, C, OH, OW, kh, kw, sh, sw, ph, pw, mode);
  else pool2d_fwd_kernel<float><<<grid, 256, 0, STREAM>>>((const float*)x, (float*)y, N, H, W, C, OH, OW, kh, kw, sh, sw, ph, pw, mode);
  return CHECK_LAUNCH();
}
// dx must be a zeroed fp32 buffer of the input's shape.
int nb_pool2d_bwd(const void* x, const void* dy, void* dx, int N, int H, int W, int C, int OH, int OW, int kh, int kw,
                  int sh, int sw, int ph, int pw, int mode, int dtype, void* stream) {
  const size_t total = (size_t)N * H * W * C;
  if (!total) return 0;
  const int grid = grid_for(total, 256);
  if (dtype) pool2d_bwd_kernel<bf16><<<grid, 256, 0, STREAM>>>((const bf16*)x, (const bf16*)dy, (bf16*)dx, N, H, W, C, OH, OW, kh, kw, sh, sw, ph, pw, mode);
  else pool2d_bwd_kernel<float><<<grid, 256, 0, STREAM>>>((const float*)x, (const float*)dy, (float*)dx, N, H, W, C, OH, OW, kh, kw, sh, sw, ph, pw, mode);
  return CHECK_LAUNCH();
}

int nb_pool2d_select(const void* x, const void* t, void* y, int N, int H, int W, int C, int OH, int OW, int kh, int kw,
                     int sh, int sw, int ph, int pw, int dtype, void* stream) {
  const size_t total = (size_t)N * OH * OW * C;
  if (!total) return 0;
  const int grid = grid_for(total, 256);
  if (dtype) pool2d_select_kernel<bf16><<<grid, 256, 0, STREAM>>>((const bf16*)x, (const bf16*)t, (bf16*)y, N, H, W, C, OH, OW, kh, kw, sh, sw, ph, pw);
  else pool2d_select_kernel<float><<<grid, 256, 0, STREAM>>>((const float*)x, (const float*)t, (float*)y, N, H, W, C, OH, OW, kh, kw, sh, sw, ph, pw);
  return CHECK_LAUNCH();
}

int nb_conv2d_direct(const void* x, const void* w, const void* bias, void* y, int N, int H, int W, int C, int R, int S,
                     int F, int OH, int OW, int sh, int sw, int pt, int pl, int dtype, void* stream) {
  const size_t total = (size_t)N * OH * OW * F;
  if (!total) return 0;
  const int grid = grid_for(total, 128, 148 * 32);
  if (dtype) conv2d_direct_kernel<bf16><<<grid, 128, 0, STREAM>>>((const bf16*)x, (const bf16*)w, (const bf16*)bias, (bf16*)y, N, H, W, C, R, S, F, OH, OW, sh, sw, pt, pl);
  else conv2d_direct_kernel<float><<<grid, 128, 0, STREAM>>>((const float*)x, (const float*)w, (const float*)bias, (float*)y, N, H, W, C, R, S, F, OH, OW, sh, sw, pt, pl);
  return CHECK_LAUNCH();
}

int nb_sum_slices(const float* part, void* out, long long n, int slices, int dtype, void* stream) {
  if (n <= 0 || slices <= 0) return 0;
  if (n & 3) return -2;
  const int grid = grid_for((size_t)n / 4, 256, 148 * 8);
  if (dtype) sum_slices_kernel<bf16><<<grid, 256, 0, STREAM>>>(part, (bf16*)out, (size_t)n, slices);
  else sum_slices_kernel<float><<<grid, 256, 0, STREAM>>>(part, (float*)out, (size_t)n, slices);
  return CHECK_LAUNCH();
}

int nb_conv2d_wgrad_direct(const void* x, const void* dy, void* dw, int N, int H, int W, int C, int R, int S, int F,
                           int OH, int OW, int sh, int sw, int pt, int pl, int dtype, void* stream) {
  if ((size_t)R * S * C * F == 0) return 0;
  const dim3 grid(R * S * C, (F + 31) / 32);
  if (dtype) conv2d_wgrad_direct_kernel<bf16><<<grid, 256, 0, STREAM>>>((const bf16*)x, (const bf16*)dy, (bf16*)dw, N, H, W, C, R, S, F, OH, OW, sh, sw, pt, pl);
  else conv2d_wgrad_direct_kernel<float><<<grid, 256, 0, STREAM>>>((const float*)x, (const float*)dy, (float*)dw, N, H, W, C, R, S, F, OH, OW, sh, sw, pt, pl);
  return CHECK_LAUNCH();
}

}  // extern "C"

NB_DEBUG_DEFINE(fused)
