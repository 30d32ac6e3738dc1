// Pointwise and reduction kernel families (fp32 / bf16, fp32 math), the long tail of ops behind
// nabla's binary / unary / reduction modules (reference: nabla/ops/binary.py, unary.py,
// reduction.py:152-217, 751-765, 821-826, which lower to MAX graph ops).
//
//   binary  out = a (op) b        b: same shape, one scalar element, or a row vector broadcast over
//                                 the leading dims (bias-style); 16-byte vectors, grid-stride
//   unary   out = f(a)            neg abs exp log sqrt rsqrt tanh sigmoid sin cos erf log1p floor ...
//   reduce  over the middle axis of an (outer, R, inner) view: sum, max, min, mean, and arg-max/min
//           inner == 1: one warp per row, 16-byte loads, two vectors in flight per lane
//           inner  > 1: a block per (outer, 32-column tile), its 8 warps split R; R is split over
//                       gridDim.y as well when there are few column tiles (second pass combines)
//   cumsum  along the middle axis of (outer, R, inner), with exclusive / reverse variants
// All kernels are bandwidth bound: one read of every input, one write of the output.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "nb_debug.cuh"

namespace nbe {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16(v); }
template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float* out) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
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

// ------------------------------------------------------------------ binary
enum BinOp { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_MAX, B_MIN, B_POW };

__device__ __forceinline__ float bin_apply(float a, float b, int op) {
  switch (op) {
    case B_ADD: return a + b;
    case B_SUB: return a - b;
    case B_MUL: return a * b;
    case B_DIV: return a / b;
    case B_MAX: return (a != a || b != b) ? NAN : fmaxf(a, b);     // propagate NaN like the framework's oracle
    case B_MIN: return (a != a || b != b) ? NAN : fminf(a, b);
    default: return powf(a, b);
  }
}

template <typename T>
__device__ __forceinline__ void unpack(const uint4& raw, float* out) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::N; ++i) out[i] = to_f<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack(const float* in) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::N; ++i) e[i] = from_f<T>(in[i]);
  return raw;
}

// bmode 0: b has n elements; 1: b is one element; 2: b has `inner` elements, index i % inner
// (inner a multiple of the vector width, so a vector never straddles two rows).
// A block owns 256 * 4 consecutive 16-byte vectors; every thread loads its four vectors (kept packed,
// 4 registers each) before it uses any, which is the memory-level parallelism a bandwidth-bound pass
// needs, and the op is selected once per vector, outside the element loop.
constexpr int EW_U = 4;

template <typename T, int BMODE>
__global__ void __launch_bounds__(256) binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                                    size_t n, int op, unsigned inner, int swap) {
  constexpr int V = Vec<T>::N;
  const size_t base = (size_t)blockIdx.x * (256 * V * EW_U) + (size_t)threadIdx.x * V;
  const float bs = BMODE == 1 ? to_f<T>(b[0]) : 0.f;
  uint4 ra[EW_U], rb[EW_U];
#pragma unroll
  for (int u = 0; u < EW_U; ++u) {
    const size_t i = base + (size_t)u * 256 * V;
    if (i + V <= n) {
      ra[u] = *reinterpret_cast<const uint4*>(a + i);
      if (BMODE == 0) rb[u] = *reinterpret_cast<const uint4*>(b + i);
      else if (BMODE == 2) rb[u] = *reinterpret_cast<const uint4*>(b + (i <= 0xffffffffull ? (size_t)((unsigned)i % inner) : i % inner));
    }
  }
#pragma unroll
  for (int u = 0; u < EW_U; ++u) {
    const size_t i = base + (size_t)u * 256 * V;
    if (i >= n) break;
    if (BMODE == 2 && !NB_IN_BOUNDS(NB_SITE_FLAT_INDEX, (i % inner) + V - 1, inner)) continue;   // debug build
    if (i + V <= n) {
      float x[V], y[V], o[V];
      unpack<T>(ra[u], x);
      if (BMODE == 1) {
#pragma unroll
        for (int j = 0; j < V; ++j) y[j] = bs;
      } else {
        unpack<T>(rb[u], y);
      }
      if (swap) {
#pragma unroll
        for (int j = 0; j < V; ++j) { const float t = x[j]; x[j] = y[j]; y[j] = t; }
      }
      switch (op) {
#define NB_CASE(OP) case OP: _Pragma("unroll") for (int j = 0; j < V; ++j) o[j] = bin_apply(x[j], y[j], OP); break;
        NB_CASE(B_ADD) NB_CASE(B_SUB) NB_CASE(B_MUL) NB_CASE(B_DIV) NB_CASE(B_MAX) NB_CASE(B_MIN)
        default: _Pragma("unroll") for (int j = 0; j < V; ++j) o[j] = bin_apply(x[j], y[j], B_POW); break;
#undef NB_CASE
      }
      *reinterpret_cast<uint4*>(out + i) = pack<T>(o);
    } else {
      for (int j = 0; j < V && i + j < n; ++j) {
        const float x = to_f<T>(a[i + j]);
        const float y = BMODE == 1 ? bs : to_f<T>(b[BMODE == 0 ? i + j : (i + j) % inner]);
        out[i + j] = from_f<T>(swap ? bin_apply(y, x, op) : bin_apply(x, y, op));
      }
    }
  }
}

// ------------------------------------------------------------------ unary
enum UnOp { U_NEG = 0, U_ABS, U_EXP, U_LOG, U_SQRT, U_RSQRT, U_TANH, U_SIGMOID, U_SIN, U_COS, U_ERF, U_LOG1P, U_FLOOR,
            U_TRUNC, U_ROUND, U_SQUARE, U_RECIP };

__device__ __forceinline__ float un_apply(float x, int op) {
  switch (op) {
    case U_NEG: return -x;
    case U_ABS: return fabsf(x);
    case U_EXP: return expf(x);
    case U_LOG: return logf(x);
    case U_SQRT: return sqrtf(x);
    case U_RSQRT: return rsqrtf(x);
    case U_TANH: return tanhf(x);
    case U_SIGMOID: return 1.f / (1.f + expf(-x));
    case U_SIN: return sinf(x);
    case U_COS: return cosf(x);
    case U_ERF: return erff(x);
    case U_LOG1P: return log1pf(x);
    case U_FLOOR: return floorf(x);
    case U_TRUNC: return truncf(x);
    case U_ROUND: return rintf(x);            // ties to even, as torch.round
    case U_SQUARE: return x * x;
    default: return 1.f / x;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) unary_kernel(const T* __restrict__ a, T* __restrict__ out, size_t n, int op) {
  constexpr int V = Vec<T>::N;
  const size_t base = (size_t)blockIdx.x * (256 * V * EW_U) + (size_t)threadIdx.x * V;
  uint4 ra[EW_U];
#pragma unroll
  for (int u = 0; u < EW_U; ++u) {
    const size_t i = base + (size_t)u * 256 * V;
    if (i + V <= n) ra[u] = *reinterpret_cast<const uint4*>(a + i);
  }
#pragma unroll
  for (int u = 0; u < EW_U; ++u) {
    const size_t i = base + (size_t)u * 256 * V;
    if (i >= n) break;
    if (i + V <= n) {
      float x[V], o[V];
      unpack<T>(ra[u], x);
      switch (op) {
#define NB_CASE(OP) case OP: _Pragma("unroll") for (int j = 0; j < V; ++j) o[j] = un_apply(x[j], OP); break;
        NB_CASE(U_NEG) NB_CASE(U_ABS) NB_CASE(U_EXP) NB_CASE(U_LOG) NB_CASE(U_SQRT) NB_CASE(U_RSQRT) NB_CASE(U_TANH)
        NB_CASE(U_SIGMOID) NB_CASE(U_SIN) NB_CASE(U_COS) NB_CASE(U_ERF) NB_CASE(U_LOG1P) NB_CASE(U_FLOOR) NB_CASE(U_TRUNC)
        NB_CASE(U_ROUND) NB_CASE(U_SQUARE)
        default: _Pragma("unroll") for (int j = 0; j < V; ++j) o[j] = un_apply(x[j], U_RECIP); break;
#undef NB_CASE
      }
      *reinterpret_cast<uint4*>(out + i) = pack<T>(o);
    } else {
      for (int j = 0; j < V && i + j < n; ++j) out[i + j] = from_f<T>(un_apply(to_f<T>(a[i + j]), op));
    }
  }
}

// ------------------------------------------------------------------ reductions
enum RedOp { R_SUM = 0, R_MAX, R_MIN, R_MEAN, R_ARGMAX, R_ARGMIN };

struct Acc {
  float v;
  long long idx;
};
__device__ __forceinline__ Acc red_init(int op) {
  return {op == R_MAX || op == R_ARGMAX ? -INFINITY : (op == R_MIN || op == R_ARGMIN ? INFINITY : 0.f), -1};
}
// NaN wins in max / min (as torch.amax / amin); arg ops keep the first extreme index.
__device__ __forceinline__ void red_step(Acc& a, float x, long long i, int op) {
  if (op == R_SUM || op == R_MEAN) { a.v += x; return; }
  const bool mx = op == R_MAX || op == R_ARGMAX;
  const bool a_nan = a.v != a.v, x_nan = x != x;
  bool take;
  if (a.idx < 0) take = true;
  else if (a_nan) take = false;
  else if (x_nan) take = true;
  else take = mx ? (x > a.v) : (x < a.v);
  if (!take && !a_nan && !x_nan && x == a.v && i < a.idx) take = true;      // first index on ties
  if (take) { a.v = x; a.idx = i; }
}
__device__ __forceinline__ void red_merge(Acc& a, const Acc& b, int op) {
  if (op == R_SUM || op == R_MEAN) { a.v += b.v; return; }
  if (b.idx >= 0) red_step(a, b.v, b.idx, op);
}
__device__ __forceinline__ Acc warp_red(Acc a, int op) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Acc b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.idx = __shfl_xor_sync(0xffffffffu, a.idx, o);
    red_merge(a, b, op);
  }
  return a;
}

// inner == 1: x viewed as (rows, R); one WARP per row (8 rows per block), 16-byte loads, two vectors
// in flight per lane; no shared memory, no block barrier.
template <typename T, typename O>
__global__ void __launch_bounds__(256) row_reduce_kernel(const T* __restrict__ x, O* __restrict__ out, long long rows,
                                                        long long R, int op) {
  constexpr int V = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  for (long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += (long long)gridDim.x * 8) {
    const T* xr = x + row * R;
    Acc a = red_init(op);
    const bool vec = (R % V == 0) && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0);
    if (vec) {
      long long c = (long long)lane * V;
      for (; c + 96 * V < R; c += 128 * V) {          // four vectors in flight per lane
        uint4 r0 = *reinterpret_cast<const uint4*>(xr + c), r1 = *reinterpret_cast<const uint4*>(xr + c + 32 * V);
        uint4 r2 = *reinterpret_cast<const uint4*>(xr + c + 64 * V), r3 = *reinterpret_cast<const uint4*>(xr + c + 96 * V);
        float f[V];
        unpack<T>(r0, f);
#pragma unroll
        for (int j = 0; j < V; ++j) red_step(a, f[j], c + j, op);
        unpack<T>(r1, f);
#pragma unroll
        for (int j = 0; j < V; ++j) red_step(a, f[j], c + 32 * V + j, op);
        unpack<T>(r2, f);
#pragma unroll
        for (int j = 0; j < V; ++j) red_step(a, f[j], c + 64 * V + j, op);
        unpack<T>(r3, f);
#pragma unroll
        for (int j = 0; j < V; ++j) red_step(a, f[j], c + 96 * V + j, op);
      }
      for (; c < R; c += 32 * V) {
        float f0[V];
        load_vec<T>(xr + c, f0);
#pragma unroll
        for (int j = 0; j < V; ++j) red_step(a, f0[j], c + j, op);
      }
    } else {
      for (long long c = lane; c < R; c += 32) red_step(a, to_f<T>(xr[c]), c, op);
    }
    a = warp_red(a, op);
    if (lane == 0) {
      if (op == R_ARGMAX || op == R_ARGMIN) out[row] = (O)a.idx;
      else out[row] = (O)from_f<T>(op == R_MEAN ? a.v / (float)R : a.v);
    }
  }
}

// inner > 1: x viewed as (outer, R, inner). A block owns one `outer` index and a tile of 32 columns;
// its 8 warps split the R rows (lane = column: 32 consecutive elements per load instruction, four
// rows in flight per thread) and meet in shared memory. gridDim.y splits R further when there are
// too few column tiles to fill the GPU; those partial results are combined by a second launch over
// the (outer, splits, inner) partials.
template <typename T, typename O>
__global__ void __launch_bounds__(256) col_reduce_kernel(const T* __restrict__ x, O* __restrict__ out, float* __restrict__ pv,
                                                        long long* __restrict__ pi, long long outer, long long R,
                                                        long long inner, int op, int splits) {
  __shared__ float sv[8][32];
  __shared__ long long si[8][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const long long tiles_i = (inner + 31) / 32;
  for (long long t = blockIdx.x; t < outer * tiles_i; t += gridDim.x) {
    const long long o = t / tiles_i, i = (t - o * tiles_i) * 32 + lane;
    const long long r0 = R * blockIdx.y / splits, r1 = R * (blockIdx.y + 1) / splits;
    Acc a = red_init(op);
    // debug build: the slice of rows and the last element this lane reads lie inside the tensor
    if (i < inner && NB_IN_BOUNDS(NB_SITE_REDUCE_INDEX, r1 - 1, R) &&
        NB_IN_BOUNDS(NB_SITE_REDUCE_INDEX, (o * R + (r1 - 1)) * inner + i, outer * R * inner)) {
      const T* p = x + o * R * inner + i;
      long long r = r0 + w;
      for (; r + 24 < r1; r += 32) {
        const float f0 = to_f<T>(p[r * inner]), f1 = to_f<T>(p[(r + 8) * inner]);
        const float f2 = to_f<T>(p[(r + 16) * inner]), f3 = to_f<T>(p[(r + 24) * inner]);
        red_step(a, f0, r, op); red_step(a, f1, r + 8, op); red_step(a, f2, r + 16, op); red_step(a, f3, r + 24, op);
      }
      for (; r < r1; r += 8) red_step(a, to_f<T>(p[r * inner]), r, op);
    }
    __syncthreads();
    sv[w][lane] = a.v; si[w][lane] = a.idx;
    __syncthreads();
    if (w == 0 && i < inner) {
      Acc tot = {sv[0][lane], si[0][lane]};
      for (int k = 1; k < 8; ++k) red_merge(tot, Acc{sv[k][lane], si[k][lane]}, op);
      if (splits > 1) {
        pv[(o * splits + blockIdx.y) * inner + i] = tot.v;
        pi[(o * splits + blockIdx.y) * inner + i] = tot.idx;
      } else if (op == R_ARGMAX || op == R_ARGMIN) {
        out[o * inner + i] = (O)tot.idx;
      } else {
        out[o * inner + i] = (O)from_f<T>(op == R_MEAN ? tot.v / (float)R : tot.v);
      }
    }
  }
}

template <typename T, typename O>
__global__ void __launch_bounds__(256) col_reduce_finish_kernel(const float* __restrict__ pv, const long long* __restrict__ pi,
                                                               O* __restrict__ out, long long outer, long long R,
                                                               long long inner, int op, int splits) {
  const long long total = outer * inner;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long o = t / inner, i = t - o * inner;
    Acc a = red_init(op);
    for (int k = 0; k < splits; ++k) red_merge(a, Acc{pv[(o * splits + k) * inner + i], pi[(o * splits + k) * inner + i]}, op);
    if (op == R_ARGMAX || op == R_ARGMIN) out[t] = (O)a.idx;
    else out[t] = (O)from_f<T>(op == R_MEAN ? a.v / (float)R : a.v);
  }
}

// cumulative sum along R of (outer, R, inner); one thread per (outer, inner) column (sequential in R)
template <typename T>
__global__ void __launch_bounds__(256) cumsum_kernel(const T* __restrict__ x, T* __restrict__ out, long long outer,
                                                    long long R, long long inner, int exclusive, int reverse) {
  const long long total = outer * inner;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long o = t / inner, i = t - o * inner;
    if (!NB_IN_BOUNDS(NB_SITE_REDUCE_INDEX, (o * R + (R - 1)) * inner + i, outer * R * inner)) continue;
    const T* p = x + o * R * inner + i;
    T* q = out + o * R * inner + i;
    float acc = 0.f;
    for (long long k = 0; k < R; ++k) {
      const long long r = reverse ? R - 1 - k : k;
      const float v = to_f<T>(p[r * inner]);
      if (exclusive) { q[r * inner] = from_f<T>(acc); acc += v; }
      else { acc += v; q[r * inner] = from_f<T>(acc); }
    }
  }
}

static inline int grid_for(size_t n, int per_block, int cap = 148 * 16) {
  size_t g = (n + per_block - 1) / per_block;
  if (g < 1) g = 1;
  return (int)(g > (size_t)cap ? cap : g);
}

}  // namespace nbe

using namespace nbe;
#define STREAM reinterpret_cast<cudaStream_t>(stream)
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : -1)

extern "C" {

// dtype: 0 fp32, 1 bf16. bmode / inner: see binary_kernel. swap = 1 computes b (op) a.
int nb_binary(const void* a, const void* b, void* out, long long n, int op, int bmode, long long inner, int swap,
              int dtype, void* stream) {
  if (n <= 0) return 0;
  const int V = dtype ? 8 : 4;
  if (bmode == 2 && (inner <= 0 || inner % V || inner > 0xffffffffll)) return -2;
  const size_t blocks = ((size_t)n + 256 * V * EW_U - 1) / (256 * V * EW_U);
  if (blocks > 0x7fffffffull) return -4;
  const unsigned grid = (unsigned)blocks;
#define NB_BIN(T, M) binary_kernel<T, M><<<grid, 256, 0, STREAM>>>((const T*)a, (const T*)b, (T*)out, (size_t)n, op, (unsigned)inner, swap)
  if (dtype) { if (bmode == 0) NB_BIN(bf16, 0); else if (bmode == 1) NB_BIN(bf16, 1); else NB_BIN(bf16, 2); }
  else { if (bmode == 0) NB_BIN(float, 0); else if (bmode == 1) NB_BIN(float, 1); else NB_BIN(float, 2); }
#undef NB_BIN
  return CHECK_LAUNCH();
}

int nb_unary(const void* a, void* out, long long n, int op, int dtype, void* stream) {
  if (n <= 0) return 0;
  const int V = dtype ? 8 : 4;
  const size_t blocks = ((size_t)n + 256 * V * EW_U - 1) / (256 * V * EW_U);
  if (blocks > 0x7fffffffull) return -4;
  const unsigned grid = (unsigned)blocks;
  if (dtype) unary_kernel<bf16><<<grid, 256, 0, STREAM>>>((const bf16*)a, (bf16*)out, (size_t)n, op);
  else unary_kernel<float><<<grid, 256, 0, STREAM>>>((const float*)a, (float*)out, (size_t)n, op);
  return CHECK_LAUNCH();
}

// x viewed as (outer, R, inner), reduced over R. Value ops write dtype of x; arg ops write int64.
// `scratch` (inner > 1 only): room for outer * splits * inner floats followed by as many int64, where
// splits = nb_reduce_splits(outer, R, inner); may be null when that is 1.
int nb_reduce_splits(long long outer, long long R, long long inner) {
  if (inner <= 1) return 1;
  const long long tiles = outer * ((inner + 31) / 32);
  long long s = (148 * 4 + tiles - 1) / tiles;
  if (s > R / 64) s = R / 64;
  if (s > 64) s = 64;
  return (int)(s < 1 ? 1 : s);
}

int nb_reduce(const void* x, void* out, void* scratch, long long outer, long long R, long long inner, int op, int dtype,
              void* stream) {
  if (outer <= 0 || inner <= 0 || R <= 0) return 0;
  const bool arg = op == R_ARGMAX || op == R_ARGMIN;
  if (inner == 1) {
    const long long want = (outer + 7) / 8;
    const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype) {
      if (arg) row_reduce_kernel<bf16, long long><<<grid, 256, 0, STREAM>>>((const bf16*)x, (long long*)out, outer, R, op);
      else row_reduce_kernel<bf16, bf16><<<grid, 256, 0, STREAM>>>((const bf16*)x, (bf16*)out, outer, R, op);
    } else {
      if (arg) row_reduce_kernel<float, long long><<<grid, 256, 0, STREAM>>>((const float*)x, (long long*)out, outer, R, op);
      else row_reduce_kernel<float, float><<<grid, 256, 0, STREAM>>>((const float*)x, (float*)out, outer, R, op);
    }
    return CHECK_LAUNCH();
  }
  const int splits = nb_reduce_splits(outer, R, inner);
  if (splits > 1 && scratch == nullptr) return -3;
  const long long tiles = outer * ((inner + 31) / 32);
  const dim3 grid((unsigned)(tiles < 148 * 16 ? tiles : 148 * 16), splits);
  float* pv = reinterpret_cast<float*>(scratch);
  long long* pi = reinterpret_cast<long long*>(pv + outer * splits * inner);
  const int fgrid = grid_for((size_t)(outer * inner), 256);
#define NB_COL(T, O) do { \
    col_reduce_kernel<T, O><<<grid, 256, 0, STREAM>>>((const T*)x, (O*)out, pv, pi, outer, R, inner, op, splits); \
    if (splits > 1) col_reduce_finish_kernel<T, O><<<fgrid, 256, 0, STREAM>>>(pv, pi, (O*)out, outer, R, inner, op, splits); \
  } while (0)
  if (dtype) { if (arg) NB_COL(bf16, long long); else NB_COL(bf16, bf16); }
  else { if (arg) NB_COL(float, long long); else NB_COL(float, float); }
#undef NB_COL
  return CHECK_LAUNCH();
}

int nb_cumsum(const void* x, void* out, long long outer, long long R, long long inner, int exclusive, int reverse, int dtype,
              void* stream) {
  if (outer <= 0 || inner <= 0 || R <= 0) return 0;
  const int grid = grid_for((size_t)(outer * inner), 256);
  if (dtype) cumsum_kernel<bf16><<<grid, 256, 0, STREAM>>>((const bf16*)x, (bf16*)out, outer, R, inner, exclusive, reverse);
  else cumsum_kernel<float><<<grid, 256, 0, STREAM>>>((const float*)x, (float*)out, outer, R, inner, exclusive, reverse);
  return CHECK_LAUNCH();
}

}  // extern "C"

NB_DEBUG_DEFINE(elementwise)
