// Column sum that brings its own scratch memory (see no_alloc_entry.h for who needs this and
// for the rules that come with a shared, fixed scratch array).
//
// Two kernels, the same split as the regular column sum: slabs of rows are summed per block into
// scratch[part][N], then one thread per column folds the parts. The scratch is a file-scope
// device array; its name is only a handle on the host side, so the device address is looked up
// once per device with cudaGetSymbolAddress and passed to the kernels as an ordinary pointer.
#include "no_alloc_entry.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace {

typedef __nv_bfloat16 bf16;

static __device__ __align__(256) float g_noalloc_scratch[NB_NOALLOC_MAX_PARTS * NB_NOALLOC_MAX_COLS];

constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {nullptr};
std::mutex g_setup_mutex;

template <typename T> struct VecOf { static constexpr int N = 16 / sizeof(T); };

__device__ __forceinline__ float as_float(float v) { return v; }
__device__ __forceinline__ float as_float(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void put(float* p, float v) { *p = v; }
__device__ __forceinline__ void put(bf16* p, float v) { *p = __float2bfloat16(v); }

// grid = (ceil(N / (32 * V)), parts); block = 256 threads = 8 warps. Warp w of a block walks rows
// r0 + w, r0 + w + 8, ... of its slab; lane l owns the 16-byte vector of columns (bx*32 + l) * V.
template <typename T>
__global__ void __launch_bounds__(256)
noalloc_colsum_slabs(const T* __restrict__ x, float* __restrict__ scratch, int rows, int N, int rows_per_part) {
  constexpr int V = VecOf<T>::N;
  __shared__ float sh[8][32 * V];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * V;
  const int r0 = blockIdx.y * rows_per_part;
  const int r1 = min(rows, r0 + rows_per_part);
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.f;
  if (c < N) {
    for (int r = r0 + warp; r < r1; r += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)r * N + c);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += as_float(e[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) sh[warp][lane * V + j] = acc[j];
  __syncthreads();
  // every column below N of this part's row is written, also by parts whose slab is empty:
  // the folding kernel therefore never reads what an earlier call left behind
  for (int i = threadIdx.x; i < 32 * V; i += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += sh[w][i];
    const int col = blockIdx.x * 32 * V + i;
    if (col < N) scratch[(size_t)blockIdx.y * N + col] = s;
  }
}

template <typename T>
__global__ void noalloc_colsum_fold(const float* __restrict__ scratch, T* __restrict__ out, int parts, int N) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float s = 0.f;
  for (int i = 0; i < parts; ++i) s += scratch[(size_t)i * N + c];
  put(out + c, s);
}

// Device address of the scratch array on the current device; looked up on first use.
float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();   // leave no sticky-looking error behind for the caller's next check
      return nullptr;
    }
    g_scratch_addr[dev] = static_cast<float*>(p);
  }
  return g_scratch_addr[dev];
}

int parts_for(int rows) {
  long long np = ((long long)rows + 511) / 512;      // 64-bit: rows close to INT_MAX must not wrap
  if (np > NB_NOALLOC_MAX_PARTS) np = NB_NOALLOC_MAX_PARTS;
  return np < 1 ? 1 : (int)np;
}

}  // namespace

extern "C" int nb_colsum_noalloc(const void* x, void* out, int rows, int N, int in_dtype, int out_dtype,
                                 void* stream) {
  const int V = in_dtype ? 8 : 4;
  if (N > NB_NOALLOC_MAX_COLS) return NB_NOALLOC_ERR_TOO_WIDE;
  if (rows < 0 || N <= 0 || (N % V) != 0 || (in_dtype != 0 && in_dtype != 1) || (out_dtype != 0 && out_dtype != 1))
    return NB_NOALLOC_ERR_BAD_SHAPE;
  if (out == nullptr || (rows > 0 && x == nullptr) || (reinterpret_cast<uintptr_t>(x) & 15))
    return NB_NOALLOC_ERR_BAD_POINTER;
  float* scratch = scratch_for_current_device();
  if (scratch == nullptr) return NB_NOALLOC_ERR_SETUP;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int parts = parts_for(rows);
  const int rows_per_part = (int)(((long long)rows + parts - 1) / parts);
  const dim3 grid((N + 32 * V - 1) / (32 * V), parts);
  // cudaPeekAtLastError after each launch: it reports a failed launch of ours without clearing (and
  // thereby swallowing) an error that the caller's earlier work may have left behind
  if (in_dtype) noalloc_colsum_slabs<bf16><<<grid, 256, 0, s>>>(static_cast<const bf16*>(x), scratch, rows, N, rows_per_part);
  else noalloc_colsum_slabs<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), scratch, rows, N, rows_per_part);
  if (cudaPeekAtLastError() != cudaSuccess) return NB_NOALLOC_ERR_LAUNCH;
  if (out_dtype) noalloc_colsum_fold<bf16><<<(N + 255) / 256, 256, 0, s>>>(scratch, static_cast<bf16*>(out), parts, N);
  else noalloc_colsum_fold<float><<<(N + 255) / 256, 256, 0, s>>>(scratch, static_cast<float*>(out), parts, N);
  return cudaPeekAtLastError() == cudaSuccess ? NB_NOALLOC_OK : NB_NOALLOC_ERR_LAUNCH;
}

extern "C" void nb_noalloc_forget_devices(void) {
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  for (int i = 0; i < MAX_DEVICES; ++i) g_scratch_addr[i] = nullptr;
}

extern "C" const char* nb_noalloc_strerror(int code) {
  switch (code) {
    case NB_NOALLOC_OK: return "ok";
    case NB_NOALLOC_ERR_TOO_WIDE: return "N exceeds NB_NOALLOC_MAX_COLS (8192): the built-in scratch array is too small";
    case NB_NOALLOC_ERR_BAD_SHAPE: return "rows < 0, N <= 0, N not a multiple of 16 bytes of elements, or unknown dtype";
    case NB_NOALLOC_ERR_BAD_POINTER: return "null pointer, or input not aligned to 16 bytes";
    case NB_NOALLOC_ERR_SETUP: return "could not obtain the device address of the built-in scratch array";
    case NB_NOALLOC_ERR_LAUNCH: return "kernel launch failed";
    default: return "unknown code";
  }
}
