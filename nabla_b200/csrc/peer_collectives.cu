// Collectives over NVLink 5 / NVSwitch peer memory for one-process-per-GPU groups.
//
// Every rank of a group owns a *symmetric workspace*: the same allocation size on every GPU,
// mapped into all peers (torch symmetric memory does the exchange of handles), optionally
// bound to an NVSwitch multicast object. Layout of a workspace:
//
//   [0, 8 KB)      barrier flags   u32 [MAX_BLOCKS][MAX_WORLD]   (monotonic epochs, never reset)
//   [16 KB, 48 KB) tile flags      u32 [8192]                    (fused GEMM + all-reduce)
//   [56 KB, 64 KB) done counters   u32
//   [64 KB, ...)   data
//
// Kernels here: cross-rank barrier, all-reduce (one-shot P2P loads, two-shot reduce-scatter +
// all-gather, NVLS multimem.ld_reduce + multimem.st), all-gather, reduce-scatter, all-to-all and
// broadcast as peer loads. They replace the MAX graph collectives the reference calls
// (nabla/ops/communication/all_reduce.py:94-108, all_gather.py:189-199,
// reduce_scatter.py:167-170, broadcast.py:56-80), and, unlike those, take the device group of
// a mesh axis, so reductions along 'tp' of a ('dp','tp') mesh stay inside each tp group.
//
// Every wait is bounded (0.5 s, WAIT_LIMIT_NS): on expiry the kernel writes NB_ERR_TIMEOUT_PEER to
// the status word and returns, so a lost peer surfaces as an error on the host instead of a hang.
// While the status word is set every kernel of this file returns at its first barrier without
// waiting, so the collectives queued behind a lost peer drain at once.
#include "sm100_ptx.cuh"
#include "nb_debug.cuh"

namespace nbc {
using namespace nb;

constexpr int MAX_WORLD = 8;
constexpr int MAX_BLOCKS = 256;
constexpr int FLAG_BYTES = 64 * 1024;
constexpr int TILE_FLAG_OFFSET = 16 * 1024;
constexpr int DONE_OFFSET = 56 * 1024;

struct Group {
  void* const* bufs;   // device array [world] of peer base pointers of the workspace
  void* mc;            // multicast base pointer of the workspace (nullptr: no NVLS)
  int rank, world;
  unsigned epoch;      // this call's number relative to *epoch_ctr (1 = the next one)
  const unsigned* epoch_ctr;   // device counter of the calls made so far on this workspace; a
                               // one-thread kernel after each collective advances it, so a launch
                               // sequence replayed from a CUDA graph keeps counting
  int* status;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_ge(const unsigned* p, unsigned target, int* status) {
  if ((int)(ld_acquire_sys(p) - target) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (true) {
    if ((int)(ld_acquire_sys(p) - target) >= 0) return true;
    if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
      atomicExch(status, NB_ERR_TIMEOUT_PEER);
      return false;
    }
  }
}

// All threads of the block call this. Block b of every rank meets block b of every other rank.
// `phase` distinguishes several barriers inside one kernel (epoch * 4 + phase is the value).
__device__ __forceinline__ bool block_barrier(const Group& g, int phase) {
  __syncthreads();
  bool ok = *reinterpret_cast<const volatile int*>(g.status) == 0;   // an earlier wait on this device gave up
  // debug build: the group fits the flag pad (blocks x world slots of 4 bytes)
  ok = ok && NB_IN_BOUNDS(NB_SITE_COMM_PEER_RANK, g.rank, g.world) &&
       NB_IN_BOUNDS(NB_SITE_COMM_PEER_RANK, g.world - 1, MAX_WORLD) &&
       NB_IN_BOUNDS(NB_SITE_COMM_FLAG, (blockIdx.x * MAX_WORLD + MAX_WORLD - 1) * 4, MAX_BLOCKS * MAX_WORLD * 4);
  if (!__syncthreads_and(ok)) return false;
  const unsigned val = (g.epoch + *reinterpret_cast<const volatile unsigned*>(g.epoch_ctr)) * 4u + (unsigned)phase;
  if (threadIdx.x < g.world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    unsigned* remote = reinterpret_cast<unsigned*>(g.bufs[peer]) + (blockIdx.x * MAX_WORLD + g.rank);
    st_release_sys(remote, val);
    const unsigned* mine = reinterpret_cast<const unsigned*>(g.bufs[g.rank]) + (blockIdx.x * MAX_WORLD + peer);
    ok = wait_ge(mine, val, g.status);
  }
  return __syncthreads_and(ok);
}

// ---------------------------------------------------------------- 16-byte vector helpers
struct alignas(16) V4 { unsigned x, y, z, w; };

template <typename T> struct Acc;
template <> struct Acc<float> {
  static constexpr int N = 4;
  __device__ static void unpack(const V4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static V4 pack(const float* f) {
    return {__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])};
  }
};
template <> struct Acc<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void unpack(const V4& v, float* f) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static V4 pack(const float* f) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<unsigned*>(&h);
    }
    return {w[0], w[1], w[2], w[3]};
  }
};

__device__ __forceinline__ float combine(float a, float b, int op) {
  return op == 0 ? a + b : op == 1 ? fmaxf(a, b) : op == 2 ? fminf(a, b) : a * b;
}

__device__ __forceinline__ V4 ld_peer(const void* p) {
  V4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_peer(void* p, const V4& v) {
  asm volatile("st.global.relaxed.sys.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T> __device__ __forceinline__ V4 mc_ld_reduce(const void* p);
template <> __device__ __forceinline__ V4 mc_ld_reduce<__nv_bfloat16>(const void* p) {
  V4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
template <> __device__ __forceinline__ V4 mc_ld_reduce<float>(const void* p) {
  V4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mc_st(void* p, const V4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---------------------------------------------------------------- all-reduce
// The caller has copied its contribution into the workspace data region (offset `off` bytes).
// algo 0: one-shot   every rank reads all peers and reduces everything          (small messages)
// algo 1: two-shot   rank r reduces chunk r in place, then everyone reads all chunks (large)
// algo 2: multimem   rank r: ld_reduce chunk r through the switch, multimem.st it back to all
// Result is written to `out` (ordinary memory, n elements).
// Thread mapping of the chunked algorithms: element j of a chunk is always handled by the thread
// with global index j mod nthreads, on every rank and in both phases. The per-block barrier pairs
// block b of all ranks, so the thread that reads an element in phase 2 is covered by the barrier
// its writer (same thread index on the owner rank) passed after phase 1, whatever the chunk size.
template <typename T>
__global__ void __launch_bounds__(512) allreduce_kernel(Group g, long long off, T* __restrict__ out, long long n,
                                                       int algo, int op) {
  constexpr int N = Acc<T>::N;
  constexpr int U = 4;                                // 16-byte vectors in flight per thread and peer
  const long long nvec = n / N;                       // n is padded to a multiple of N * world by the host
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  // debug build: 16-byte vectors at a 16-byte offset, whole vectors per rank
  if (!(NB_ALIGNED(NB_SITE_COMM_OFFSET, off, 16) && NB_IN_BOUNDS(NB_SITE_COMM_OFFSET, n % (N * g.world), 1))) return;
  if (!block_barrier(g, 0)) return;
  const char* mine = reinterpret_cast<const char*>(g.bufs[g.rank]) + FLAG_BYTES + off;
  if (algo == 0) {
    for (long long i0 = tid; i0 < nvec; i0 += nthreads * U) {
      float acc[U][N];
      V4 r[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        r[u] = i < nvec ? ld_peer(mine + i * 16) : V4{0u, 0u, 0u, 0u};
      }
#pragma unroll
      for (int u = 0; u < U; ++u) Acc<T>::unpack(r[u], acc[u]);
      for (int p = 1; p < g.world; ++p) {
        const char* src = reinterpret_cast<const char*>(g.bufs[(g.rank + p) % g.world]) + FLAG_BYTES + off;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * nthreads;
          r[u] = i < nvec ? ld_peer(src + i * 16) : V4{0u, 0u, 0u, 0u};
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float v[N];
          Acc<T>::unpack(r[u], v);
#pragma unroll
          for (int j = 0; j < N; ++j) acc[u][j] = combine(acc[u][j], v[j], op);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < nvec) reinterpret_cast<V4*>(out)[i] = Acc<T>::pack(acc[u]);
      }
    }
    block_barrier(g, 1);      // nobody may overwrite its buffer while peers still read it
    return;
  }
  const long long chunk = nvec / g.world;
  const long long c0 = chunk * g.rank;
  if (algo == 1) {
    // phase 1: reduce the own chunk in place
    for (long long i0 = tid; i0 < chunk; i0 += nthreads * U) {
      float acc[U][N];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < N; ++j) acc[u][j] = op == 0 ? 0.f : op == 1 ? -INFINITY : op == 2 ? INFINITY : 1.f;
      for (int p = 0; p < g.world; ++p) {
        const char* src = reinterpret_cast<const char*>(g.bufs[(g.rank + p) % g.world]) + FLAG_BYTES + off + c0 * 16;
        V4 r[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * nthreads;
          r[u] = i < chunk ? ld_peer(src + i * 16) : V4{0u, 0u, 0u, 0u};
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float v[N];
          Acc<T>::unpack(r[u], v);
#pragma unroll
          for (int j = 0; j < N; ++j) acc[u][j] = combine(acc[u][j], v[j], op);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < chunk) *reinterpret_cast<V4*>(const_cast<char*>(mine) + (c0 + i) * 16) = Acc<T>::pack(acc[u]);
      }
    }
  } else {
    // multimem (sum only): the switch adds the ranks' copies of the own chunk and stores the sum back to all
    char* mc = reinterpret_cast<char*>(g.mc) + FLAG_BYTES + off + c0 * 16;
    for (long long i0 = tid; i0 < chunk; i0 += nthreads * U) {
      V4 r[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < chunk) r[u] = mc_ld_reduce<T>(mc + i * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < chunk) mc_st(mc + i * 16, r[u]);
      }
    }
  }
  if (!block_barrier(g, 1)) return;
  // phase 2: collect every owner's reduced chunk with the SAME (thread <-> element of a chunk) mapping.
  // After the multimem store every rank holds all chunks in its own buffer; the two-shot variant
  // reads each chunk from its owner.
  for (int q = 0; q < g.world; ++q) {
    const int owner = (g.rank + q) % g.world;
    const char* src = (algo == 1 ? reinterpret_cast<const char*>(g.bufs[owner]) + FLAG_BYTES + off : mine) + owner * chunk * 16;
    V4* dst = reinterpret_cast<V4*>(out) + owner * chunk;
    for (long long i0 = tid; i0 < chunk; i0 += nthreads * U) {
      V4 r[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < chunk) r[u] = ld_peer(src + i * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < chunk) dst[i] = r[u];
      }
    }
  }
  block_barrier(g, 2);
}

// ---------------------------------------------------------------- gather-style collectives
// mode 0 all_gather    : out[p * chunk + i] = peer p's data[i]                  (chunk bytes each)
// mode 1 reduce_scatter: out[i] = sum_p peer p's data[rank * chunk + i]
// mode 2 all_to_all    : out[p * chunk + i] = peer p's data[rank * chunk + i]
// mode 3 broadcast     : out[i] = root's data[i]            (root in `op`)
template <typename T>
__global__ void __launch_bounds__(512) gather_kernel(Group g, long long off, T* __restrict__ out, long long chunk_elems,
                                                    int mode, int op) {
  constexpr int N = Acc<T>::N;
  const long long cvec = chunk_elems / N;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  if (!(NB_ALIGNED(NB_SITE_COMM_OFFSET, off, 16) && NB_IN_BOUNDS(NB_SITE_COMM_OFFSET, chunk_elems % N, 1))) return;
  if (!block_barrier(g, 0)) return;
  if (mode == 1) {
    for (long long i = tid; i < cvec; i += nthreads) {
      float acc[N];
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = 0.f;
      for (int p = 0; p < g.world; ++p) {
        const int peer = (g.rank + p) % g.world;
        float v[N];
        Acc<T>::unpack(ld_peer(reinterpret_cast<const char*>(g.bufs[peer]) + FLAG_BYTES + off + (g.rank * cvec + i) * 16), v);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] += v[j];
      }
      reinterpret_cast<V4*>(out)[i] = Acc<T>::pack(acc);
    }
  } else if (mode == 3) {
    for (long long i = tid; i < cvec; i += nthreads)
      reinterpret_cast<V4*>(out)[i] = ld_peer(reinterpret_cast<const char*>(g.bufs[op]) + FLAG_BYTES + off + i * 16);
  } else {
    for (int p = 0; p < g.world; ++p) {
      const int peer = (g.rank + p) % g.world;
      const char* src = reinterpret_cast<const char*>(g.bufs[peer]) + FLAG_BYTES + off + (mode == 2 ? g.rank * cvec * 16 : 0);
      for (long long i = tid; i < cvec; i += nthreads) reinterpret_cast<V4*>(out)[peer * cvec + i] = ld_peer(src + i * 16);
    }
  }
  block_barrier(g, 1);
}

__global__ void barrier_kernel(Group g) { block_barrier(g, 0); }

// ---------------------------------------------------------------- point-to-point shift (ppermute)
// Every rank of the group runs this kernel in the same call, on a workspace that only these calls
// use. Rank r stores `in` (nvec 16-byte vectors) into the inbox of rank `dst` (dst < 0: r sends
// nothing), all ranks meet, and r copies its own inbox to `out` (src < 0: nobody sends to r, `out` is
// zero-filled). The inbox has two slots used in turn (slot = call number & 1, `slot_bytes` apart):
// a sender that is one call ahead writes the other slot, and it cannot be two calls ahead, because
// leaving call n + 1 takes every rank's arrival at that call's barrier, which a rank reaches only
// after it has read its inbox of call n. So one barrier per call is enough. Block b of the sender
// writes the vectors that block b of the receiver reads (same grid and same thread <-> vector
// mapping on every rank), so the per-block barrier covers them. One launch replaces a grouped
// NCCL send / recv pair, which for the pipeline's 0.5 MB activations is all latency.
__global__ void __launch_bounds__(512) permute_kernel(Group g, long long slot_bytes, const V4* __restrict__ in,
                                                     V4* __restrict__ out, long long nvec, int dst, int src) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const unsigned call = g.epoch + *reinterpret_cast<const volatile unsigned*>(g.epoch_ctr);
  const long long off = (long long)(call & 1u) * slot_bytes;
  if (!(NB_ALIGNED(NB_SITE_COMM_OFFSET, slot_bytes, 16) && NB_IN_BOUNDS(NB_SITE_COMM_OFFSET, nvec * 16, slot_bytes + 1) &&
        NB_IN_BOUNDS(NB_SITE_COMM_PEER_RANK, dst + 1, g.world + 1) &&
        NB_IN_BOUNDS(NB_SITE_COMM_PEER_RANK, src + 1, g.world + 1)))
    return;
  if (*reinterpret_cast<const volatile int*>(g.status) != 0) return;   // an earlier wait on this device gave up
  if (dst >= 0) {
    char* remote = reinterpret_cast<char*>(g.bufs[dst]) + FLAG_BYTES + off;
    for (long long i = tid; i < nvec; i += nthreads) st_peer(remote + i * 16, in[i]);
  }
  if (!block_barrier(g, 0)) return;
  if (src >= 0) {
    const char* mine = reinterpret_cast<const char*>(g.bufs[g.rank]) + FLAG_BYTES + off;
    for (long long i = tid; i < nvec; i += nthreads) out[i] = ld_peer(mine + i * 16);
  } else {
    for (long long i = tid; i < nvec; i += nthreads) out[i] = V4{0u, 0u, 0u, 0u};
  }
}

// ---------------------------------------------------------------- gradient all-reduce + AdamW
// One kernel for the data-parallel update of one parameter: every rank's gradient (bf16) sits at
// the same offset of a symmetric arena; after a barrier (all gradients written) each rank sums them
// (multimem.ld_reduce through the switch, or one load per peer), scales, and applies AdamW to its
// own copy of p / m / v in place; a closing barrier keeps the gradients alive until every peer has
// read them. No reduced gradient is ever written to memory, and the replicas stay bit-identical
// because every rank adds the same values in the same order.
//   hyper = [lr, 1 - b1^t, 1 - b2^t, grad_scale] (device) overrides the scalar arguments.
__global__ void __launch_bounds__(256) adamw_reduce_kernel(Group g, void* const* grad_bufs, const char* grad_mc,
                                                          long long grad_off, __nv_bfloat16* p, float* m, float* v,
                                                          long long n, float lr, float b1, float b2, float eps, float wd,
                                                          float bc1, float bc2, float grad_scale, const float* hyper) {
  if (!block_barrier(g, 0)) return;
  if (hyper) { lr = hyper[0]; bc1 = hyper[1]; bc2 = hyper[2]; grad_scale = hyper[3]; }
  const float ibc1 = 1.f / bc1, ibc2 = 1.f / bc2;
  const long long nv = n / 8;                                  // 16-byte vectors of bf16 (n % 8 == 0)
  constexpr int U = 4;                                         // vectors per thread in flight per peer
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthr = (long long)gridDim.x * blockDim.x;
  for (long long i0 = tid; i0 < nv; i0 += nthr * U) {
    float gr[U][8];
    if (grad_mc != nullptr) {
      V4 r[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthr;
        if (i < nv)
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                       : "=r"(r[u].x), "=r"(r[u].y), "=r"(r[u].z), "=r"(r[u].w)
                       : "l"(grad_mc + grad_off + i * 16)
                       : "memory");
      }
#pragma unroll
      for (int u = 0; u < U; ++u) Acc<__nv_bfloat16>::unpack(r[u], gr[u]);
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) gr[u][j] = 0.f;
      for (int q = 0; q < g.world; ++q) {
        const char* src = reinterpret_cast<const char*>(grad_bufs[q]) + grad_off;
        V4 r[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * nthr;
          r[u] = V4{0u, 0u, 0u, 0u};
          if (i < nv)
            asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r[u].x), "=r"(r[u].y), "=r"(r[u].z), "=r"(r[u].w)
                         : "l"(src + i * 16)
                         : "memory");
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float f[8];
          Acc<__nv_bfloat16>::unpack(r[u], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) gr[u][j] += f[j];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * nthr;
      if (i >= nv) break;
      float pv[8], mv[8], vv[8];
      Acc<__nv_bfloat16>::unpack(reinterpret_cast<const V4*>(p)[i], pv);
      const float4 m0 = reinterpret_cast<const float4*>(m)[2 * i], m1 = reinterpret_cast<const float4*>(m)[2 * i + 1];
      const float4 v0 = reinterpret_cast<const float4*>(v)[2 * i], v1 = reinterpret_cast<const float4*>(v)[2 * i + 1];
      mv[0] = m0.x; mv[1] = m0.y; mv[2] = m0.z; mv[3] = m0.w; mv[4] = m1.x; mv[5] = m1.y; mv[6] = m1.z; mv[7] = m1.w;
      vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gj = gr[u][j] * grad_scale;
        mv[j] = b1 * mv[j] + (1.f - b1) * gj;
        vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
        pv[j] -= lr * ((mv[j] * ibc1) / (sqrtf(vv[j] * ibc2) + eps) + wd * pv[j]);
      }
      reinterpret_cast<V4*>(p)[i] = Acc<__nv_bfloat16>::pack(pv);
      reinterpret_cast<float4*>(m)[2 * i] = make_float4(mv[0], mv[1], mv[2], mv[3]);
      reinterpret_cast<float4*>(m)[2 * i + 1] = make_float4(mv[4], mv[5], mv[6], mv[7]);
      reinterpret_cast<float4*>(v)[2 * i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      reinterpret_cast<float4*>(v)[2 * i + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    }
  }
  block_barrier(g, 1);
}

// A wait on a flag that nobody sets: exercises the bounded-wait error path without any fault.
__global__ void wait_flag_kernel(const unsigned* flag, unsigned target, int* status, unsigned long long limit_ns) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const unsigned long long t0 = globaltimer_ns();
    while ((int)(ld_acquire_sys(flag) - target) < 0) {
      if (globaltimer_ns() - t0 > limit_ns) {
        atomicExch(status, NB_ERR_TIMEOUT_PEER);
        break;
      }
    }
  }
}

}  // namespace nbc

using namespace nbc;
#define STREAM reinterpret_cast<cudaStream_t>(stream)

static Group make_group(void* const* bufs, void* mc, int rank, int world, unsigned* epoch_ctr, int* status) {
  Group g;
  g.bufs = bufs; g.mc = mc; g.rank = rank; g.world = world; g.epoch = 1u; g.epoch_ctr = epoch_ctr; g.status = status;
  return g;
}

__global__ void bump_kernel(unsigned* ctr, unsigned inc) { *ctr += inc; }

extern "C" {

int nb_comm_flag_bytes() { return FLAG_BYTES; }
int nb_comm_tile_flag_offset() { return TILE_FLAG_OFFSET; }
int nb_comm_done_offset() { return DONE_OFFSET; }

// `epoch_ctr`: device counter owned by the workspace (zero at creation); advanced here after the kernel.
int nb_comm_barrier(void* const* bufs, int rank, int world, unsigned* epoch_ctr, int* status, void* stream) {
  barrier_kernel<<<1, 32, 0, STREAM>>>(make_group(bufs, nullptr, rank, world, epoch_ctr, status));
  bump_kernel<<<1, 1, 0, STREAM>>>(epoch_ctr, 1u);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// n must be a multiple of (16 / sizeof(T)) * world; dtype 0 fp32, 1 bf16; op 0 sum 1 max 2 min 3 prod.
int nb_comm_allreduce(void* const* bufs, void* mc, int rank, int world, unsigned* epoch_ctr, long long off, void* out,
                      long long n, int dtype, int algo, int op, int blocks, int* status, void* stream) {
  if (world > MAX_WORLD || blocks > MAX_BLOCKS) return -2;
  if (algo == 2 && (mc == nullptr || op != 0)) return -3;
  Group g = make_group(bufs, mc, rank, world, epoch_ctr, status);
  if (dtype) allreduce_kernel<__nv_bfloat16><<<blocks, 512, 0, STREAM>>>(g, off, (__nv_bfloat16*)out, n, algo, op);
  else allreduce_kernel<float><<<blocks, 512, 0, STREAM>>>(g, off, (float*)out, n, algo, op);
  bump_kernel<<<1, 1, 0, STREAM>>>(epoch_ctr, 1u);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int nb_comm_gather(void* const* bufs, int rank, int world, unsigned* epoch_ctr, long long off, void* out, long long chunk_elems,
                   int dtype, int mode, int op, int blocks, int* status, void* stream) {
  if (world > MAX_WORLD || blocks > MAX_BLOCKS) return -2;
  Group g = make_group(bufs, nullptr, rank, world, epoch_ctr, status);
  if (dtype) gather_kernel<__nv_bfloat16><<<blocks, 512, 0, STREAM>>>(g, off, (__nv_bfloat16*)out, chunk_elems, mode, op);
  else gather_kernel<float><<<blocks, 512, 0, STREAM>>>(g, off, (float*)out, chunk_elems, mode, op);
  bump_kernel<<<1, 1, 0, STREAM>>>(epoch_ctr, 1u);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Fused data-parallel gradient all-reduce + AdamW step (see adamw_reduce_kernel). `grad_bufs`:
// device array [world] of the arena base pointers, `grad_mc`: the arena's multicast base or null,
// `grad_off`: byte offset of this parameter's bf16 gradient in the arena; n must be a multiple of 8;
// p bf16, m / v fp32, all 16-byte aligned, updated in place.
int nb_comm_adamw_reduce(void* const* bufs, int rank, int world, unsigned* epoch_ctr, void* const* grad_bufs,
                         void* grad_mc, long long grad_off, void* p, float* m, float* v, long long n, float lr,
                         float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
                         const float* hyper, int blocks, int* status, void* stream) {
  if (world > MAX_WORLD || blocks > MAX_BLOCKS || blocks < 1) return -2;
  if ((n & 7) || (grad_off & 15)) return -12;
  Group g = make_group(bufs, nullptr, rank, world, epoch_ctr, status);
  adamw_reduce_kernel<<<blocks, 256, 0, STREAM>>>(g, grad_bufs, reinterpret_cast<const char*>(grad_mc), grad_off,
                                                  reinterpret_cast<__nv_bfloat16*>(p), m, v, n, lr, b1, b2, eps, wd, bc1,
                                                  bc2, grad_scale, hyper);
  bump_kernel<<<1, 1, 0, STREAM>>>(epoch_ctr, 1u);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Shift of `nbytes` (a multiple of 16, at most `slot_bytes`) from `in` to rank `dst`'s `out`; see
// permute_kernel. `dst` / `src` are ranks of the group or -1. The workspace behind `bufs` holds the
// flag pad followed by two inbox slots of `slot_bytes` each and serves no other collective.
int nb_comm_permute(void* const* bufs, int rank, int world, unsigned* epoch_ctr, long long slot_bytes, const void* in,
                    void* out, long long nbytes, int dst, int src, int blocks, int* status, void* stream) {
  if (world > MAX_WORLD || blocks > MAX_BLOCKS || blocks < 1) return -2;
  if ((nbytes & 15) || (slot_bytes & 15) || nbytes > slot_bytes || dst >= world || src >= world) return -12;
  if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -11;
  Group g = make_group(bufs, nullptr, rank, world, epoch_ctr, status);
  permute_kernel<<<blocks, 512, 0, STREAM>>>(g, slot_bytes, reinterpret_cast<const V4*>(in), reinterpret_cast<V4*>(out),
                                             nbytes / 16, dst, src);
  bump_kernel<<<1, 1, 0, STREAM>>>(epoch_ctr, 1u);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int nb_comm_wait_flag(const unsigned* flag, unsigned target, int* status, unsigned long long limit_ns, void* stream) {
  wait_flag_kernel<<<1, 32, 0, STREAM>>>(flag, target, status, limit_ns);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"

NB_DEBUG_DEFINE(comm)
