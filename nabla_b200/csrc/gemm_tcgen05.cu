// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   D[b] = epilogue( A[b] (M x K)  *  B[b] (K x N) )        fp32 accumulation in TMEM
//
// Structure (one persistent CTA per SM, 256 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of A/B tiles into a shared-memory ring
//   warp 1      MMA issuer:   one thread issues tcgen05.mma (128 x BN x 16) from smem descriptors
//   warp 2      TMEM allocator (2 accumulator buffers of BN columns each)
//   warps 4..7  epilogue: tcgen05.ld the accumulator, bias / relu / gelu / d-activation /
//               residual add, cast and store; overlaps the next tile's MMAs (double-buffered TMEM)
//
// Both operands may be K-major (row = M or N index, K contiguous) or MN-major (row = K index,
// M or N contiguous), so x@W, dY@W^T and X^T@dY all run without materialising a transpose.
// No TMA multicast is used anywhere: every CTA loads its own tiles.
//
// Replaces what the reference obtains from MAX's matmul (nabla/ops/binary.py:197-198) and the
// matmul + add + relu/gelu composition of nabla/nn/functional/layers.py:30-35.
#include "sm100_ptx.cuh"
#include <stdio.h>

namespace nb {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 256;
constexpr int EPI_THREADS = 128;

enum Epi : int { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_RELU = 2, EPI_BIAS_GELU = 3 };
enum Aux : int { AUX_NONE = 0, AUX_STORE_PREACT = 1, AUX_MUL_DRELU = 2, AUX_MUL_DGELU = 3, AUX_ADD = 4 };

struct GemmArgs {
  int M, N, K, batch;
  void* out;                // bf16 or fp32
  const void* bias;         // [N] bf16 or fp32, may be null
  const __nv_bfloat16* aux_in;
  __nv_bfloat16* aux_out;
  long long ldc, stride_c;  // elements
  long long ld_aux, stride_aux;
  int a_mn, b_mn;           // 1 = MN-major operand
  int out_fp32, bias_fp32;
  int epi, aux, accumulate, gelu_tanh;
  int vec_ok;               // output/aux rows are 16-byte aligned
  float alpha;              // scale applied to the accumulator before the epilogue
  int* status;              // device status word (0 = ok)
};

template <int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = BN * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BIAS_BYTES = BN * 4;
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int TOTAL = RING_BYTES + BIAS_BYTES + BAR_BYTES + 1024;  // + alignment slack
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& b, int& m, int& n) {
  const int per_batch = num_m * num_n;
  b = t / per_batch;
  int r = t - b * per_batch;
  constexpr int GROUP_M = 8;
  const int group = GROUP_M * num_n;
  const int gid = r / group;
  const int first_m = gid * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int rr = r - gid * group;
  m = first_m + rr % gsz;
  n = rr / gsz;
}

// Fused GEMM + all-reduce: where the tiles go and how ranks tell each other about them.
struct CommArgs {
  void* const* bufs;        // device array [world]: peer base pointers of the symmetric workspace
  char* mc;                 // multicast base of the workspace (nullptr: plain peer loads/stores)
  long long data_off;       // byte offset of the C matrix inside the workspace
  int flag_off, done_off;   // byte offsets of the tile flags / done counter inside the workspace
  int rank, world;
  unsigned tile_target;     // value a tile flag reaches when every rank has written the tile
  unsigned done_target;     // value the done counter reaches when every CTA of every rank is through
  int* ticket;              // device int, zeroed before the launch: next reduce job of this rank
};

// One CTA's share of the GEMM. `cta` / `nctas` replace blockIdx / gridDim so that the fused
// kernel can dedicate some CTAs to communication. Returns false if the CTA left early.
template <int BN, bool FUSED>
__device__ __forceinline__ bool gemm_cta(const CUtensorMap* tmAp, const CUtensorMap* tmBp, const GemmArgs& args,
                                         const CommArgs& comm, const int cta, const int nctas) {
  const CUtensorMap& tmA = *tmAp;
  const CUtensorMap& tmB = *tmBp;
  using L = SmemLayout<BN>;
  constexpr int STAGES = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  float* sbias = reinterpret_cast<float*>(smem + L::RING_BYTES);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::RING_BYTES + L::BIAS_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // a previous bounded wait failed on this device: do not pile more waits on top of it
  {
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = *reinterpret_cast<volatile int*>(args.status);
    __syncthreads();
    if (s_abort != 0) return false;   // uniform for the whole CTA
  }

  const int num_m = (args.M + BLOCK_M - 1) / BLOCK_M;
  const int num_n = (args.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n * args.batch;
  const int num_kb = (args.K + BLOCK_K - 1) / BLOCK_K;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    mbar_init(&tmem_empty[0], EPI_THREADS);
    mbar_init(&tmem_empty[1], EPI_THREADS);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += nctas) {
        int b, tm, tn;
        tile_coords(t, num_m, num_n, b, tm, tn);
        const int m0 = tm * BLOCK_M, n0 = tn * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            ok = false;
            atomicExch(args.status, NB_ERR_TIMEOUT_PRODUCER);
            break;
          }
          uint8_t* sA = ring + stage * L::STAGE_BYTES;
          uint8_t* sB = sA + L::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          const int k0 = kb * BLOCK_K;
          if (!args.a_mn) {
            tma_load_3d(sA, &tmA, &full_bar[stage], k0, m0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_M / 64; ++j)
              tma_load_3d(sA + j * (BLOCK_K * 128), &tmA, &full_bar[stage], m0 + j * 64, k0, b);
          }
          if (!args.b_mn) {
            tma_load_3d(sB, &tmB, &full_bar[stage], k0, n0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sB + j * (BLOCK_K * 128), &tmB, &full_bar[stage], n0 + j * 64, k0, b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BLOCK_M, BN, args.a_mn, args.b_mn);
      // Per-operand descriptor constants.
      const uint32_t a_lbo = args.a_mn ? BLOCK_K * 128 : 16, a_sbo = 1024;
      const uint32_t b_lbo = args.b_mn ? BLOCK_K * 128 : 16, b_sbo = 1024;
      // Descriptor start-address step per UMMA_K (in 16-byte units).
      const uint32_t a_kstep = args.a_mn ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
      const uint32_t b_kstep = args.b_mn ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = cta; t < num_tiles && ok; t += nctas, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1)) {
          atomicExch(args.status, NB_ERR_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            atomicExch(args.status, NB_ERR_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(ring + stage * L::STAGE_BYTES);
          const uint32_t sB = sA + L::A_BYTES;
          const uint64_t da = make_smem_desc_sw128(sA, a_lbo, a_sbo);
          const uint64_t db = make_smem_desc_sw128(sB, b_lbo, b_sbo);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            umma_f16_ss(tmem_d, da + static_cast<uint64_t>(k * a_kstep), db + static_cast<uint64_t>(k * b_kstep),
                        idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);   // frees the smem slot when these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[buf]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue
    const int wq = warp & 3;                 // TMEM lane quarter this warp may read
    const int et = threadIdx.x - 128;        // 0..127
    bool ok = true;
    int it = 0;
    for (int t = cta; t < num_tiles; t += nctas, ++it) {
      int b, tm, tn;
      tile_coords(t, num_m, num_n, b, tm, tn);
      const int m0 = tm * BLOCK_M, n0 = tn * BN;
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      // stage the bias slice of this tile
      named_bar_sync(1, EPI_THREADS);
      for (int j = et; j < BN; j += EPI_THREADS) {
        float bv = 0.f;
        if (args.bias != nullptr && args.epi != EPI_NONE && n0 + j < args.N) {
          bv = args.bias_fp32 ? reinterpret_cast<const float*>(args.bias)[n0 + j]
                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(args.bias)[n0 + j]);
        }
        sbias[j] = bv;
      }
      named_bar_sync(1, EPI_THREADS);
      if (ok && !mbar_wait(&tmem_full[buf], acc_phase)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) continue;   // keep barrier participation uniform, skip the work
      tc_fence_after();
      const int row = m0 + wq * 32 + lane;
      const bool row_ok = row < args.M;
      const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(wq * 32) << 16);
      const long long out_off = static_cast<long long>(b) * args.stride_c + static_cast<long long>(row) * args.ldc;
      const long long aux_off =
          static_cast<long long>(b) * args.stride_aux + static_cast<long long>(row) * args.ld_aux;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int nb0 = n0 + c * 32;
        if (nb0 >= args.N) break;   // warp-uniform
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * args.alpha + sbias[c * 32 + j];
        const bool full = (nb0 + 32 <= args.N) && args.vec_ok;
        // ---- auxiliary output: pre-activation
        if (args.aux == AUX_STORE_PREACT && row_ok) {
          __nv_bfloat16* ap = args.aux_out + aux_off + nb0;
          if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 pk;
              uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(f[q * 8 + 2 * j], f[q * 8 + 2 * j + 1]);
                pw[j] = *reinterpret_cast<uint32_t*>(&h);
              }
              reinterpret_cast<uint4*>(ap)[q] = pk;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (nb0 + j < args.N) ap[j] = __float2bfloat16(f[j]);
          }
        }
        // ---- activation
        if (args.epi == EPI_BIAS_RELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = fmaxf(f[j], 0.f);
        } else if (args.epi == EPI_BIAS_GELU) {
          if (args.gelu_tanh) {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = gelu_tanh(f[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = gelu_erf(f[j]);
          }
        }
        // ---- auxiliary input: d-activation multiply or residual add
        if (args.aux >= AUX_MUL_DRELU && row_ok) {
          const __nv_bfloat16* ap = args.aux_in + aux_off + nb0;
          float a[32];
          if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 pk = reinterpret_cast<const uint4*>(ap)[q];
              const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 x = __bfloat1622float2(ph[j]);
                a[q * 8 + 2 * j] = x.x;
                a[q * 8 + 2 * j + 1] = x.y;
              }
            }
          } else {
            for (int j = 0; j < 32; ++j) a[j] = (nb0 + j < args.N) ? __bfloat162float(ap[j]) : 0.f;
          }
          if (args.aux == AUX_MUL_DRELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = a[j] > 0.f ? f[j] : 0.f;
          } else if (args.aux == AUX_MUL_DGELU) {
            if (args.gelu_tanh) {
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] *= dgelu_tanh(a[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] *= dgelu_erf(a[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] += a[j];
          }
        }
        // ---- store
        if (row_ok) {
          if (args.out_fp32) {
            float* op = reinterpret_cast<float*>(args.out) + out_off + nb0;
            if (full) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                float4 o = make_float4(f[q * 4], f[q * 4 + 1], f[q * 4 + 2], f[q * 4 + 3]);
                if (args.accumulate) {
                  float4 old = reinterpret_cast<float4*>(op)[q];
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                reinterpret_cast<float4*>(op)[q] = o;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (nb0 + j < args.N) op[j] = args.accumulate ? op[j] + f[j] : f[j];
            }
          } else {
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(args.out) + out_off + nb0;
            if (full) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 pk;
                uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
                if (args.accumulate) {
                  uint4 old = reinterpret_cast<uint4*>(op)[q];
                  const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    float2 x = __bfloat1622float2(ph[j]);
                    f[q * 8 + 2 * j] += x.x;
                    f[q * 8 + 2 * j + 1] += x.y;
                  }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(f[q * 8 + 2 * j], f[q * 8 + 2 * j + 1]);
                  pw[j] = *reinterpret_cast<uint32_t*>(&h);
                }
                reinterpret_cast<uint4*>(op)[q] = pk;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (nb0 + j < args.N)
                  op[j] = __float2bfloat16(args.accumulate ? __bfloat162float(op[j]) + f[j] : f[j]);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[buf]);
      if (FUSED) {
        // the tile is in this rank's workspace: make it visible system-wide, then count it on
        // the rank that reduces this tile (tile t belongs to rank t % world)
        __threadfence_system();
        named_bar_sync(2, EPI_THREADS);
        if (et == 0)
          asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(reinterpret_cast<char*>(comm.bufs[t % comm.world]) +
                                                                         comm.flag_off + 4ll * t),
                       "r"(1u)
                       : "memory");
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
  return true;
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmArgs args) {
  CommArgs none{};
  gemm_cta<BN, false>(&tmA, &tmB, args, none, blockIdx.x, gridDim.x);
}

// ------------------------------------------------------------------ fused GEMM + all-reduce
// CTAs [0, n_gemm) compute tiles of this rank's partial product into the symmetric workspace and
// raise per-tile flags on all ranks. Every CTA (the dedicated communication CTAs from the start,
// the GEMM CTAs once they run out of tiles) then takes reduce jobs from a ticket counter: job k of
// rank r is tile r + k * world. A job waits until all ranks have written the tile, sums the
// copies (multimem.ld_reduce in the switch, or peer loads) and writes the sum into every rank's
// workspace (multimem.st, or peer stores). The kernel leaves once every CTA of every rank is
// through, so the next kernel on the stream finds the reduced matrix in the local workspace.
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_flag_ge(const unsigned* p, unsigned target) {
  if ((int)(ld_acquire_sys_u32(p) - target) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (true) {
    if ((int)(ld_acquire_sys_u32(p) - target) >= 0) return true;
    if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
}

template <int BN>
__device__ __forceinline__ void reduce_jobs(const GemmArgs& args, const CommArgs& comm) {
  __shared__ int s_job;
  __shared__ int s_ok;
  const int num_m = (args.M + BLOCK_M - 1) / BLOCK_M;
  const int num_n = (args.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n * args.batch;
  char* local = reinterpret_cast<char*>(comm.bufs[comm.rank]);
  const unsigned* flags = reinterpret_cast<const unsigned*>(local + comm.flag_off);
  while (true) {
    __syncthreads();
    if (threadIdx.x == 0) {
      const int k = atomicAdd(comm.ticket, 1);
      const int t = comm.rank + k * comm.world;
      s_job = t;
      s_ok = 1;
      if (t < num_tiles) {
        if (!wait_flag_ge(flags + t, comm.tile_target)) {
          atomicExch(args.status, NB_ERR_TIMEOUT_PEER);
          s_ok = 0;
        } else {
          // every rank has counted: nobody touches this flag again before the closing
          // barrier, so it can go back to zero for the next call
          *const_cast<volatile unsigned*>(flags + t) = 0u;
        }
      }
    }
    __syncthreads();
    const int t = s_job;
    if (t >= num_tiles || !s_ok) break;
    int b, tm, tn;
    tile_coords(t, num_m, num_n, b, tm, tn);
    const int m0 = tm * BLOCK_M, n0 = tn * BN;
    const int rows = min(BLOCK_M, args.M - m0);
    const int vpr = (min(BN, args.N - n0) * 2) / 16;       // 16-byte vectors per tile row (N % 8 == 0)
    const long long base = comm.data_off + ((long long)b * args.stride_c + (long long)m0 * args.ldc + n0) * 2;
    const int total = rows * vpr;
    if (comm.mc != nullptr) {
      for (int i = threadIdx.x; i < total; i += 4 * NUM_THREADS) {
        uint4 v[4];
        long long off[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = i + u * NUM_THREADS;
          off[u] = base + ((long long)(idx / vpr) * args.ldc) * 2 + (idx % vpr) * 16;
          if (idx < total)
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                         : "l"(comm.mc + off[u])
                         : "memory");
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i + u * NUM_THREADS < total)
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(comm.mc + off[u]), "r"(v[u].x),
                         "r"(v[u].y), "r"(v[u].z), "r"(v[u].w)
                         : "memory");
      }
    } else {
      for (int idx = threadIdx.x; idx < total; idx += NUM_THREADS) {
        const long long off = base + ((long long)(idx / vpr) * args.ldc) * 2 + (idx % vpr) * 16;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int p = 0; p < comm.world; ++p) {
          uint4 v;
          asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                       : "l"(reinterpret_cast<char*>(comm.bufs[p]) + off)
                       : "memory");
          const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] += __uint_as_float(w[j] << 16);
            acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
          }
        }
        uint4 o;
        unsigned* ow = reinterpret_cast<unsigned*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
          ow[j] = *reinterpret_cast<unsigned*>(&h);
        }
        for (int p = 0; p < comm.world; ++p)
          *reinterpret_cast<uint4*>(reinterpret_cast<char*>(comm.bufs[p]) + off) = o;
      }
    }
  }
  // this CTA is through: tell every rank, and let the last CTA wait for everybody
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (comm.mc != nullptr) {
      asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(comm.mc + comm.done_off), "r"(1u) : "memory");
    } else {
      for (int p = 0; p < comm.world; ++p)
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(reinterpret_cast<char*>(comm.bufs[p]) + comm.done_off),
                     "r"(1u)
                     : "memory");
    }
    if (blockIdx.x == gridDim.x - 1) {
      if (!wait_flag_ge(reinterpret_cast<const unsigned*>(local + comm.done_off), comm.done_target))
        atomicExch(args.status, NB_ERR_TIMEOUT_PEER);
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_allreduce_fused_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                            const GemmArgs args, const CommArgs comm, const int n_gemm) {
  if ((int)blockIdx.x < n_gemm) {
    if (!gemm_cta<BN, true>(&tmA, &tmB, args, comm, blockIdx.x, n_gemm)) return;
  } else {
    __shared__ int s_abort2;
    if (threadIdx.x == 0) s_abort2 = *reinterpret_cast<volatile int*>(args.status);
    __syncthreads();
    if (s_abort2 != 0) return;
  }
  reduce_jobs<BN>(args, comm);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map over a bf16 operand seen as [batch][rows][cols] with cols contiguous.
// Box = 64 cols (128 B, SWIZZLE_128B) x box_rows x 1.
static int make_map(CUtensorMap* map, const void* ptr, long long cols, long long rows, long long batch,
                    long long ld, long long stride_b, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  if (batch == 1 || stride_b == 0) stride_b = rows * ld;
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)stride_b * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

static int g_num_sms = 0;

template <int BN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, int max_ctas,
                  cudaStream_t stream) {
  using L = SmemLayout<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         L::TOTAL);
    if (e != cudaSuccess) return -2;
    configured = true;
  }
  const int num_m = (a.M + BLOCK_M - 1) / BLOCK_M, num_n = (a.N + BN - 1) / BN;
  long long tiles = (long long)num_m * num_n * a.batch;
  int grid = (int)(tiles < max_ctas ? tiles : max_ctas);
  if (grid < 1) return 0;
  gemm_bf16_tcgen05_kernel<BN><<<grid, NUM_THREADS, L::TOTAL, stream>>>(ta, tb, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace nb

// C entry point. All leading dimensions / strides are in elements.
//   A: a_mn == 0 -> [batch][M][K] (K contiguous, row stride lda); a_mn == 1 -> [batch][K][M]
//   B: b_mn == 0 -> [batch][N][K] (K contiguous, row stride ldb); b_mn == 1 -> [batch][K][N]
// Requirements: base pointers 16-byte aligned, lda/ldb/strides multiples of 8 elements.
// Returns 0 on launch success; the device status word reports bounded-wait failures.
extern "C" int nb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, const void* aux_in,
                            void* aux_out, int M, int N, int K, int batch, long long lda, long long ldb,
                            long long ldc, long long stride_a, long long stride_b, long long stride_c,
                            long long ld_aux, long long stride_aux, int a_mn, int b_mn, int out_fp32,
                            int bias_fp32, int epi, int aux, int accumulate, int gelu_tanh, float alpha,
                            int block_n, int max_ctas, int* status, void* stream) {
  using namespace nb;
  if (M <= 0 || N <= 0 || batch <= 0) return 0;
  if (K <= 0) return -10;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -11;
  if ((lda & 7) || (ldb & 7) || (batch > 1 && ((stride_a & 7) || (stride_b & 7)))) return -12;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (max_ctas <= 0 || max_ctas > g_num_sms) max_ctas = g_num_sms;
  int bn = block_n;
  if (bn != 256 && bn != 128 && bn != 64) {
    // Largest tile that still gives every SM a tile; small problems use narrower tiles.
    const long long m_tiles = (M + BLOCK_M - 1) / BLOCK_M;
    bn = 256;
    if (N <= 64 || m_tiles * ((N + 255) / 256) * batch < g_num_sms / 2) bn = 128;
    if (N <= 64 || (bn == 128 && m_tiles * ((N + 127) / 128) * batch < g_num_sms / 2)) bn = 64;
  }
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_map(&ta, A, K, M, batch, lda, stride_a, BLOCK_M);
  else       r = make_map(&ta, A, M, K, batch, lda, stride_a, BLOCK_K);
  if (r) return r;
  if (!b_mn) r = make_map(&tb, B, K, N, batch, ldb, stride_b, bn);
  else       r = make_map(&tb, B, N, K, batch, ldb, stride_b, BLOCK_K);
  if (r) return r;
  GemmArgs g;
  g.M = M; g.N = N; g.K = K; g.batch = batch;
  g.out = C; g.bias = bias;
  g.aux_in = reinterpret_cast<const __nv_bfloat16*>(aux_in);
  g.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out);
  g.ldc = ldc; g.stride_c = stride_c; g.ld_aux = ld_aux; g.stride_aux = stride_aux;
  g.a_mn = a_mn; g.b_mn = b_mn; g.out_fp32 = out_fp32; g.bias_fp32 = bias_fp32;
  g.epi = epi; g.aux = aux; g.accumulate = accumulate; g.gelu_tanh = gelu_tanh;
  g.alpha = alpha;
  g.status = status;
  const int oes = out_fp32 ? 4 : 2;
  bool vec = ((reinterpret_cast<uintptr_t>(C) & 15) == 0) && ((ldc * oes) % 16 == 0) &&
             (batch == 1 || (stride_c * oes) % 16 == 0);
  if (aux != AUX_NONE) {
    const void* ap = aux == AUX_STORE_PREACT ? aux_out : aux_in;
    vec = vec && ((reinterpret_cast<uintptr_t>(ap) & 15) == 0) && ((ld_aux * 2) % 16 == 0) &&
          (batch == 1 || (stride_aux * 2) % 16 == 0);
  }
  g.vec_ok = vec ? 1 : 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 256) return launch<256>(ta, tb, g, max_ctas, s);
  if (bn == 128) return launch<128>(ta, tb, g, max_ctas, s);
  return launch<64>(ta, tb, g, max_ctas, s);
}

// Fused row-parallel GEMM + all-reduce over a symmetric workspace.
//   ws_local      this rank's workspace base pointer;  ws_bufs  device array [world] of all bases
//   mc            multicast base of the workspace or null;  data_off  byte offset of C (M x N bf16)
//   call_index    1, 2, 3, ... counts the fused calls on this workspace (flags are monotonic)
//   ticket        device int used as job counter (zeroed here on `stream`)
// After the kernel, every rank's workspace holds sum_r A_r @ B_r at data_off.
extern "C" int nb_gemm_allreduce_bf16(const void* A, const void* B, void* ws_local, void* const* ws_bufs, void* mc,
                                      long long data_off, int flag_off, int done_off, int M, int N, int K, long long lda,
                                      long long ldb, int a_mn, int b_mn, int rank, int world, unsigned call_index,
                                      int n_comm_ctas, int* ticket, int* status, void* stream) {
  using namespace nb;
  constexpr int BN = 256;
  if (M <= 0 || N <= 0 || K <= 0) return -10;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (data_off & 15)) return -11;
  if ((lda & 7) || (ldb & 7) || (N & 7)) return -12;
  const int num_m = (M + BLOCK_M - 1) / BLOCK_M, num_n = (N + BN - 1) / BN;
  const long long tiles = (long long)num_m * num_n;
  if (tiles > 8192) return -13;   // tile-flag region holds 8192 flags
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (n_comm_ctas < 1) n_comm_ctas = 1;
  if (n_comm_ctas > g_num_sms / 2) n_comm_ctas = g_num_sms / 2;
  const int grid = g_num_sms;                 // every rank must launch the same grid
  const int n_gemm = grid - n_comm_ctas;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_map(&ta, A, K, M, 1, lda, 0, BLOCK_M);
  else       r = make_map(&ta, A, M, K, 1, lda, 0, BLOCK_K);
  if (r) return r;
  if (!b_mn) r = make_map(&tb, B, K, N, 1, ldb, 0, BN);
  else       r = make_map(&tb, B, N, K, 1, ldb, 0, BLOCK_K);
  if (r) return r;
  GemmArgs g{};
  g.M = M; g.N = N; g.K = K; g.batch = 1;
  g.out = reinterpret_cast<char*>(ws_local) + data_off;
  g.bias = nullptr; g.aux_in = nullptr; g.aux_out = nullptr;
  g.ldc = N; g.stride_c = (long long)M * N; g.ld_aux = 0; g.stride_aux = 0;
  g.a_mn = a_mn; g.b_mn = b_mn; g.out_fp32 = 0; g.bias_fp32 = 0;
  g.epi = EPI_NONE; g.aux = AUX_NONE; g.accumulate = 0; g.gelu_tanh = 0;
  g.vec_ok = 1; g.alpha = 1.0f; g.status = status;
  CommArgs c{};
  c.bufs = ws_bufs; c.mc = reinterpret_cast<char*>(mc); c.data_off = data_off;
  c.flag_off = flag_off; c.done_off = done_off; c.rank = rank; c.world = world;
  c.tile_target = (unsigned)world;
  c.done_target = (unsigned)world * (unsigned)grid * call_index;
  c.ticket = ticket;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_allreduce_fused_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SmemLayout<BN>::TOTAL) != cudaSuccess)
      return -2;
    configured = true;
  }
  if (cudaMemsetAsync(ticket, 0, sizeof(int), s) != cudaSuccess) return -4;
  gemm_allreduce_fused_kernel<BN><<<grid, NUM_THREADS, SmemLayout<BN>::TOTAL, s>>>(ta, tb, g, c, n_gemm);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
