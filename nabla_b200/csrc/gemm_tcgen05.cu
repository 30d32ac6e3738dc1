// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   D[b] = epilogue( A[b] (M x K)  *  B[b] (K x N) )        fp32 accumulation in TMEM
//
// Structure (one persistent CTA per SM, 384 threads):
//   warp 0       TMA producer: cp.async.bulk.tensor loads of A/B tiles into a shared-memory ring
//   warp 1       MMA issuer:   one thread issues tcgen05.mma (128 x BN x 16) from smem descriptors
//   warp 2       TMEM allocator (2 accumulator buffers of BN columns each)
//   warps 4..11  epilogue, two groups of four warps (a warp reads the TMEM lane quarter warp % 4):
//                tcgen05.ld the accumulator, bias / relu / gelu / d-activation / residual add, cast
//                and store. For the erf-gelu and d-gelu epilogues the groups take alternate
//                64-column pairs of the tile, which keeps them shorter than the tile's MMAs; plain
//                epilogues run on group 0 alone. The epilogue overlaps the next tile's MMAs
//                (double-buffered TMEM).
//
// Both operands may be K-major (row = M or N index, K contiguous) or MN-major (row = K index,
// M or N contiguous), so x@W, dY@W^T and X^T@dY all run without materialising a transpose.
// No TMA multicast is used anywhere: every CTA loads its own tiles.
//
// Replaces what the reference obtains from MAX's matmul (nabla/ops/binary.py:197-198) and the
// matmul + add + relu/gelu composition of nabla/nn/functional/layers.py:30-35.
#include "sm100_ptx.cuh"
#include "nb_debug.cuh"
#include <stdio.h>

namespace nb {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 384;   // warps 0-3: TMA / MMA / TMEM alloc / idle; warps 4-11: two epilogue groups
constexpr int EPI_THREADS = 256;

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
  int vec32_ok;             // ... and 32-byte aligned: a lane's 32 columns go out as 32-byte stores (whole sectors)
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
  // per epilogue warp: 32 rows x 64 bf16 (+16 B pad) used to turn row-per-lane accumulators into
  // 128-byte row segments before they are stored to a peer (reduce-scatter push)
  static constexpr int OUT_ROW_BYTES = 64 * 2 + 16;
  static constexpr int OUT_STAGE_BYTES = 4 * 32 * OUT_ROW_BYTES;
  static constexpr int TOTAL = RING_BYTES + BIAS_BYTES + BAR_BYTES + 112 + OUT_STAGE_BYTES + 1024;  // + alignment slack
};

// CTA-pair variant (cta_group::2): a 256 x BN tile per pair; each CTA stages its own 128 rows of A and
// BN / 2 columns of B per k-block (32 KB for BN = 256, against 48 KB for a lone CTA), which is what
// cuts the shared-memory bytes the tensor core reads per FLOP by a third.
template <int BN>
struct SmemLayoutPair {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = (BN / 2) * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 6 : 8;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BIAS_BYTES = BN * 4;
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int OUT_ROW_BYTES = 64 * 2 + 16;
  static constexpr int OUT_STAGE_BYTES = 4 * 32 * OUT_ROW_BYTES;
  static constexpr int TOTAL = RING_BYTES + BIAS_BYTES + BAR_BYTES + 112 + OUT_STAGE_BYTES + 1024;
};
template <int BN, bool PAIR> struct SmemSelect { using type = SmemLayout<BN>; };
template <int BN> struct SmemSelect<BN, true> { using type = SmemLayoutPair<BN>; };

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

// Fused GEMM + collective: what the launch does besides the GEMM.
//   MODE_AR  C = sum_r A_r @ B_r on every rank        (tiles -> workspace, reduced in place)
//   MODE_RS  rank r keeps its row chunks of that sum   (tiles -> workspace, reduced into rs_out)
//   MODE_AG  C = epilogue(gather_r(A_r) @ B)           (peers' row chunks of A are pulled into
//            a_full by copy CTAs of the same launch; GEMM tiles wait for their rows only)
// Row chunks: the gathered / scattered matrix has M = G * world * chunk_rows rows; rows
// [(g * world + p) * chunk_rows, +chunk_rows) belong to rank p (chunk_rows a multiple of 128).
enum FusedMode : int { MODE_NONE = 0, MODE_AR = 1, MODE_RS = 2, MODE_AG = 3 };

constexpr int AG_FLAG_BASE = 8192;   // index of the first per-M-tile "rows are here" flag
constexpr int READY_OFF = 64;        // byte offset, after the done counter, of the per-rank ready flags

struct CommArgs {
  void* const* bufs;        // device array [world]: peer base pointers of the symmetric workspace
  char* mc;                 // multicast base of the workspace (nullptr: plain peer loads/stores)
  long long data_off;       // byte offset inside the workspace of C (AR/RS) or of the staged A shard (AG)
  int flag_off, done_off;   // byte offsets of the tile flags / done counter inside the workspace
  int rank, world;
  unsigned tile_target;     // value a tile flag reaches when every rank has written the tile
  unsigned done_target;     // value the done counter reaches when every participant of every rank is through
  int* ticket;              // device int, zeroed before the launch: next reduce job of this rank
  int mpc;                  // M tiles per row chunk (chunk_rows / 128); RS and AG
  int per;                  // M tiles per rank (num_m / world); AG
  unsigned epoch;           // AG: value of the ready / row flags of this call (relative to ctr[1])
  const unsigned* ctr;      // device counters of the workspace: [1] all-gather calls so far, [2] done
                            // counts so far; epoch and done_target are relative to them, and a
                            // one-thread kernel advances them after the launch (CUDA-graph replay safe)
  __nv_bfloat16* rs_out;    // RS: this rank's rows of the sum, [M / world][N]
  char* a_full;             // AG: the gathered A, [M][K] dense
  long long unit_bytes;     // AG: bytes of one 128-row block of A
  // AG push variant: the gathered A of every rank lives at the same offset of a symmetric arena;
  // copy CTAs read this rank's own rows and store them into every rank's gathered A
  void* const* abufs;       // device array [world] of arena base pointers (nullptr: pull variant)
  long long a_off;          // byte offset of the gathered A inside the arena
  const char* own_src;      // this rank's own rows, [M / world][K] dense
  char* a_mc;               // multicast base of the arena (nullptr: one store per peer). With it a
                            // single multimem.st reaches the gathered A of EVERY rank of the group
                            // through the switch: the rows leave this GPU once instead of world - 1 times
};

// Order in which the GEMM walks the M tiles -> the tile's real row block.
//   RS: consecutive tiles rotate over the owning ranks, so that every rank's reducers get work
//       from the start;  AG: own rows first, then the peers' blocks in the order they arrive.
template <int MODE>
__device__ __forceinline__ int remap_m(int tm, const CommArgs& c) {
  if (MODE == MODE_RS) {
    const int q = tm / c.world, p = tm - q * c.world;
    const int g = q / c.mpc, j = q - g * c.mpc;
    return (g * c.world + p) * c.mpc + j;
  }
  if (MODE == MODE_AG) {
    // own rows first; then the peers' blocks in ARRIVAL order. Every rank sends its block v to all
    // peers at the same time, so the blocks with the same index v of all peers land together: the
    // walk takes block 0 of peer +1, +2, ..., then block 1 of each, and so on. (Walking one peer's
    // rows to the end before the next peer's would wait for the end of the whole exchange after the
    // first quarter of the work.)
    int dist = 0, rem = tm;
    if (tm >= c.per) {
      const int t2 = tm - c.per, nw = c.world - 1;
      rem = t2 / nw;
      dist = 1 + (t2 - rem * nw);
    }
    const int g = rem / c.mpc, j = rem - g * c.mpc;
    int p = c.rank + dist;
    if (p >= c.world) p -= c.world;
    return (g * c.world + p) * c.mpc + j;
  }
  return tm;
}

__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// 32-byte store (one whole sector per lane and instruction; the address must be 32-byte aligned).
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
               "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

// One CTA's share of the GEMM. `cta` / `nctas` replace blockIdx / gridDim so that the fused
// kernel can dedicate some CTAs to communication. Returns false if the CTA left early.
// PAIR: this CTA is one of a cluster of two (cta_group::2). `cta` / `nctas` then count pairs; a pair
// takes the 128-row tiles 2 * i and 2 * i + 1 (one each: the two CTAs share only the tile of B, so
// their row blocks need not be neighbours once a fused mode has re-ordered them), the tensor map of
// B has a box of BN / 2 rows, the loads of both CTAs complete on the leader's full barriers, and the
// leader's MMA warp issues for both CTAs.
template <int BN, int MODE, bool PAIR = false>
__device__ __forceinline__ bool gemm_cta(const CUtensorMap* tmAp, const CUtensorMap* tmBp, const GemmArgs& args,
                                         const CommArgs& comm, const int cta, const int nctas,
                                         const CUtensorMap* tmAownp = nullptr) {
  const CUtensorMap& tmA = *tmAp;
  const CUtensorMap& tmB = *tmBp;
  using L = typename SmemSelect<BN, PAIR>::type;
  constexpr int TILE_M = PAIR ? 2 * BLOCK_M : BLOCK_M;
  constexpr int BNL = PAIR ? BN / 2 : BN;            // columns of B this CTA stages
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = crank == 0u;
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
  uint8_t* out_stage = smem + ((L::RING_BYTES + L::BIAS_BYTES + L::BAR_BYTES + 127) & ~127);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // a previous bounded wait failed on this device: do not pile more waits on top of it
  // (a pair does not leave early: both CTAs must reach the cluster barriers below, and their waits
  // are bounded anyway)
  if (!PAIR) {
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = *reinterpret_cast<volatile int*>(args.status);
    __syncthreads();
    if (s_abort != 0) return false;   // uniform for the whole CTA
  }

  // pair: tiles are counted in pairs of 128-row tiles; an odd last tile leaves the second CTA a tile
  // past the edge (its loads read the fill value and its epilogue stores nothing)
  const int num_m = (args.M + TILE_M - 1) / TILE_M;
  const int num_n = (args.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n * args.batch;
  const int num_kb = (args.K + BLOCK_K - 1) / BLOCK_K;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      // pair: only the leader's full barriers are used; the loads of both CTAs complete on them
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    // pair: one arrival per epilogue warp of both CTAs, all on the leader's barrier
    mbar_init(&tmem_empty[0], PAIR ? 2 * (EPI_THREADS / 32) : EPI_THREADS);
    mbar_init(&tmem_empty[1], PAIR ? 2 * (EPI_THREADS / 32) : EPI_THREADS);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (PAIR) {
    __syncthreads();
    cluster_sync_all();              // the other CTA is running before the allocator is asked for the pair
  }
  if (warp == 2) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, 2 * BN);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 2 * BN);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();      // the other CTA's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t leader_full = PAIR ? mapa_shared(smem_u32(&full_bar[0]), 0u) : 0u;
      (void)leader_full;
      for (int t = cta; t < num_tiles && ok; t += nctas) {
        int b, tm, tn;
        tile_coords(t, num_m, num_n, b, tm, tn);
        if (PAIR) tm = 2 * tm + (int)crank;
        tm = remap_m<MODE>(tm, comm);
        const int m0 = tm * BLOCK_M, n0 = tn * BN + (int)crank * BNL;
        // MODE_AG: this rank's own rows are read from its shard directly (no copy to wait for)
        const CUtensorMap* tmAuse = tmAp;
        int ma0 = m0;
        bool own = false;
        if (MODE == MODE_AG) {
          const int blk = tm / comm.mpc;
          own = (blk % comm.world) == comm.rank;
          if (own) {
            tmAuse = tmAownp;
            ma0 = ((blk / comm.world) * comm.mpc + (tm - blk * comm.mpc)) * BLOCK_M;
          }
        }
        if (MODE == MODE_AG && !own) {
          // rows m0 .. m0+127 of the gathered A must have been copied in by a copy CTA
          const unsigned* f = reinterpret_cast<const unsigned*>(reinterpret_cast<char*>(comm.bufs[comm.rank]) +
                                                                comm.flag_off) + AG_FLAG_BASE + tm;
          const unsigned long long t0 = globaltimer_ns();
          unsigned spins = 0;
          while ((int)(ld_acquire_sys_u32(f) - comm.epoch) < 0) {
            if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
              ok = false;
              atomicExch(args.status, NB_ERR_TIMEOUT_PEER);
              break;
            }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");   // the rows were written by bulk copies
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(PAIR ? mbar_wait_cluster(&empty_bar[stage], phase ^ 1) : mbar_wait(&empty_bar[stage], phase ^ 1))) {
            ok = false;
            atomicExch(args.status, NB_ERR_TIMEOUT_PRODUCER);
            break;
          }
          uint8_t* sA = ring + stage * L::STAGE_BYTES;
          uint8_t* sB = sA + L::A_BYTES;
          // pair: the leader expects the bytes of both CTAs on its barrier; the other CTA only loads
          if (!PAIR) mbar_arrive_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          else if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * L::STAGE_BYTES);
          const int k0 = kb * BLOCK_K;
          // debug build: every tile origin lies inside its tensor and the innermost coordinate
          // starts on a 16-byte boundary; a failed check skips the copies (the consumers' bounded
          // waits then end the kernel) instead of issuing them
          // (in a pair the second CTA's half tile may start past the edge: those loads read the fill value)
          if (!(NB_IN_BOUNDS(NB_SITE_GEMM_TMA_COORD, k0, args.K) &&
                NB_IN_BOUNDS(NB_SITE_GEMM_TMA_COORD, m0, args.M + (PAIR ? BLOCK_M : 0)) &&
                NB_IN_BOUNDS(NB_SITE_GEMM_TMA_COORD, n0, args.N + (PAIR ? BNL : 0)) &&
                NB_IN_BOUNDS(NB_SITE_GEMM_TMA_COORD, b, args.batch) &&
                NB_IN_BOUNDS(NB_SITE_GEMM_TMA_COORD, ma0, args.M + (PAIR ? BLOCK_M : 0)) &&
                NB_ALIGNED(NB_SITE_GEMM_TMA_ALIGN, (args.a_mn ? m0 : k0) * 2, 16) &&
                NB_ALIGNED(NB_SITE_GEMM_TMA_ALIGN, (args.b_mn ? n0 : k0) * 2, 16))) {
            ok = false;
            break;
          }
          if (PAIR) {
            const uint32_t lbar = leader_full + 8u * stage;   // the leader's full barrier of this stage
            if (!args.a_mn) {
              tma_load_3d_pair(sA, tmAuse, lbar, k0, ma0, b);
            } else {
#pragma unroll
              for (int j = 0; j < BLOCK_M / 64; ++j)
                tma_load_3d_pair(sA + j * (BLOCK_K * 128), &tmA, lbar, m0 + j * 64, k0, b);
            }
            if (!args.b_mn) {
              tma_load_3d_pair(sB, &tmB, lbar, k0, n0, b);
            } else {
#pragma unroll
              for (int j = 0; j < BNL / 64; ++j)
                tma_load_3d_pair(sB + j * (BLOCK_K * 128), &tmB, lbar, n0 + j * 64, k0, b);
            }
          } else {
            if (!args.a_mn) {
              tma_load_3d(sA, tmAuse, &full_bar[stage], k0, ma0, b);
            } else {
#pragma unroll
              for (int j = 0; j < BLOCK_M / 64; ++j)
                tma_load_3d(sA + j * (BLOCK_K * 128), &tmA, &full_bar[stage], m0 + j * 64, k0, b);
            }
            if (!args.b_mn) {
              tma_load_3d(sB, &tmB, &full_bar[stage], k0, n0, b);
            } else {
#pragma unroll
              for (int j = 0; j < BNL / 64; ++j)
                tma_load_3d(sB + j * (BLOCK_K * 128), &tmB, &full_bar[stage], n0 + j * 64, k0, b);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (PAIR && !leader) {
      // the other CTA of the pair issues nothing: the leader's thread drives both tensor cores
    } else if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(TILE_M, BN, args.a_mn, args.b_mn);
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
        if (!(PAIR ? mbar_wait_cluster(&tmem_empty[buf], acc_phase ^ 1) : mbar_wait(&tmem_empty[buf], acc_phase ^ 1))) {
          atomicExch(args.status, NB_ERR_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(PAIR ? mbar_wait_cluster(&full_bar[stage], phase) : mbar_wait(&full_bar[stage], phase))) {
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
            if (PAIR)
              umma_f16_ss_pair(tmem_d, da + static_cast<uint64_t>(k * a_kstep), db + static_cast<uint64_t>(k * b_kstep),
                               idesc, (kb | k) != 0 ? 1u : 0u);
            else
              umma_f16_ss(tmem_d, da + static_cast<uint64_t>(k * a_kstep), db + static_cast<uint64_t>(k * b_kstep),
                          idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // frees the smem slot (of both CTAs of a pair) when these MMAs retire
          if (PAIR) umma_commit_pair(&empty_bar[stage], 3);
          else umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          if (PAIR) umma_commit_pair(&tmem_full[buf], 3);
          else umma_commit(&tmem_full[buf]);
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue
    const int wq = warp & 3;                 // TMEM lane quarter this warp may read
    const int et = threadIdx.x - 128;        // 0..255
    // two epilogue groups share every tile: group g takes the 64-column pairs with (pair & 1) == g,
    // so the per-element math of the gelu / d-gelu epilogues fits under the tile's MMAs
    const int grp = (warp - 4) >> 2;
    const bool heavy = args.epi == EPI_BIAS_GELU || args.aux == AUX_MUL_DGELU;
    bool ok = true;
    int it = 0;
    for (int t = cta; t < num_tiles; t += nctas, ++it) {
      int b, tm, tn;
      tile_coords(t, num_m, num_n, b, tm, tn);
      if (PAIR) tm = 2 * tm + (int)crank;
      const int tm_order = tm;
      tm = remap_m<MODE>(tm, comm);
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
      long long out_off = static_cast<long long>(b) * args.stride_c + static_cast<long long>(row) * args.ldc;
      // debug build: the first element of this lane's output row lies inside the output
      const bool row_ok =
          row < args.M && NB_IN_BOUNDS(NB_SITE_GEMM_STORE, out_off,
                                       static_cast<long long>(args.batch - 1) * args.stride_c +
                                           static_cast<long long>(args.M - 1) * args.ldc + 1);
      const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(wq * 32) << 16);
      void* out_ptr = args.out;
      if (MODE == MODE_RS) {
        // push: the tile goes straight into the memory of the rank that owns these rows, into
        // the slot of this rank ([world][M / world][N] at data_off of the owner's workspace)
        const int q = tm_order / comm.world, p = tm_order - q * comm.world;
        out_ptr = reinterpret_cast<char*>(comm.bufs[p]) + comm.data_off;
        out_off = (static_cast<long long>(comm.rank) * (args.M / comm.world) + q * BLOCK_M + wq * 32 + lane) * args.N;
      }
      const long long aux_off =
          static_cast<long long>(b) * args.stride_aux + static_cast<long long>(row) * args.ld_aux;
      // epilogues with per-element transcendental math are split between the two groups by
      // 64-column pairs; the plain ones (and the peer-store path, whose staging buffers exist
      // once per lane quarter) stay with group 0, whose warps then stream the whole tile.
      // next_chunk(c): the first 32-column chunk after c that this warp handles (BN / 32: none)
      auto next_chunk = [&](int c) -> int {
        for (++c; c < BN / 32; ++c) {
          if (n0 + c * 32 >= args.N) break;   // warp-uniform
          if (MODE != MODE_RS && heavy) {
            if (((c >> 1) & 1) == grp) return c;
          } else {
            return grp == 0 ? c : BN / 32;
          }
        }
        return BN / 32;
      };
      // the accumulator chunk after the current one is fetched from tensor memory while the current
      // one goes through the epilogue math and its stores
      uint32_t v[32];
      int c = next_chunk(-1);
      if (c < BN / 32) tmem_ld_32x32(taddr + c * 32, v);
#pragma unroll 1
      while (c < BN / 32) {
        const int nb0 = n0 + c * 32;
        tmem_ld_wait_regs(v);
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * args.alpha + sbias[c * 32 + j];
        const int c_next = next_chunk(c);
        if (c_next < BN / 32) tmem_ld_32x32(taddr + c_next * 32, v);
        const bool full = (nb0 + 32 <= args.N) && args.vec_ok;
        // ---- auxiliary output: pre-activation
        if (args.aux == AUX_STORE_PREACT && row_ok) {
          __nv_bfloat16* ap = args.aux_out + aux_off + nb0;
          if (full && args.vec32_ok) {
            uint32_t pw[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
              pw[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            st_global_v8(ap, pw);
            st_global_v8(ap + 16, pw + 8);
          } else if (full) {
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
              const uint4 pk = reinterpret_cast<const uint4*>(ap)[q];
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
        if (MODE == MODE_RS) {
          // to a peer: stage two 32-column chunks per warp in shared memory, then write whole
          // 128-byte row segments (4 rows per warp instruction) instead of 16-byte pieces of
          // 32 different rows, which NVLink would carry as 32 small packets
          uint8_t* mine = out_stage + wq * (32 * L::OUT_ROW_BYTES);
          uint8_t* rowp = mine + lane * L::OUT_ROW_BYTES + (c & 1) * 64;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 pk;
            uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 h = __floats2bfloat162_rn(f[q * 8 + 2 * j], f[q * 8 + 2 * j + 1]);
              pw[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(rowp + q * 16) = pk;
          }
          const bool last_chunk = (c == BN / 32 - 1) || (nb0 + 32 >= args.N);
          if ((c & 1) || last_chunk) {
            __syncwarp();
            const int col0 = n0 + (c & ~1) * 32;               // first column held in the stage
            const int sub = lane >> 3, piece = lane & 7;       // 4 rows x 8 pieces of 16 bytes
            __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(out_ptr) + (out_off - (long long)lane * args.N);
#pragma unroll
            for (int it8 = 0; it8 < 8; ++it8) {
              const int r = it8 * 4 + sub;
              const int col = col0 + piece * 8;
              const bool have = ((c & 1) || piece < 4) && col < args.N;
              if (have) {
                const uint4 v = *reinterpret_cast<const uint4*>(mine + r * L::OUT_ROW_BYTES + piece * 16);
                *reinterpret_cast<uint4*>(base + (long long)r * args.N + col) = v;
              }
            }
            __syncwarp();
          }
        } else if (row_ok) {
          if (args.out_fp32) {
            float* op = reinterpret_cast<float*>(args.out) + out_off + nb0;
            if (full && args.vec32_ok && !args.accumulate) {
#pragma unroll
              for (int q = 0; q < 4; ++q) st_global_v8(op + q * 8, reinterpret_cast<const uint32_t*>(f) + q * 8);
            } else if (full) {
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
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(out_ptr) + out_off + nb0;
            if (full && args.vec32_ok && !args.accumulate) {
              uint32_t pw[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
                pw[j] = *reinterpret_cast<uint32_t*>(&h);
              }
              st_global_v8(op, pw);
              st_global_v8(op + 16, pw + 8);
            } else if (full) {
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
        c = c_next;
      }
      tc_fence_before();
      if (PAIR) {
        // one arrival per warp, on the leader's barrier (it holds the MMA issuer of both CTAs)
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive(&tmem_empty[buf]);
          else mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[buf]), 0u));
        }
      } else {
        mbar_arrive(&tmem_empty[buf]);
      }
      if (MODE == MODE_AR) {
        // the tile is in this rank's workspace: make it visible system-wide, then count it on
        // the rank that reduces it (tile (tm_order, tn) belongs to rank tm_order % world)
        __threadfence_system();
        named_bar_sync(2, EPI_THREADS);
        if (et == 0)
          asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(
                           reinterpret_cast<char*>(comm.bufs[tm_order % comm.world]) + comm.flag_off +
                           4ll * (tm_order * num_n + tn)),
                       "r"(1u)
                       : "memory");
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // neither CTA's shared or tensor memory goes away while the other may still use it
  if (warp == 2) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN);
    else tmem_dealloc(tmem_base, 2 * BN);
  }
  return true;
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmArgs args) {
  CommArgs none{};
  gemm_cta<BN, MODE_NONE>(&tmA, &tmB, args, none, blockIdx.x, gridDim.x);
}

// The same GEMM on CTA pairs: launched as clusters of two CTAs, one pair per two SMs.
template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                              const GemmArgs args) {
  CommArgs none{};
  gemm_cta<BN, MODE_NONE, true>(&tmA, &tmB, args, none, blockIdx.x >> 1, gridDim.x >> 1);
}

// Probe of the tensor-memory allocator for CTA pairs, run once before the pair GEMM is used: both
// CTAs of one cluster ask for 256 columns with cta_group::2 and report the base they were given.
// 2 x 256 columns fit the 512 of an SM, so neither request can wait for the other whichever way the
// hardware counts them; equal bases mean that the two requests were one allocation made together.
__global__ void __launch_bounds__(32, 1) pair_alloc_probe_kernel(unsigned* out) {
  __shared__ uint32_t slot;
  cluster_sync_all();              // the other CTA is running before the allocator is asked for the pair
  tmem_alloc_pair(&slot, 256);
  tmem_relinquish_pair();
  tc_fence_before();
  __syncwarp();
  tc_fence_after();
  const uint32_t base = slot;
  if (threadIdx.x == 0) out[cluster_ctarank()] = base;
  cluster_sync_all();
  tmem_dealloc_pair(base, 256);
}

// ------------------------------------------------------------------ fused GEMM + all-reduce
// CTAs [0, n_gemm) compute tiles of this rank's partial product into the symmetric workspace and
// raise per-tile flags on all ranks. Every CTA (the dedicated communication CTAs from the start,
// the GEMM CTAs once they run out of tiles) then takes reduce jobs from a ticket counter: job k of
// rank r is tile r + k * world. A job waits until all ranks have written the tile, sums the
// copies (multimem.ld_reduce in the switch, or peer loads) and writes the sum into every rank's
// workspace (multimem.st, or peer stores). The kernel leaves once every CTA of every rank is
// through, so the next kernel on the stream finds the reduced matrix in the local workspace.
__device__ __forceinline__ bool wait_flag_ge(const unsigned* p, unsigned target) {
  if ((int)(ld_acquire_sys_u32(p) - target) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (true) {
    if ((int)(ld_acquire_sys_u32(p) - target) >= 0) return true;
    if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
}

constexpr int RED_UNROLL = 16;

// Reduce jobs of MODE_AR / MODE_RS. Job k of this rank is tile (tm_order = (k / num_n) * world +
// rank, tn = k % num_n): wait until every rank has counted it, then sum the ranks' copies.
//   AR: multimem.ld_reduce + multimem.st in place on every rank (or peer loads + peer stores)
//   RS: multimem.ld_reduce (or peer loads) + a plain store into this rank's rs_out
template <int BN, int MODE>
__device__ __forceinline__ void reduce_jobs(const GemmArgs& args, const CommArgs& comm) {
  __shared__ int s_job;
  __shared__ int s_ok;
  const int num_m = (args.M + BLOCK_M - 1) / BLOCK_M;
  const int num_n = (args.N + BN - 1) / BN;
  char* local = reinterpret_cast<char*>(comm.bufs[comm.rank]);
  const unsigned* flags = reinterpret_cast<const unsigned*>(local + comm.flag_off);
  // comm.ticket == nullptr (deterministic replay): CTA c takes jobs c, c + grid, ... in that order
  // whatever the timing, so which CTA reduces which tile, and after which other tile, is the same in
  // every run; with the counter the first free CTA takes the next job
  int fixed_k = (int)blockIdx.x;
  while (true) {
    __syncthreads();
    if (threadIdx.x == 0) {
      int k;
      if (comm.ticket != nullptr) {
        k = atomicAdd(comm.ticket, 1);
      } else {
        k = fixed_k;
        fixed_k += (int)gridDim.x;
      }
      const int tmo = (k / num_n) * comm.world + comm.rank;
      s_job = k;
      s_ok = 1;
      if (tmo < num_m) {
        const unsigned* f = flags + tmo * num_n + (k % num_n);
        if (!wait_flag_ge(f, comm.tile_target)) {
          atomicExch(args.status, NB_ERR_TIMEOUT_PEER);
          s_ok = 0;
        } else {
          // every rank has counted: nobody touches this flag again before the closing
          // barrier, so it can go back to zero for the next call
          *const_cast<volatile unsigned*>(f) = 0u;
        }
      }
    }
    __syncthreads();
    const int k = s_job;
    const int q = k / num_n, tn = k - q * num_n;
    const int tmo = q * comm.world + comm.rank;
    if (tmo >= num_m || !s_ok) break;
    const int tm = remap_m<MODE>(tmo, comm);
    const int m0 = tm * BLOCK_M, n0 = tn * BN;
    const int rows = min(BLOCK_M, args.M - m0);
    const int vpr = (min(BN, args.N - n0) * 2) / 16;       // 16-byte vectors per tile row (N % 8 == 0)
    const long long base = comm.data_off + ((long long)m0 * args.ldc + n0) * 2;
    // RS: the tile's rows in this rank's output (its row blocks are numbered q = 0, 1, ...)
    char* rs_base = reinterpret_cast<char*>(comm.rs_out) + ((long long)q * BLOCK_M * args.N + n0) * 2;
    const int total = rows * vpr;
    if (comm.mc != nullptr) {
      // RED_UNROLL 16-byte vectors in flight per thread: one 128 x 256 tile is a single round
      // trip through the switch for a 256-thread CTA
      for (int i = threadIdx.x; i < total; i += RED_UNROLL * NUM_THREADS) {
        uint4 v[RED_UNROLL];
#pragma unroll
        for (int u = 0; u < RED_UNROLL; ++u) {
          const int idx = i + u * NUM_THREADS;
          if (idx < total) {
            const long long off = base + ((long long)(idx / vpr) * args.ldc) * 2 + (idx % vpr) * 16;
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                         : "l"(comm.mc + off)
                         : "memory");
          }
        }
#pragma unroll
        for (int u = 0; u < RED_UNROLL; ++u) {
          const int idx = i + u * NUM_THREADS;
          if (idx < total) {
            if (MODE == MODE_RS) {
              *reinterpret_cast<uint4*>(rs_base + ((long long)(idx / vpr) * args.N) * 2 + (idx % vpr) * 16) = v[u];
            } else {
              const long long off = base + ((long long)(idx / vpr) * args.ldc) * 2 + (idx % vpr) * 16;
              asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(comm.mc + off),
                           "r"(v[u].x), "r"(v[u].y), "r"(v[u].z), "r"(v[u].w)
                           : "memory");
            }
          }
        }
      }
    } else {
      constexpr int PU = 8;   // vectors in flight per thread and peer
      for (int i = threadIdx.x; i < total; i += PU * NUM_THREADS) {
        float acc[PU][8];
#pragma unroll
        for (int u = 0; u < PU; ++u)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
        for (int p = 0; p < comm.world; ++p) {
          const char* src = reinterpret_cast<const char*>(comm.bufs[p]);
          uint4 v[PU];
#pragma unroll
          for (int u = 0; u < PU; ++u) {
            const int idx = i + u * NUM_THREADS;
            v[u] = make_uint4(0u, 0u, 0u, 0u);
            if (idx < total) {
              const long long off = base + ((long long)(idx / vpr) * args.ldc) * 2 + (idx % vpr) * 16;
              asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                           : "l"(src + off)
                           : "memory");
            }
          }
#pragma unroll
          for (int u = 0; u < PU; ++u) {
            const unsigned w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              acc[u][2 * j] += __uint_as_float(w[j] << 16);
              acc[u][2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < PU; ++u) {
          const int idx = i + u * NUM_THREADS;
          if (idx < total) {
            uint4 o;
            unsigned* ow = reinterpret_cast<unsigned*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 h = __floats2bfloat162_rn(acc[u][2 * j], acc[u][2 * j + 1]);
              ow[j] = *reinterpret_cast<unsigned*>(&h);
            }
            if (MODE == MODE_RS) {
              *reinterpret_cast<uint4*>(rs_base + ((long long)(idx / vpr) * args.N) * 2 + (idx % vpr) * 16) = o;
            } else {
              const long long off = base + ((long long)(idx / vpr) * args.ldc) * 2 + (idx % vpr) * 16;
              for (int p = 0; p < comm.world; ++p)
                *reinterpret_cast<uint4*>(reinterpret_cast<char*>(comm.bufs[p]) + off) = o;
            }
          }
        }
      }
    }
  }
}

// Closing step of a fused launch: count this CTA on every rank; the last CTA of the grid waits
// until every participant of every rank is through, so no rank's workspace is reused (or its
// kernel gone) while a peer still reads or writes it.
__device__ __forceinline__ void closing_count(const GemmArgs& args, const CommArgs& comm) {
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
      const char* local = reinterpret_cast<const char*>(comm.bufs[comm.rank]);
      if (!wait_flag_ge(reinterpret_cast<const unsigned*>(local + comm.done_off), comm.done_target))
        atomicExch(args.status, NB_ERR_TIMEOUT_PEER);
    }
  }
}

// ---- MODE_AG copy CTAs -----------------------------------------------------------------------
// One thread per copy CTA drives a ring of bulk copies: peer (or own) staged rows -> shared
// memory -> a_full. No multicast; every byte crosses NVLink once. After the last piece of a
// 128-row block has landed, the block's flag is raised for the GEMM producers of this GPU.
constexpr int AG_PIECE = 32 * 1024;
constexpr int AG_STAGES = 6;      // 192 KB of the GEMM's shared-memory ring

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}

// Copy order of the 128-row blocks: the peers' rows in ring order, as the GEMM will ask for them.
// This rank's own rows (the last num_m / world positions of this order) are not copied here: the
// GEMM reads them from the shard, and the caller writes them into the gathered matrix itself.
__device__ __forceinline__ int ag_unit(int u, int num_m, const CommArgs& c) {
  u += c.per;
  return u >= num_m ? u - num_m : u;
}

template <int BN>
__device__ __forceinline__ void gather_jobs(const GemmArgs& args, const CommArgs& comm, int cidx, int ncomm) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  static_assert(AG_PIECE * AG_STAGES <= SmemLayout<BN>::RING_BYTES, "copy ring must fit the GEMM ring");
  __shared__ uint64_t bars[AG_STAGES];
  if (threadIdx.x != 0) return;
  char* local = reinterpret_cast<char*>(comm.bufs[comm.rank]);
  const int num_m = (args.M + BLOCK_M - 1) / BLOCK_M;
  // tell every peer that this rank's rows are staged (the staging copy ran before this kernel)
  if (cidx == 0) {
    for (int p = 0; p < comm.world; ++p)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<char*>(comm.bufs[p]) + comm.done_off +
                                                                READY_OFF + 4 * comm.rank),
                   "r"(comm.epoch)
                   : "memory");
  }
  for (int s = 0; s < AG_STAGES; ++s) mbar_init(&bars[s], 1);
  fence_mbar_init();
  fence_proxy_async_smem();
  const int ppu = (int)((comm.unit_bytes + AG_PIECE - 1) / AG_PIECE);   // pieces per 128-row block
  int n_units = 0;
  for (int u = cidx; u < num_m - comm.per; u += ncomm) ++n_units;     // the peers' blocks; own rows are the caller's
  const int total = n_units * ppu;
  unsigned ready_mask = 0;
  bool ok = true;
  // piece i -> (unit, piece in unit) -> source / destination
  auto issue_load = [&](int i) -> bool {
    const int ui = i / ppu, pi = i - ui * ppu;
    const int tm = remap_m<MODE_AG>(ag_unit(cidx + ui * ncomm, num_m, comm), comm);
    const int blk = tm / comm.mpc;                     // row chunk index in the gathered matrix
    const int p = blk % comm.world, g = blk / comm.world, j = tm - blk * comm.mpc;
    // debug build: the owner is a rank of the group and the block lies inside its staged shard
    if (!(NB_IN_BOUNDS(NB_SITE_GEMM_PEER_RANK, p, comm.world) &&
          NB_IN_BOUNDS(NB_SITE_GEMM_PEER_OFFSET, g * comm.mpc + j, comm.per)))
      return false;
    if (!((ready_mask >> p) & 1u)) {
      if (!wait_flag_ge(reinterpret_cast<const unsigned*>(local + comm.done_off + READY_OFF + 4 * p), comm.epoch))
        return false;
      ready_mask |= 1u << p;
    }
    const long long off = (long long)pi * AG_PIECE;
    const uint32_t bytes = (uint32_t)min((long long)AG_PIECE, comm.unit_bytes - off);
    const char* src = reinterpret_cast<const char*>(comm.bufs[p]) + comm.data_off +
                      (long long)(g * comm.mpc + j) * comm.unit_bytes + off;
    const int st = i % AG_STAGES;
    mbar_arrive_expect_tx(&bars[st], bytes);
    bulk_g2s(ring + st * AG_PIECE, src, bytes, &bars[st]);
    return true;
  };
  auto publish = [&](int i) {   // piece i has landed in a_full; raise its block's flag if it was the last piece
    const int ui = i / ppu, pi = i - ui * ppu;
    if (pi != ppu - 1) return;
    const int tm = remap_m<MODE_AG>(ag_unit(cidx + ui * ncomm, num_m, comm), comm);
    asm volatile("fence.proxy.async;" ::: "memory");
    __threadfence();
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(reinterpret_cast<unsigned*>(local + comm.flag_off) +
                                                              AG_FLAG_BASE + tm),
                 "r"(comm.epoch)
                 : "memory");
  };
  // Ring of AG_STAGES pieces. Stores trail loads by AG_LAG groups: after committing store i only
  // stores up to i - AG_LAG are awaited, so loads and stores of several pieces are in flight and
  // neither the peer's latency nor the store's is paid per piece.
  constexpr int AG_LAG = 2;
  int issued = 0;
  for (; issued < total && issued < AG_STAGES && ok; ++issued) ok = issue_load(issued);
  for (int i = 0; i < total && ok; ++i) {
    const int st = i % AG_STAGES;
    const uint32_t phase = (i / AG_STAGES) & 1;
    if (!mbar_wait(&bars[st], phase)) { ok = false; break; }
    const int ui = i / ppu, pi = i - ui * ppu;
    const int tm = remap_m<MODE_AG>(ag_unit(cidx + ui * ncomm, num_m, comm), comm);
    const long long off = (long long)pi * AG_PIECE;
    const uint32_t bytes = (uint32_t)min((long long)AG_PIECE, comm.unit_bytes - off);
    bulk_s2g(comm.a_full + (long long)tm * comm.unit_bytes + off, ring + st * AG_PIECE, bytes);
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    if (i >= AG_LAG) {
      asm volatile("cp.async.bulk.wait_group %0;" ::"n"(AG_LAG) : "memory");   // stores <= i - AG_LAG are complete
      publish(i - AG_LAG);
      if (issued < total) {          // piece `issued` reuses the stage of piece i - AG_LAG (AG_STAGES apart)
        ok = issue_load(issued);
        ++issued;
      }
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if (ok)
    for (int i = max(0, total - AG_LAG); i < total; ++i) publish(i);
  if (!ok) atomicExch(args.status, NB_ERR_TIMEOUT_PEER);
}

// Push variant of the MODE_AG copy CTAs: all threads read this rank's own rows (local memory,
// short latency) and store them into the gathered A of every rank. The peer stores are posted:
// nothing waits for a round trip, so a few CTAs keep the link busy. After each 128-row block a
// barrier and one release store per peer raise the block's flag there. A peer is written only
// after it announced (ready flag) that its gathered A may be overwritten.
template <int BN>
__device__ __forceinline__ void push_jobs(const GemmArgs& args, const CommArgs& comm, int cidx, int ncomm) {
  __shared__ int s_ok;
  char* local = reinterpret_cast<char*>(comm.bufs[comm.rank]);
  if (threadIdx.x == 0) {
    if (cidx == 0) {
      for (int p = 0; p < comm.world; ++p)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<char*>(comm.bufs[p]) + comm.done_off +
                                                                  READY_OFF + 4 * comm.rank),
                     "r"(comm.epoch)
                     : "memory");
    }
    bool ok = true;
    for (int p = 0; p < comm.world && ok; ++p)
      ok = wait_flag_ge(reinterpret_cast<const unsigned*>(local + comm.done_off + READY_OFF + 4 * p), comm.epoch);
    if (!ok) atomicExch(args.status, NB_ERR_TIMEOUT_PEER);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  constexpr int PU = 16;                                   // 16-byte vectors in flight per thread
  const long long nvec = comm.unit_bytes / 16;
  for (int v = cidx; v < comm.per; v += ncomm) {           // this CTA's own 128-row blocks
    const int g = v / comm.mpc, j = v - g * comm.mpc;
    const int tm = (g * comm.world + comm.rank) * comm.mpc + j;   // the block's place in the gathered A
    if (!NB_IN_BOUNDS(NB_SITE_GEMM_PEER_OFFSET, tm, comm.per * comm.world)) continue;   // CTA-uniform
    const uint4* src = reinterpret_cast<const uint4*>(comm.own_src + (long long)v * comm.unit_bytes);
    const long long dst_off = comm.a_off + (long long)tm * comm.unit_bytes;
    for (long long base = 0; base < nvec; base += (long long)PU * NUM_THREADS) {
      uint4 val[PU];
#pragma unroll
      for (int u = 0; u < PU; ++u) {
        const long long idx = base + u * NUM_THREADS + threadIdx.x;
        if (idx < nvec) val[u] = src[idx];
      }
      if (comm.a_mc != nullptr) {                          // one store, replicated by the switch (own copy included)
        char* dst = comm.a_mc + dst_off;
#pragma unroll
        for (int u = 0; u < PU; ++u) {
          const long long idx = base + u * NUM_THREADS + threadIdx.x;
          if (idx < nvec)
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst + idx * 16),
                         "r"(val[u].x), "r"(val[u].y), "r"(val[u].z), "r"(val[u].w)
                         : "memory");
        }
      } else {
        for (int d = 1; d < comm.world; ++d) {             // the peers in ring order (the own copy is the caller's)
          int q = comm.rank + d;
          if (q >= comm.world) q -= comm.world;
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(comm.abufs[q]) + dst_off);
#pragma unroll
          for (int u = 0; u < PU; ++u) {
            const long long idx = base + u * NUM_THREADS + threadIdx.x;
            if (idx < nvec) dst[idx] = val[u];
          }
        }
      }
    }
    __syncthreads();                                       // every thread's stores precede the flags
    if (threadIdx.x == 0) {
      __threadfence_system();
      for (int d = 1; d < comm.world; ++d) {
        int q = comm.rank + d;
        if (q >= comm.world) q -= comm.world;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<unsigned*>(
                                                                      reinterpret_cast<char*>(comm.bufs[q]) + comm.flag_off) +
                                                                  AG_FLAG_BASE + tm),
                     "r"(comm.epoch)
                     : "memory");
      }
    }
  }
}

// PAIR: the grid is launched as clusters of two CTAs and n_gemm is even; CTAs 2i and 2i + 1 below
// n_gemm work as a pair (see gemm_cta), the communication CTAs are unaffected.
template <int BN, int MODE, bool PAIR = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fused_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmAown, const GemmArgs args, const CommArgs comm_in,
                  const int n_gemm) {
  CommArgs comm = comm_in;
  comm.epoch += *reinterpret_cast<const volatile unsigned*>(comm_in.ctr + 1);
  comm.done_target += *reinterpret_cast<const volatile unsigned*>(comm_in.ctr + 2);
  const bool is_gemm = (int)blockIdx.x < n_gemm;
  if (is_gemm) {
    if (!gemm_cta<BN, MODE, PAIR>(&tmA, &tmB, args, comm, PAIR ? blockIdx.x >> 1 : blockIdx.x,
                                  PAIR ? n_gemm >> 1 : n_gemm, &tmAown))
      return;
  } else {
    __shared__ int s_abort2;
    if (threadIdx.x == 0) s_abort2 = *reinterpret_cast<volatile int*>(args.status);
    __syncthreads();
    if (s_abort2 != 0) return;
  }
  if (MODE == MODE_AG) {
    if (is_gemm) return;                      // GEMM CTAs touch no peer memory
    if (comm.abufs != nullptr) {
      // push: nobody reads this rank's memory, and the GEMM has waited for every block that was
      // pushed to it, so no closing barrier is needed
      push_jobs<BN>(args, comm, (int)blockIdx.x - n_gemm, (int)gridDim.x - n_gemm);
      return;
    }
    gather_jobs<BN>(args, comm, (int)blockIdx.x - n_gemm, (int)gridDim.x - n_gemm);
  } else if (MODE == MODE_AR) {
    reduce_jobs<BN, MODE>(args, comm);
  }
  // MODE_RS: the tiles were pushed by the epilogue; once every CTA of every rank has counted,
  // all partial sums of this rank's rows are in its workspace and rs_reduce_kernel adds them up
  closing_count(args, comm);
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

// bit 0: CTA pairs for 256-wide tiles of plain GEMMs with at least one tile pair per two SMs;
// bit 1: CTA pairs in the fused GEMM + collective kernels (even number of 128-row tiles). 0: lone CTAs only
static int g_pair_mode = 0;
static int g_pair_max_clusters = -1;   // co-resident clusters of the pair kernel (set at its first launch)

template <int BN>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, int max_ctas,
                       cudaStream_t stream) {
  using L = SmemLayoutPair<BN>;
  int& max_clusters = g_pair_max_clusters;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_clusters < 0) {
    if (cudaFuncSetAttribute(gemm_bf16_tcgen05_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::TOTAL) != cudaSuccess)
      return -2;
    cfg.gridDim = dim3(2 * (g_num_sms / 2));
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_tcgen05_pair_kernel<BN>, &cfg) != cudaSuccess || n < 1) return -2;
    max_clusters = n;
  }
  const int num_m = (a.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M), num_n = (a.N + BN - 1) / BN;
  long long tiles = (long long)num_m * num_n * a.batch;
  int pairs = max_clusters < max_ctas / 2 ? max_clusters : max_ctas / 2;
  if (tiles < pairs) pairs = (int)tiles;
  if (pairs < 1) return 0;
  cfg.gridDim = dim3(2 * pairs);
  return cudaLaunchKernelEx(&cfg, gemm_bf16_tcgen05_pair_kernel<BN>, ta, tb, a) == cudaSuccess ? 0 : -3;
}

}  // namespace nb

// CTA pairs: bit 0 plain GEMM, bit 1 fused GEMM + collective kernels. Returns the previous setting.
extern "C" int nb_gemm_set_pair_mode(int mode) {
  const int old = nb::g_pair_mode;
  nb::g_pair_mode = mode;
  return old;
}

// Co-resident clusters of the pair kernel on this device (-1 before its first launch).
extern "C" int nb_gemm_pair_max_clusters() { return nb::g_pair_max_clusters; }

// Runs pair_alloc_probe_kernel on one cluster; out2 = device unsigned[2] (tensor-memory base of CTA 0, 1).
extern "C" int nb_gemm_pair_alloc_probe(unsigned* out2, void* stream) {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(2);
  cfg.blockDim = dim3(32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = reinterpret_cast<cudaStream_t>(stream);
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, nb::pair_alloc_probe_kernel, out2) == cudaSuccess ? 0 : -3;
}

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
  // CTA pairs: wide tiles of problems with enough 256 x 256 tiles to give every pair of SMs one
  const bool pair = (g_pair_mode & 1) && bn == 256 && M >= 2 * BLOCK_M &&
                    (long long)((M + 2 * BLOCK_M - 1) / (2 * BLOCK_M)) * ((N + 255) / 256) * batch >= g_num_sms / 2;
  if (!b_mn) r = make_map(&tb, B, K, N, batch, ldb, stride_b, pair ? bn / 2 : bn);
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
  bool vec32 = vec && ((reinterpret_cast<uintptr_t>(C) & 31) == 0) && ((ldc * oes) % 32 == 0) &&
               (batch == 1 || (stride_c * oes) % 32 == 0);
  if (aux == AUX_STORE_PREACT)
    vec32 = vec32 && ((reinterpret_cast<uintptr_t>(aux_out) & 31) == 0) && ((ld_aux * 2) % 32 == 0) &&
            (batch == 1 || (stride_aux * 2) % 32 == 0);
  g.vec32_ok = vec32 ? 1 : 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (pair) return launch_pair<256>(ta, tb, g, max_ctas, s);
  if (bn == 256) return launch<256>(ta, tb, g, max_ctas, s);
  if (bn == 128) return launch<128>(ta, tb, g, max_ctas, s);
  return launch<64>(ta, tb, g, max_ctas, s);
}

// Fused GEMM + collective over a symmetric workspace (one launch; see FusedMode).
//   mode          1 all-reduce, 2 reduce-scatter, 3 all-gather
//   ws_local      this rank's workspace base;  ws_bufs  device array [world] of all ranks' bases
//   mc            multicast base of the workspace or null (plain peer loads/stores)
//   data_off      byte offset in the workspace of C (modes 1, 2) or of the staged A shard (mode 3)
//   out           mode 2: this rank's rows [M/world][N];  mode 3: C [M][N] (ldc = N);  mode 1: unused
//   bias, aux_out mode 2: optional bias[N] (bf16) and residual [M/world][N] added while the partial
//                 sums are folded;  mode 3: GEMM epilogue bias and stored pre-activation
//   a_full        mode 3: the gathered A [M][K] (dense, regular device memory); A = this rank's own rows
//                 [M / world][K], dense (the same data that was staged at data_off for the peers)
//   chunk_rows    modes 2, 3: rows per contiguous chunk of a rank (multiple of 128, M % (world*chunk_rows) == 0)
//   arena_bufs    mode 3, push variant: device array [world] of the base pointers of a symmetric arena
//                 in which a_full sits at byte offset a_off on EVERY rank (null: pull variant)
//   ctr           device counters of the workspace (unsigned[4], zero at creation): the kernel
//                 takes its all-gather epoch and done target relative to them and a one-thread
//                 kernel advances them afterwards, so replaying the launches from a CUDA graph works
//   ticket        device int used as job counter (zeroed here on `stream`); nullptr = fixed job order
// Returns 0, or a negative code when the shape does not fit (the caller then runs the unfused path).
extern "C" int nb_gemm_fused_grid() {
  if (nb::g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&nb::g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return nb::g_num_sms;
}

// Sum of the `world` partial row blocks that the peers pushed into this rank's workspace
// ([world][rows][N] bf16), plus optional bias[N] and residual[rows][N]: out = sum_s part[s] + bias + res.
__global__ void __launch_bounds__(256) rs_reduce_kernel(const __nv_bfloat16* __restrict__ parts, int world,
                                                        long long n_vec, int n_cols_vec, long long slot_vec,
                                                        const __nv_bfloat16* __restrict__ bias,
                                                        const __nv_bfloat16* __restrict__ residual,
                                                        __nv_bfloat16* __restrict__ out) {
  const uint4* pv = reinterpret_cast<const uint4*>(parts);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < world; ++s) {
      const uint4 v = pv[s * slot_vec + i];
      const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
      }
    }
    if (bias != nullptr) {
      const uint4 v = reinterpret_cast<const uint4*>(bias)[i % n_cols_vec];
      const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
      }
    }
    if (residual != nullptr) {
      const uint4 v = reinterpret_cast<const uint4*>(residual)[i];
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
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

__global__ void bump_fused_kernel(unsigned* ctr, unsigned add_epoch, unsigned add_done) {
  ctr[1] += add_epoch;
  ctr[2] += add_done;
}

template <int MODE>
static int launch_fused(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ta_own, const nb::GemmArgs& g,
                        const nb::CommArgs& c, int grid, int n_gemm, cudaStream_t s) {
  using namespace nb;
  constexpr int BN = 256;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_fused_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SmemLayout<BN>::TOTAL) != cudaSuccess)
      return -2;
    configured = true;
  }
  gemm_fused_kernel<BN, MODE><<<grid, NUM_THREADS, SmemLayout<BN>::TOTAL, s>>>(ta, tb, ta_own, g, c, n_gemm);
  bump_fused_kernel<<<1, 1, 0, s>>>(const_cast<unsigned*>(c.ctr), MODE == nb::MODE_AG ? 1u : 0u, c.done_target);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// The same launch with the GEMM CTAs working as pairs (grid and n_gemm even; B's tensor map has a box
// of BN / 2 rows).
template <int MODE>
static int launch_fused_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ta_own,
                             const nb::GemmArgs& g, const nb::CommArgs& c, int grid, int n_gemm, cudaStream_t s) {
  using namespace nb;
  constexpr int BN = 256;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_fused_kernel<BN, MODE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SmemLayoutPair<BN>::TOTAL) != cudaSuccess)
      return -2;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SmemLayoutPair<BN>::TOTAL;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm_fused_kernel<BN, MODE, true>, ta, tb, ta_own, g, c, n_gemm) != cudaSuccess) return -3;
  bump_fused_kernel<<<1, 1, 0, s>>>(const_cast<unsigned*>(c.ctr), MODE == nb::MODE_AG ? 1u : 0u, c.done_target);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int nb_gemm_fused_bf16(int mode, const void* A, const void* B, void* out, const void* bias, void* aux_out,
                                  void* a_full, void* ws_local, void* const* ws_bufs, void* mc, long long data_off,
                                  int flag_off, int done_off, int M, int N, int K, long long lda, long long ldb,
                                  int a_mn, int b_mn, int bias_fp32, int epi, int aux, int gelu_tanh, int rank,
                                  int world, int chunk_rows, unsigned* ctr, int n_comm_ctas, int* ticket, int* status,
                                  void* const* arena_bufs, long long a_off, void* arena_mc, void* stream) {
  using namespace nb;
  constexpr int BN = 256;
  if (mode < MODE_AR || mode > MODE_AG) return -9;
  if (M <= 0 || N <= 0 || K <= 0) return -10;
  const void* Aop = mode == MODE_AG ? a_full : A;
  if ((reinterpret_cast<uintptr_t>(Aop) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (data_off & 15)) return -11;
  if (mode == MODE_AG) { lda = K; a_mn = 0; }
  if ((lda & 7) || (ldb & 7) || (N & 7) || (K & 7)) return -12;
  const int num_m = (M + BLOCK_M - 1) / BLOCK_M, num_n = (N + BN - 1) / BN;
  if (mode != MODE_AG && (long long)num_m * num_n > AG_FLAG_BASE) return -13;   // tile-flag region
  if (mode == MODE_AG && num_m > 2048) return -13;
  int mpc = 1, per = num_m;
  if (mode != MODE_AR) {
    if (chunk_rows <= 0 || (chunk_rows % BLOCK_M) || (M % (world * chunk_rows))) return -14;
    mpc = chunk_rows / BLOCK_M;
    per = num_m / world;
  }
  const int grid = nb_gemm_fused_grid();      // every rank must launch the same grid
  if (n_comm_ctas < 1) n_comm_ctas = 1;
  if (n_comm_ctas > grid / 2) n_comm_ctas = grid / 2;
  if (mode == MODE_RS) n_comm_ctas = 0;        // the epilogue pushes the tiles; no communication CTAs
  // CTA pairs: clusters of two, so the GEMM CTAs and the whole grid come in even numbers (the same
  // rule on every rank)
  const bool pair = (g_pair_mode & 2) && (num_m % 2 == 0) && (grid % 2 == 0) && grid >= 4;
  if (pair && (n_comm_ctas & 1)) n_comm_ctas += 1;
  const int n_gemm = grid - n_comm_ctas;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_map(&ta, Aop, K, M, 1, lda, 0, BLOCK_M);
  else       r = make_map(&ta, Aop, M, K, 1, lda, 0, BLOCK_K);
  if (r) return r;
  if (!b_mn) r = make_map(&tb, B, K, N, 1, ldb, 0, pair ? BN / 2 : BN);
  else       r = make_map(&tb, B, N, K, 1, ldb, 0, BLOCK_K);
  if (r) return r;
  GemmArgs g{};
  g.M = M; g.N = N; g.K = K; g.batch = 1;
  g.ldc = N; g.stride_c = (long long)M * N;
  g.a_mn = a_mn; g.b_mn = b_mn; g.out_fp32 = 0; g.accumulate = 0;
  g.alpha = 1.0f; g.status = status; g.vec_ok = 1;
  g.vec32_ok = 0;   // set below for the mode whose epilogue stores to ordinary memory
  if (mode == MODE_AG) {
    if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(aux_out) & 15)) return -11;
    g.out = out; g.bias = bias; g.bias_fp32 = bias_fp32; g.epi = epi; g.gelu_tanh = gelu_tanh;
    // aux 1: aux_out receives the pre-activation; aux 2 / 3: aux_out holds z and the result is
    // multiplied by relu'(z) / gelu'(z) (activation backward fused into the epilogue)
    g.aux = (aux == AUX_STORE_PREACT || aux == AUX_MUL_DRELU || aux == AUX_MUL_DGELU) ? aux : AUX_NONE;
    g.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out);
    g.aux_in = reinterpret_cast<const __nv_bfloat16*>(aux_out);
    g.ld_aux = N; g.stride_aux = (long long)M * N;
    g.vec32_ok = (((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(aux_out)) & 31) == 0 && (N % 16) == 0) ? 1 : 0;
  } else {
    g.out = reinterpret_cast<char*>(ws_local) + data_off;
    g.epi = EPI_NONE; g.aux = AUX_NONE;
  }
  CommArgs c{};
  c.bufs = ws_bufs; c.mc = reinterpret_cast<char*>(mc); c.data_off = data_off;
  c.flag_off = flag_off; c.done_off = done_off; c.rank = rank; c.world = world;
  c.tile_target = (unsigned)world;
  c.done_target = (unsigned)world * (unsigned)(mode == MODE_AG ? n_comm_ctas : grid);   // + ctr[2] on the device
  c.ticket = ticket;
  c.mpc = mpc; c.per = per; c.epoch = 1u; c.ctr = ctr;
  c.rs_out = reinterpret_cast<__nv_bfloat16*>(out);
  c.a_full = reinterpret_cast<char*>(a_full);
  c.unit_bytes = (long long)BLOCK_M * K * 2;
  c.abufs = mode == MODE_AG ? arena_bufs : nullptr;
  c.a_off = a_off;
  c.a_mc = (mode == MODE_AG && arena_bufs != nullptr) ? reinterpret_cast<char*>(arena_mc) : nullptr;
  c.own_src = reinterpret_cast<const char*>(A);
  if (mode == MODE_AG && arena_bufs != nullptr) c.done_target = 0;   // push: no closing barrier, nothing counted
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (mode != MODE_AG && ticket != nullptr && cudaMemsetAsync(ticket, 0, sizeof(int), s) != cudaSuccess) return -4;
  if (mode == MODE_AR)
    return pair ? launch_fused_pair<MODE_AR>(ta, tb, ta, g, c, grid, n_gemm, s)
                : launch_fused<MODE_AR>(ta, tb, ta, g, c, grid, n_gemm, s);
  if (mode == MODE_RS) {
    r = pair ? launch_fused_pair<MODE_RS>(ta, tb, ta, g, c, grid, n_gemm, s)
             : launch_fused<MODE_RS>(ta, tb, ta, g, c, grid, n_gemm, s);
    if (r) return r;
    const long long rows = M / world;
    const long long n_vec = rows * N / 8;
    const int blocks = (int)((n_vec + 255) / 256 < 148 * 8 ? (n_vec + 255) / 256 : 148 * 8);
    rs_reduce_kernel<<<blocks, 256, 0, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<char*>(ws_local) + data_off), world, n_vec, N / 8, n_vec,
        reinterpret_cast<const __nv_bfloat16*>(bias), reinterpret_cast<const __nv_bfloat16*>(aux_out),
        reinterpret_cast<__nv_bfloat16*>(out));
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  }
  // mode 3: A = this rank's own rows (dense [M / world][K]); the GEMM reads them in place
  CUtensorMap ta_own;
  if ((reinterpret_cast<uintptr_t>(A) & 15)) return -11;
  r = make_map(&ta_own, A, K, M / world, 1, K, 0, BLOCK_M);
  if (r) return r;
  return pair ? launch_fused_pair<MODE_AG>(ta, tb, ta_own, g, c, grid, n_gemm, s)
              : launch_fused<MODE_AG>(ta, tb, ta_own, g, c, grid, n_gemm, s);
}

NB_DEBUG_DEFINE(gemm)
