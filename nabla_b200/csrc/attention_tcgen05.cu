// Flash attention for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
//   O = softmax(Q K^T * scale [+ causal mask]) V        per (batch, head), never materialising
//                                                       the (seq_q, seq_k) score matrix
//
// Replaces the reference's composed attention (matmul, mul, tril, where, softmax, matmul:
// nabla/nn/functional/layers.py:106-153), whose memory is O(seq^2).
//
// Forward: one CTA per (batch, head, 128 query rows), 256 threads:
//   warp 0     TMA producer: Q once, K/V tiles (128 keys) into a 2-stage ring (4-D tensor maps
//              over strided (B, H, S, D) views, so packed qkv projections are read in place)
//   warp 1     MMA issuer: S_j = Q K_j^T into one of two TMEM score buffers, O += P_j V_j
//   warp 2     TMEM allocator
//   warps 4-7  softmax: thread r owns query row r (TMEM lane r): scale, mask, online max/sum in
//              the log2 domain, P (bf16) to swizzled smem as the A operand of the second MMA,
//              lazy rescaling of the O accumulator in TMEM, final normalisation and store
// S is double buffered so the tensor core computes S_{j+1} while the softmax works on S_j.
//
// Backward: see attn_bwd_* below (dK/dV per key tile with tensor-core GEMMs for S^T, dP^T,
// dV, dK and dQ; dQ accumulated with fp32 reductions).
#include "sm100_ptx.cuh"

namespace nba {
using namespace nb;

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int NTHREADS = 256;

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}

struct FwdArgs {
  int B, H, Sq, Skv;
  float scale_log2;   // softmax scale * log2(e)
  int causal;
  __nv_bfloat16* O;
  long long o_sb, o_sh, o_ss;   // element strides of O for batch, head, row
  float* lse;                   // [B][H][Sq]
  int* status;
};

template <int HD>
struct FwdSmem {
  static constexpr int Q_BYTES = BM * HD * 2;
  static constexpr int KV_BYTES = BN * HD * 2;
  static constexpr int P_BYTES = BM * BN * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int RAW = OFF_BAR + 16 * 8 + 16 + 1024;
  static constexpr int TOTAL = RAW < 120 * 1024 ? 120 * 1024 : RAW;   // keep one CTA per SM (TMEM)
};

template <int HD>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FwdArgs args) {
  using L = FwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sP = smem + L::OFF_P;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* p_full = bars + 7;
  uint64_t* pv_done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    __shared__ int s_abort;   // an earlier bounded wait on this device already failed: leave (uniformly)
    if (threadIdx.x == 0) s_abort = *reinterpret_cast<volatile int*>(args.status);
    __syncthreads();
    if (s_abort != 0) return;
  }
  const int nqt = (args.Sq + BM - 1) / BM;
  int bid = blockIdx.x;
  const int qt = nqt - 1 - (bid % nqt);   // heavy (late) causal tiles first
  bid /= nqt;
  const int h = bid % args.H;
  const int b = bid / args.H;
  const int q0 = qt * BM;
  const int off = args.Skv - args.Sq;     // causal: row i sees keys <= i + off
  int n_tiles = (args.Skv + BN - 1) / BN;
  if (args.causal) {
    const int last_key = min(args.Skv - 1, q0 + BM - 1 + off);
    n_tiles = last_key < 0 ? 0 : last_key / BN + 1;
  }

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_arrive_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) tma_load_4d(sQ + c * (BM * 128), &tmQ, q_full, c * 64, q0, h, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1)) {
          atomicExch(args.status, NB_ERR_TIMEOUT_PRODUCER);
          break;
        }
        mbar_arrive_expect_tx(&kv_full[st], 2 * L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          tma_load_4d(sK + st * L::KV_BYTES + c * (BN * 128), &tmK, &kv_full[st], c * 64, j * BN, h, b);
          tma_load_4d(sV + st * L::KV_BYTES + c * (BN * 128), &tmV, &kv_full[st], c * 64, j * BN, h, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_qk = make_idesc_bf16(BM, BN, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(BM, HD, 0, 1);
      bool ok = mbar_wait(q_full, 0);
      auto issue_qk = [&](int j) {
        const int st = j & 1;
        const uint32_t a0 = smem_u32(sQ), b0 = smem_u32(sK + st * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(a0 + (k >> 2) * (BM * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(b0 + (k >> 2) * (BN * 128) + (k & 3) * 32, 16, 1024);
          umma_f16_ss(tmem_base + (j & 1) * BN, da, db, idesc_qk, k != 0);
        }
        umma_commit(&s_full[j & 1]);
      };
      auto issue_pv = [&](int j) {
        const int st = j & 1;
        const uint32_t a0 = smem_u32(sP), b0 = smem_u32(sV + st * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(a0 + (k >> 2) * (BM * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(b0 + k * (16 * 128), BN * 128, 1024);
          umma_f16_ss(tmem_o, da, db, idesc_pv, (j | k) != 0);
        }
        umma_commit(&kv_empty[st]);   // K_j / V_j slot reusable once these MMAs retire
        umma_commit(pv_done);
      };
      if (!ok) atomicExch(args.status, NB_ERR_TIMEOUT_MMA);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (!mbar_wait(&kv_full[j & 1], (j >> 1) & 1)) { ok = false; break; }
        tc_fence_after();
        issue_qk(j);
        if (j > 0) {
          if (!mbar_wait(p_full, (j - 1) & 1)) { ok = false; break; }
          tc_fence_after();
          issue_pv(j - 1);
        }
      }
      if (ok) {
        if (mbar_wait(p_full, (n_tiles - 1) & 1)) {
          tc_fence_after();
          issue_pv(n_tiles - 1);
        } else {
          ok = false;
        }
      }
      if (!ok) atomicExch(args.status, NB_ERR_TIMEOUT_MMA);
    }
  } else if (warp >= 4) {
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int q_idx = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      if (ok && !mbar_wait(&s_full[sb], (j >> 1) & 1)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float s[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + sb * BN + lane_addr + c * 32, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(v[i]);
      }
      tmem_ld_wait();
      const int kv0 = j * BN;
      const bool need_mask = (kv0 + BN > args.Skv) || (args.causal && (kv0 + BN - 1 > q0 + off));
      float mx = -INFINITY;
      if (need_mask) {
        const int lim = args.causal ? min(args.Skv - 1, q_idx + off) : args.Skv - 1;
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          const float x = (kv0 + c <= lim) ? s[c] * args.scale_log2 : -INFINITY;
          s[c] = x;
          mx = fmaxf(mx, x);
        }
      } else {
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          s[c] *= args.scale_log2;
          mx = fmaxf(mx, s[c]);
        }
      }
      // lazy rescale: keep the old reference maximum unless the new one exceeds it by 2^8
      float alpha = 1.f;
      bool resc = false;
      if (j == 0) {
        m_used = (mx == -INFINITY) ? 0.f : mx;
      } else if (mx > m_used + 8.f) {
        alpha = exp2f(m_used - mx);
        m_used = mx;
        resc = true;
      }
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < BN; ++c) {
        s[c] = exp2f(s[c] - m_used);
        sum += s[c];
      }
      l = l * alpha + sum;
      if (j > 0) {
        if (!mbar_wait(pv_done, (j - 1) & 1)) {
          atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
          ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, resc)) {
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_o + lane_addr + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(tmem_o + lane_addr + c * 32, v);
          }
          tmem_st_wait();
        }
      }
      // P (bf16) into the K-major SWIZZLE_128B layout the second MMA reads
#pragma unroll
      for (int cc = 0; cc < BN / 64; ++cc) {
        uint8_t* rowp = sP + cc * (BM * 128) + r * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          uint4 pk;
          uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(s[cc * 64 + u * 8 + 2 * e], s[cc * 64 + u * 8 + 2 * e + 1]);
            pw[e] = *reinterpret_cast<uint32_t*>(&hh);
          }
          *reinterpret_cast<uint4*>(rowp + ((u ^ (r & 7)) << 4)) = pk;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok && n_tiles > 0) {
      if (!mbar_wait(pv_done, (n_tiles - 1) & 1)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = (n_tiles > 0 && l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = args.O + (long long)b * args.o_sb + (long long)h * args.o_sh + (long long)q_idx * args.o_ss;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(tmem_o + lane_addr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (q_idx < args.Sq) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 pk;
            uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 2 * e]) * inv,
                                                        __uint_as_float(v[u * 8 + 2 * e + 1]) * inv);
              pw[e] = *reinterpret_cast<uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = pk;
          }
        }
      }
      if (q_idx < args.Sq)
        args.lse[((long long)b * args.H + h) * args.Sq + q_idx] =
            (n_tiles > 0 && l > 0.f) ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ====================================================================== backward
// One CTA per (batch, head, 128 keys). K_j and V_j stay in shared memory; the CTA walks over the
// query tiles (64 rows) that see these keys. Per query tile, on the tensor cores:
//   S^T  = K_j Q_i^T            (128 x 64, TMEM)       dP^T = V_j dO_i^T        (128 x 64, TMEM)
//   P^T  = exp2(S^T * c - lse_i),  dS^T = P^T * (dP^T - delta_i) * scale      (softmax warps,
//          thread = key row; both written as bf16 A operands into swizzled smem)
//   dV  += P^T dO_i   dK += dS^T Q_i   (128 x 128 accumulators in TMEM for the whole loop)
//   dQ_i^T = K_j^T dS^T (128 x 64)  -> fp32 vector reductions into a [B][H][D][Sq_pad] scratch
// Two small kernels bracket it: delta_i = rowsum(dO_i * O_i), and the conversion of the dQ
// scratch (transposed, fp32) to the caller's bf16 layout.
//
// Two query tiles are in flight: math group 0 (warps 4-7) owns the even tiles, group 1 (warps
// 8-11) the odd ones, each with its own S^T / dP^T columns in TMEM and its own P^T / dS^T buffers
// in shared memory, so the tensor pipe works on one tile's five MMAs while the other tile's
// exponentials and dS are computed. dQ_i^T is written over tile i's dP^T columns (which the math
// threads have consumed by then): 2 x (64 + 64) + 128 + 128 = 512 TMEM columns.
constexpr int BQ = 64;
constexpr int BWD_THREADS = 384;

struct BwdArgs {
  int B, H, Sq, Skv, Sq_pad;
  float scale, scale_log2;
  int causal;
  const float* lse;     // [B][H][Sq] natural log
  const float* delta;   // [B][H][Sq]
  float* dq_acc;        // [B][H][128][Sq_pad]
  __nv_bfloat16 *dK, *dV;
  long long dk_sb, dk_sh, dk_ss, dv_sb, dv_sh, dv_ss;
  int* status;
};

struct BwdSmem {
  static constexpr int HD = 128;
  static constexpr int KV_BYTES = BN * HD * 2;        // 32 KB
  static constexpr int QT_BYTES = BQ * HD * 2;        // 16 KB
  static constexpr int XY_BYTES = BN * BQ * 2;        // 16 KB
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + KV_BYTES;
  static constexpr int OFF_Q = OFF_V + KV_BYTES;      // 2 stages
  static constexpr int OFF_DO = OFF_Q + 2 * QT_BYTES;
  static constexpr int OFF_X = OFF_DO + 2 * QT_BYTES;  // 2 buffers (one per math group)
  static constexpr int OFF_Y = OFF_X + 2 * XY_BYTES;   // 2 buffers
  static constexpr int OFF_STAT = OFF_Y + 2 * XY_BYTES;   // lse2[2][64], delta[2][64]
  static constexpr int OFF_BAR = OFF_STAT + 4 * BQ * 4;
  static constexpr int TOTAL = OFF_BAR + 24 * 8 + 16 + 1024;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const BwdArgs args) {
  using L = BwdSmem;
  constexpr int HD = 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sDO = smem + L::OFF_DO;
  uint8_t* sX = smem + L::OFF_X;
  uint8_t* sY = smem + L::OFF_Y;
  float* s_lse2 = reinterpret_cast<float*>(smem + L::OFF_STAT);   // [2][64]
  float* s_delta = s_lse2 + 2 * BQ;                               // [2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;    // [2]  Q_i / dO_i landed in stage i & 1
  uint64_t* qdo_empty = bars + 3;   // [2]  the MMAs that read the stage have retired
  uint64_t* sdp_full = bars + 5;    // [2]  S^T and dP^T of the group's tile are in TMEM
  uint64_t* xy_full = bars + 7;     // [2]  P^T and dS^T of the group's tile are in shared memory (128 arrivals)
  uint64_t* g2_done = bars + 9;     // [2]  dV / dK / dQ^T MMAs of the group's tile have retired
  uint64_t* dq_free = bars + 11;    // [2]  dQ^T of the group's tile has been drained (128 arrivals)
  uint64_t* all_done = bars + 13;   //      every MMA of the CTA has retired
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    __shared__ int s_abort;   // an earlier bounded wait on this device already failed: leave (uniformly)
    if (threadIdx.x == 0) s_abort = *reinterpret_cast<volatile int*>(args.status);
    __syncthreads();
    if (s_abort != 0) return;
  }
  const int nkt = (args.Skv + BN - 1) / BN;
  // key tile 0 sees every query tile, the last one only a few: tile index slowest, so that the
  // long CTAs start first and the short ones fill the end of the grid
  int bid = blockIdx.x;
  const int bh = args.H * args.B;
  const int jt = bid / bh;
  bid -= jt * bh;
  const int h = bid % args.H;
  const int b = bid / args.H;
  const int k0 = jt * BN;
  const int off = args.Skv - args.Sq;
  const int nqt = (args.Sq + BQ - 1) / BQ;
  int i_start = 0;
  if (args.causal) {
    const int first_q = k0 - off;             // first query row that sees key k0
    i_start = first_q <= 0 ? 0 : first_q / BQ;
  }
  const int n_it = max(0, nqt - i_start);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
      mbar_init(&xy_full[i], 128);
      mbar_init(&g2_done[i], 1);
      mbar_init(&dq_free[i], 128);
    }
    mbar_init(all_done, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_dv = tmem_base + 256, t_dk = tmem_base + 384;
  // group g: S^T at columns g*128 .. +63, dP^T (later dQ^T) at g*128 + 64 .. +127

  if (warp == 0) {
    if (lane == 0 && n_it > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * L::KV_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_4d(sK + c * (BN * 128), &tmK, kv_full, c * 64, k0, h, b);
        tma_load_4d(sV + c * (BN * 128), &tmV, kv_full, c * 64, k0, h, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1;
        if (!mbar_wait(&qdo_empty[st], ((it >> 1) & 1) ^ 1)) {
          atomicExch(args.status, NB_ERR_TIMEOUT_PRODUCER);
          break;
        }
        mbar_arrive_expect_tx(&qdo_full[st], 2 * L::QT_BYTES);
        const int q0 = (i_start + it) * BQ;
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          tma_load_4d(sQ + st * L::QT_BYTES + c * (BQ * 128), &tmQ, &qdo_full[st], c * 64, q0, h, b);
          tma_load_4d(sDO + st * L::QT_BYTES + c * (BQ * 128), &tmDO, &qdo_full[st], c * 64, q0, h, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      const uint32_t id_g1 = make_idesc_bf16(128, BQ, 0, 0);    // S^T, dP^T : A K-major, B K-major
      const uint32_t id_g2 = make_idesc_bf16(128, HD, 0, 1);    // dV, dK    : A K-major, B MN-major
      const uint32_t id_dq = make_idesc_bf16(128, BQ, 1, 1);    // dQ^T      : A MN-major, B MN-major
      // Descriptors are built once; inside the loops an operand advances by adding a constant to
      // the descriptor's start-address field (16-byte units), so the issuing thread spends a few
      // instructions per MMA and keeps ahead of the tensor pipe (the MMAs are only 128 x 64 x 16).
      const uint64_t dK_k = make_smem_desc_sw128(smem_u32(sK), 16, 1024);            // K as K-major A
      const uint64_t dV_k = make_smem_desc_sw128(smem_u32(sV), 16, 1024);
      const uint64_t dK_mn = make_smem_desc_sw128(smem_u32(sK), BN * 128, 1024);     // K as MN-major A (dQ^T)
      // stage / group 1 operands sit a fixed distance after stage / group 0: one add selects them
      const uint64_t dQ_k0 = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t dDO_k0 = make_smem_desc_sw128(smem_u32(sDO), 16, 1024);
      const uint64_t dQ_mn0 = make_smem_desc_sw128(smem_u32(sQ), BQ * 128, 1024);
      const uint64_t dDO_mn0 = make_smem_desc_sw128(smem_u32(sDO), BQ * 128, 1024);
      const uint64_t dX0 = make_smem_desc_sw128(smem_u32(sX), 16, 1024);
      const uint64_t dY_k0 = make_smem_desc_sw128(smem_u32(sY), 16, 1024);
      const uint64_t dY_mn0 = make_smem_desc_sw128(smem_u32(sY), BN * 128, 1024);
      auto g1 = [&](int it) {       // S^T and dP^T of tile `it` into its group's columns
        const int g = it & 1;
        const uint32_t t_s = tmem_base + g * 128, t_dp = t_s + 64;
        const uint64_t bq = dQ_k0 + (uint64_t)(g * (L::QT_BYTES >> 4)), bdo = dDO_k0 + (uint64_t)(g * (L::QT_BYTES >> 4));
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t ko = (uint64_t)(((k >> 2) * (BN * 128) + (k & 3) * 32) >> 4);     // K/V chunk + in-row offset
          const uint64_t qo = (uint64_t)(((k >> 2) * (BQ * 128) + (k & 3) * 32) >> 4);
          umma_f16_ss(t_s, dK_k + ko, bq + qo, id_g1, k != 0);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t ko = (uint64_t)(((k >> 2) * (BN * 128) + (k & 3) * 32) >> 4);
          const uint64_t qo = (uint64_t)(((k >> 2) * (BQ * 128) + (k & 3) * 32) >> 4);
          umma_f16_ss(t_dp, dV_k + ko, bdo + qo, id_g1, k != 0);
        }
        umma_commit(&sdp_full[g]);
      };
      bool ok = mbar_wait(kv_full, 0);
      for (int t = 0; t < 2 && t < n_it && ok; ++t) {
        ok = mbar_wait(&qdo_full[t], 0);
        if (ok) {
          tc_fence_after();
          g1(t);
        }
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int g = it & 1;
        if (!mbar_wait(&xy_full[g], (it >> 1) & 1)) { ok = false; break; }
        tc_fence_after();
        const uint64_t gq = (uint64_t)(g * (L::QT_BYTES >> 4)), gx = (uint64_t)(g * (L::XY_BYTES >> 4));
        const uint64_t dXg = dX0 + gx, dYkg = dY_k0 + gx, dYmng = dY_mn0 + gx;
        const uint64_t dQmng = dQ_mn0 + gq, dDOmng = dDO_mn0 + gq;
        // dV += P^T dO_i ; dK += dS^T Q_i   (K = 64 query rows -> 4 k-steps)
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)
          umma_f16_ss(t_dv, dXg + (uint64_t)((k * 32) >> 4), dDOmng + (uint64_t)((k * 16 * 128) >> 4), id_g2,
                      (it | k) != 0);
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)
          umma_f16_ss(t_dk, dYkg + (uint64_t)((k * 32) >> 4), dQmng + (uint64_t)((k * 16 * 128) >> 4), id_g2,
                      (it | k) != 0);
        // dQ_i^T = K_j^T dS^T : M = head dim, N = 64 queries, K = 128 keys; over the tile's dP^T columns
        const uint32_t t_dq = tmem_base + g * 128 + 64;
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)
          umma_f16_ss(t_dq, dK_mn + (uint64_t)((k * 16 * 128) >> 4), dYmng + (uint64_t)((k * 16 * 128) >> 4), id_dq,
                      k != 0);
        umma_commit(&qdo_empty[g]);
        umma_commit(&g2_done[g]);
        if (it >= 1 && it + 1 < n_it) {
          // tile it + 1 belongs to the other group: its columns are free once dQ of tile it - 1 is drained
          const int o = g ^ 1;
          if (!mbar_wait(&dq_free[o], ((it - 1) >> 1) & 1)) { ok = false; break; }
          if (!mbar_wait(&qdo_full[o], ((it + 1) >> 1) & 1)) { ok = false; break; }
          tc_fence_after();
          g1(it + 1);
        }
      }
      if (ok) umma_commit(all_done);
      else atomicExch(args.status, NB_ERR_TIMEOUT_MMA);
    }
  } else if (warp >= 4) {
    const int grp = (warp - 4) >> 2;        // math group: 0 = even query tiles, 1 = odd ones
    const int wq = warp & 3;                // TMEM lane quarter this warp may read
    const int r = wq * 32 + lane;           // key row inside the tile / head-dim row for dQ^T
    const int et = (threadIdx.x - 128) & 127;
    const int key = k0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t t_s = tmem_base + grp * 128, t_dp = t_s + 64;
    const long long bh = (long long)b * args.H + h;
    uint8_t* xr = sX + grp * L::XY_BYTES + r * 128;
    uint8_t* yr = sY + grp * L::XY_BYTES + r * 128;
    const bool key_ok = key < args.Skv;
    bool ok = true;
    for (int it = grp; it < n_it; it += 2) {
      const int q0 = (i_start + it) * BQ;
      const uint32_t ph = (it >> 1) & 1;
      // stage the per-query statistics of this tile (the group's previous tile is fully consumed)
      {
        const int qi = q0 + (et & 63);
        const bool inr = qi < args.Sq;
        if (et < 64) s_lse2[grp * BQ + et] = inr ? args.lse[bh * args.Sq + qi] * 1.4426950408889634f : INFINITY;
        else s_delta[grp * BQ + (et - 64)] = inr ? args.delta[bh * args.Sq + qi] : 0.f;
      }
      named_bar_sync(1 + grp, 128);
      if (ok && !mbar_wait(&sdp_full[grp], ph)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = args.causal && (k0 + BN - 1 > q0 + off);
      // the MMAs that read this group's P^T / dS^T buffers belong to its previous tile; their
      // retirement was awaited before that tile's dQ was drained, so the buffers are free
#pragma unroll
      for (int c = 0; c < BQ / 32; ++c) {
        uint32_t v[32], w[32];
        tmem_ld_32x32(t_s + lane_addr + c * 32, v);
        tmem_ld_32x32(t_dp + lane_addr + c * 32, w);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int qc = c * 32 + i;
          float pv = exp2f(__uint_as_float(v[i]) * args.scale_log2 - s_lse2[grp * BQ + qc]);
          if (!key_ok || (need_mask && key > q0 + qc + off)) pv = 0.f;
          const float dsv = pv * (__uint_as_float(w[i]) - s_delta[grp * BQ + qc]) * args.scale;
          v[i] = __float_as_uint(pv);
          w[i] = __float_as_uint(dsv);
        }
        // X = P^T, Y = dS^T as bf16, one 128-byte swizzled row per key (4 x 16 bytes per 32 queries)
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint4 px, py;
          uint32_t* wx = reinterpret_cast<uint32_t*>(&px);
          uint32_t* wy = reinterpret_cast<uint32_t*>(&py);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 a = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 2 * e]), __uint_as_float(v[u * 8 + 2 * e + 1]));
            __nv_bfloat162 d2 = __floats2bfloat162_rn(__uint_as_float(w[u * 8 + 2 * e]), __uint_as_float(w[u * 8 + 2 * e + 1]));
            wx[e] = *reinterpret_cast<uint32_t*>(&a);
            wy[e] = *reinterpret_cast<uint32_t*>(&d2);
          }
          const int sw = ((c * 4 + u) ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(xr + sw) = px;
          *reinterpret_cast<uint4*>(yr + sw) = py;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&xy_full[grp]);
      // dQ^T of this tile: wait for its MMAs, then reduce it into the fp32 scratch
      if (!mbar_wait(&g2_done[grp], ph)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      {
        float* dst = args.dq_acc + (bh * HD + r) * (long long)args.Sq_pad + q0;
#pragma unroll
        for (int c = 0; c < BQ / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_dp + lane_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 8; ++u)
            red_add_v4(dst + c * 32 + u * 4, __uint_as_float(v[u * 4]), __uint_as_float(v[u * 4 + 1]),
                       __uint_as_float(v[u * 4 + 2]), __uint_as_float(v[u * 4 + 3]));
        }
      }
      tc_fence_before();
      mbar_arrive(&dq_free[grp]);
    }
    if (ok && n_it > 0) {
      if (!mbar_wait(all_done, 0)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) tc_fence_after();
    }
    if (ok) {
      // group 0 writes this key's dK row, group 1 its dV row
      __nv_bfloat16* dst = grp == 0
          ? args.dK + (long long)b * args.dk_sb + (long long)h * args.dk_sh + (long long)key * args.dk_ss
          : args.dV + (long long)b * args.dv_sb + (long long)h * args.dv_sh + (long long)key * args.dv_ss;
      const uint32_t src = grp == 0 ? t_dk : t_dv;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        if (n_it > 0) {
          tmem_ld_32x32(src + lane_addr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (key_ok) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 pk;
            uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 2 * e]), __uint_as_float(v[u * 8 + 2 * e + 1]));
              pw[e] = *reinterpret_cast<uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(dst + c * 32 + u * 8) = pk;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b][h][q] = sum_d dO * O ; one warp per row, head dim 128 (4 elements per lane)
__global__ void __launch_bounds__(128) attn_delta_kernel(const __nv_bfloat16* __restrict__ dO,
                                                        const __nv_bfloat16* __restrict__ O, float* __restrict__ delta,
                                                        int B, int H, int Sq, int D, long long do_sb, long long do_sh,
                                                        long long do_ss, long long o_sb, long long o_sh, long long o_ss) {
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (long long)B * H * Sq) return;
  const int q = row % Sq;
  const int h = (row / Sq) % H;
  const int b = row / ((long long)Sq * H);
  const __nv_bfloat16* a = dO + b * do_sb + h * do_sh + q * do_ss;
  const __nv_bfloat16* c = O + b * o_sb + h * o_sh + q * o_ss;
  float acc = 0.f;
  for (int d = lane * 4; d < D; d += 128) {
    const uint2 ra = *reinterpret_cast<const uint2*>(a + d);
    const uint2 rc = *reinterpret_cast<const uint2*>(c + d);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
    const __nv_bfloat162* pc = reinterpret_cast<const __nv_bfloat162*>(&rc);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float2 x = __bfloat1622float2(pa[e]), y = __bfloat1622float2(pc[e]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) delta[row] = acc;
}

// dq[b][h][q][d] (bf16, strided) = dq_acc[b][h][d][q] (fp32): 32 x 32 transposing tiles
__global__ void __launch_bounds__(256) attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                                             int H, int Sq, int Sq_pad, int D, long long sb, long long sh,
                                                             long long ss) {
  __shared__ float tile[32][33];
  const int bh = blockIdx.z;
  const int b = bh / H, h = bh % H;
  const int q0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  for (int i = ty; i < 32; i += 8) {
    const int d = d0 + i, q = q0 + tx;
    tile[i][tx] = (d < D && q < Sq) ? acc[((long long)bh * D + d) * Sq_pad + q] : 0.f;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int q = q0 + i, d = d0 + tx;
    if (q < Sq && d < D) dq[b * sb + h * sh + q * ss + d] = __float2bfloat16(tile[tx][i]);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}
// (B, H, S, D) bf16 view with D contiguous; element strides sb, sh, ss. Box = 64 x rows x 1 x 1.
static int make_map4(CUtensorMap* map, const void* ptr, int B, int H, int S, int D, long long sb, long long sh,
                     long long ss, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)(H > 1 ? sh : ss * S) * 2, (cuuint64_t)(B > 1 ? sb : sh * H) * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

template <int HD>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdArgs& a,
                      cudaStream_t stream) {
  using L = FwdSmem<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return -2;
    configured = true;
  }
  const int nqt = (a.Sq + BM - 1) / BM;
  const long long grid = (long long)nqt * a.H * a.B;
  if (grid <= 0) return 0;
  attn_fwd_kernel<HD><<<(unsigned)grid, NTHREADS, L::TOTAL, stream>>>(tq, tk, tv, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace nba

// q, k, v: bf16 (B, H, S, D) views, D contiguous, strides in elements (multiples of 8, 16-byte
// aligned bases). o: bf16 with its own strides. lse: fp32 [B][H][Sq]. D in {64, 128}.
extern "C" int nb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int Sq,
                           int Skv, int D, long long q_sb, long long q_sh, long long q_ss, long long k_sb,
                           long long k_sh, long long k_ss, long long v_sb, long long v_sh, long long v_ss,
                           long long o_sb, long long o_sh, long long o_ss, float scale, int causal, int* status,
                           void* stream) {
  using namespace nba;
  if (D != 64 && D != 128) return -10;
  if (B <= 0 || H <= 0 || Sq <= 0) return 0;
  const long long strides[] = {q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_ss, o_sh, o_sb};
  for (long long s : strides)
    if (s & 7) return -12;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return -11;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_map4(&tq, q, B, H, Sq, D, q_sb, q_sh, q_ss, BM))) return r;
  if ((r = make_map4(&tk, k, B, H, Skv, D, k_sb, k_sh, k_ss, BN))) return r;
  if ((r = make_map4(&tv, v, B, H, Skv, D, v_sb, v_sh, v_ss, BN))) return r;
  FwdArgs a;
  a.B = B; a.H = H; a.Sq = Sq; a.Skv = Skv;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.O = reinterpret_cast<__nv_bfloat16*>(o);
  a.o_sb = o_sb; a.o_sh = o_sh; a.o_ss = o_ss;
  a.lse = lse;
  a.status = status;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return D == 128 ? launch_fwd<128>(tq, tk, tv, a, s) : launch_fwd<64>(tq, tk, tv, a, s);
}

// Backward. All tensors are (B, H, S, 128) bf16 views with the head dim contiguous (element strides
// given per tensor); lse fp32 [B][H][Sq] from the forward; dq_acc: zeroed fp32 scratch of
// B*H*128*Sq_pad elements (Sq_pad = Sq rounded up to 64); delta: fp32 scratch [B][H][Sq].
extern "C" int nb_attn_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o, const float* lse,
                           void* dq, void* dk, void* dv, float* dq_acc, int B, int H, int Sq, int Skv, int D,
                           long long q_sb, long long q_sh, long long q_ss, long long k_sb, long long k_sh, long long k_ss,
                           long long v_sb, long long v_sh, long long v_ss, long long do_sb, long long do_sh,
                           long long do_ss, long long o_sb, long long o_sh, long long o_ss, long long dq_sb,
                           long long dq_sh, long long dq_ss, long long dk_sb, long long dk_sh, long long dk_ss,
                           long long dv_sb, long long dv_sh, long long dv_ss, float scale, int causal, float* delta,
                           int* status, void* stream) {
  using namespace nba;
  if (D != 128) return -10;
  if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long st[] = {q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, do_sb, do_sh, do_ss,
                          o_sb, o_sh, o_ss, dq_sb, dq_sh, dq_ss, dk_sb, dk_sh, dk_ss, dv_sb, dv_sh, dv_ss};
  for (long long x : st)
    if (x & 7) return -12;
  const int Sq_pad = (Sq + BQ - 1) / BQ * BQ;
  const long long rows = (long long)B * H * Sq;
  attn_delta_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(dO), reinterpret_cast<const __nv_bfloat16*>(o), delta, B, H, Sq, D, do_sb,
      do_sh, do_ss, o_sb, o_sh, o_ss);
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_map4(&tq, q, B, H, Sq, D, q_sb, q_sh, q_ss, BQ))) return r;
  if ((r = make_map4(&tdo, dO, B, H, Sq, D, do_sb, do_sh, do_ss, BQ))) return r;
  if ((r = make_map4(&tk, k, B, H, Skv, D, k_sb, k_sh, k_ss, BN))) return r;
  if ((r = make_map4(&tv, v, B, H, Skv, D, v_sb, v_sh, v_ss, BN))) return r;
  BwdArgs a;
  a.B = B; a.H = H; a.Sq = Sq; a.Skv = Skv; a.Sq_pad = Sq_pad;
  a.scale = scale; a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.lse = lse; a.delta = delta; a.dq_acc = dq_acc;
  a.dK = reinterpret_cast<__nv_bfloat16*>(dk); a.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  a.dk_sb = dk_sb; a.dk_sh = dk_sh; a.dk_ss = dk_ss; a.dv_sb = dv_sb; a.dv_sh = dv_sh; a.dv_ss = dv_ss;
  a.status = status;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::TOTAL) != cudaSuccess)
      return -2;
    configured = true;
  }
  const int nkt = (Skv + BN - 1) / BN;
  attn_bwd_kernel<<<(unsigned)((long long)nkt * H * B), BWD_THREADS, BwdSmem::TOTAL, s>>>(tq, tk, tv, tdo, a);
  dim3 grid((Sq + 31) / 32, (D + 31) / 32, B * H);
  attn_dq_convert_kernel<<<grid, 256, 0, s>>>(dq_acc, reinterpret_cast<__nv_bfloat16*>(dq), H, Sq, Sq_pad, D, dq_sb, dq_sh,
                                              dq_ss);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

