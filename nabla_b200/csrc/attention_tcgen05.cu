// Flash attention for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
//   O = softmax(Q K^T * scale [+ mask] [+ causal mask]) V     per (batch, head), never materialising
//                                                             the (seq_q, seq_k) score matrix
//
// Replaces the reference's composed attention (matmul, mul, tril, where, softmax, matmul:
// nabla/nn/functional/layers.py:106-153), whose memory is O(seq^2).
//
// Three kernels, all with the same warp roles (384 threads, one CTA per SM):
//   warp 0      TMA producer (4-D tensor maps over strided (B, H, S, D) views, so q/k/v sliced out
//               of a packed projection are read in place)
//   warp 1      MMA issuer (one elected thread)
//   warp 2      TMEM allocator
//   warps 4-11  two math warpgroups of 128 threads; thread r of a group owns TMEM lane r
//
// The probabilities never touch shared memory: the math threads write P (bf16, two values per
// 32-bit TMEM column) over the score columns they have just read, and the second MMA takes its A
// operand from TMEM. Shared memory then only feeds Q / K / V / dO, which halves the operand
// traffic of the PV-type products.
//
// forward (attn_fwd_kernel): one CTA owns TWO query tiles (2 x 128 rows) that share the K / V
//   stream. Group A works on the softmax of tile A while the tensor core runs tile B's products
//   and vice versa (S_A, S_B, O_A, O_B = 512 TMEM columns at head_dim 128).
// backward, dK / dV (attn_bwd_dkdv_kernel): one CTA owns 128 keys and walks over the query
//   tiles: S^T = K Q^T, dP^T = V dO^T, P^T and dS^T written back into TMEM as A operands of
//   dV += P^T dO and dK += dS^T Q. The two groups split the 128 query columns of a tile.
// backward, dQ (attn_bwd_dq_kernel): one CTA owns 128 queries and walks over the key tiles:
//   S = Q K^T (double buffered), dP = dO V^T, dS into TMEM, dQ += dS K accumulated in TMEM and
//   stored once as bf16: no atomics, no fp32 scratch, deterministic.
// A small kernel before the backward computes delta = rowsum(dO * O) and log2-domain row
// statistics padded to whole tiles.
#include "sm100_ptx.cuh"
#include "nb_debug.cuh"

namespace nba {
using namespace nb;

constexpr int BT = 128;          // tile edge, queries and keys
constexpr int NTHREADS = 384;
constexpr float LOG2E = 1.4426950408889634f;

// Tile load at (column c0, row c1, head c2, batch c3) of a [batch][heads][rows][head_dim] bf16 tensor.
// Debug build: the origin lies inside the tensor and c0 starts on a 16-byte boundary, else the copy is
// not issued (the consumer's bounded wait then ends the kernel with an error status).
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2,
                                            int c3, int rows, int heads, int batch) {
  if (!(NB_ALIGNED(NB_SITE_ATTN_TMA_COORD, c0 * 2, 16) && NB_IN_BOUNDS(NB_SITE_ATTN_TMA_COORD, c1, rows) &&
        NB_IN_BOUNDS(NB_SITE_ATTN_TMA_COORD, c2, heads) && NB_IN_BOUNDS(NB_SITE_ATTN_TMA_COORD, c3, batch)))
    return;
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
// tcgen05.wait::ld that names the 32 loaded registers as in/out operands: everything that reads
// them afterwards depends on the wait, so the compiler cannot schedule a use above it. This lets a
// loop issue the load of the next chunk before it works on the current one.
__device__ __forceinline__ void tmem_ld_wait32(uint32_t (&v)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                 "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
                 "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
                 "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
               :
               : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float2 f2(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }

// D[128 x 128] = A[128 x HD] B[128 x HD]^T : both operands K-major tiles of HD / 64 swizzled chunks.
template <int HD>
__device__ __forceinline__ void mma_scores(uint32_t d_tmem, uint32_t a0, uint32_t b0) {
  constexpr uint32_t idesc = make_idesc_bf16(BT, BT, 0, 0);
#pragma unroll
  for (int k = 0; k < HD / 16; ++k) {
    const uint64_t da = make_smem_desc_sw128(a0 + (k >> 2) * (BT * 128) + (k & 3) * 32, 16, 1024);
    const uint64_t db = make_smem_desc_sw128(b0 + (k >> 2) * (BT * 128) + (k & 3) * 32, 16, 1024);
    umma_f16_ss(d_tmem, da, db, idesc, k != 0);
  }
}
// D[128 x HD] (+)= A[128 x 128] B[128 x HD] : A (bf16 pairs) in TMEM, B in shared memory with the
// reduction index as rows and HD contiguous. `split`: the A columns of k-steps 4-7 start 64 TMEM
// columns after those of k-steps 0-3 (each math group writes inside the columns it has read).
template <int HD>
__device__ __forceinline__ void mma_accum(uint32_t d_tmem, uint32_t a_tmem, bool split, uint32_t b0, bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(BT, HD, 0, 1);
#pragma unroll
  for (int k = 0; k < BT / 16; ++k) {
    const uint64_t db = make_smem_desc_sw128(b0 + k * (16 * 128), BT * 128, 1024);
    const uint32_t a = a_tmem + (split ? 64 * (k >> 2) + 8 * (k & 3) : 8 * k);
    umma_f16_ts(d_tmem, a, db, idesc, (accumulate || k != 0) ? 1u : 0u);
  }
}

// Optional additive mask (fp32, natural-log domain), element (b, h, q, key) at
// mask[b * sb + h * sh + q * sq + key]; strides of 0 broadcast.
struct MaskArg {
  const float* ptr;
  long long sb, sh, sq;
};

// ====================================================================== forward
struct FwdArgs {
  int B, H, Sq, Skv;
  float scale_log2;   // softmax scale * log2(e)
  int causal;
  __nv_bfloat16* O;
  long long o_sb, o_sh, o_ss;   // element strides of O for batch, head, row
  float* lse;                   // [B][H][Sq]
  MaskArg mask;
  int* status;
};

template <int HD>
struct FwdSmem {
  static constexpr int TILE_BYTES = BT * HD * 2;
  static constexpr int OFF_Q = 0;                          // 2 query tiles
  static constexpr int OFF_K = OFF_Q + 2 * TILE_BYTES;     // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * TILE_BYTES;     // 2 stages
  static constexpr int OFF_BAR = OFF_V + 2 * TILE_BYTES;
  static constexpr int RAW = OFF_BAR + 16 * 8 + 16 + 1024;
  static constexpr int TOTAL = RAW < 120 * 1024 ? 120 * 1024 : RAW;   // one CTA per SM (it takes all of TMEM)
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
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars + 0;     // [2] per query tile
  uint64_t* k_full = bars + 2;     // [2]
  uint64_t* k_empty = bars + 4;    // [2]
  uint64_t* v_full = bars + 6;     // [2]
  uint64_t* v_empty = bars + 8;    // [2]
  uint64_t* s_full = bars + 10;    // [2] per query tile: scores of the next key tile are in TMEM
  uint64_t* p_full = bars + 12;    // [2] per query tile: probabilities are in TMEM (128 arrivals)
  uint64_t* o_done = bars + 14;    // [2] per query tile: last PV product has retired
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    __shared__ int s_abort;   // an earlier bounded wait on this device already failed: leave (uniformly)
    if (threadIdx.x == 0) s_abort = *reinterpret_cast<volatile int*>(args.status);
    __syncthreads();
    if (s_abort != 0) return;
  }
  const int nqt = (args.Sq + 2 * BT - 1) / (2 * BT);
  int bid = blockIdx.x;
  const int qt = nqt - 1 - (bid % nqt);   // heavy (late) causal tiles first
  bid /= nqt;
  const int h = bid % args.H;
  const int b = bid / args.H;
  const int q0 = qt * 2 * BT;
  const int off = args.Skv - args.Sq;     // causal: row i sees keys <= i + off
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0t = q0 + t * BT;
    int n = (args.Skv + BT - 1) / BT;
    if (args.causal) {
      const int last_key = min(args.Skv - 1, q0t + BT - 1 + off);
      n = last_key < 0 ? 0 : last_key / BT + 1;
    }
    n_t[t] = q0t < args.Sq ? n : 0;
  }
  const int n_max = max(n_t[0], n_t[1]);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_done[i], 1);
    }
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
  // tile t: scores (and P over their first 64 columns) at t * 128, output accumulator at 256 + t * HD

  if (warp == 0) {
    if (lane == 0 && n_max > 0) {
      for (int t = 0; t < 2; ++t) {
        if (n_t[t] == 0) continue;
        mbar_arrive_expect_tx(&q_full[t], L::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(sQ + t * L::TILE_BYTES + c * (BT * 128), &tmQ, &q_full[t], c * 64, q0 + t * BT, h, b, args.Sq, args.H, args.B);
      }
      for (int j = 0; j < n_max; ++j) {
        const int st = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], ph)) { atomicExch(args.status, NB_ERR_TIMEOUT_PRODUCER); break; }
        mbar_arrive_expect_tx(&k_full[st], L::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(sK + st * L::TILE_BYTES + c * (BT * 128), &tmK, &k_full[st], c * 64, j * BT, h, b, args.Skv, args.H, args.B);
        if (!mbar_wait(&v_empty[st], ph)) { atomicExch(args.status, NB_ERR_TIMEOUT_PRODUCER); break; }
        mbar_arrive_expect_tx(&v_full[st], L::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(sV + st * L::TILE_BYTES + c * (BT * 128), &tmV, &v_full[st], c * 64, j * BT, h, b, args.Skv, args.H, args.B);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_max > 0) {
      bool ok = true;
      auto qk = [&](int t, int j) {
        mma_scores<HD>(tmem_base + t * BT, smem_u32(sQ + t * L::TILE_BYTES), smem_u32(sK + (j & 1) * L::TILE_BYTES));
        umma_commit(&s_full[t]);
      };
      auto pv = [&](int t, int j) {
        mma_accum<HD>(tmem_base + 256 + t * HD, tmem_base + t * BT, false, smem_u32(sV + (j & 1) * L::TILE_BYTES), j != 0);
        if (j == n_t[t] - 1) umma_commit(&o_done[t]);
      };
      for (int t = 0; t < 2 && ok; ++t)
        if (n_t[t] > 0) ok = mbar_wait(&q_full[t], 0);
      ok = ok && mbar_wait(&k_full[0], 0);
      if (ok) {
        tc_fence_after();
        if (n_t[0] > 0) qk(0, 0);
        if (n_t[1] > 0) qk(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const bool more = j + 1 < n_max;
        if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1)) { ok = false; break; }
        if (more && !mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1)) { ok = false; break; }
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j < n_t[t]) {
            if (!mbar_wait(&p_full[t], j & 1)) { ok = false; break; }
            tc_fence_after();
            pv(t, j);
          }
          if (t == 1) umma_commit(&v_empty[j & 1]);
          if (j + 1 < n_t[t]) qk(t, j + 1);
        }
        if (!ok) break;
        if (more) umma_commit(&k_empty[(j + 1) & 1]);
      }
      if (!ok) atomicExch(args.status, NB_ERR_TIMEOUT_MMA);
    }
  } else if (warp >= 4) {
    const int t = (warp - 4) >> 2;          // query tile of this math group
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int q_idx = q0 + t * BT + r;
    const int n = n_t[t];
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t t_s = tmem_base + t * BT + lane_addr;
    const uint32_t t_o = tmem_base + 256 + t * HD + lane_addr;
    const float* mrow = nullptr;
    if (args.mask.ptr != nullptr && q_idx < args.Sq)
      mrow = args.mask.ptr + b * args.mask.sb + h * args.mask.sh + (long long)q_idx * args.mask.sq;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      if (ok && !mbar_wait(&s_full[t], j & 1)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int kv0 = j * BT;
      const bool general = (kv0 + BT > args.Skv) || (args.causal && (kv0 + BT - 1 > q0 + t * BT + off)) ||
                           (args.mask.ptr != nullptr);
      if (general) {
        // masked tile (diagonal, tail or user mask): rewrite the scores in place, -inf where a key is
        // not visible, so that the two passes below carry no mask logic
        const int lim = args.causal ? min(args.Skv - 1, q_idx + off) : args.Skv - 1;
        const float mask_mul = LOG2E / args.scale_log2;
#pragma unroll 1
        for (int c = 0; c < BT / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_s + c * 32, v);
          tmem_ld_wait32(v);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kc = kv0 + c * 32 + i;
            float x = __uint_as_float(v[i]);
            if (mrow != nullptr && kc < args.Skv) x = fmaf(mrow[kc], mask_mul, x);
            v[i] = __float_as_uint(kc <= lim ? x : -INFINITY);
          }
          tmem_st_32x32(t_s + c * 32, v);
        }
        tmem_st_wait();
      }
      // pass 1: row maximum. The load of the next 32 columns is in flight while the current ones
      // are reduced (four independent chains of three-input max).
      uint32_t va[32], vb[32];
      tmem_ld_32x32(t_s, va);
      float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < BT / 32; ++c) {
        uint32_t (&v)[32] = (c & 1) ? vb : va;
        uint32_t (&nx)[32] = (c & 1) ? va : vb;
        tmem_ld_wait32(v);
        tmem_ld_32x32(t_s + ((c + 1) & 3) * 32, nx);       // after the last chunk: chunk 0 again, for pass 2
#pragma unroll
        for (int i = 0; i < 16; ++i) mxa[i & 3] = max3(mxa[i & 3], __uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
      }
      const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])) * args.scale_log2;
      // lazy rescale: keep the old reference maximum unless the new one exceeds it by 2^8
      float alpha = 1.f;
      bool resc = false;
      if (m_used == -INFINITY) {
        m_used = mx;                       // may stay -inf: every key so far is masked for this row
      } else if (mx > m_used + 8.f) {
        alpha = ex2(m_used - mx);
        m_used = mx;
        resc = true;
      }
      const float m_sub = m_used == -INFINITY ? 0.f : m_used;
      if (__any_sync(0xffffffffu, resc)) {
        // s_full of this tile also tracks the previous PV product: O is not being written now
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_o + c * 32, v);
          tmem_ld_wait32(v);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(t_o + c * 32, v);
        }
      }
      // pass 2: probabilities (bf16 pairs) written over the first 64 score columns; packed fp32x2
      // arithmetic: per pair one FFMA2, two EX2, one FADD2, one pack
      const float2 sc2 = make_float2(args.scale_log2, args.scale_log2), nm2 = make_float2(-m_sub, -m_sub);
      float2 acc[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int c = 0; c < BT / 32; ++c) {
        uint32_t (&v)[32] = (c & 1) ? vb : va;
        uint32_t (&nx)[32] = (c & 1) ? va : vb;
        tmem_ld_wait32(v);
        if (c + 1 < BT / 32) tmem_ld_32x32(t_s + (c + 1) * 32, nx);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 x = __ffma2_rn(f2(v[2 * i], v[2 * i + 1]), sc2, nm2);
          const float2 pr = make_float2(ex2(x.x), ex2(x.y));
          acc[i & 1] = __fadd2_rn(acc[i & 1], pr);
          pk[i] = pack_bf16(pr.x, pr.y);
        }
        tmem_st_32x16(t_s + c * 16, pk);
      }
      const float sum = (acc[0].x + acc[0].y) + (acc[1].x + acc[1].y);
      l = l * alpha + sum;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[t]);
    }
    if (ok && n > 0) {
      if (!mbar_wait(&o_done[t], 0)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && q0 + t * BT < args.Sq) {
      tc_fence_after();
      const bool have = n > 0 && l > 0.f;
      const float inv = have ? 1.f / l : 0.f;
      __nv_bfloat16* orow = args.O + (long long)b * args.o_sb + (long long)h * args.o_sh + (long long)q_idx * args.o_ss;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        if (n > 0) {
          tmem_ld_32x32(t_o + c * 32, v);
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
            for (int e = 0; e < 4; ++e)
              pw[e] = pack_bf16(__uint_as_float(v[u * 8 + 2 * e]) * inv, __uint_as_float(v[u * 8 + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = pk;
          }
        }
      }
      if (q_idx < args.Sq)
        args.lse[((long long)b * args.H + h) * args.Sq + q_idx] =
            have ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
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
struct BwdArgs {
  int B, H, Sq, Skv, Sq_pad;
  float scale, scale_log2;
  int causal;
  const float* nlse2;   // [B][H][Sq_pad]  -(log-sum-exp) in the log2 domain; -inf on padding rows and rows without keys
  const float* ndelta;  // [B][H][Sq_pad]  -rowsum(dO * O), 0 on padding rows
  __nv_bfloat16 *dQ, *dK, *dV;
  long long dq_sb, dq_sh, dq_ss, dk_sb, dk_sh, dk_ss, dv_sb, dv_sh, dv_ss;
  MaskArg mask;
  int* status;
};

// ---------------------------------------------------------------------- dK / dV
template <int HD>
struct DkvSmem {
  static constexpr int TILE_BYTES = BT * HD * 2;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE_BYTES;
  static constexpr int OFF_Q = OFF_V + TILE_BYTES;        // 2 stages
  static constexpr int OFF_DO = OFF_Q + 2 * TILE_BYTES;   // 2 stages
  static constexpr int OFF_STAT = OFF_DO + 2 * TILE_BYTES;   // lse2[2][128], delta[2][128]
  static constexpr int OFF_BAR = OFF_STAT + 4 * BT * 4;
  static constexpr int RAW = OFF_BAR + 24 * 8 + 16 + 1024;
  static constexpr int TOTAL = RAW < 120 * 1024 ? 120 * 1024 : RAW;
};

template <int HD>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const BwdArgs args) {
  using L = DkvSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sDO = smem + L::OFF_DO;
  float* s_nlse2 = reinterpret_cast<float*>(smem + L::OFF_STAT);   // [2][128]
  float* s_ndelta = s_nlse2 + 2 * BT;                              // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;     // [2]  Q_i and its lse2 landed in stage i & 1
  uint64_t* q_empty = bars + 3;    // [2]
  uint64_t* do_full = bars + 5;    // [2]  dO_i and its delta landed
  uint64_t* do_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;     //      S^T of the current tile is in TMEM
  uint64_t* dp_full = bars + 10;   //      dP^T of the current tile is in TMEM
  uint64_t* p_full = bars + 11;    //      P^T written back (256 arrivals)
  uint64_t* ds_full = bars + 12;   //      dS^T written back (256 arrivals)
  uint64_t* all_done = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = *reinterpret_cast<volatile int*>(args.status);
    __syncthreads();
    if (s_abort != 0) return;
  }
  // key tile 0 sees every query tile, the last one only a few: tile index slowest, so that the
  // long CTAs start first and the short ones fill the end of the grid
  int bid = blockIdx.x;
  const int nbh = args.H * args.B;
  const int jt = bid / nbh;
  bid -= jt * nbh;
  const int h = bid % args.H;
  const int b = bid / args.H;
  const int k0 = jt * BT;
  const int off = args.Skv - args.Sq;
  const int nqt = (args.Sq + BT - 1) / BT;
  int i_start = 0;
  if (args.causal) {
    const int first_q = k0 - off;             // first query row that sees key k0
    i_start = first_q <= 0 ? 0 : first_q / BT;
  }
  const int n_it = max(0, nqt - i_start);
  const long long bh = (long long)b * args.H + h;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&do_full[i], 1);
      mbar_init(&do_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_full, 256);
    mbar_init(ds_full, 256);
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
  const uint32_t t_st = tmem_base, t_dpt = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 256 + HD;

  if (warp == 0) {
    if (lane == 0 && n_it > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * L::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_4d(sK + c * (BT * 128), &tmK, kv_full, c * 64, k0, h, b, args.Skv, args.H, args.B);
        tma_load_4d(sV + c * (BT * 128), &tmV, kv_full, c * 64, k0, h, b, args.Skv, args.H, args.B);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1;
        const uint32_t ph = ((it >> 1) & 1) ^ 1;
        const int q0 = (i_start + it) * BT;
        if (!mbar_wait(&q_empty[st], ph)) { atomicExch(args.status, NB_ERR_TIMEOUT_PRODUCER); break; }
        mbar_arrive_expect_tx(&q_full[st], L::TILE_BYTES + BT * 4);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(sQ + st * L::TILE_BYTES + c * (BT * 128), &tmQ, &q_full[st], c * 64, q0, h, b, args.Sq, args.H, args.B);
        if (!NB_IN_BOUNDS(NB_SITE_ATTN_STAT_INDEX, q0 + BT - 1, args.Sq_pad)) break;   // debug build only
        bulk_load_1d(s_nlse2 + st * BT, args.nlse2 + bh * args.Sq_pad + q0, BT * 4, &q_full[st]);
        if (!mbar_wait(&do_empty[st], ph)) { atomicExch(args.status, NB_ERR_TIMEOUT_PRODUCER); break; }
        mbar_arrive_expect_tx(&do_full[st], L::TILE_BYTES + BT * 4);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(sDO + st * L::TILE_BYTES + c * (BT * 128), &tmDO, &do_full[st], c * 64, q0, h, b, args.Sq, args.H, args.B);
        bulk_load_1d(s_ndelta + st * BT, args.ndelta + bh * args.Sq_pad + q0, BT * 4, &do_full[st]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      bool ok = mbar_wait(kv_full, 0) && mbar_wait(&q_full[0], 0);
      if (ok) {
        tc_fence_after();
        mma_scores<HD>(t_st, smem_u32(sK), smem_u32(sQ));            // S^T_0 = K Q_0^T
        umma_commit(s_full);
        ok = mbar_wait(&do_full[0], 0);
      }
      if (ok) {
        tc_fence_after();
        mma_scores<HD>(t_dpt, smem_u32(sV), smem_u32(sDO));          // dP^T_0 = V dO_0^T
        umma_commit(dp_full);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1;
        const bool more = it + 1 < n_it;
        if (!mbar_wait(p_full, it & 1)) { ok = false; break; }
        tc_fence_after();
        mma_accum<HD>(t_dv, t_st, true, smem_u32(sDO + st * L::TILE_BYTES), it != 0);     // dV += P^T dO_i
        umma_commit(&do_empty[st]);
        if (more) {
          if (!mbar_wait(&q_full[st ^ 1], ((it + 1) >> 1) & 1)) { ok = false; break; }
          tc_fence_after();
          mma_scores<HD>(t_st, smem_u32(sK), smem_u32(sQ + (st ^ 1) * L::TILE_BYTES));
          umma_commit(s_full);
        }
        if (!mbar_wait(ds_full, it & 1)) { ok = false; break; }
        tc_fence_after();
        mma_accum<HD>(t_dk, t_dpt, true, smem_u32(sQ + st * L::TILE_BYTES), it != 0);     // dK += dS^T Q_i
        umma_commit(&q_empty[st]);
        if (more) {
          if (!mbar_wait(&do_full[st ^ 1], ((it + 1) >> 1) & 1)) { ok = false; break; }
          tc_fence_after();
          mma_scores<HD>(t_dpt, smem_u32(sV), smem_u32(sDO + (st ^ 1) * L::TILE_BYTES));
          umma_commit(dp_full);
        }
      }
      if (ok) umma_commit(all_done);
      else atomicExch(args.status, NB_ERR_TIMEOUT_MMA);
    }
  } else if (warp >= 4) {
    const int grp = (warp - 4) >> 2;        // query columns [64 grp, 64 grp + 64) of every tile
    const int wq = warp & 3;
    const int r = wq * 32 + lane;           // key row inside the tile
    const int key = k0 + r;
    const bool key_ok = key < args.Skv;
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t a_s = t_st + lane_addr + grp * 64, a_dp = t_dpt + lane_addr + grp * 64;
    const float* mbase = args.mask.ptr == nullptr ? nullptr : args.mask.ptr + b * args.mask.sb + h * args.mask.sh + key;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int st = it & 1;
      const int q0 = (i_start + it) * BT + grp * 64;
      if (ok && !(mbar_wait(&q_full[st], (it >> 1) & 1) && mbar_wait(s_full, it & 1))) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool general = (args.causal && (k0 + BT - 1 > q0 + off)) || (k0 + BT > args.Skv) || (mbase != nullptr);
      if (general) {
        // masked tile: rewrite S^T in place with -inf where (key, query) is not visible
        const float mask_mul = LOG2E / args.scale_log2;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(a_s + c * 32, v);
          tmem_ld_wait32(v);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int q = q0 + c * 32 + i;
            float x = __uint_as_float(v[i]);
            if (mbase != nullptr && key_ok && q < args.Sq) x = fmaf(mbase[(long long)q * args.mask.sq], mask_mul, x);
            if (!key_ok || (args.causal && key > q + off)) x = -INFINITY;
            v[i] = __float_as_uint(x);
          }
          tmem_st_32x32(a_s + c * 32, v);
        }
        tmem_st_wait();
      }
      const float2* nl2 = reinterpret_cast<const float2*>(s_nlse2 + st * BT + grp * 64);
      const float2 sc2 = make_float2(args.scale_log2, args.scale_log2);
      float2 p[32];
      uint32_t va[32], vb[32];
      tmem_ld_32x32(a_s, va);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t (&v)[32] = c ? vb : va;
        tmem_ld_wait32(v);
        if (c == 0) tmem_ld_32x32(a_s + 32, vb);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 x = __ffma2_rn(f2(v[2 * i], v[2 * i + 1]), sc2, nl2[c * 16 + i]);
          p[c * 16 + i] = make_float2(ex2(x.x), ex2(x.y));
          pk[i] = pack_bf16(p[c * 16 + i].x, p[c * 16 + i].y);
        }
        tmem_st_32x16(a_s + c * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(p_full);
      if (!(mbar_wait(&do_full[st], (it >> 1) & 1) && mbar_wait(dp_full, it & 1))) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float2* nd2 = reinterpret_cast<const float2*>(s_ndelta + st * BT + grp * 64);
      tmem_ld_32x32(a_dp, va);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t (&v)[32] = c ? vb : va;
        tmem_ld_wait32(v);
        if (c == 0) tmem_ld_32x32(a_dp + 32, vb);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          // dS^T / scale = P^T * (dP^T - delta); the scale is applied once, to dK, in the epilogue
          const float2 d = __fmul2_rn(p[c * 16 + i], __fadd2_rn(f2(v[2 * i], v[2 * i + 1]), nd2[c * 16 + i]));
          pk[i] = pack_bf16(d.x, d.y);
        }
        tmem_st_32x16(a_dp + c * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(ds_full);
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
      const uint32_t src = (grp == 0 ? t_dk : t_dv) + lane_addr;
      const float mul = grp == 0 ? args.scale : 1.f;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        if (n_it > 0) {
          tmem_ld_32x32(src + c * 32, v);
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
            for (int e = 0; e < 4; ++e)
              pw[e] = pack_bf16(__uint_as_float(v[u * 8 + 2 * e]) * mul, __uint_as_float(v[u * 8 + 2 * e + 1]) * mul);
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

// ---------------------------------------------------------------------- dQ
template <int HD>
struct DqSmem {
  static constexpr int TILE_BYTES = BT * HD * 2;
  static constexpr int KST = 3;                             // K stages (a K tile is held until its dQ product retires)
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = OFF_Q + TILE_BYTES;
  static constexpr int OFF_K = OFF_DO + TILE_BYTES;
  static constexpr int OFF_V = OFF_K + KST * TILE_BYTES;    // 2 stages
  static constexpr int OFF_BAR = OFF_V + 2 * TILE_BYTES;
  static constexpr int RAW = OFF_BAR + 24 * 8 + 16 + 1024;
  static constexpr int TOTAL = RAW < 120 * 1024 ? 120 * 1024 : RAW;
};

template <int HD>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const BwdArgs args) {
  using L = DqSmem<HD>;
  constexpr int KST = L::KST;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sDO = smem + L::OFF_DO;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* qdo_full = bars + 0;
  uint64_t* k_full = bars + 1;     // [3]
  uint64_t* k_empty = bars + 4;    // [3]
  uint64_t* v_full = bars + 7;     // [2]
  uint64_t* v_empty = bars + 9;    // [2]
  uint64_t* s_full = bars + 11;    // [2]  score buffer j & 1 holds S_j
  uint64_t* dp_full = bars + 13;   //      dP_j is in TMEM
  uint64_t* ds_full = bars + 14;   //      dS_j written back (256 arrivals)
  uint64_t* dq_done = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = *reinterpret_cast<volatile int*>(args.status);
    __syncthreads();
    if (s_abort != 0) return;
  }
  const int nqt = (args.Sq + BT - 1) / BT;
  int bid = blockIdx.x;
  const int qt = nqt - 1 - (bid % nqt);   // heavy (late) causal tiles first
  bid /= nqt;
  const int h = bid % args.H;
  const int b = bid / args.H;
  const int q0 = qt * BT;
  const int off = args.Skv - args.Sq;
  int n = (args.Skv + BT - 1) / BT;
  if (args.causal) {
    const int last_key = min(args.Skv - 1, q0 + BT - 1 + off);
    n = last_key < 0 ? 0 : last_key / BT + 1;
  }
  const long long bh = (long long)b * args.H + h;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    mbar_init(qdo_full, 1);
    for (int i = 0; i < KST; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(dp_full, 1);
    mbar_init(ds_full, 256);
    mbar_init(dq_done, 1);
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
  const uint32_t t_dp = tmem_base + 256, t_dq = tmem_base + 384;   // S buffers at 0 and 128

  if (warp == 0) {
    if (lane == 0 && n > 0) {
      mbar_arrive_expect_tx(qdo_full, 2 * L::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_4d(sQ + c * (BT * 128), &tmQ, qdo_full, c * 64, q0, h, b, args.Sq, args.H, args.B);
        tma_load_4d(sDO + c * (BT * 128), &tmDO, qdo_full, c * 64, q0, h, b, args.Sq, args.H, args.B);
      }
      for (int j = 0; j < n; ++j) {
        const int ks = j % KST, vs = j & 1;
        if (!mbar_wait(&k_empty[ks], ((j / KST) & 1) ^ 1)) { atomicExch(args.status, NB_ERR_TIMEOUT_PRODUCER); break; }
        mbar_arrive_expect_tx(&k_full[ks], L::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(sK + ks * L::TILE_BYTES + c * (BT * 128), &tmK, &k_full[ks], c * 64, j * BT, h, b, args.Skv, args.H, args.B);
        if (!mbar_wait(&v_empty[vs], ((j >> 1) & 1) ^ 1)) { atomicExch(args.status, NB_ERR_TIMEOUT_PRODUCER); break; }
        mbar_arrive_expect_tx(&v_full[vs], L::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(sV + vs * L::TILE_BYTES + c * (BT * 128), &tmV, &v_full[vs], c * 64, j * BT, h, b, args.Skv, args.H, args.B);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n > 0) {
      auto scores = [&](int j) {          // S_j = Q K_j^T into buffer j & 1
        mma_scores<HD>(tmem_base + (j & 1) * BT, smem_u32(sQ), smem_u32(sK + (j % KST) * L::TILE_BYTES));
        umma_commit(&s_full[j & 1]);
      };
      auto dprobs = [&](int j) {          // dP_j = dO V_j^T
        mma_scores<HD>(t_dp, smem_u32(sDO), smem_u32(sV + (j & 1) * L::TILE_BYTES));
        umma_commit(dp_full);
        umma_commit(&v_empty[j & 1]);
      };
      bool ok = mbar_wait(qdo_full, 0) && mbar_wait(&k_full[0], 0);
      if (ok) {
        tc_fence_after();
        scores(0);
        ok = mbar_wait(&v_full[0], 0);
      }
      if (ok) {
        tc_fence_after();
        dprobs(0);
        if (n > 1) {
          ok = mbar_wait(&k_full[1], 0);
          if (ok) {
            tc_fence_after();
            scores(1);
          }
        }
      }
      for (int j = 0; j < n && ok; ++j) {
        if (!mbar_wait(ds_full, j & 1)) { ok = false; break; }
        tc_fence_after();
        mma_accum<HD>(t_dq, t_dp, true, smem_u32(sK + (j % KST) * L::TILE_BYTES), j != 0);   // dQ += dS_j K_j
        umma_commit(&k_empty[j % KST]);
        if (j + 1 < n) {
          if (!mbar_wait(&v_full[(j + 1) & 1], ((j + 1) >> 1) & 1)) { ok = false; break; }
          tc_fence_after();
          dprobs(j + 1);
        }
        if (j + 2 < n) {
          if (!mbar_wait(&k_full[(j + 2) % KST], ((j + 2) / KST) & 1)) { ok = false; break; }
          tc_fence_after();
          scores(j + 2);
        }
      }
      if (ok) umma_commit(dq_done);
      else atomicExch(args.status, NB_ERR_TIMEOUT_MMA);
    }
  } else if (warp >= 4) {
    const int grp = (warp - 4) >> 2;        // key columns [64 grp, 64 grp + 64) of every tile
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int q_idx = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t a_dp = t_dp + lane_addr + grp * 64;
    // padded to whole tiles, so always in range (the debug build checks it and reads nothing otherwise)
    const bool stat_ok = NB_IN_BOUNDS(NB_SITE_ATTN_STAT_INDEX, q_idx, args.Sq_pad);
    const float nlse2 = stat_ok ? args.nlse2[bh * args.Sq_pad + q_idx] : -INFINITY;
    const float ndelta = stat_ok ? args.ndelta[bh * args.Sq_pad + q_idx] : 0.f;
    const float* mrow = nullptr;
    if (args.mask.ptr != nullptr && q_idx < args.Sq)
      mrow = args.mask.ptr + b * args.mask.sb + h * args.mask.sh + (long long)q_idx * args.mask.sq;
    const int lim = args.causal ? min(args.Skv - 1, q_idx + off) : args.Skv - 1;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      if (ok && !mbar_wait(&s_full[j & 1], (j >> 1) & 1)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int kv0 = j * BT + grp * 64;
      const bool general = (kv0 + 64 > args.Skv) || (args.causal && (kv0 + 63 > q0 + off)) || (args.mask.ptr != nullptr);
      const uint32_t a_s = tmem_base + (j & 1) * BT + lane_addr + grp * 64;
      if (general) {
        // masked tile: rewrite the scores in place with -inf where the key is not visible
        const float mask_mul = LOG2E / args.scale_log2;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(a_s + c * 32, v);
          tmem_ld_wait32(v);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kc = kv0 + c * 32 + i;
            float x = __uint_as_float(v[i]);
            if (mrow != nullptr && kc < args.Skv) x = fmaf(mrow[kc], mask_mul, x);
            v[i] = __float_as_uint(kc <= lim ? x : -INFINITY);
          }
          tmem_st_32x32(a_s + c * 32, v);
        }
        tmem_st_wait();
      }
      const float2 sc2 = make_float2(args.scale_log2, args.scale_log2), nl2 = make_float2(nlse2, nlse2);
      float2 p[32];
      uint32_t va[32], vb[32];
      tmem_ld_32x32(a_s, va);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t (&v)[32] = c ? vb : va;
        tmem_ld_wait32(v);
        if (c == 0) tmem_ld_32x32(a_s + 32, vb);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 x = __ffma2_rn(f2(v[2 * i], v[2 * i + 1]), sc2, nl2);
          p[c * 16 + i] = make_float2(ex2(x.x), ex2(x.y));
        }
      }
      if (!mbar_wait(dp_full, j & 1)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float2 nd2 = make_float2(ndelta, ndelta);
      tmem_ld_32x32(a_dp, va);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t (&v)[32] = c ? vb : va;
        tmem_ld_wait32(v);
        if (c == 0) tmem_ld_32x32(a_dp + 32, vb);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          // dS / scale = P * (dP - delta); the scale is applied once, to dQ, in the epilogue
          const float2 d = __fmul2_rn(p[c * 16 + i], __fadd2_rn(f2(v[2 * i], v[2 * i + 1]), nd2));
          pk[i] = pack_bf16(d.x, d.y);
        }
        tmem_st_32x16(a_dp + c * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(ds_full);
    }
    if (ok && n > 0) {
      if (!mbar_wait(dq_done, 0)) {
        atomicExch(args.status, NB_ERR_TIMEOUT_EPILOGUE);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) tc_fence_after();
    }
    if (ok) {
      // each group stores half of the head dim of its query row
      constexpr int HALF = HD / 2;
      __nv_bfloat16* dst = args.dQ + (long long)b * args.dq_sb + (long long)h * args.dq_sh + (long long)q_idx * args.dq_ss +
                           grp * HALF;
#pragma unroll
      for (int c = 0; c < HALF / 32; ++c) {
        uint32_t v[32];
        if (n > 0) {
          tmem_ld_32x32(t_dq + lane_addr + grp * HALF + c * 32, v);
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
            for (int e = 0; e < 4; ++e)
              pw[e] = pack_bf16(__uint_as_float(v[u * 8 + 2 * e]) * args.scale, __uint_as_float(v[u * 8 + 2 * e + 1]) * args.scale);
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

// ndelta[b][h][q] = -sum_d dO * O and nlse2 = -lse * log2(e), both padded to Sq_pad rows per
// (b, h): padding rows and rows whose lse is -inf (no visible key) get nlse2 = -inf (probability 0)
// and ndelta = 0. D / 8 lanes per row, 16-byte loads.
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ dO,
                                                           const __nv_bfloat16* __restrict__ O,
                                                           const float* __restrict__ lse, float* __restrict__ ndelta,
                                                           float* __restrict__ nlse2, int B, int H, int Sq, int Sq_pad, int D,
                                                           long long do_sb, long long do_sh, long long do_ss,
                                                           long long o_sb, long long o_sh, long long o_ss) {
  const int lpr = D / 8;                                  // lanes per row: 16 (D = 128) or 8 (D = 64)
  const int rows_per_block = 256 / lpr;
  const long long row = (long long)blockIdx.x * rows_per_block + threadIdx.x / lpr;
  const int sub = threadIdx.x % lpr;
  const bool in_range = row < (long long)B * H * Sq_pad;
  const int q = in_range ? (int)(row % Sq_pad) : 0;
  const long long bh = in_range ? row / Sq_pad : 0;
  const int h = bh % H;
  const int b = bh / H;
  float acc = 0.f;
  if (in_range && q < Sq) {
    const uint4 ra = *reinterpret_cast<const uint4*>(dO + b * do_sb + h * do_sh + q * do_ss + sub * 8);
    const uint4 rc = *reinterpret_cast<const uint4*>(O + b * o_sb + h * o_sh + q * o_ss + sub * 8);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
    const __nv_bfloat162* pc = reinterpret_cast<const __nv_bfloat162*>(&rc);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(pa[e]), y = __bfloat1622float2(pc[e]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  for (int o = lpr / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (in_range && sub == 0) {
    if (q < Sq) {
      const float l = lse[bh * Sq + q];
      ndelta[row] = -acc;
      nlse2[row] = (l == -INFINITY) ? -INFINITY : -l * LOG2E;
    } else {
      ndelta[row] = 0.f;
      nlse2[row] = -INFINITY;
    }
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
// (B, H, S, D) bf16 view with D contiguous; element strides sb, sh, ss. Box = 64 x 128 rows x 1 x 1.
static int make_map4(CUtensorMap* map, const void* ptr, int B, int H, int S, int D, long long sb, long long sh,
                     long long ss) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)(H > 1 ? sh : ss * S) * 2, (cuuint64_t)(B > 1 ? sb : sh * H) * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)BT, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

template <typename K>
static int set_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -2;
}

template <int HD>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdArgs& a,
                      cudaStream_t stream) {
  using L = FwdSmem<HD>;
  static bool configured = false;
  if (!configured) {
    if (set_smem(attn_fwd_kernel<HD>, L::TOTAL)) return -2;
    configured = true;
  }
  const int nqt = (a.Sq + 2 * BT - 1) / (2 * BT);
  const long long grid = (long long)nqt * a.H * a.B;
  if (grid <= 0) return 0;
  attn_fwd_kernel<HD><<<(unsigned)grid, NTHREADS, L::TOTAL, stream>>>(tq, tk, tv, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

template <int HD>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                      const BwdArgs& a, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (set_smem(attn_bwd_dkdv_kernel<HD>, DkvSmem<HD>::TOTAL)) return -2;
    if (set_smem(attn_bwd_dq_kernel<HD>, DqSmem<HD>::TOTAL)) return -2;
    configured = true;
  }
  const long long bh = (long long)a.H * a.B;
  const int nkt = (a.Skv + BT - 1) / BT, nqt = (a.Sq + BT - 1) / BT;
  attn_bwd_dkdv_kernel<HD><<<(unsigned)(nkt * bh), NTHREADS, DkvSmem<HD>::TOTAL, stream>>>(tq, tk, tv, tdo, a);
  attn_bwd_dq_kernel<HD><<<(unsigned)(nqt * bh), NTHREADS, DqSmem<HD>::TOTAL, stream>>>(tq, tk, tv, tdo, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace nba

// q, k, v: bf16 (B, H, S, D) views, D contiguous, strides in elements (multiples of 8, 16-byte
// aligned bases). o: bf16 with its own strides. lse: fp32 [B][H][Sq]. D in {64, 128}.
// mask: optional fp32 additive mask (null = none), element strides m_sb, m_sh, m_sq (0 = broadcast),
// key stride 1.
extern "C" int nb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int Sq,
                           int Skv, int D, long long q_sb, long long q_sh, long long q_ss, long long k_sb,
                           long long k_sh, long long k_ss, long long v_sb, long long v_sh, long long v_ss,
                           long long o_sb, long long o_sh, long long o_ss, float scale, int causal, const float* mask,
                           long long m_sb, long long m_sh, long long m_sq, int* status, void* stream) {
  using namespace nba;
  if (D != 64 && D != 128) return -10;
  if (!(scale > 0.f)) return -13;
  if (B <= 0 || H <= 0 || Sq <= 0) return 0;
  const long long strides[] = {q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_ss, o_sh, o_sb};
  for (long long s : strides)
    if (s & 7) return -12;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return -11;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_map4(&tq, q, B, H, Sq, D, q_sb, q_sh, q_ss))) return r;
  if ((r = make_map4(&tk, k, B, H, Skv, D, k_sb, k_sh, k_ss))) return r;
  if ((r = make_map4(&tv, v, B, H, Skv, D, v_sb, v_sh, v_ss))) return r;
  FwdArgs a;
  a.B = B; a.H = H; a.Sq = Sq; a.Skv = Skv;
  a.scale_log2 = scale * LOG2E;
  a.causal = causal;
  a.O = reinterpret_cast<__nv_bfloat16*>(o);
  a.o_sb = o_sb; a.o_sh = o_sh; a.o_ss = o_ss;
  a.lse = lse;
  a.mask = MaskArg{mask, m_sb, m_sh, m_sq};
  a.status = status;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return D == 128 ? launch_fwd<128>(tq, tk, tv, a, s) : launch_fwd<64>(tq, tk, tv, a, s);
}

// Backward. All tensors are (B, H, S, D) bf16 views with the head dim contiguous (element strides
// given per tensor), D in {64, 128}; lse fp32 [B][H][Sq] from the forward. `stats`: fp32 scratch of
// 2 * B * H * Sq_pad elements (Sq_pad = Sq rounded up to 128), filled here (delta, then lse2).
extern "C" int nb_attn_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o, const float* lse,
                           void* dq, void* dk, void* dv, float* stats, int B, int H, int Sq, int Skv, int D,
                           long long q_sb, long long q_sh, long long q_ss, long long k_sb, long long k_sh, long long k_ss,
                           long long v_sb, long long v_sh, long long v_ss, long long do_sb, long long do_sh,
                           long long do_ss, long long o_sb, long long o_sh, long long o_ss, long long dq_sb,
                           long long dq_sh, long long dq_ss, long long dk_sb, long long dk_sh, long long dk_ss,
                           long long dv_sb, long long dv_sh, long long dv_ss, float scale, int causal, const float* mask,
                           long long m_sb, long long m_sh, long long m_sq, int* status, void* stream) {
  using namespace nba;
  if (D != 64 && D != 128) return -10;
  if (!(scale > 0.f)) return -13;
  if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long st[] = {q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, do_sb, do_sh, do_ss,
                          o_sb, o_sh, o_ss, dq_sb, dq_sh, dq_ss, dk_sb, dk_sh, dk_ss, dv_sb, dv_sh, dv_ss};
  for (long long x : st)
    if (x & 7) return -12;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
       reinterpret_cast<uintptr_t>(dv) | reinterpret_cast<uintptr_t>(stats) | reinterpret_cast<uintptr_t>(o)) & 15)
    return -11;
  const int Sq_pad = (Sq + BT - 1) / BT * BT;
  const long long rows = (long long)B * H * Sq_pad;
  float* ndelta = stats;
  float* nlse2 = stats + rows;
  const int rpb = 256 / (D / 8);
  attn_bwd_prep_kernel<<<(unsigned)((rows + rpb - 1) / rpb), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(dO), reinterpret_cast<const __nv_bfloat16*>(o), lse, ndelta, nlse2, B, H, Sq,
      Sq_pad, D, do_sb, do_sh, do_ss, o_sb, o_sh, o_ss);
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_map4(&tq, q, B, H, Sq, D, q_sb, q_sh, q_ss))) return r;
  if ((r = make_map4(&tdo, dO, B, H, Sq, D, do_sb, do_sh, do_ss))) return r;
  if ((r = make_map4(&tk, k, B, H, Skv, D, k_sb, k_sh, k_ss))) return r;
  if ((r = make_map4(&tv, v, B, H, Skv, D, v_sb, v_sh, v_ss))) return r;
  BwdArgs a;
  a.B = B; a.H = H; a.Sq = Sq; a.Skv = Skv; a.Sq_pad = Sq_pad;
  a.scale = scale; a.scale_log2 = scale * LOG2E;
  a.causal = causal;
  a.nlse2 = nlse2; a.ndelta = ndelta;
  a.dQ = reinterpret_cast<__nv_bfloat16*>(dq);
  a.dK = reinterpret_cast<__nv_bfloat16*>(dk); a.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  a.dq_sb = dq_sb; a.dq_sh = dq_sh; a.dq_ss = dq_ss;
  a.dk_sb = dk_sb; a.dk_sh = dk_sh; a.dk_ss = dk_ss; a.dv_sb = dv_sb; a.dv_sh = dv_sh; a.dv_ss = dv_ss;
  a.mask = MaskArg{mask, m_sb, m_sh, m_sq};
  a.status = status;
  return D == 128 ? launch_bwd<128>(tq, tk, tv, tdo, a, s) : launch_bwd<64>(tq, tk, tv, tdo, a, s);
}

NB_DEBUG_DEFINE(attention)
