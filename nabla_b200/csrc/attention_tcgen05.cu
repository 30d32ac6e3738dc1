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
