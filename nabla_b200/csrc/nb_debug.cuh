// Debug-build index checks for the kernels of this package.
//
// Built with -DNB_DEBUG_CHECKS (`python -m nabla_b200.csrc.build --debug`, libraries in
// nabla_b200/lib/debug, selected at run time with NABLA_B200_DEBUG_KERNELS=1) every global, peer
// and TMA coordinate that a kernel derives from data or from its launch geometry goes through
// NB_IN_BOUNDS / NB_ALIGNED before it is used. A check that fails never traps and never touches
// the address: it records the first failure in the bound record
//     rec[0] = NB_ERR_BOUNDS (5) or NB_ERR_ALIGN (6)     rec[1] = site id (NbSite)
//     rec[2..3] = offending value (lo, hi)               rec[4..5] = limit (lo, hi)
//     rec[6] = number of failed checks so far
// and evaluates to false, and the caller skips the access. The host reads the record with
// `nabla_b200.native.debug_report()`. In a release build both macros are the constant `true` and
// cost nothing.
//
// Each translation unit has its own copy of the record pointer (the libraries are not linked with
// relocatable device code); NB_DEBUG_DEFINE(tu) emits `nb_debug_bind_<tu>(void* rec)` to set it and
// `nb_debug_enabled_<tu>()` so that the host can tell which build it loaded.
#pragma once
#include <cuda_runtime.h>

enum NbDebugCode : int { NB_ERR_BOUNDS = 5, NB_ERR_ALIGN = 6 };

// Where a check sits. The numbers are part of the host-side report; append, do not renumber.
enum NbSite : int {
  NB_SITE_EMB_GATHER_ID = 1,     // embedding gather: row id vs vocabulary
  NB_SITE_EMB_SCATTER_ID = 2,    // embedding scatter-add: row id vs vocabulary
  NB_SITE_XENT_TARGET = 3,       // cross-entropy: class id vs number of classes
  NB_SITE_ROW_INDEX = 4,         // row-wise kernels: row vs number of rows
  NB_SITE_FLAT_INDEX = 5,        // flat element index vs element count
  NB_SITE_POOL_INPUT = 6,        // pooling: input pixel vs image
  NB_SITE_CONV_INPUT = 7,        // direct convolution: input pixel vs image
  NB_SITE_NF4_BLOCK = 8,         // NF4 dequantisation: scale block vs number of blocks
  NB_SITE_REDUCE_INDEX = 9,      // reduction kernels: (outer, r, inner) vs extents
  NB_SITE_GEMM_TMA_COORD = 10,   // GEMM: TMA tile coordinate vs tensor extent
  NB_SITE_GEMM_TMA_ALIGN = 11,   // GEMM: innermost TMA coordinate x element size vs 16 bytes
  NB_SITE_GEMM_STORE = 12,       // GEMM epilogue: (row, col) vs (M, N)
  NB_SITE_GEMM_PEER_RANK = 13,   // fused GEMM + collective: peer rank vs world size
  NB_SITE_GEMM_PEER_OFFSET = 14, // fused GEMM + collective: byte offset vs arena size
  NB_SITE_ATTN_TMA_COORD = 15,   // attention: TMA tile coordinate vs tensor extent
  NB_SITE_ATTN_STAT_INDEX = 16,  // attention: row-statistics index vs padded length
  NB_SITE_ATTN_STORE = 17,       // attention: output row vs sequence length
  NB_SITE_COMM_PEER_RANK = 18,   // peer collectives: peer rank vs world size
  NB_SITE_COMM_OFFSET = 19,      // peer collectives: element offset vs buffer length
  NB_SITE_COMM_FLAG = 20,        // peer collectives: flag slot vs flag pad
};

#ifdef NB_DEBUG_CHECKS
static __device__ int* nb_dbg_rec = nullptr;

static __device__ __noinline__ bool nb_dbg_fail(int code, int site, long long value, long long limit) {
  int* r = nb_dbg_rec;
  if (r != nullptr) {
    if (atomicCAS(r, 0, code) == 0) {
      r[1] = site;
      r[2] = (int)(value & 0xffffffffll);
      r[3] = (int)(value >> 32);
      r[4] = (int)(limit & 0xffffffffll);
      r[5] = (int)(limit >> 32);
    }
    atomicAdd(r + 6, 1);
  }
  return false;
}
// 0 <= value < limit
#define NB_IN_BOUNDS(site, value, limit)                                            \
  (((unsigned long long)(long long)(value) < (unsigned long long)(long long)(limit)) \
       ? true                                                                       \
       : nb_dbg_fail(NB_ERR_BOUNDS, (site), (long long)(value), (long long)(limit)))
// value is a multiple of `align` (a power of two)
#define NB_ALIGNED(site, value, align)                          \
  ((((unsigned long long)(value)) & ((unsigned long long)(align) - 1ull)) == 0ull \
       ? true                                                   \
       : nb_dbg_fail(NB_ERR_ALIGN, (site), (long long)(value), (long long)(align)))
// One thread evaluates one bounds check and one alignment check on the given numbers and touches no
// memory besides the record: the host uses it to see that a failed check of this translation unit
// reaches the record.
static __global__ void nb_dbg_selftest_kernel(long long value, long long limit, long long addr, long long align) {
  (void)NB_IN_BOUNDS(NB_SITE_FLAT_INDEX, value, limit);
  (void)NB_ALIGNED(NB_SITE_FLAT_INDEX, addr, align);
}
#define NB_DEBUG_DEFINE(tu)                                                         \
  extern "C" int nb_debug_bind_##tu(void* rec) {                                    \
    int* p = static_cast<int*>(rec);                                                \
    return (int)cudaMemcpyToSymbol(nb_dbg_rec, &p, sizeof(p));                      \
  }                                                                                 \
  extern "C" int nb_debug_enabled_##tu() { return 1; }                              \
  extern "C" int nb_debug_selftest_##tu(long long value, long long limit, long long addr, long long align, \
                                        void* stream) {                             \
    nb_dbg_selftest_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(value, limit, addr, align); \
    return (int)cudaGetLastError();                                                 \
  }
#else
#define NB_IN_BOUNDS(site, value, limit) true
#define NB_ALIGNED(site, value, align) true
#define NB_DEBUG_DEFINE(tu)                                         \
  extern "C" int nb_debug_bind_##tu(void*) { return 0; }            \
  extern "C" int nb_debug_enabled_##tu() { return 0; }              \
  extern "C" int nb_debug_selftest_##tu(long long, long long, long long, long long, void*) { return 0; }
#endif
