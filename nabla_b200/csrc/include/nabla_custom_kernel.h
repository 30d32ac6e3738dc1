// ABI of user kernels callable through nabla_b200.call_custom_kernel.
//
// A custom kernel library is a .cu (or built .so) file that defines, for each kernel NAME,
//
//     extern "C" int NAME(const NbTensor* inputs, int n_inputs,
//                         NbTensor* outputs, int n_outputs, void* cuda_stream);
//
// Inputs and pre-allocated outputs are dense row-major device (or host) buffers. The function
// launches its work on `cuda_stream` (a cudaStream_t; null for host tensors) and returns 0 on
// success. Counterpart of the reference's Mojo `@compiler.register("name")` kernels
// (tests/mojo/kernels/custom_kernel.mojo).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum NbDType { NB_F32 = 0, NB_BF16 = 1, NB_F16 = 2, NB_F64 = 3, NB_I32 = 4, NB_I64 = 5, NB_U8 = 6, NB_BOOL = 7 };

typedef struct NbTensor {
  void* data;
  int64_t numel;
  int32_t rank;
  int32_t dtype;      // NbDType
  int64_t shape[8];
} NbTensor;

#ifdef __cplusplus
}
#endif
