// Column sum with built-in scratch memory: an entry point that never allocates.
//
// This entry point has no counterpart in the reference framework. It exists for callers that
// must not allocate device memory at the moment they need a column sum (a bias gradient, a
// per-feature statistic):
//   * code that runs with all of the device memory already handed out, such as a serving
//     process that sized its KV cache to fill the GPU, where an allocation could fail or push
//     the caching allocator into a synchronising free-and-retry;
//   * code that runs between other people's kernels under a latency limit, where a device-wide
//     synchronisation hidden inside an allocation or a free stalls every stream of the process;
//   * hosts that call this library from C, C++ or another runtime and have no torch allocator
//     to hand scratch tensors to the regular entry point (`nb_colsum`, which expects the caller
//     to provide the `partial` buffer).
//
// The scratch lives in one fixed array in the library's device data segment
// (NB_NOALLOC_MAX_PARTS x NB_NOALLOC_MAX_COLS floats = 2 MiB per device). Consequences:
//   * Limits: N <= NB_NOALLOC_MAX_COLS columns; rows may be anything that fits an int.
//     N must be a multiple of 8 for bf16 input and of 4 for fp32 input (16-byte rows), as for
//     `nb_colsum`. Anything else is rejected with a negative code before any launch.
//   * All calls on one device share the array. Two calls whose kernels can overlap on the GPU
//     (different streams, no dependency between them) race on it and give wrong sums:
//     serialise such calls yourself, e.g. by issuing them on one stream.
//   * The array keeps whatever the previous call left in it. This routine needs no zeroed
//     scratch: every element that the second kernel reads is written by the first kernel of the
//     same call, so stale contents are never observed.
//   * Set-up: the first call on each device looks up the device address of the array (with that
//     device current) and caches it. Make that first call outside any stream capture; later
//     calls only launch kernels. With lazy module loading that first call is also the moment
//     the driver loads this library's code and commits its 2 MiB data segment on the device, so
//     make it while the device still has that much memory to spare, i.e. before the process
//     fills the GPU. A host that resets the device (cudaDeviceReset) must call
//     nb_noalloc_forget_devices() afterwards: the cached addresses belong to the old context.
//   * The routine itself calls no cudaMalloc, cudaFree or other allocating routine, and takes
//     nothing from torch.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define NB_NOALLOC_MAX_COLS 8192
#define NB_NOALLOC_MAX_PARTS 64

#define NB_NOALLOC_OK 0
#define NB_NOALLOC_ERR_TOO_WIDE (-1)      /* N > NB_NOALLOC_MAX_COLS */
#define NB_NOALLOC_ERR_BAD_SHAPE (-2)     /* rows < 0, N <= 0 or N not a multiple of the vector width */
#define NB_NOALLOC_ERR_BAD_POINTER (-3)   /* null or not 16-byte aligned */
#define NB_NOALLOC_ERR_SETUP (-4)         /* the scratch array's device address could not be found */
#define NB_NOALLOC_ERR_LAUNCH (-5)        /* a kernel launch failed */

/* out[c] = sum over r of x[r][c] for a row-major, contiguous x[rows][N] on the current device.
 * in_dtype / out_dtype: 0 = float32, 1 = bfloat16. The sum is accumulated in float32.
 * `stream` is a cudaStream_t (null = the default stream). Returns NB_NOALLOC_OK or a negative
 * code; nothing is launched when the code is one of the argument errors. */
int nb_colsum_noalloc(const void* x, void* out, int rows, int N, int in_dtype, int out_dtype, void* stream);

/* Drop the cached per-device addresses of the scratch array; the next call on a device looks
 * its address up again. Needed only after the host destroyed the device's context. */
void nb_noalloc_forget_devices(void);

/* A one-line description of a code returned by nb_colsum_noalloc. */
const char* nb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
