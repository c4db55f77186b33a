// Allocation-free norm backward.  This entry point has no counterpart in the reference library.
//
// mlb_norm_bwd (norm.cu) needs a caller-provided fp32 workspace for the per-block partial sums of
// dgamma / dbeta.  Some callers cannot provide one because they may not allocate device memory at
// the point of the call: code that runs under a frozen memory plan (a serving process that has
// handed every byte of its budget to its own pools), code that must not risk the implicit device
// synchronisation of cudaMalloc / cudaFree in the middle of a step, and code called from inside
// another allocator's hooks, where asking for memory would re-enter that allocator.
//
// mlb_norm_bwd_noalloc computes exactly what mlb_norm_bwd computes, but keeps the partial sums in
// an array that is part of the library image:  static __device__ float [148 * 2 * 8192]  (about
// 9.7 MB).  Every GPU on which the library is used holds that array until the process exits.
//
// Limits and rules
//   * h must be a multiple of 8 and at most mlb_norm_bwd_noalloc_max_h() (8192); rows >= 1.
//     Anything else is refused with MLB_NOALLOC_BAD_SIZE and nothing is launched.
//   * The call allocates nothing and frees nothing: no cudaMalloc / cudaFree, no library routine
//     that allocates.  Inputs and outputs are the caller's.
//   * The first call on each device resolves the device address of the array (once per device,
//     with that device current) and remembers it.  Make that first call during set-up, before any
//     stream capture begins on that device.
//   * All calls on a device share the one array.  Calls are safe back to back on one stream; two
//     calls that can overlap on the GPU (different streams, no dependency) race on it.
//   * The array keeps whatever the previous call left.  Nothing has to be cleared between calls:
//     every block rewrites its whole row of partials (blocks without rows write zeros) before the
//     fold kernel reads them.
//
// Return value: 0 on success, a positive cudaError_t if the runtime reported one, or one of the
// negative codes below.
#pragma once
#include <cuda_runtime.h>

#define MLB_NOALLOC_BAD_SIZE   (-20)   /* h not a multiple of 8, h above the maximum, or rows < 1 */
#define MLB_NOALLOC_BAD_DTYPE  (-21)   /* dtype code is none of 0 (fp32), 1 (bf16), 2 (fp16) */
#define MLB_NOALLOC_NO_SYMBOL  (-22)   /* the scratch array's device address could not be resolved */

#ifdef __cplusplus
extern "C" {
#endif

// Largest hidden size the built-in scratch array supports.
int mlb_norm_bwd_noalloc_max_h(void);

// dtype: 0 fp32, 1 bf16, 2 fp16 (activations dy, x, gamma, dx).  rms != 0 selects RMSNorm (mean and dbeta are
// ignored and may be null), else LayerNorm.  mean / rstd: fp32 [rows] saved by the forward.  dgamma / dbeta: fp32 [h],
// overwritten, or added to when accumulate != 0.
int mlb_norm_bwd_noalloc(int dtype, int rms, const void* dy, const void* x, const void* gamma, const float* mean,
                         const float* rstd, void* dx, float* dgamma, float* dbeta, int rows, int h, int zero_centered,
                         int accumulate, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
