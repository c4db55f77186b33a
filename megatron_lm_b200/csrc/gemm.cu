// Plain (single-GPU) entry point of the tcgen05 GEMM; the kernel lives in gemm_core.cuh.
#include "gemm_core.cuh"

using namespace mlb;

// D[M,N] (=|+=) op(A) * op(B) (+ bias).
//   a_mn == 0: A is [M, K] with row stride lda (K contiguous).  a_mn == 1: A is stored [K, M] with row stride lda.
//   b_mn == 0: B is [N, K] with row stride ldb (K contiguous).  b_mn == 1: B is stored [K, N] with row stride ldb.
// lda/ldb/ldd are in elements; operand bases 16-byte aligned and lda, ldb multiples of 8.
// max_ctas > 0 caps the persistent grid (to leave SMs to a concurrent communication kernel).
MLB_API int mlb_gemm(int lp_fmt, const void* A, long lda, int a_mn, const void* B, long ldb, int b_mn, void* D,
                     long ldd, int out_mode, const void* bias, int M, int N, int K, int max_ctas, int* status,
                     cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  int sms = sm_count_cached();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  CommParams cp = {};
  cp.mode = COMM_NONE;
  return run_gemm(lp_fmt, A, lda, a_mn, B, ldb, b_mn, D, ldd, out_mode, bias, M, N, K, sms, status, cp, st);
}

// FP8 variant: A [M, K] and B [N, K] hold one byte per element (format 0 = e4m3, 1 = e5m2), K contiguous, lda/ldb
// multiples of 16.  D = (A B^T) * (*scale_a) * (*scale_b) (+ bias) with D bf16 / fp16 (out_lp_fmt 1 / 0), fp32 or
// fp32-accumulate as out_mode says; the scales are device scalars (dequantisation factors), either may be null.
MLB_API int mlb_gemm_fp8(int a_fmt, int b_fmt, const void* A, long lda, const void* B, long ldb, void* D, long ldd,
                         int out_mode, int out_lp_fmt, const void* bias, const float* scale_a, const float* scale_b,
                         int M, int N, int K, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return run_gemm_fp8(a_fmt, b_fmt, A, lda, B, ldb, D, ldd, out_mode, out_lp_fmt, bias, scale_a, scale_b, M, N, K,
                      sm_count_cached(), status, st);
}
