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
