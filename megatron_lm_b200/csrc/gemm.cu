// Plain (single-GPU) entry point of the tcgen05 GEMM; the kernel lives in gemm_core.cuh.
#include "gemm_core.cuh"
#include "gemm2.cuh"

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
  {
    static int pair = -1;
    if (pair < 0) { const char* e = getenv("MLB_GEMM_PAIR"); pair = (e && e[0] == '0') ? 0 : 1; }
    const int esz = out_mode == OUT_LP ? 2 : 4;
    if (pair && M >= 256 && N >= 256 && (((size_t)ldd * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(D) & 15) == 0))
      return run_gemm2_fp8(a_fmt, b_fmt, A, lda, B, ldb, D, ldd, out_mode, out_lp_fmt, bias, scale_a, scale_b, M, N, K,
                           sm_count_cached(), status, st);
  }
  return run_gemm_fp8(a_fmt, b_fmt, A, lda, B, ldb, D, ldd, out_mode, out_lp_fmt, bias, scale_a, scale_b, M, N, K,
                      sm_count_cached(), status, st);
}

// Grouped (mixture-of-experts) product in one launch: rows of A [T, K] are sorted by expert, `tiles` is a device
// array of n_tiles records {row_begin, row_end, expert, 0} (each at most 128 rows of one expert), B stacks the
// experts' matrices: b_mn == 0 -> [E * N, K] (forward, y = x W_e^T); b_mn == 1 -> [E * K, N] (data gradient,
// dx = dy W_e with W_e stored [K, N]; K a multiple of 64).  D [T, N] gets only the rows the tiles cover.
MLB_API int mlb_gemm_grouped(int lp_fmt, const void* A, long lda, const void* B, long ldb, int b_mn, void* D, long ldd,
                             const void* tiles, int n_tiles, int E, int T, int N, int K, int* status, cudaStream_t st) {
  if (n_tiles <= 0 || N <= 0 || K <= 0) return 0;
  return run_gemm_grouped(lp_fmt, A, lda, B, ldb, b_mn, D, ldd, reinterpret_cast<const int4*>(tiles), n_tiles, E, T, N,
                          K, sm_count_cached(), status, st);
}

// CTA-pair (cta_group::2) variant of mlb_gemm for plain products whose output rows are 16-byte aligned.
// sched: null for the static tile schedule, or two zeroed device words for the dynamic one (tiles are drawn from a
// counter by the blocks that are running, so the product does not take a second wave when another stream's
// long-running kernel holds some SMs); launches that share the words must be ordered on one stream.
MLB_API int mlb_gemm_pair(int lp_fmt, const void* A, long lda, int a_mn, const void* B, long ldb, int b_mn, void* D,
                          long ldd, int out_mode, const void* bias, int M, int N, int K, int max_ctas, int* status,
                          cudaStream_t st, uint32_t* sched) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  int sms = sm_count_cached();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (sched == nullptr)
    return run_gemm2(lp_fmt, A, lda, a_mn, B, ldb, b_mn, D, ldd, out_mode, bias, M, N, K, sms, status, st);
  CommParams cp = {};
  cp.mode = COMM_NONE;
  cp.sched = sched;
  return run_gemm2(lp_fmt, A, lda, a_mn, B, ldb, b_mn, D, ldd, out_mode, bias, M, N, K, sms, status, st, &cp);
}
