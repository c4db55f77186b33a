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
// tile_count: null, or a device int32 holding how many of the n_tiles records are valid (the table was built on the
// device from the per-expert token counts; n_tiles is then its capacity).
MLB_API int mlb_gemm_grouped(int lp_fmt, const void* A, long lda, const void* B, long ldb, int b_mn, void* D, long ldd,
                             const void* tiles, int n_tiles, int E, int T, int N, int K, int* status, cudaStream_t st,
                             const void* tile_count) {
  if (n_tiles <= 0 || N <= 0 || K <= 0) return 0;
  return run_gemm_grouped(lp_fmt, A, lda, B, ldb, b_mn, D, ldd, reinterpret_cast<const int4*>(tiles), n_tiles, E, T, N,
                          K, sm_count_cached(), status, st, reinterpret_cast<const int*>(tile_count));
}

// Row-tile table of the grouped GEMM and expert row offsets, computed on the device from the per-expert token
// counts (int64 [E]): tiles [cap] records {row_begin, row_end, expert, 0} of at most 128 rows, never across two
// experts; count[0] = records written; offsets int32 [E + 1].  No host read of the counts is needed.
__global__ void moe_tile_table_kernel(const long long* __restrict__ counts, int E, int4* __restrict__ tiles, int cap,
                                      int* __restrict__ count, int* __restrict__ offsets) {
  __shared__ int s_off[257], s_tile[257];
  if (threadIdx.x == 0) {
    int o = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = o; s_tile[e] = t;
      const int n = (int)counts[e];
      o += n; t += (n + 127) / 128;
    }
    s_off[E] = o; s_tile[E] = t;
    count[0] = t < cap ? t : cap;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = s_off[e];
  for (int e = 0; e < E; ++e) {
    const int nt = s_tile[e + 1] - s_tile[e], end = s_off[e + 1];
    for (int i = threadIdx.x; i < nt; i += blockDim.x) {
      const int idx = s_tile[e] + i;
      if (idx < cap) {
        const int r0 = s_off[e] + i * 128;
        tiles[idx] = make_int4(r0, (r0 + 128 < end) ? r0 + 128 : end, e, 0);
      }
    }
  }
}
MLB_API int mlb_moe_tile_table(const void* counts, int E, void* tiles, int cap, void* count, void* offsets,
                               cudaStream_t st) {
  if (E < 1 || E > 256 || cap < 1) return -3;
  moe_tile_table_kernel<<<1, 256, 0, st>>>(reinterpret_cast<const long long*>(counts), E, reinterpret_cast<int4*>(tiles),
                                           cap, reinterpret_cast<int*>(count), reinterpret_cast<int*>(offsets));
  MLB_CHECK_LAUNCH();
  return 0;
}

// dW [E, N_out, K_in] fp32 (=|+=) dy_e^T x_e for all experts in one launch (see run_gemm_grouped_wgrad).
MLB_API int mlb_gemm_grouped_wgrad(int lp_fmt, const void* dy, long ld_dy, const void* x, long ld_x, void* dW,
                                   const void* offsets, int E, int T, int N_out, int K_in, int accumulate, int* status,
                                   cudaStream_t st) {
  if (E <= 0 || T <= 0 || N_out <= 0 || K_in <= 0) return 0;
  return run_gemm_grouped_wgrad(lp_fmt, dy, ld_dy, x, ld_x, reinterpret_cast<float*>(dW),
                                reinterpret_cast<const int*>(offsets), E, T, N_out, K_in, accumulate, sm_count_cached(),
                                status, st);
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
