// Tensor-parallel products fused with their sequence-parallel collective, one launch each
// (the kernel is gemm_core.cuh in its AG / RS communication mode):
//   mlb_ag_gemm : D = allgather_rows(X_r) * op(B)      column-parallel forward, row-parallel dgrad
//   mlb_gemm_rs : out = reduce_scatter_rows(A * op(B)) (+ residual)   row-parallel forward, column-parallel dgrad
// They replace the userbuffer-overlapped GEMMs the reference configures through
// megatron/training/initialize.py:238-294 and megatron/core/extensions/transformer_engine.py:188-221.
#include "gemm_core.cuh"
#include "gemm2.cuh"

using namespace mlb;

// MLB_GEMM_PAIR=0 selects the single-CTA kernel for the fused products too
static bool pair_ok() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("MLB_GEMM_PAIR"); v = (e && e[0] == '0') ? 0 : 1; }
  return v == 1;
}

// peer_x / peer_sig: host arrays of tp device addresses (symmetric-memory mappings, this rank's own included).
// gathered: local [tp*rows_per_rank, K]; chunk_flags: local uint32[tp*rows_per_rank/128]; comm_counter: local uint32.
// seq: 1, 2, 3, ... per call on this buffer set (flags and signals are monotonic, never reset).
// comm_target: the sum of n_comm over all calls on this buffer set so far, this one included.
// sched: two zeroed local words for the CTA-pair kernel's dynamic tile schedule (see gemm2.cuh), or null for the
// static schedule; calls that share the words must be ordered on one stream.
MLB_API int mlb_ag_gemm(int lp_fmt, const void* const* peer_x, uint32_t* const* peer_sig, void* gathered,
                        uint32_t* chunk_flags, uint32_t* comm_counter, int rank, int tp, int rows_per_rank,
                        unsigned seq, unsigned comm_target, int n_comm, const void* B, long ldb, int b_mn, void* D, long ldd, int out_mode,
                        const void* bias, int N, int K, int* status, cudaStream_t st, uint32_t* sched) {
  if (tp < 2 || tp > kMaxPeers || rows_per_rank % BM || K % 8) return -7;
  const int sms = sm_count_cached();
  if (n_comm < 1 || n_comm >= sms) return -7;
  CommParams cp = {};
  cp.mode = COMM_AG; cp.rank = rank; cp.tp = tp; cp.n_comm = n_comm; cp.bpr = rows_per_rank / BM; cp.seq = seq;
  for (int i = 0; i < tp; ++i) { cp.peer_x[i] = peer_x[i]; cp.peer_sig[i] = peer_sig[i]; }
  cp.gathered = gathered; cp.chunk_flags = chunk_flags; cp.comm_counter = comm_counter; cp.comm_target = comm_target;
  cp.shard_bytes = (long)rows_per_rank * K * 2;
  cp.sched = sched;
  ExtraMaps xm = {};
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)rows_per_rank}, strides[1] = {(uint64_t)K * 2};
    uint32_t box[2] = {BK, BM};
    int rc = make_tmap(&xm.m[0], peer_x[rank], 2, dims, strides, box);
    if (rc) return rc;
  }
  // CTA-pair kernel when 256-row tiles fit the rank layout and the output is TMA-addressable
  if (pair_ok() && (cp.bpr % 2 == 0) && (n_comm % 2 == 0) && N >= 256) {
    const int esz = out_mode == OUT_LP ? 2 : 4;
    if ((((size_t)ldd * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(D) & 15) == 0))
      return run_gemm2(lp_fmt, gathered, K, 0, B, ldb, b_mn, D, ldd, out_mode, bias, tp * rows_per_rank, N, K, sms,
                       status, st, &cp, &xm);
  }
  return run_gemm(lp_fmt, gathered, K, 0, B, ldb, b_mn, D, ldd, out_mode, bias, tp * rows_per_rank, N, K, sms, status,
                  cp, st, &xm);
}

// A: local [tp*rows_per_rank, K] (a_mn = 0).  peer_recv[i]: rank i's receive buffer [tp][rows_per_rank][N];
// peer_cnt[i]: rank i's uint32[rows_per_rank/128] arrival counters.  cnt_target: cumulative arrivals expected on
// this counter set once this call is complete (each call adds (tp - 1) * ceil(N/BN) * 4 per row block: one per
// epilogue warp per tile from every peer; the owner's own tiles are summed in registers and do not count).
MLB_API int mlb_gemm_rs(int lp_fmt, const void* A, long lda, const void* B, long ldb, int b_mn, void* const* peer_recv,
                        uint32_t* const* peer_cnt, unsigned cnt_target, int rank, int tp, int rows_per_rank,
                        const void* residual, long ld_res, void* out, long ld_out, int N, int K, int* status,
                        cudaStream_t st, uint32_t* sched) {
  if (tp < 2 || tp > kMaxPeers || rows_per_rank % BM || N % 64) return -7;
  CommParams cp = {};
  cp.mode = COMM_RS; cp.rank = rank; cp.tp = tp; cp.bpr = rows_per_rank / BM; cp.cnt_target = cnt_target;
  for (int i = 0; i < tp; ++i) { cp.peer_recv[i] = peer_recv[i]; cp.peer_cnt[i] = peer_cnt[i]; }
  cp.residual = residual; cp.ld_res = ld_res; cp.out = out; cp.ld_out = ld_out;
  cp.sched = sched;
  ExtraMaps xm = {};
  for (int q = 0; q < tp; ++q) {
    const uint8_t* slot = reinterpret_cast<const uint8_t*>(peer_recv[q]) + (size_t)rank * rows_per_rank * N * 2;
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)rows_per_rank}, strides[1] = {(uint64_t)N * 2};
    uint32_t box[2] = {64, 32};
    int rc = make_tmap(&xm.m[q], slot, 2, dims, strides, box);
    if (rc) return rc;
  }
  if (pair_ok() && (cp.bpr % 2 == 0) && N >= 256 && (((size_t)ld_out * 2) % 16 == 0) &&
      ((reinterpret_cast<uintptr_t>(out) & 15) == 0))
    return run_gemm2(lp_fmt, A, lda, 0, B, ldb, b_mn, out, ld_out, OUT_LP, nullptr, tp * rows_per_rank, N, K,
                     sm_count_cached(), status, st, &cp, &xm);
  return run_gemm(lp_fmt, A, lda, 0, B, ldb, b_mn, out /*unused*/, ld_out, OUT_LP, nullptr, tp * rows_per_rank, N, K,
                  sm_count_cached(), status, cp, st, &xm);
}

// 1 when mlb_ag_gemm / mlb_gemm_rs with these sizes run on the CTA-pair kernel (the one with the dynamic schedule)
MLB_API int mlb_tp_fused_uses_pair(int rows_per_rank, int N, int n_comm) {
  return (pair_ok() && ((rows_per_rank / BM) % 2 == 0) && (n_comm % 2 == 0) && N >= 256) ? 1 : 0;
}

// Arrivals one mlb_gemm_rs call adds to each 128-row block counter: one per epilogue warp per column tile from every
// peer (4 warps in the single-CTA kernel, 8 in the CTA-pair kernel; the choice mirrors mlb_gemm_rs).
MLB_API int mlb_gemm_rs_arrivals(int tp, int N, int rows_per_rank) {
  const int bn = (N > 128) ? 256 : 128;
  const bool pair = pair_ok() && ((rows_per_rank / BM) % 2 == 0) && N >= 256;
  return (tp - 1) * ((N + bn - 1) / bn) * (pair ? 8 : 4);
}

// Test aid: `n_ctas` blocks that each claim `smem_bytes` of shared memory and idle for `usec` microseconds (at most
// half a second), then leave.  It stands in for long-running kernels of other streams (NCCL send / receive kernels,
// gradient reductions) that keep part of the GPU away from a fused kernel's grid.
__global__ void occupy_kernel(long long ns) {
  extern __shared__ uint8_t occ_smem[];
  if (threadIdx.x == 0) occ_smem[0] = 1;
  unsigned long long t0, t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  do {
    __nanosleep(2000);
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
  } while ((long long)(t1 - t0) < ns);
}
MLB_API int mlb_occupy_sms(int n_ctas, int smem_bytes, int usec, cudaStream_t st) {
  if (n_ctas < 1 || smem_bytes < 0 || smem_bytes > 227 * 1024 || usec < 0) return -7;
  if (usec > 500000) usec = 500000;
  cudaError_t e = cudaFuncSetAttribute(occupy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e != cudaSuccess) return (int)e;
  occupy_kernel<<<n_ctas, 32, smem_bytes, st>>>((long long)usec * 1000LL);
  MLB_CHECK_LAUNCH();
  return 0;
}
