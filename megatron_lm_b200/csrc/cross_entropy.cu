// Vocab-parallel cross entropy in two passes over the logits (one forward, one
// backward).  The forward computes, per row of this rank's vocab shard, an
// online-softmax pair (max, sum exp(x - max)), the raw target logit when the
// target falls in the shard, and the sum of logits (for label smoothing); the
// cross-rank combination is then a reduction over three [rows] vectors instead
// of the reference's three passes with an all-reduce between each
// (megatron/core/tensor_parallel/cross_entropy.py:124-232).
#include "common.cuh"

namespace mlb {

constexpr int kCeThreads = 256;

// Peer-memory variant of the cross-rank combination: instead of leaving its four per-row statistics for an
// all-reduce, each rank stores them (one 16-byte store per peer and row) into slot `rank` of every rank's
// statistics table [tp][rows][4]; after a barrier ce_combine_kernel reads the tp slots of its own table.
struct CePeers { float4* table[8]; int n, rank; long rows; };

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ target, float* __restrict__ row_max,
              float* __restrict__ row_sumexp, float* __restrict__ row_tgt, float* __restrict__ row_sumx,
              int v_local, long ld, int64_t v0, const CePeers peers) {
  __shared__ float sh[64];
  const size_t row = blockIdx.x;
  const T* x = logits + row * ld;
  float m = -INFINITY, s = 0.f, sx = 0.f;
  const int nvec = v_local >> 3;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    float a[8];
    load8(x + v * 8, a);
    float lm = a[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) lm = fmaxf(lm, a[k]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { acc += __expf(a[k] - nm); sx += a[k]; }
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int j = (nvec << 3) + threadIdx.x; j < v_local; j += kCeThreads) {
    const float a = to_f(x[j]);
    const float nm = fmaxf(m, a);
    s = s * __expf(m - nm) + __expf(a - nm);
    m = nm; sx += a;
  }
  const float gm = block_max(m, sh);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  block_sum2(s, sx, sh);
  if (threadIdx.x == 0) {
    row_max[row] = gm;
    row_sumexp[row] = s;
    row_sumx[row] = sx;
    const int64_t t = target[row] - v0;
    const float tg = (t >= 0 && t < v_local) ? to_f(x[t]) : 0.f;
    row_tgt[row] = tg;
    for (int q = 0; q < peers.n; ++q)
      peers.table[q][(size_t)peers.rank * peers.rows + row] = make_float4(gm, s, tg, sx);
  }
}

// loss, global max and global sum(exp(x - gmax)) per row from the tp slots of this rank's statistics table
__global__ void ce_combine_kernel(const float4* __restrict__ table, int tp, long rows, float label_smoothing, int v_total,
                                  float* __restrict__ loss, float* __restrict__ gmax, float* __restrict__ gsum) {
  const long row = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float m = -INFINITY;
  for (int q = 0; q < tp; ++q) m = fmaxf(m, table[(size_t)q * rows + row].x);
  float s = 0.f, tg = 0.f, sx = 0.f;
  for (int q = 0; q < tp; ++q) {
    const float4 v = table[(size_t)q * rows + row];
    s += v.y * __expf(v.x - m); tg += v.z; sx += v.w;
  }
  const float lse = logf(s) + m;
  float l = lse - tg;
  if (label_smoothing > 0.f) l = (1.f - label_smoothing) * l + label_smoothing * (lse - sx / (float)v_total);
  loss[row] = l; gmax[row] = m; gsum[row] = s;
}

// grad = (softmax - onehot*(1-ls) - ls/V_total) * gscale[row]; written to dlogits (may alias logits)
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_bwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ target, const float* __restrict__ gmax,
              const float* __restrict__ gsum, const float* __restrict__ gscale, T* __restrict__ dlogits,
              int v_local, long ld, int64_t v0, float label_smoothing, int v_total) {
  const size_t row = blockIdx.x;
  const T* x = logits + row * ld;
  T* d = dlogits + row * ld;
  const float m = gmax[row], inv = 1.f / gsum[row], g = gscale[row];
  const int64_t t = target[row] - v0;
  const float on = 1.f - label_smoothing, off = label_smoothing / (float)v_total;
  const int nvec = v_local >> 3;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    float a[8];
    load8(x + v * 8, a);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float p = __expf(a[k] - m) * inv - off;
      if ((int64_t)(v * 8 + k) == t) p -= on;
      a[k] = p * g;
    }
    store8(d + v * 8, a);
  }
  for (int j = (nvec << 3) + threadIdx.x; j < v_local; j += kCeThreads) {
    float p = __expf(to_f(x[j]) - m) * inv - off;
    if ((int64_t)j == t) p -= on;
    d[j] = from_f<T>(p * g);
  }
}

}  // namespace mlb

using namespace mlb;

// logits [rows, v_local] with row stride ld (elements, multiple of 8, 16-byte aligned base)
MLB_API int mlb_ce_fwd(int dtype, const void* logits, const int64_t* target, float* row_max, float* row_sumexp,
                       float* row_tgt, float* row_sumx, long rows, int v_local, long ld, int64_t v0,
                       cudaStream_t st) {
  if (ld % 8 || rows <= 0) return -3;
  MLB_DISPATCH_ACT(dtype, T, (ce_fwd_kernel<T><<<(unsigned)rows, kCeThreads, 0, st>>>(
      (const T*)logits, target, row_max, row_sumexp, row_tgt, row_sumx, v_local, ld, v0, CePeers{})));
  MLB_CHECK_LAUNCH(); return 0;
}
// Same forward, additionally storing the row statistics into slot `rank` of every rank's table
// (tables: host array of tp device addresses of float4 [tp][table_rows]).
MLB_API int mlb_ce_fwd_peer(int dtype, const void* logits, const int64_t* target, float* row_max, float* row_sumexp,
                            float* row_tgt, float* row_sumx, long rows, int v_local, long ld, int64_t v0,
                            void* const* tables, int tp, int rank, long table_rows, cudaStream_t st) {
  if (ld % 8 || rows <= 0 || tp > 8 || rows > table_rows) return -3;
  CePeers pe = {};
  pe.n = tp; pe.rank = rank; pe.rows = table_rows;
  for (int i = 0; i < tp; ++i) pe.table[i] = reinterpret_cast<float4*>(tables[i]);
  MLB_DISPATCH_ACT(dtype, T, (ce_fwd_kernel<T><<<(unsigned)rows, kCeThreads, 0, st>>>(
      (const T*)logits, target, row_max, row_sumexp, row_tgt, row_sumx, v_local, ld, v0, pe)));
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_ce_combine(const void* table, int tp, long rows, long table_rows, float label_smoothing, int v_total,
                           float* loss, float* gmax, float* gsum, cudaStream_t st) {
  if (rows <= 0) return 0;
  // the table is laid out with table_rows per slot; only the first `rows` of each slot are valid
  if (rows != table_rows) return -3;
  ce_combine_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(reinterpret_cast<const float4*>(table), tp, rows,
                                                                   label_smoothing, v_total, loss, gmax, gsum);
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_ce_bwd(int dtype, const void* logits, const int64_t* target, const float* gmax, const float* gsum,
                       const float* gscale, void* dlogits, long rows, int v_local, long ld, int64_t v0,
                       float label_smoothing, int v_total, cudaStream_t st) {
  if (ld % 8 || rows <= 0) return -3;
  MLB_DISPATCH_ACT(dtype, T, (ce_bwd_kernel<T><<<(unsigned)rows, kCeThreads, 0, st>>>(
      (const T*)logits, target, gmax, gsum, gscale, (T*)dlogits, v_local, ld, v0, label_smoothing, v_total)));
  MLB_CHECK_LAUNCH(); return 0;
}
