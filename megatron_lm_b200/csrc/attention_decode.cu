// Single-query ("decode") attention over a KV cache, contiguous or paged.
// One block per (sequence, query head); its warps split the cached positions, each keeps an
// online-softmax state (max, sum, weighted V accumulator spread over lanes), and the warps are
// merged through shared memory.  Memory bound: K and V are each read once, 16 bytes per lane.
// Covers the flash-decode call sites of the reference (megatron/core/transformer/attention.py:391,437)
// and the chunked KV cache of its dynamic context (inference/contexts/dynamic_context.py:453).
#include "common.cuh"

namespace mlb {

constexpr int kDecThreads = 128;

// q [nseq, ng, qpg, D]; out same.  Cache layout per token: [ng, D].
//  contiguous: k_cache/v_cache [nseq, max_len, ng, D], block_table == nullptr
//  paged     : k_cache/v_cache [num_chunks, chunk, ng, D], block_table [nseq, max_chunks] (chunk ids)
template <typename T, int D>
__global__ void __launch_bounds__(kDecThreads)
attn_decode_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                   const int* __restrict__ lens, const int* __restrict__ block_table, T* __restrict__ out,
                   int ng, int qpg, long max_len, int chunk, int max_chunks, float scale_log2) {
  constexpr int EPL = D / 32;                       // elements per lane
  __shared__ float s_m[kDecThreads / 32], s_l[kDecThreads / 32];
  __shared__ float s_acc[kDecThreads / 32][D];
  const int seq = blockIdx.x / (ng * qpg);
  const int hh = blockIdx.x % (ng * qpg);
  const int g = hh / qpg;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = lens[seq];
  float qv[EPL];
  {
    const T* qp = q + ((size_t)seq * ng * qpg + hh) * D + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) qv[e] = to_f(qp[e]) * scale_log2;
  }
  float m = -INFINITY, l = 0.f, acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
  for (int t = warp; t < len; t += kDecThreads / 32) {
    size_t tok;
    if (block_table != nullptr) tok = (size_t)block_table[(size_t)seq * max_chunks + t / chunk] * chunk + (t % chunk);
    else tok = (size_t)seq * max_len + t;
    const T* kp = k_cache + (tok * ng + g) * D + lane * EPL;
    const T* vp = v_cache + (tok * ng + g) * D + lane * EPL;
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) s += qv[e] * to_f(kp[e]);
    s = warp_sum(s);
    const float nm = fmaxf(m, s);
    const float a = exp2f(m - nm), p = exp2f(s - nm);
    l = l * a + p;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * a + p * to_f(vp[e]);
    m = nm;
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int e = 0; e < EPL; ++e) s_acc[warp][lane * EPL + e] = acc[e];
  __syncthreads();
  if (warp == 0) {
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecThreads / 32; ++w) gm = fmaxf(gm, s_m[w]);
    float tl = 0.f, o[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[e] = 0.f;
#pragma unroll
    for (int w = 0; w < kDecThreads / 32; ++w) {
      const float sc = (s_m[w] == -INFINITY) ? 0.f : exp2f(s_m[w] - gm);
      tl += s_l[w] * sc;
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[e] += s_acc[w][lane * EPL + e] * sc;
    }
    const float inv = tl > 0.f ? 1.f / tl : 0.f;
    T* op = out + ((size_t)seq * ng * qpg + hh) * D + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) op[e] = from_f<T>(o[e] * inv);
  }
}

// Append this step's K/V ([n_tokens, ng, D], token i belongs to sequence seq_of[i] at position pos_of[i]).
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ k_cache,
                                 T* __restrict__ v_cache, const int* __restrict__ seq_of, const int* __restrict__ pos_of,
                                 const int* __restrict__ block_table, long src_stride, int row /*ng*D*/, long max_len,
                                 int chunk, int max_chunks, int n_tokens) {
  const int vec = row / 8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < (size_t)n_tokens * vec; i += (size_t)gridDim.x * blockDim.x) {
    const int tkn = (int)(i / vec), c = (int)(i % vec) * 8;
    const int seq = seq_of[tkn], pos = pos_of[tkn];
    size_t tok;
    if (block_table != nullptr) tok = (size_t)block_table[(size_t)seq * max_chunks + pos / chunk] * chunk + (pos % chunk);
    else tok = (size_t)seq * max_len + pos;
    *reinterpret_cast<uint4*>(k_cache + tok * row + c) = *reinterpret_cast<const uint4*>(k + (size_t)tkn * src_stride + c);
    *reinterpret_cast<uint4*>(v_cache + tok * row + c) = *reinterpret_cast<const uint4*>(v + (size_t)tkn * src_stride + c);
  }
}

}  // namespace mlb

using namespace mlb;

MLB_API int mlb_attn_decode(int dtype, const void* q, const void* k_cache, const void* v_cache, const int* lens,
                            const int* block_table, void* out, int nseq, int ng, int qpg, int D, long max_len,
                            int chunk, int max_chunks, float scale, cudaStream_t st) {
  if (nseq <= 0) return 0;
  const float sl2 = scale * 1.4426950408889634f;
  const unsigned grid = (unsigned)(nseq * ng * qpg);
#define GO(T, DD) attn_decode_kernel<T, DD><<<grid, kDecThreads, 0, st>>>((const T*)q, (const T*)k_cache, (const T*)v_cache, \
    lens, block_table, (T*)out, ng, qpg, max_len, chunk, max_chunks, sl2)
  if (dtype == MLB_BF16) { if (D == 128) GO(__nv_bfloat16, 128); else if (D == 64) GO(__nv_bfloat16, 64); else return -5; }
  else if (dtype == MLB_F16) { if (D == 128) GO(__half, 128); else if (D == 64) GO(__half, 64); else return -5; }
  else if (dtype == MLB_F32) { if (D == 128) GO(float, 128); else if (D == 64) GO(float, 64); else return -5; }
  else return -1;
#undef GO
  MLB_CHECK_LAUNCH();
  return 0;
}

// k, v: [n_tokens, ...] with row stride src_stride (elements) and ng*D contiguous elements per token (2-byte dtypes)
MLB_API int mlb_kv_append(const void* k, const void* v, void* k_cache, void* v_cache, const int* seq_of, const int* pos_of,
                          const int* block_table, long src_stride, int row, long max_len, int chunk, int max_chunks,
                          int n_tokens, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (row % 8 || src_stride % 8) return -3;
  size_t work = (size_t)n_tokens * (row / 8);
  unsigned grid = (unsigned)((work + 255) / 256 > 148 * 8 ? 148 * 8 : (work + 255) / 256);
  kv_append_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)k, (const uint16_t*)v, (uint16_t*)k_cache,
                                                   (uint16_t*)v_cache, seq_of, pos_of, block_table, src_stride, row,
                                                   max_len, chunk, max_chunks, n_tokens);
  MLB_CHECK_LAUNCH();
  return 0;
}
