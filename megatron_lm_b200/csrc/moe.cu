// Mixture-of-experts token movement fused with the expert-parallel exchange over peer memory.
//   scatter_rows : "permute + all-to-all" - every routed copy of a token is written straight into its destination
//                  rank's receive buffer (a peer store over NVLink), at the row the layout [local expert][source
//                  rank][token order] assigns to it; optional per-copy scale (the combine gradient).
//   gather_sum   : "all-to-all + unpermute + weighting" - every token pulls its top-k expert outputs from the
//                  ranks that computed them (peer loads) and accumulates prob-weighted in fp32; optionally
//                  keeps the pulled rows for the router-probability gradient.
// They replace the permute / all_to_all_single / sort_chunks / unpermute chain of the reference's all-to-all
// dispatcher (megatron/core/transformer/moe/token_dispatcher.py:588-788) and the fused dispatch/combine it gets from
// an external library (moe/fused_a2a.py:68,162).
#include "common.cuh"

namespace mlb {

constexpr int kMoeMaxRanks = 64;
struct MoePtrs { unsigned long long base[kMoeMaxRanks]; };

template <typename T>
__global__ void __launch_bounds__(128)
moe_scatter_rows_kernel(const T* __restrict__ src, const int* __restrict__ src_row, const MoePtrs dst,
                        const int* __restrict__ dst_rank, const int* __restrict__ dst_row,
                        const float* __restrict__ scale, int n_copies, int h) {
  for (int i = blockIdx.x; i < n_copies; i += gridDim.x) {
    const T* s = src + (size_t)(src_row ? src_row[i] : i) * h;
    T* d = reinterpret_cast<T*>(dst.base[dst_rank[i]]) + (size_t)dst_row[i] * h;
    const float sc = scale ? scale[i] : 1.f;
    for (int c = threadIdx.x * 8; c < h; c += blockDim.x * 8) {
      if (scale) {
        float v[8]; load8(s + c, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] *= sc;
        store8(d + c, v);
      } else {
        *reinterpret_cast<uint4*>(d + c) = *reinterpret_cast<const uint4*>(s + c);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_sum_kernel(const MoePtrs src, const int* __restrict__ src_rank, const int* __restrict__ src_row,
                      const float* __restrict__ weight, T* __restrict__ out, T* __restrict__ pulled, int n_tokens,
                      int topk, int h) {
  for (int t = blockIdx.x; t < n_tokens; t += gridDim.x) {
    for (int c = threadIdx.x * 8; c < h; c += blockDim.x * 8) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int k = 0; k < topk; ++k) {
        const int i = t * topk + k;
        const T* s = reinterpret_cast<const T*>(src.base[src_rank[i]]) + (size_t)src_row[i] * h + c;
        const uint4 raw = *reinterpret_cast<const uint4*>(s);
        if (pulled) *reinterpret_cast<uint4*>(pulled + (size_t)i * h + c) = raw;
        const T* e = reinterpret_cast<const T*>(&raw);
        const float w = weight ? weight[i] : 1.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += w * to_f(e[q]);
      }
      store8(out + (size_t)t * h + c, acc);
    }
  }
}

}  // namespace mlb

using namespace mlb;

// dst_bases: host array of n_ranks device addresses (peer-mapped buffers of [rows, h] elements of the 2-byte dtype).
MLB_API int mlb_moe_scatter_rows(int dtype, const void* src, const int* src_row, const void* const* dst_bases,
                                 int n_ranks, const int* dst_rank, const int* dst_row, const float* scale,
                                 int n_copies, int h, cudaStream_t st) {
  if (n_copies <= 0) return 0;
  if (n_ranks > kMoeMaxRanks || h % 8) return -3;
  MoePtrs p = {};
  for (int i = 0; i < n_ranks; ++i) p.base[i] = reinterpret_cast<unsigned long long>(dst_bases[i]);
  const unsigned grid = (unsigned)(n_copies < 148 * 16 ? n_copies : 148 * 16);
  if (dtype == MLB_BF16)
    moe_scatter_rows_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)src, src_row, p, dst_rank, dst_row,
                                                                 scale, n_copies, h);
  else if (dtype == MLB_F16)
    moe_scatter_rows_kernel<__half><<<grid, 128, 0, st>>>((const __half*)src, src_row, p, dst_rank, dst_row, scale,
                                                          n_copies, h);
  else return -1;
  MLB_CHECK_LAUNCH();
  return 0;
}

MLB_API int mlb_moe_gather_sum(int dtype, const void* const* src_bases, int n_ranks, const int* src_rank,
                               const int* src_row, const float* weight, void* out, void* pulled, int n_tokens, int topk,
                               int h, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (n_ranks > kMoeMaxRanks || h % 8) return -3;
  MoePtrs p = {};
  for (int i = 0; i < n_ranks; ++i) p.base[i] = reinterpret_cast<unsigned long long>(src_bases[i]);
  const unsigned grid = (unsigned)(n_tokens < 148 * 16 ? n_tokens : 148 * 16);
  if (dtype == MLB_BF16)
    moe_gather_sum_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(p, src_rank, src_row, weight, (__nv_bfloat16*)out,
                                                               (__nv_bfloat16*)pulled, n_tokens, topk, h);
  else if (dtype == MLB_F16)
    moe_gather_sum_kernel<__half><<<grid, 128, 0, st>>>(p, src_rank, src_row, weight, (__half*)out, (__half*)pulled,
                                                        n_tokens, topk, h);
  else return -1;
  MLB_CHECK_LAUNCH();
  return 0;
}
