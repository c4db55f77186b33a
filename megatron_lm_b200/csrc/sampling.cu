// Token sampling for generation: temperature, top-k, top-p (nucleus) filtering and the multinomial draw in one kernel,
// one thread block per sequence, without sorting the vocabulary.
//
//   1. max and sum of exp((x - max) / T) over the row;
//   2. the filter threshold by a 4-pass radix select over the order-preserving integer image of the logits: the
//      k-th largest value for top-k (buckets count elements), or the value at which the probability mass of the
//      strictly larger logits first stays within p for top-p (buckets hold probability mass);
//   3. the draw: every warp owns a contiguous slice of the vocabulary, sums the kept mass of its slice, the block
//      scans the 32 slice sums, and the warp whose slice contains u * (kept mass) walks it 32 tokens at a time.
//
// Replaces the sort / cumsum / masked_fill / multinomial chain of the reference sampler
// (megatron/core/inference/text_generation_controllers/text_generation_controller.py:164 sample_from_logits,
// megatron/inference/text_generation/sampling.py:45).  Ties at the threshold are all kept, as in the reference's
// `logits < kth` / cumulative-mass rule.
#include "common.cuh"
#include <math.h>

namespace mlb {

constexpr int kSampleThreads = 1024;
constexpr int kSampleWarps = kSampleThreads / 32;

// float -> unsigned that sorts the same way (larger float -> larger key)
__device__ __forceinline__ unsigned order_key(float x) {
  const unsigned b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(unsigned k) {
  const unsigned b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(b);
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const T* __restrict__ logits, const float* __restrict__ uniform, long long* __restrict__ out,
              int V, long long row_stride, float inv_temp, int top_k, float top_p) {
  __shared__ float red[2 * 32];
  __shared__ float hist[256];
  __shared__ unsigned sh_prefix;
  __shared__ float sh_remaining;
  __shared__ float warp_mass[kSampleWarps];
  __shared__ int sh_token;
  const T* row = logits + (size_t)blockIdx.x * row_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---- 1. max (and arg-max for the greedy case), then the softmax denominator
  float m = -INFINITY; int am = 0x7fffffff;
  for (int i = tid; i < V; i += kSampleThreads) {
    const float x = to_f(row[i]) * inv_temp;
    if (x > m) { m = x; am = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const int oa = __shfl_xor_sync(0xffffffffu, am, o);
    if (om > m || (om == m && oa < am)) { m = om; am = oa; }
  }
  __shared__ int red_i[32];
  if (lane == 0) { red[warp] = m; red_i[warp] = am; }
  __syncthreads();
  if (warp == 0) {
    m = red[lane]; am = red_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oa = __shfl_xor_sync(0xffffffffu, am, o);
      if (om > m || (om == m && oa < am)) { m = om; am = oa; }
    }
    if (lane == 0) { red[0] = m; red_i[0] = am; }
  }
  __syncthreads();
  m = red[0]; am = red_i[0];
  __syncthreads();
  if (top_k == 1) {
    if (tid == 0) out[blockIdx.x] = am;
    return;
  }
  float z = 0.f;
  for (int i = tid; i < V; i += kSampleThreads) z += __expf(to_f(row[i]) * inv_temp - m);
  z = block_sum(z, red);
  const float inv_z = 1.f / z;

  // ---- 2. threshold key: everything with key >= thr is kept
  unsigned thr = 0u;
  const bool by_count = top_k > 1 && top_k < V;
  const bool by_mass = !by_count && top_p > 0.f && top_p < 1.f;
  if (by_count || by_mass) {
    if (tid == 0) { sh_prefix = 0u; sh_remaining = by_count ? (float)top_k : top_p; }
    __syncthreads();
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      const unsigned prefix = sh_prefix;
      if (tid < 256) hist[tid] = 0.f;
      __syncthreads();
      // Logits of one row crowd into a few buckets (in the first pass: the same sign and exponent), so lanes of a
      // warp mostly hit one address.  Lanes that share a bucket are combined first: counts by a peer mask, masses
      // by a warp sum when the whole warp agrees; only the rest falls back to one atomic per lane.
      const int v_round = (V + kSampleThreads - 1) / kSampleThreads * kSampleThreads;
      for (int i = tid; i < v_round; i += kSampleThreads) {
        float x = 0.f; unsigned k = 0u; bool in = false;
        if (i < V) { x = to_f(row[i]) * inv_temp; k = order_key(x); in = (k & mask) == prefix; }
        const unsigned bucket = in ? ((k >> shift) & 255u) : 256u;          // 256: not a candidate
        const unsigned peers = __match_any_sync(0xffffffffu, bucket);
        if (by_count) {
          if (in && lane == __ffs(peers) - 1) atomicAdd(&hist[bucket], (float)__popc(peers));
        } else {
          const float w = in ? __expf(x - m) * inv_z : 0.f;
          if (peers == 0xffffffffu) {                                        // warp-uniform bucket
            const float sum = warp_sum(w);
            if (in && lane == 0) atomicAdd(&hist[bucket], sum);
          } else {
            // mixed buckets in the warp: every lane adds up the weights of the lanes that share its bucket (all
            // lanes run the same 32 shuffles), and the lowest lane of each group issues the one atomic
            float sum = 0.f;
#pragma unroll
            for (int src = 0; src < 32; ++src) {
              const float ws = __shfl_sync(0xffffffffu, w, src);
              if ((peers >> src) & 1u) sum += ws;
            }
            if (in && lane == __ffs(peers) - 1) atomicAdd(&hist[bucket], sum);
          }
        }
      }
      __syncthreads();
      if (tid == 0) {
        // walk the buckets from the largest values down; stop in the bucket where the budget runs out
        float rem = sh_remaining;
        int b = 255;
        for (; b > 0; --b) {
          const float h = hist[b];
          if (by_count ? (h >= rem) : (h > rem)) break;
          rem -= h;
        }
        sh_prefix = prefix | ((unsigned)b << shift);
        sh_remaining = rem;
      }
      __syncthreads();
    }
    thr = sh_prefix;
  }
  const float thr_f = (by_count || by_mass) ? key_to_float(thr) : -INFINITY;

  // ---- 3. draw in index order
  const int per_warp = ((V + kSampleWarps - 1) / kSampleWarps + 31) & ~31;
  const int begin = warp * per_warp, end = min(V, begin + per_warp);
  float mass = 0.f;
  for (int i = begin + lane; i < end; i += 32) {
    const float x = to_f(row[i]) * inv_temp;
    mass += (x >= thr_f) ? __expf(x - m) : 0.f;
  }
  mass = warp_sum(mass);
  if (lane == 0) warp_mass[warp] = mass;
  if (tid == 0) sh_token = -1;
  __syncthreads();
  float total = 0.f, before = 0.f;
  for (int w = 0; w < kSampleWarps; ++w) { if (w == warp) before = total; total += warp_mass[w]; }
  const float target = uniform[blockIdx.x] * total;
  // the owning warp: the first whose cumulative mass exceeds the target (the last non-empty one catches rounding)
  const bool mine = target >= before && target < before + mass;
  if (mine && mass > 0.f) {
    float run = before; int found = -1, last_kept = -1;
    for (int base = begin; base < end && found < 0; base += 32) {
      const int i = base + lane;
      float p = 0.f;
      if (i < end) { const float x = to_f(row[i]) * inv_temp; p = (x >= thr_f) ? __expf(x - m) : 0.f; }
      float inc = p;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const float v = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += v; }
      const bool hit = p > 0.f && run + inc > target;
      const unsigned ballot = __ballot_sync(0xffffffffu, hit);
      const unsigned kept = __ballot_sync(0xffffffffu, p > 0.f);
      if (kept) last_kept = base + 31 - __clz(kept);
      if (ballot) found = base + __ffs(ballot) - 1;
      run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (found < 0) found = last_kept;
    if (lane == 0) sh_token = found;
  }
  __syncthreads();
  if (tid == 0) {
    int tok = sh_token;
    if (tok < 0) tok = am;                 // rounding left no owner: the most likely token
    out[blockIdx.x] = tok;
  }
}

}  // namespace mlb

// logits [rows, V] (row stride in elements), uniform [rows] in [0, 1), out [rows] int64.
// top_k == 1: arg-max.  top_k > 1: keep the k largest.  else 0 < top_p < 1: nucleus.  else: plain multinomial.
MLB_API int mlb_sample(int dtype, const void* logits, const void* uniform, void* out, int rows, int V,
                       long long row_stride, float temperature, int top_k, float top_p, void* stream) {
  if (rows <= 0) return 0;
  if (V <= 0 || temperature <= 0.f) return 1;
  cudaStream_t st = (cudaStream_t)stream;
  const float it = 1.f / temperature;
  switch (dtype) {
    case MLB_F32:
      mlb::sample_kernel<float><<<rows, mlb::kSampleThreads, 0, st>>>((const float*)logits, (const float*)uniform,
                                                                      (long long*)out, V, row_stride, it, top_k, top_p);
      break;
    case MLB_BF16:
      mlb::sample_kernel<__nv_bfloat16><<<rows, mlb::kSampleThreads, 0, st>>>(
          (const __nv_bfloat16*)logits, (const float*)uniform, (long long*)out, V, row_stride, it, top_k, top_p);
      break;
    case MLB_F16:
      mlb::sample_kernel<__half><<<rows, mlb::kSampleThreads, 0, st>>>((const __half*)logits, (const float*)uniform,
                                                                       (long long*)out, V, row_stride, it, top_k, top_p);
      break;
    default: return 2;
  }
  MLB_CHECK_LAUNCH();
  return 0;
}
