// Mixture-of-experts router: score function, top-k choice, dense probability / routing-map rows and the
// per-expert statistics of the load-balancing and z losses in one pass over the logits, and the matching backward
// pass that folds the three gradient sources (token weighting, load-balancing loss, z loss) into one write of
// d(logits).  A group of LPT lanes (4, 8, 16 or 32) owns one token - a warp works on 32 / LPT tokens at a time, so
// the reductions take log2(LPT) shuffle steps and the tokens' dependency chains overlap; lane g of a group holds
// experts g, g + LPT, ... in registers.
//
// Replaces the softmax / topk / scatter / sum chain of the reference router
// (megatron/core/transformer/moe/moe_utils.py:529 topk_softmax_with_capacity, :35 switch_load_balancing_loss_func,
// :107 z_loss_func) for the configurations without capacity dropping or group-limited choice.
#include "common.cuh"
#include <math.h>

namespace mlb {

enum : int { ROUTER_SOFTMAX_POST = 0, ROUTER_SOFTMAX_PRE = 1, ROUTER_SIGMOID = 2 };

constexpr int kRouterWarps = 8;
// resident blocks the register budget is planned for: fewer experts per lane leave room for more warps
constexpr int router_blocks_per_sm(int vpt) { return vpt <= 4 ? 4 : (vpt <= 8 ? 3 : 1); }

struct RouterFwdArgs {
  const float* logits;       // [T, E]
  const float* bias;         // [E] or null: added to the scores for the choice only (sigmoid mode)
  float* probs;              // [T, E] dense, zero off the chosen experts
  unsigned char* rmap;       // [T, E] 1 where chosen
  int* tokens_per_expert;    // [E]  += count
  float* score_sum;          // [E]  += sum over tokens of the full (all-expert) score
  float* z_sum;              // [1]  += sum over tokens of logsumexp^2
  int T, E, topk, mode;
  float scale;               // multiplies the chosen probabilities
};

template <int LPT> __device__ __forceinline__ float grp_sum(float v) {
#pragma unroll
  for (int o = LPT / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <int LPT> __device__ __forceinline__ float grp_max(float v) {
#pragma unroll
  for (int o = LPT / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <int VPT, int LPT>
__global__ void __launch_bounds__(kRouterWarps * 32, router_blocks_per_sm(VPT))
router_fwd_kernel(const RouterFwdArgs a) {
  extern __shared__ float sh[];            // [E] score sums, [E] counts (as int)
  float* sh_score = sh;
  int* sh_cnt = reinterpret_cast<int*>(sh + a.E);
  for (int i = threadIdx.x; i < a.E; i += blockDim.x) { sh_score[i] = 0.f; sh_cnt[i] = 0; }
  __syncthreads();
  constexpr int TPW = 32 / LPT;            // tokens a warp works on at a time
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gl = lane % LPT, grp = lane / LPT;
  float zacc = 0.f;
  // a lane owns the same experts for every token of its group: their statistics stay in registers until the end
  float sacc[VPT]; int cacc[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) { sacc[j] = 0.f; cacc[j] = 0; }
  const int stride = gridDim.x * kRouterWarps * TPW;
  // every lane of the warp runs every iteration (the shuffles are warp-wide); groups past the end work on zeros
  for (int tb = (blockIdx.x * kRouterWarps + warp) * TPW; tb < a.T; tb += stride) {
    const int t = tb + grp;
    const bool valid = t < a.T;
    const float* row = a.logits + (size_t)(valid ? t : 0) * a.E;
    float l[VPT], s[VPT], v[VPT];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int e = gl + LPT * j;
      l[j] = e < a.E ? (valid ? row[e] : 0.f) : -INFINITY;
      m = fmaxf(m, l[j]);
    }
    m = grp_max<LPT>(m);
    float se = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) se += (gl + LPT * j < a.E) ? __expf(l[j] - m) : 0.f;
    se = grp_sum<LPT>(se);
    const float lse = m + __logf(se);
    if (gl == 0 && valid) zacc += lse * lse;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int e = gl + LPT * j;
      const bool ok = e < a.E;
      if (a.mode == ROUTER_SIGMOID) s[j] = ok ? 1.f / (1.f + __expf(-l[j])) : 0.f;
      else s[j] = ok ? __expf(l[j] - lse) : 0.f;
      if (a.mode == ROUTER_SOFTMAX_POST) v[j] = l[j];
      else v[j] = ok ? s[j] + ((a.mode == ROUTER_SIGMOID && a.bias) ? a.bias[e] : 0.f) : -INFINITY;
    }
    // top-k by repeated group arg-max; ties go to the lower expert index
    unsigned chosen = 0;                   // bit j: this lane's j-th expert is chosen
    float first = 0.f, denom = 0.f;        // post-softmax: exp(l - first) summed; sigmoid: chosen scores summed
    for (int k = 0; k < a.topk; ++k) {
      float bv = -INFINITY; int be = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int e = gl + LPT * j;
        if (e < a.E && !((chosen >> j) & 1u) && (v[j] > bv || (v[j] == bv && e < be))) { bv = v[j]; be = e; }
      }
#pragma unroll
      for (int o = LPT / 2; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
      }
      if (be != 0x7fffffff) {              // (topk <= E is checked by the host: an expert is always left)
        if (k == 0) first = bv;
        if (be % LPT == gl) chosen |= 1u << (be / LPT);
        if (a.mode == ROUTER_SOFTMAX_POST) denom += __expf(bv - first);
      }
    }
    if (a.mode == ROUTER_SIGMOID) {
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) d += ((chosen >> j) & 1u) ? s[j] : 0.f;
      denom = grp_sum<LPT>(d) + 1e-20f;
    }
    if (!valid) continue;                  // after the last shuffle of the iteration
    float* prow = a.probs + (size_t)t * a.E;
    unsigned char* mrow = a.rmap + (size_t)t * a.E;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int e = gl + LPT * j;
      if (e >= a.E) continue;
      const bool c = (chosen >> j) & 1u;
      float p = 0.f;
      if (c) {
        if (a.mode == ROUTER_SOFTMAX_POST) p = __expf(l[j] - first) / denom;
        else if (a.mode == ROUTER_SOFTMAX_PRE) p = s[j];
        else p = a.topk > 1 ? s[j] / denom : s[j];
        p *= a.scale;
        cacc[j] += 1;
      }
      prow[e] = p;
      mrow[e] = c ? 1 : 0;
      sacc[j] += s[j];
    }
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int e = gl + LPT * j;
    if (e < a.E) {
      if (cacc[j]) atomicAdd(&sh_cnt[e], cacc[j]);
      if (sacc[j] != 0.f) atomicAdd(&sh_score[e], sacc[j]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < a.E; i += blockDim.x) {
    if (sh_cnt[i]) atomicAdd(a.tokens_per_expert + i, sh_cnt[i]);
    atomicAdd(a.score_sum + i, sh_score[i]);
  }
  if (gl == 0 && zacc != 0.f) atomicAdd(a.z_sum, zacc);
}

struct RouterBwdArgs {
  const float* logits;       // [T, E]
  const unsigned char* rmap; // [T, E]
  const float* dprobs;       // [T, E] gradient of the dense probabilities (read at the chosen experts only)
  const float* aux_coef;     // [E] or null: d(loss)/d(full score of expert e), the same for every token
  float* dlogits;            // [T, E]
  int T, E, topk, mode;
  float scale;               // the forward's scale
  float z_coef;              // d(loss)/d(logsumexp^2) per token (coeff * loss scale / T), 0 to skip
};

template <int VPT, int LPT>
__global__ void __launch_bounds__(kRouterWarps * 32, router_blocks_per_sm(VPT))
router_bwd_kernel(const RouterBwdArgs a) {
  constexpr int TPW = 32 / LPT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gl = lane % LPT, grp = lane / LPT;
  const int stride = gridDim.x * kRouterWarps * TPW;
  for (int tb = (blockIdx.x * kRouterWarps + warp) * TPW; tb < a.T; tb += stride) {
    const int t = tb + grp;
    const bool valid = t < a.T;
    const size_t off = (size_t)(valid ? t : 0) * a.E;
    float l[VPT], g[VPT], dl[VPT];
    unsigned chosen = 0;
    float m = -INFINITY, mc = -INFINITY;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int e = gl + LPT * j;
      const bool ok = e < a.E;
      l[j] = ok ? (valid ? a.logits[off + e] : 0.f) : -INFINITY;
      const bool c = ok && valid && a.rmap[off + e];
      if (c) chosen |= 1u << j;
      g[j] = c ? a.dprobs[off + e] * a.scale : 0.f;
      dl[j] = 0.f;
      m = fmaxf(m, l[j]);
      if (c) mc = fmaxf(mc, l[j]);
    }
    m = grp_max<LPT>(m); mc = grp_max<LPT>(mc);
    float se = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) se += (gl + LPT * j < a.E) ? __expf(l[j] - m) : 0.f;
    se = grp_sum<LPT>(se);
    const float lse = m + __logf(se);
    const bool need_soft = a.mode != ROUTER_SIGMOID || a.z_coef != 0.f;
    float sf[VPT];                          // softmax over all experts
#pragma unroll
    for (int j = 0; j < VPT; ++j) sf[j] = (need_soft && gl + LPT * j < a.E) ? __expf(l[j] - lse) : 0.f;

    if (a.mode == ROUTER_SOFTMAX_POST) {
      float p[VPT], den = 0.f, dot = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) { p[j] = ((chosen >> j) & 1u) ? __expf(l[j] - mc) : 0.f; den += p[j]; }
      den = grp_sum<LPT>(den);
      const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) { p[j] *= inv; dot += p[j] * g[j]; }
      dot = grp_sum<LPT>(dot);
#pragma unroll
      for (int j = 0; j < VPT; ++j) dl[j] = p[j] * (g[j] - dot);
    } else if (a.mode == ROUTER_SOFTMAX_PRE) {
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) dot += sf[j] * g[j];
      dot = grp_sum<LPT>(dot);
#pragma unroll
      for (int j = 0; j < VPT; ++j) dl[j] = sf[j] * (g[j] - dot);
    } else {
      float sg[VPT], den = 0.f, dot = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        sg[j] = (gl + LPT * j < a.E) ? 1.f / (1.f + __expf(-l[j])) : 0.f;
        if ((chosen >> j) & 1u) { den += sg[j]; dot += g[j] * sg[j]; }
      }
      if (a.topk > 1) {
        den = grp_sum<LPT>(den) + 1e-20f; dot = grp_sum<LPT>(dot);
#pragma unroll
        for (int j = 0; j < VPT; ++j)
          if ((chosen >> j) & 1u) dl[j] = (g[j] / den - dot / (den * den)) * sg[j] * (1.f - sg[j]);
      } else {
#pragma unroll
        for (int j = 0; j < VPT; ++j) dl[j] = g[j] * sg[j] * (1.f - sg[j]);
      }
      if (a.aux_coef) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
          const int e = gl + LPT * j;
          if (e < a.E) dl[j] += a.aux_coef[e] * sg[j] * (1.f - sg[j]);
        }
      }
    }
    if (a.aux_coef && a.mode != ROUTER_SIGMOID) {
      float dot = 0.f, c[VPT];
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int e = gl + LPT * j;
        c[j] = e < a.E ? a.aux_coef[e] : 0.f;
        dot += sf[j] * c[j];
      }
      dot = grp_sum<LPT>(dot);
#pragma unroll
      for (int j = 0; j < VPT; ++j) dl[j] += sf[j] * (c[j] - dot);
    }
    if (a.z_coef != 0.f) {
      const float f = 2.f * a.z_coef * lse;
#pragma unroll
      for (int j = 0; j < VPT; ++j) dl[j] += f * sf[j];
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int e = gl + LPT * j;
      if (e < a.E && valid) a.dlogits[off + e] = dl[j];
    }
  }
}

static int router_grid(int T, int tokens_per_warp, int blocks_per_sm) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int per_block = kRouterWarps * tokens_per_warp;
  const int want = (T + per_block - 1) / per_block;
  const int cap = sms * blocks_per_sm;
  return want < cap ? (want > 0 ? want : 1) : cap;
}

}  // namespace mlb

// lanes per token: the smallest group that keeps at most 8 experts per lane (32 lanes from 256 experts on)
#define ROUTER_LAUNCH(KERNEL, V, L, SMEM, ARGS)                                                   \
  mlb::KERNEL<V, L><<<mlb::router_grid(ARGS.T, 32 / L, mlb::router_blocks_per_sm(V)), dim3(mlb::kRouterWarps * 32), SMEM, st>>>(ARGS)
#define ROUTER_DISPATCH(KERNEL, SMEM, ARGS)                                                      \
  do {                                                                                           \
    const int E_ = ARGS.E;                                                                       \
    if (E_ <= 8) ROUTER_LAUNCH(KERNEL, 2, 4, SMEM, ARGS);                                        \
    else if (E_ <= 16) ROUTER_LAUNCH(KERNEL, 4, 4, SMEM, ARGS);                                  \
    else if (E_ <= 32) ROUTER_LAUNCH(KERNEL, 8, 4, SMEM, ARGS);                                  \
    else if (E_ <= 64) ROUTER_LAUNCH(KERNEL, 8, 8, SMEM, ARGS);                                  \
    else if (E_ <= 128) ROUTER_LAUNCH(KERNEL, 8, 16, SMEM, ARGS);                                \
    else if (E_ <= 256) ROUTER_LAUNCH(KERNEL, 8, 32, SMEM, ARGS);                                \
    else if (E_ <= 512) ROUTER_LAUNCH(KERNEL, 16, 32, SMEM, ARGS);                               \
    else ROUTER_LAUNCH(KERNEL, 32, 32, SMEM, ARGS);                                              \
  } while (0)

// tokens_per_expert, score_sum and z_sum are accumulated into: zero them before the call.
MLB_API int mlb_moe_router_fwd(const void* logits, const void* bias, void* probs, void* rmap, void* tokens_per_expert,
                               void* score_sum, void* z_sum, int T, int E, int topk, int mode, float scale,
                               void* stream) {
  if (E < 1 || E > 1024 || topk < 1 || topk > E || mode < 0 || mode > 2) return 1;
  if (T <= 0) return 0;
  mlb::RouterFwdArgs a{(const float*)logits, (const float*)bias, (float*)probs, (unsigned char*)rmap,
                       (int*)tokens_per_expert, (float*)score_sum, (float*)z_sum, T, E, topk, mode, scale};
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)E * 8;
  ROUTER_DISPATCH(router_fwd_kernel, smem, a);
  MLB_CHECK_LAUNCH();
  return 0;
}

MLB_API int mlb_moe_router_bwd(const void* logits, const void* rmap, const void* dprobs, const void* aux_coef,
                               void* dlogits, int T, int E, int topk, int mode, float scale, float z_coef,
                               void* stream) {
  if (E < 1 || E > 1024 || topk < 1 || topk > E || mode < 0 || mode > 2) return 1;
  if (T <= 0) return 0;
  mlb::RouterBwdArgs a{(const float*)logits, (const unsigned char*)rmap, (const float*)dprobs, (const float*)aux_coef,
                       (float*)dlogits, T, E, topk, mode, scale, z_coef};
  cudaStream_t st = (cudaStream_t)stream;
  ROUTER_DISPATCH(router_bwd_kernel, 0, a);
  MLB_CHECK_LAUNCH();
  return 0;
}
