// Optimizer kernels over flat buffers: chunk-table AdamW / SGD with fused
// gradient unscale+clip and low-precision parameter write-back, two-stage sum
// of squares, in-place scale, zero count.  One launch covers every parameter of
// a buffer regardless of its hyper-parameter group (replaces the multi-tensor
// Apex/TE kernels the reference selects at megatron/core/optimizer/__init__.py:10-25
// and clip_grads.py:51-178, and the copy kernels of distrib_optimizer.py:2030-2125).
#include "common.cuh"

namespace mlb {

struct OptChunk { long long start; int len; int group; };
struct OptGroups {
  float lr[16]; float wd[16];
  float beta1, beta2, eps, bc1, bc2;   // bc = 1 - beta^step
  float momentum;
};

constexpr int kOptThreads = 256;

// Additional destinations of the low-precision parameter copy: the same element range of the parameter buffers of
// the other data-parallel ranks (peer-mapped addresses), so that the update doubles as the parameter all-gather.
struct PeerOut { __nv_bfloat16* ptr[8]; int n; };

// grads are multiplied by *grad_scale (device scalar, may be null = 1); whole launch is a
// no-op when *skip != 0 (overflow found).  p_lp (bf16, optional) receives the updated value.
template <typename G>
__global__ void __launch_bounds__(kOptThreads)
adam_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, const G* __restrict__ g,
            __nv_bfloat16* __restrict__ p_lp, const OptChunk* __restrict__ chunks, OptGroups hp,
            const float* __restrict__ grad_scale, const float* __restrict__ skip, const PeerOut peers) {
  if (skip != nullptr && *skip != 0.f) return;
  const OptChunk c = chunks[blockIdx.x];
  const float gs = grad_scale ? *grad_scale : 1.f;
  const float lr = hp.lr[c.group], wd = hp.wd[c.group];
  const float decay = 1.f - lr * wd, step = lr / hp.bc1, rbc2 = rsqrtf(hp.bc2);
  for (int i = threadIdx.x * 4; i < c.len; i += kOptThreads * 4) {
    const long long o = c.start + i;
    if (i + 4 <= c.len && (o & 3) == 0) {
      float4 pp = *reinterpret_cast<float4*>(p + o), mm = *reinterpret_cast<float4*>(m + o),
             vv = *reinterpret_cast<float4*>(v + o);
      float gg[4];
      if constexpr (sizeof(G) == 4) {
        float4 t = *reinterpret_cast<const float4*>(g + o); gg[0] = t.x; gg[1] = t.y; gg[2] = t.z; gg[3] = t.w;
      } else {
        uint2 t = *reinterpret_cast<const uint2*>(g + o);
        const G* h = reinterpret_cast<const G*>(&t);
        gg[0] = to_f(h[0]); gg[1] = to_f(h[1]); gg[2] = to_f(h[2]); gg[3] = to_f(h[3]);
      }
      float* P = &pp.x; float* M = &mm.x; float* V = &vv.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gr = gg[k] * gs;
        M[k] = hp.beta1 * M[k] + (1.f - hp.beta1) * gr;
        V[k] = hp.beta2 * V[k] + (1.f - hp.beta2) * gr * gr;
        P[k] = P[k] * decay - step * M[k] / (sqrtf(V[k]) * rbc2 + hp.eps);
      }
      *reinterpret_cast<float4*>(p + o) = pp; *reinterpret_cast<float4*>(m + o) = mm;
      *reinterpret_cast<float4*>(v + o) = vv;
      if (p_lp) {
        uint2 t; __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(&t);
#pragma unroll
        for (int k = 0; k < 4; ++k) h[k] = __float2bfloat16_rn(P[k]);
        *reinterpret_cast<uint2*>(p_lp + o) = t;
        for (int q = 0; q < peers.n; ++q) *reinterpret_cast<uint2*>(peers.ptr[q] + o) = t;
      }
    } else {
      for (int k = 0; k < 4 && i + k < c.len; ++k) {
        const long long q = o + k;
        const float gr = to_f(g[q]) * gs;
        const float mk = hp.beta1 * m[q] + (1.f - hp.beta1) * gr;
        const float vk = hp.beta2 * v[q] + (1.f - hp.beta2) * gr * gr;
        const float pk = p[q] * decay - step * mk / (sqrtf(vk) * rbc2 + hp.eps);
        m[q] = mk; v[q] = vk; p[q] = pk;
        if (p_lp) {
          p_lp[q] = __float2bfloat16_rn(pk);
          for (int r = 0; r < peers.n; ++r) peers.ptr[r][q] = __float2bfloat16_rn(pk);
        }
      }
    }
  }
}

template <typename G>
__global__ void __launch_bounds__(kOptThreads)
sgd_kernel(float* __restrict__ p, float* __restrict__ mom, const G* __restrict__ g, __nv_bfloat16* __restrict__ p_lp,
           const OptChunk* __restrict__ chunks, OptGroups hp, const float* __restrict__ grad_scale,
           const float* __restrict__ skip, int first_step) {
  if (skip != nullptr && *skip != 0.f) return;
  const OptChunk c = chunks[blockIdx.x];
  const float gs = grad_scale ? *grad_scale : 1.f;
  const float lr = hp.lr[c.group], wd = hp.wd[c.group];
  for (int i = threadIdx.x; i < c.len; i += kOptThreads) {
    const long long q = c.start + i;
    float gr = to_f(g[q]) * gs + wd * p[q];
    if (hp.momentum != 0.f) {
      const float b = first_step ? gr : hp.momentum * mom[q] + gr;
      mom[q] = b; gr = b;
    }
    const float pk = p[q] - lr * gr;
    p[q] = pk;
    if (p_lp) p_lp[q] = __float2bfloat16_rn(pk);
  }
}

template <typename T>
__global__ void __launch_bounds__(kOptThreads)
sumsq_partial_kernel(const T* __restrict__ x, size_t n, float* __restrict__ partial) {
  __shared__ float sh[64];
  float acc = 0.f;
  const size_t nv = n >> 3;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    float a[8];
    load8(x + i * 8, a);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc += a[k] * a[k];
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) { const float a = to_f(x[(nv << 3) + threadIdx.x]); acc += a * a; }
  acc = block_sum(acc, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int n, float* __restrict__ out, int accumulate) {
  __shared__ float sh[64];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
  acc = block_sum(acc, sh);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + acc : acc;
}

// Gradient reduce-scatter as a pull: out[i] = scale * sum_q src[q][i] over the data-parallel ranks' buffers (peer
// loads), fused with the averaging scale and the sum of squares of the result (per-block partials).
// With `flags` set the kernel first waits (bounded) until every peer has published, in this rank's flag words, that
// its part of the bucket is complete for this step (flags[q] >= target): the pull can then be launched on a side
// stream as soon as the *local* bucket is complete, while the backward pass goes on.
struct PeerIn { const float* ptr[8]; int n; };
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__global__ void __launch_bounds__(kOptThreads)
grad_pull_kernel(const PeerIn src, float* __restrict__ out, size_t n, float scale, float* __restrict__ partial,
                 const uint32_t* __restrict__ flags, int n_flags, uint32_t target, int* status) {
  __shared__ float sh[64];
  __shared__ int give_up;
  if (flags != nullptr) {
    if (threadIdx.x == 0) {
      give_up = 0;
      const long long t0 = clock64();
      for (int q = 0; q < n_flags && !give_up; ++q) {
        uint32_t it = 0;
        while ((int32_t)(ld_acquire_sys_u32(flags + q) - target) < 0) {
          if ((++it & 63u) == 0u) {
            // about twenty seconds: data-parallel ranks may be further apart than tensor-parallel ones
            if (clock64() - t0 > 40000000000LL || (status && *reinterpret_cast<volatile int*>(status) != 0)) {
              if (status) atomicCAS(status, 0, 61);
              give_up = 1;
              break;
            }
            __nanosleep(256);
          }
        }
      }
      __threadfence_system();
    }
    __syncthreads();
    if (give_up) { if (threadIdx.x == 0) partial[blockIdx.x] = 0.f; return; }
  }
  float acc = 0.f;
  const size_t nv = n >> 2;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (q >= src.n) break;
      const float4 t = reinterpret_cast<const float4*>(src.ptr[q])[i];
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = block_sum(acc, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

// one thread publishes `value` in a word of every peer (after everything earlier on the stream has completed)
struct PeerFlags { uint32_t* ptr[8]; int n; };
__global__ void peer_signal_kernel(const PeerFlags f, uint32_t value) {
  __threadfence_system();
  for (int q = 0; q < f.n; ++q) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f.ptr[q]), "r"(value) : "memory");
}

template <typename T>
__global__ void scale_kernel(T* __restrict__ x, size_t n, const float* __restrict__ scale_ptr, float scale) {
  const float s = scale_ptr ? *scale_ptr * scale : scale;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = from_f<T>(to_f(x[i]) * s);
}

template <typename T>
__global__ void count_zeros_kernel(const T* __restrict__ x, size_t n, unsigned long long* __restrict__ out) {
  unsigned long long c = 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    c += (to_f(x[i]) == 0.f);
  c += __shfl_xor_sync(0xffffffffu, c, 16); c += __shfl_xor_sync(0xffffffffu, c, 8);
  c += __shfl_xor_sync(0xffffffffu, c, 4);  c += __shfl_xor_sync(0xffffffffu, c, 2);
  c += __shfl_xor_sync(0xffffffffu, c, 1);
  if ((threadIdx.x & 31) == 0 && c) atomicAdd(out, c);
}

}  // namespace mlb

using namespace mlb;

MLB_API int mlb_sumsq_parts();

static OptGroups make_groups(const float* lr, const float* wd, int ngroups, float b1, float b2, float eps,
                             float bc1, float bc2, float momentum) {
  OptGroups hp;
  for (int i = 0; i < 16; ++i) { hp.lr[i] = i < ngroups ? lr[i] : 0.f; hp.wd[i] = i < ngroups ? wd[i] : 0.f; }
  hp.beta1 = b1; hp.beta2 = b2; hp.eps = eps; hp.bc1 = bc1; hp.bc2 = bc2; hp.momentum = momentum;
  return hp;
}

// chunks: device array of {int64 start, int32 len, int32 group}; lr/wd: host arrays [ngroups<=16]
MLB_API int mlb_adam(int grad_dtype, float* p, float* m, float* v, const void* g, void* p_lp, const void* chunks,
                     int nchunks, const float* lr, const float* wd, int ngroups, float beta1, float beta2,
                     float eps, float bc1, float bc2, const float* grad_scale, const float* skip, cudaStream_t st) {
  if (nchunks <= 0) return 0;
  if (ngroups > 16) return -4;
  OptGroups hp = make_groups(lr, wd, ngroups, beta1, beta2, eps, bc1, bc2, 0.f);
  if (grad_dtype == MLB_F32)
    adam_kernel<float><<<nchunks, kOptThreads, 0, st>>>(p, m, v, (const float*)g, (__nv_bfloat16*)p_lp,
                                                        (const OptChunk*)chunks, hp, grad_scale, skip, PeerOut{});
  else if (grad_dtype == MLB_BF16)
    adam_kernel<__nv_bfloat16><<<nchunks, kOptThreads, 0, st>>>(p, m, v, (const __nv_bfloat16*)g, (__nv_bfloat16*)p_lp,
                                                                (const OptChunk*)chunks, hp, grad_scale, skip, PeerOut{});
  else return -1;
  MLB_CHECK_LAUNCH(); return 0;
}
// AdamW on this rank's shard whose bf16 result is also stored into the same range of n_peers other ranks' parameter
// buffers (peer_lp: host array of device addresses, each already offset to the shard's first element).
MLB_API int mlb_adam_push(float* p, float* m, float* v, const float* g, void* p_lp, void* const* peer_lp, int n_peers,
                          const void* chunks, int nchunks, const float* lr, const float* wd, int ngroups, float beta1,
                          float beta2, float eps, float bc1, float bc2, const float* grad_scale, const float* skip,
                          cudaStream_t st) {
  if (nchunks <= 0) return 0;
  if (ngroups > 16 || n_peers > 8 || p_lp == nullptr) return -4;
  OptGroups hp = make_groups(lr, wd, ngroups, beta1, beta2, eps, bc1, bc2, 0.f);
  PeerOut po = {};
  po.n = n_peers;
  for (int i = 0; i < n_peers; ++i) po.ptr[i] = reinterpret_cast<__nv_bfloat16*>(peer_lp[i]);
  adam_kernel<float><<<nchunks, kOptThreads, 0, st>>>(p, m, v, g, (__nv_bfloat16*)p_lp, (const OptChunk*)chunks, hp,
                                                      grad_scale, skip, po);
  MLB_CHECK_LAUNCH(); return 0;
}
// out[0:n] = scale * sum over n_src buffers (local and peer addresses, fp32, 16-byte aligned, n % 4 == 0);
// sumsq_out[0] (+)= sum of squares of the result.  workspace: fp32 [mlb_sumsq_parts()].
MLB_API int mlb_grad_pull(const void* const* src, int n_src, float* out, long n, float scale, float* sumsq_out,
                          float* workspace, int accumulate, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n_src < 1 || n_src > 8 || (n % 4)) return -3;
  PeerIn pi = {};
  pi.n = n_src;
  for (int i = 0; i < n_src; ++i) pi.ptr[i] = reinterpret_cast<const float*>(src[i]);
  const int parts = mlb_sumsq_parts();
  grad_pull_kernel<<<parts, kOptThreads, 0, st>>>(pi, out, (size_t)n, scale, workspace, nullptr, 0, 0u, nullptr);
  MLB_CHECK_LAUNCH();
  if (sumsq_out) { sumsq_final_kernel<<<1, 256, 0, st>>>(workspace, parts, sumsq_out, accumulate); MLB_CHECK_LAUNCH(); }
  return 0;
}
// The same pull behind a wait on `n_flags` local flag words (each >= target), on at most `max_blocks` blocks
// (0 = the usual grid; a small grid leaves the SMs to the backward pass it overlaps).  workspace: fp32
// [mlb_sumsq_parts()], private to the stream the call runs on.
MLB_API int mlb_grad_pull_when_ready(const void* const* src, int n_src, float* out, long n, float scale,
                                     float* workspace, const void* flags, int n_flags, unsigned target, int max_blocks,
                                     int* status, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n_src < 1 || n_src > 8 || (n % 4) || n_flags < 0 || n_flags > 8) return -3;
  PeerIn pi = {};
  pi.n = n_src;
  for (int i = 0; i < n_src; ++i) pi.ptr[i] = reinterpret_cast<const float*>(src[i]);
  int parts = mlb_sumsq_parts();
  if (max_blocks > 0 && max_blocks < parts) parts = max_blocks;
  grad_pull_kernel<<<parts, kOptThreads, 0, st>>>(pi, out, (size_t)n, scale, workspace,
                                                  reinterpret_cast<const uint32_t*>(flags), n_flags, target, status);
  MLB_CHECK_LAUNCH();
  return 0;
}
// *dst[q] = value for q < n (peer-mapped addresses of 32-bit words), ordered after all earlier work of the stream
MLB_API int mlb_peer_signal(void* const* dst, int n, unsigned value, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n > 8) return -3;
  PeerFlags f = {};
  f.n = n;
  for (int i = 0; i < n; ++i) f.ptr[i] = reinterpret_cast<uint32_t*>(dst[i]);
  peer_signal_kernel<<<1, 1, 0, st>>>(f, value);
  MLB_CHECK_LAUNCH();
  return 0;
}
MLB_API int mlb_sgd(int grad_dtype, float* p, float* mom, const void* g, void* p_lp, const void* chunks, int nchunks,
                    const float* lr, const float* wd, int ngroups, float momentum, int first_step,
                    const float* grad_scale, const float* skip, cudaStream_t st) {
  if (nchunks <= 0) return 0;
  if (ngroups > 16) return -4;
  OptGroups hp = make_groups(lr, wd, ngroups, 0, 0, 0, 1, 1, momentum);
  if (grad_dtype == MLB_F32)
    sgd_kernel<float><<<nchunks, kOptThreads, 0, st>>>(p, mom, (const float*)g, (__nv_bfloat16*)p_lp,
                                                       (const OptChunk*)chunks, hp, grad_scale, skip, first_step);
  else if (grad_dtype == MLB_BF16)
    sgd_kernel<__nv_bfloat16><<<nchunks, kOptThreads, 0, st>>>(p, mom, (const __nv_bfloat16*)g, (__nv_bfloat16*)p_lp,
                                                               (const OptChunk*)chunks, hp, grad_scale, skip, first_step);
  else return -1;
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_sumsq_parts() { return 148 * 4; }
// out[0] (+)= sum x^2.  workspace: fp32 [mlb_sumsq_parts()]
MLB_API int mlb_sumsq(int dtype, const void* x, long n, float* out, float* workspace, int accumulate, cudaStream_t st) {
  const int parts = mlb_sumsq_parts();
  MLB_DISPATCH_ACT(dtype, T, (sumsq_partial_kernel<T><<<parts, kOptThreads, 0, st>>>((const T*)x, (size_t)n, workspace)));
  MLB_CHECK_LAUNCH();
  sumsq_final_kernel<<<1, 256, 0, st>>>(workspace, parts, out, accumulate);
  MLB_CHECK_LAUNCH(); return 0;
}
// x *= (*scale_ptr if given) * scale
MLB_API int mlb_scale(int dtype, void* x, long n, const float* scale_ptr, float scale, cudaStream_t st) {
  size_t g = ((size_t)n + 255) / 256; if (g > 148 * 16) g = 148 * 16; if (g < 1) g = 1;
  MLB_DISPATCH_ACT(dtype, T, (scale_kernel<T><<<(int)g, 256, 0, st>>>((T*)x, (size_t)n, scale_ptr, scale)));
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_count_zeros(int dtype, const void* x, long n, unsigned long long* out, cudaStream_t st) {
  size_t g = ((size_t)n + 255) / 256; if (g > 148 * 8) g = 148 * 8; if (g < 1) g = 1;
  MLB_DISPATCH_ACT(dtype, T, (count_zeros_kernel<T><<<(int)g, 256, 0, st>>>((const T*)x, (size_t)n, out)));
  MLB_CHECK_LAUNCH(); return 0;
}
