// Bandwidth-bound fused elementwise ops: SwiGLU, bias+GeLU, RoPE,
// bias+dropout+residual, embedding gather / scatter-add, column sums, casts.
// Each replaces an inductor/ATen/TE kernel the reference reaches through
// megatron/core/fusions/fused_bias_swiglu.py:16-98, fused_bias_gelu.py:17-36,
// fused_bias_dropout.py:11-81, models/common/embeddings/rope_utils.py:73-143 and
// tensor_parallel/layers.py:262-295.
#include "common.cuh"

namespace mlb {

constexpr int kEwThreads = 256;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// ---------------------------------------------------------------- SwiGLU
// in [rows, 2f] (first half gate, second half linear), out [rows, f]
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ in, T* __restrict__ out, size_t rows, int f) {
  const int fv = f >> 3;
  const size_t total = rows * (size_t)fv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / fv; const int c = (int)(i % fv) * 8;
    float a[8], b[8], o[8];
    load8(in + r * 2 * f + c, a);
    load8(in + r * 2 * f + f + c, b);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = a[k] * sigmoidf_(a[k]) * b[k];
    store8(out + r * f + c, o);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ in, T* __restrict__ din,
                                  size_t rows, int f) {
  const int fv = f >> 3;
  const size_t total = rows * (size_t)fv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / fv; const int c = (int)(i % fv) * 8;
    float a[8], b[8], g[8], da[8], db[8];
    load8(in + r * 2 * f + c, a);
    load8(in + r * 2 * f + f + c, b);
    load8(dy + r * f + c, g);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = sigmoidf_(a[k]);
      da[k] = g[k] * b[k] * s * (1.f + a[k] * (1.f - s));
      db[k] = g[k] * a[k] * s;
    }
    store8(din + r * 2 * f + c, da);
    store8(din + r * 2 * f + f + c, db);
  }
}

// ---------------------------------------------------------------- bias + GeLU (tanh form)
__device__ __forceinline__ float gelu_f(float x) {
  return 0.5f * x * (1.f + tanhf(0.79788456f * x * (1.f + 0.044715f * x * x)));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float t = tanhf(0.79788456f * x * (1.f + 0.044715f * x * x));
  return 0.5f * x * ((1.f - t * t) * (0.79788456f + 0.1070322243f * x * x)) + 0.5f * (1.f + t);
}
template <typename T>
__global__ void bias_gelu_fwd_kernel(const T* __restrict__ in, const T* __restrict__ bias, T* __restrict__ out,
                                     size_t rows, int f) {
  const int fv = f >> 3;
  const size_t total = rows * (size_t)fv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % fv) * 8;
    float a[8], b[8], o[8];
    load8(in + i * 8, a);
    if (bias) load8(bias + c, b);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = gelu_f(a[k] + (bias ? b[k] : 0.f));
    store8(out + i * 8, o);
  }
}
template <typename T>
__global__ void bias_gelu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ in, const T* __restrict__ bias,
                                     T* __restrict__ din, size_t rows, int f) {
  const int fv = f >> 3;
  const size_t total = rows * (size_t)fv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % fv) * 8;
    float a[8], b[8], g[8], o[8];
    load8(in + i * 8, a);
    load8(dy + i * 8, g);
    if (bias) load8(bias + c, b);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] * gelu_grad_f(a[k] + (bias ? b[k] : 0.f));
    store8(din + i * 8, o);
  }
}

// ---------------------------------------------------------------- column sum (bias gradients)
// x [rows, cols] -> partial [grid.y, cols]; then folded by colsum_reduce.
template <typename T>
__global__ void colsum_partial_kernel(const T* __restrict__ x, float* __restrict__ partial, size_t rows, int cols) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= cols) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (size_t r = blockIdx.y; r < rows; r += gridDim.y) {
    float v[8];
    load8(x + r * cols + c, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += v[k];
  }
  store8(partial + (size_t)blockIdx.y * cols + c, acc);
}
__global__ void colsum_reduce_kernel(const float* __restrict__ partial, int nparts, int cols,
                                     float* __restrict__ out, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float a = 0.f;
  for (int p = 0; p < nparts; ++p) a += partial[(size_t)p * cols + c];
  out[c] = accumulate ? out[c] + a : a;
}

// ---------------------------------------------------------------- RoPE
// t viewed as [s, b, n_outer, n_inner, hn] with element strides; cos/sin fp32 [s, rot/2].
// sign = +1 forward, -1 backward (inverse rotation).  May run in place (src == dst, same strides).
template <typename T>
__global__ void rope_kernel(const T* __restrict__ src, T* __restrict__ dst, const float* __restrict__ cs,
                            const float* __restrict__ sn, int s, int b, int n_outer, int n_inner, int hn,
                            int rot, int interleaved, float sign,
                            long ss_s, long ss_b, long ss_o, long ss_i,
                            long ds_s, long ds_b, long ds_o, long ds_i) {
  const int half = rot >> 1;
  const size_t per_head = (size_t)(hn - half);   // work items per head: half pairs + (hn - rot) passthrough
  const size_t heads = (size_t)s * b * n_outer * n_inner;
  const size_t total = heads * per_head;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int e = (int)(i % per_head);
    size_t hidx = i / per_head;
    const int ii = (int)(hidx % n_inner); hidx /= n_inner;
    const int oo = (int)(hidx % n_outer); hidx /= n_outer;
    const int bb = (int)(hidx % b);
    const int sidx = (int)(hidx / b);
    const T* sp = src + sidx * ss_s + bb * ss_b + oo * ss_o + ii * ss_i;
    T* dp = dst + sidx * ds_s + bb * ds_b + oo * ds_o + ii * ds_i;
    if (e < half) {
      const int i0 = interleaved ? 2 * e : e;
      const int i1 = interleaved ? 2 * e + 1 : e + half;
      const float c = cs[(size_t)sidx * half + e], sv = sign * sn[(size_t)sidx * half + e];
      const float x0 = to_f(sp[i0]), x1 = to_f(sp[i1]);
      dp[i0] = from_f<T>(x0 * c - x1 * sv);
      dp[i1] = from_f<T>(x1 * c + x0 * sv);
    } else {
      const int j = rot + (e - half);
      if (dp != sp) dp[j] = sp[j];
    }
  }
}

// Vector form for the common case: rotate-half pairing, rot/2 a multiple of 8, 16-byte aligned heads.
// One thread rotates 8 pairs: two 16-byte loads of activations, four of cos/sin.
template <typename T>
__global__ void rope_vec_kernel(const T* __restrict__ src, T* __restrict__ dst, const float* __restrict__ cs,
                                const float* __restrict__ sn, int s, int b, int n_outer, int n_inner, int hn,
                                int rot, float sign, long ss_s, long ss_b, long ss_o, long ss_i,
                                long ds_s, long ds_b, long ds_o, long ds_i) {
  const int half = rot >> 1;
  const int vec_per_head = half >> 3;
  const int tail_vec = (hn - rot) >> 3;                     // pass-through channels (copied when out of place)
  const int per_head = vec_per_head + ((src != dst) ? tail_vec : 0);
  const size_t heads = (size_t)s * b * n_outer * n_inner;
  const size_t total = heads * per_head;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % per_head);
    size_t hidx = i / per_head;
    const int ii = (int)(hidx % n_inner); hidx /= n_inner;
    const int oo = (int)(hidx % n_outer); hidx /= n_outer;
    const int bb = (int)(hidx % b);
    const int sidx = (int)(hidx / b);
    const T* sp = src + sidx * ss_s + bb * ss_b + oo * ss_o + ii * ss_i;
    T* dp = dst + sidx * ds_s + bb * ds_b + oo * ds_o + ii * ds_i;
    if (v < vec_per_head) {
      float x0[8], x1[8], c[8], sv[8], o0[8], o1[8];
      load8(sp + v * 8, x0);
      load8(sp + half + v * 8, x1);
      load8(cs + (size_t)sidx * half + v * 8, c);
      load8(sn + (size_t)sidx * half + v * 8, sv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float sg = sign * sv[k];
        o0[k] = x0[k] * c[k] - x1[k] * sg;
        o1[k] = x1[k] * c[k] + x0[k] * sg;
      }
      store8(dp + v * 8, o0);
      store8(dp + half + v * 8, o1);
    } else {
      const int j = rot + (v - vec_per_head) * 8;
      float t[8];
      load8(sp + j, t);
      store8(dp + j, t);
    }
  }
}

// ---------------------------------------------------------------- bias + dropout + residual
__device__ __forceinline__ uint32_t hash32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
  return (uint32_t)x;
}
// out = residual + dropout(x + bias); mask (uint8, optional) saved for backward when p > 0
template <typename T>
__global__ void bias_dropout_add_kernel(const T* __restrict__ x, const T* __restrict__ bias,
                                        const T* __restrict__ residual, T* __restrict__ out,
                                        uint8_t* __restrict__ mask, size_t rows, int h, float p,
                                        uint64_t seed, uint64_t offset) {
  const int hv = h >> 3;
  const size_t total = rows * (size_t)hv;
  const float scale = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const uint32_t thresh = (uint32_t)(p * 4294967295.0);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % hv) * 8;
    float a[8], b[8], r[8], o[8];
    load8(x + i * 8, a);
    load8(residual + i * 8, r);
    if (bias) load8(bias + c, b);
    uint8_t m = 0xff;
    if (p > 0.f) {
      m = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t rnd = hash32(seed * 0x9E3779B97F4A7C15ULL + offset + i * 8 + k);
        if (rnd >= thresh) m |= (uint8_t)(1u << k);
      }
      if (mask) mask[i] = m;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float v = a[k] + (bias ? b[k] : 0.f);
      o[k] = r[k] + (((m >> k) & 1) ? v * scale : 0.f);
    }
    store8(out + i * 8, o);
  }
}
// dx = dout * mask * scale  (residual gradient is dout itself)
template <typename T>
__global__ void dropout_bwd_kernel(const T* __restrict__ dout, const uint8_t* __restrict__ mask, T* __restrict__ dx,
                                   size_t nvec, float p) {
  const float scale = 1.f / (1.f - p);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    float g[8], o[8];
    load8(dout + i * 8, g);
    const uint8_t m = mask[i];
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = ((m >> k) & 1) ? g[k] * scale : 0.f;
    store8(dx + i * 8, o);
  }
}

// ---------------------------------------------------------------- embedding
// out[row] = W[idx[row]-v0] when v0 <= idx < v1, else zeros (vocab-parallel shard)
template <typename T>
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ idx, const T* __restrict__ w, T* __restrict__ out,
                                     size_t rows, int h, int64_t v0, int64_t v1) {
  const int hv = h >> 3;
  const size_t total = rows * (size_t)hv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / hv; const int c = (int)(i % hv) * 8;
    const int64_t t = idx[r];
    uint4 val = make_uint4(0, 0, 0, 0);
    if constexpr (sizeof(T) == 2) {
      if (t >= v0 && t < v1) val = *reinterpret_cast<const uint4*>(w + (size_t)(t - v0) * h + c);
      *reinterpret_cast<uint4*>(out + r * h + c) = val;
    } else {
      float o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (t >= v0 && t < v1) load8(w + (size_t)(t - v0) * h + c, o);
      store8(out + r * h + c, o);
    }
  }
}
// dW[idx[row]-v0] += dy[row]   (fp32 accumulate buffer)
template <typename T>
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ idx, const T* __restrict__ dy,
                                     float* __restrict__ dw, size_t rows, int h, int64_t v0, int64_t v1) {
  const int hv = h >> 3;
  const size_t total = rows * (size_t)hv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / hv; const int c = (int)(i % hv) * 8;
    const int64_t t = idx[r];
    if (t < v0 || t >= v1) continue;
    float g[8];
    load8(dy + r * h + c, g);
    float* d = dw + (size_t)(t - v0) * h + c;
#pragma unroll
    for (int k = 0; k < 8; ++k) atomicAdd(d + k, g[k]);
  }
}

// ---------------------------------------------------------------- casts / axpy
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n, float scale, int accumulate) {
  const size_t nv = n >> 3;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    float a[8];
    load8(in + i * 8, a);
    if (accumulate) {
      float o[8];
      load8(out + i * 8, o);
#pragma unroll
      for (int k = 0; k < 8; ++k) a[k] = o[k] + a[k] * scale;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) a[k] *= scale;
    }
    store8(out + i * 8, a);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    const size_t j = (nv << 3) + threadIdx.x;
    const float v = to_f(in[j]) * scale;
    out[j] = from_f<TO>(accumulate ? to_f(out[j]) + v : v);
  }
}

static inline int ew_grid(size_t work) {
  size_t g = (work + kEwThreads - 1) / kEwThreads;
  const size_t cap = 148 * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace mlb

using namespace mlb;

MLB_API int mlb_swiglu_fwd(int dtype, const void* in, void* out, long rows, int f, cudaStream_t st) {
  if (f % 8) return -3;
  MLB_DISPATCH_ACT(dtype, T, (swiglu_fwd_kernel<T><<<ew_grid(rows * (size_t)(f / 8)), kEwThreads, 0, st>>>(
      (const T*)in, (T*)out, (size_t)rows, f)));
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_swiglu_bwd(int dtype, const void* dy, const void* in, void* din, long rows, int f, cudaStream_t st) {
  if (f % 8) return -3;
  MLB_DISPATCH_ACT(dtype, T, (swiglu_bwd_kernel<T><<<ew_grid(rows * (size_t)(f / 8)), kEwThreads, 0, st>>>(
      (const T*)dy, (const T*)in, (T*)din, (size_t)rows, f)));
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_bias_gelu_fwd(int dtype, const void* in, const void* bias, void* out, long rows, int f, cudaStream_t st) {
  if (f % 8) return -3;
  MLB_DISPATCH_ACT(dtype, T, (bias_gelu_fwd_kernel<T><<<ew_grid(rows * (size_t)(f / 8)), kEwThreads, 0, st>>>(
      (const T*)in, (const T*)bias, (T*)out, (size_t)rows, f)));
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_bias_gelu_bwd(int dtype, const void* dy, const void* in, const void* bias, void* din, long rows, int f,
                              cudaStream_t st) {
  if (f % 8) return -3;
  MLB_DISPATCH_ACT(dtype, T, (bias_gelu_bwd_kernel<T><<<ew_grid(rows * (size_t)(f / 8)), kEwThreads, 0, st>>>(
      (const T*)dy, (const T*)in, (const T*)bias, (T*)din, (size_t)rows, f)));
  MLB_CHECK_LAUNCH(); return 0;
}
// Number of partial rows the column sum uses; workspace is fp32 [parts, cols].
MLB_API int mlb_colsum_parts(long rows) { return rows < 256 ? (rows > 0 ? (int)rows : 1) : 256; }
MLB_API int mlb_colsum(int dtype, const void* x, float* out, float* workspace, long rows, int cols, int accumulate,
                       cudaStream_t st) {
  if (cols % 8) return -3;
  const int parts = mlb_colsum_parts(rows);
  dim3 grid((cols / 8 + 127) / 128, parts);
  MLB_DISPATCH_ACT(dtype, T, (colsum_partial_kernel<T><<<grid, 128, 0, st>>>((const T*)x, workspace, (size_t)rows, cols)));
  MLB_CHECK_LAUNCH();
  colsum_reduce_kernel<<<(cols + 255) / 256, 256, 0, st>>>(workspace, parts, cols, out, accumulate);
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_rope(int dtype, const void* src, void* dst, const float* cs, const float* sn, int s, int b,
                     int n_outer, int n_inner, int hn, int rot, int interleaved, float sign,
                     long ss_s, long ss_b, long ss_o, long ss_i, long ds_s, long ds_b, long ds_o, long ds_i,
                     cudaStream_t st) {
  if (rot % 2 || rot > hn) return -3;
  const int half = rot / 2;
  const long strides[] = {ss_s, ss_b, ss_o, ss_i, ds_s, ds_b, ds_o, ds_i};
  bool vec_ok = !interleaved && half % 8 == 0 && (hn - rot) % 8 == 0 && dtype != MLB_F32 &&
                (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0 &&
                (reinterpret_cast<uintptr_t>(cs) & 31) == 0 && (reinterpret_cast<uintptr_t>(sn) & 31) == 0;
  for (long st_ : strides) vec_ok = vec_ok && (st_ % 8 == 0);
  if (vec_ok) {
    const size_t vwork = (size_t)s * b * n_outer * n_inner * ((half + (src != dst ? hn - rot : 0)) / 8);
    MLB_DISPATCH_ACT(dtype, T, (rope_vec_kernel<T><<<ew_grid(vwork), kEwThreads, 0, st>>>(
        (const T*)src, (T*)dst, cs, sn, s, b, n_outer, n_inner, hn, rot, sign,
        ss_s, ss_b, ss_o, ss_i, ds_s, ds_b, ds_o, ds_i)));
    MLB_CHECK_LAUNCH(); return 0;
  }
  const size_t work = (size_t)s * b * n_outer * n_inner * (hn - rot / 2);
  MLB_DISPATCH_ACT(dtype, T, (rope_kernel<T><<<ew_grid(work), kEwThreads, 0, st>>>(
      (const T*)src, (T*)dst, cs, sn, s, b, n_outer, n_inner, hn, rot, interleaved, sign,
      ss_s, ss_b, ss_o, ss_i, ds_s, ds_b, ds_o, ds_i)));
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_bias_dropout_add(int dtype, const void* x, const void* bias, const void* residual, void* out,
                                 uint8_t* mask, long rows, int h, float p, uint64_t seed, uint64_t offset,
                                 cudaStream_t st) {
  if (h % 8) return -3;
  MLB_DISPATCH_ACT(dtype, T, (bias_dropout_add_kernel<T><<<ew_grid(rows * (size_t)(h / 8)), kEwThreads, 0, st>>>(
      (const T*)x, (const T*)bias, (const T*)residual, (T*)out, mask, (size_t)rows, h, p, seed, offset)));
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_dropout_bwd(int dtype, const void* dout, const uint8_t* mask, void* dx, long n, float p, cudaStream_t st) {
  if (n % 8) return -3;
  MLB_DISPATCH_ACT(dtype, T, (dropout_bwd_kernel<T><<<ew_grid(n / 8), kEwThreads, 0, st>>>(
      (const T*)dout, mask, (T*)dx, (size_t)(n / 8), p)));
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_embedding_fwd(int dtype, const int64_t* idx, const void* w, void* out, long rows, int h,
                              int64_t v0, int64_t v1, cudaStream_t st) {
  if (h % 8) return -3;
  MLB_DISPATCH_ACT(dtype, T, (embedding_fwd_kernel<T><<<ew_grid(rows * (size_t)(h / 8)), kEwThreads, 0, st>>>(
      idx, (const T*)w, (T*)out, (size_t)rows, h, v0, v1)));
  MLB_CHECK_LAUNCH(); return 0;
}
MLB_API int mlb_embedding_bwd(int dtype, const int64_t* idx, const void* dy, float* dw, long rows, int h,
                              int64_t v0, int64_t v1, cudaStream_t st) {
  if (h % 8) return -3;
  MLB_DISPATCH_ACT(dtype, T, (embedding_bwd_kernel<T><<<ew_grid(rows * (size_t)(h / 8)), kEwThreads, 0, st>>>(
      idx, (const T*)dy, dw, (size_t)rows, h, v0, v1)));
  MLB_CHECK_LAUNCH(); return 0;
}
// out = (accumulate ? out : 0) + in * scale, with dtype conversion.  Pointers 16-byte aligned.
MLB_API int mlb_cast(int in_dtype, int out_dtype, const void* in, void* out, long n, float scale, int accumulate,
                     cudaStream_t st) {
  const int grid = ew_grid((size_t)n / 8 + 1);
#define C(TI, TO) cast_kernel<TI, TO><<<grid, kEwThreads, 0, st>>>((const TI*)in, (TO*)out, (size_t)n, scale, accumulate)
  if (in_dtype == MLB_F32 && out_dtype == MLB_BF16) C(float, __nv_bfloat16);
  else if (in_dtype == MLB_BF16 && out_dtype == MLB_F32) C(__nv_bfloat16, float);
  else if (in_dtype == MLB_F32 && out_dtype == MLB_F32) C(float, float);
  else if (in_dtype == MLB_BF16 && out_dtype == MLB_BF16) C(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == MLB_F32 && out_dtype == MLB_F16) C(float, __half);
  else if (in_dtype == MLB_F16 && out_dtype == MLB_F32) C(__half, float);
  else return -1;
#undef C
  MLB_CHECK_LAUNCH(); return 0;
}
