// State-space (Mamba-2) kernels: depthwise causal conv1d with SiLU (forward, backward) and the
// selective state-space recurrence (forward, with carried state for decoding).
// They stand in for the external causal-conv1d and mamba-ssm kernels the reference calls from
// megatron/core/ssm/mamba_mixer.py:426,480,515,586,661.
//
//   conv : y[b,t,c] = act(bias[c] + sum_j w[c,j] * x[b, t-(K-1)+j, c])        x channel-last [b, l, c]
//   scan : h_t = exp(dt_t A) h_{t-1} + dt_t * x_t (outer) B_t ;  y_t = h_t C_t + D x_t
//          x [b,l,H,P], dt [b,l,H] (already softplus'ed, fp32), A,D [H] fp32, B,C [b,l,G,N], state [b,H,P,N] fp32
#include "common.cuh"

namespace mlb {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }
__device__ __forceinline__ float dsilu_f(float v) { const float s = 1.f / (1.f + __expf(-v)); return s * (1.f + v * (1.f - s)); }

constexpr int kConvSeg = 64;
constexpr int kMaxConvK = 8;

// mode 0: y = act(conv(x));  mode 1: y = dy * act'(conv(x))  (the pre-activation gradient, fp32 out)
template <typename T, typename TO, int MODE>
__global__ void conv1d_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                  const T* __restrict__ dy, TO* __restrict__ out, int L, int C, int K, int silu,
                                  const T* __restrict__ init /* [b, K-1, C] or null */) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t0 = blockIdx.y * kConvSeg, b = blockIdx.z;
  float wk[kMaxConvK], win[kMaxConvK];
  for (int j = 0; j < K; ++j) wk[j] = w[c * K + j];
  const float bs = bias ? bias[c] : 0.f;
  const T* xb = x + (size_t)b * L * C + c;
  for (int j = 0; j < K - 1; ++j) {
    const int t = t0 - (K - 1) + j;
    win[j] = t >= 0 ? to_f(xb[(size_t)t * C]) : (init ? to_f(init[((size_t)b * (K - 1) + (K - 1 + t)) * C + c]) : 0.f);
  }
  for (int t = t0; t < t0 + kConvSeg && t < L; ++t) {
    win[K - 1] = to_f(xb[(size_t)t * C]);
    float acc = bs;
    for (int j = 0; j < K; ++j) acc += wk[j] * win[j];
    float r;
    if (MODE == 0) r = silu ? silu_f(acc) : acc;
    else r = to_f(dy[(size_t)b * L * C + (size_t)t * C + c]) * (silu ? dsilu_f(acc) : 1.f);
    out[(size_t)b * L * C + (size_t)t * C + c] = from_f<TO>(r);
    for (int j = 0; j < K - 1; ++j) win[j] = win[j + 1];
  }
}

// dx[t] = sum_j w[j] * g[t + (K-1-j)];  dw[j] += sum_t g[t] * x[t-(K-1)+j];  dbias += sum_t g[t]
template <typename T>
__global__ void conv1d_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ g,
                                  T* __restrict__ dx, float* __restrict__ dw, float* __restrict__ dbias, int L, int C,
                                  int K) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t0 = blockIdx.y * kConvSeg, b = blockIdx.z;
  float wk[kMaxConvK], dwk[kMaxConvK];
  for (int j = 0; j < K; ++j) { wk[j] = w[c * K + j]; dwk[j] = 0.f; }
  float db = 0.f;
  const size_t base = (size_t)b * L * C + c;
  for (int t = t0; t < t0 + kConvSeg && t < L; ++t) {
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
      const int tt = t + (K - 1 - j);
      if (tt < L) acc += wk[j] * g[base + (size_t)tt * C];
    }
    dx[base + (size_t)t * C] = from_f<T>(acc);
    const float gt = g[base + (size_t)t * C];
    db += gt;
    for (int j = 0; j < K; ++j) {
      const int tt = t - (K - 1) + j;
      if (tt >= 0) dwk[j] += gt * to_f(x[base + (size_t)tt * C]);
    }
  }
  for (int j = 0; j < K; ++j) atomicAdd(dw + c * K + j, dwk[j]);
  if (dbias) atomicAdd(dbias + c, db);
}

// One block per (batch, head).  Thread (p, s) owns state[p][s*NPT .. s*NPT+NPT); the S = N/NPT threads of a row are
// adjacent lanes, so y[p] is a shuffle reduction.  Inputs of kScanChunk steps are staged in shared memory.
constexpr int kScanChunk = 32;
constexpr int NPT = 16;
template <typename T>
__global__ void ssd_scan_kernel(const T* __restrict__ x, const float* __restrict__ dt, const float* __restrict__ A,
                                const T* __restrict__ Bm, const T* __restrict__ Cm, const float* __restrict__ D,
                                const T* __restrict__ z, T* __restrict__ y, float* __restrict__ state, int L, int H,
                                int P, int G, int N, int has_init) {
  extern __shared__ float sm[];
  float* sx = sm;                         // [chunk][P]
  float* sB = sx + kScanChunk * P;        // [chunk][N]
  float* sC = sB + kScanChunk * N;        // [chunk][N]
  float* sdt = sC + kScanChunk * N;       // [chunk]
  const int b = blockIdx.x / H, h = blockIdx.x % H, g = h / (H / G);
  const int S = N / NPT;
  const int p = threadIdx.x / S, s = threadIdx.x % S;
  const float a = A[h], d = D ? D[h] : 0.f;
  float st[NPT];
  float* sp = state ? state + (((size_t)b * H + h) * P + p) * N + s * NPT : nullptr;
#pragma unroll
  for (int i = 0; i < NPT; ++i) st[i] = (has_init && sp) ? sp[i] : 0.f;
  for (int t0 = 0; t0 < L; t0 += kScanChunk) {
    const int nt = min(kScanChunk, L - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * P; i += blockDim.x)
      sx[i] = to_f(x[(((size_t)b * L + t0 + i / P) * H + h) * P + i % P]);
    for (int i = threadIdx.x; i < nt * N; i += blockDim.x) {
      const size_t o = (((size_t)b * L + t0 + i / N) * G + g) * N + i % N;
      sB[i] = to_f(Bm[o]); sC[i] = to_f(Cm[o]);
    }
    for (int i = threadIdx.x; i < nt; i += blockDim.x) sdt[i] = dt[((size_t)b * L + t0 + i) * H + h];
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float dtv = sdt[t], decay = __expf(dtv * a), xv = sx[t * P + p] * dtv;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        st[i] = st[i] * decay + xv * sB[t * N + s * NPT + i];
        acc += st[i] * sC[t * N + s * NPT + i];
      }
      for (int o = S >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (s == 0) {
        float out = acc + d * sx[t * P + p];
        const size_t oi = (((size_t)b * L + t0 + t) * H + h) * P + p;
        if (z) out *= silu_f(to_f(z[oi]));
        y[oi] = from_f<T>(out);
      }
    }
  }
  if (sp) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) sp[i] = st[i];
  }
}

}  // namespace mlb

using namespace mlb;

MLB_API int mlb_causal_conv1d_fwd(int dtype, const void* x, const float* w, const float* bias, const void* init, void* y,
                                  int B, int L, int C, int K, int silu, cudaStream_t st) {
  if (K < 1 || K > kMaxConvK) return -5;
  dim3 grid((C + 127) / 128, (L + kConvSeg - 1) / kConvSeg, B);
  MLB_DISPATCH_ACT(dtype, T, (conv1d_fwd_kernel<T, T, 0><<<grid, 128, 0, st>>>((const T*)x, w, bias, nullptr, (T*)y, L, C, K,
                                                                              silu, (const T*)init)));
  MLB_CHECK_LAUNCH();
  return 0;
}

// g_scratch: fp32 [B, L, C]; dw [C, K] and dbias [C] are accumulated into (fp32, caller zeroes them when needed)
MLB_API int mlb_causal_conv1d_bwd(int dtype, const void* x, const float* w, const float* bias, const void* dy,
                                  float* g_scratch, void* dx, float* dw, float* dbias, int B, int L, int C, int K,
                                  int silu, cudaStream_t st) {
  if (K < 1 || K > kMaxConvK) return -5;
  dim3 grid((C + 127) / 128, (L + kConvSeg - 1) / kConvSeg, B);
  MLB_DISPATCH_ACT(dtype, T, {
    conv1d_fwd_kernel<T, float, 1><<<grid, 128, 0, st>>>((const T*)x, w, bias, (const T*)dy, g_scratch, L, C, K, silu,
                                                         (const T*)nullptr);
    conv1d_bwd_kernel<T><<<grid, 128, 0, st>>>((const T*)x, w, g_scratch, (T*)dx, dw, dbias, L, C, K);
  });
  MLB_CHECK_LAUNCH();
  return 0;
}

// z (optional): gate, y *= silu(z).  state (optional): fp32 [B,H,P,N], read when has_init, always written back.
MLB_API int mlb_ssd_scan_fwd(int dtype, const void* x, const float* dt, const float* A, const void* Bm, const void* Cm,
                             const float* D, const void* z, void* y, float* state, int B, int L, int H, int P, int G, int N,
                             int has_init, cudaStream_t st) {
  if (N % NPT || H % G) return -5;
  const int S = N / NPT;
  if (S > 32 || (S & (S - 1)) || P * S > 1024 || (P * S) % 32) return -5;
  const size_t smem = (size_t)(kScanChunk * (P + 2 * N) + kScanChunk) * sizeof(float);
  if (smem > 48 * 1024) return -5;
  MLB_DISPATCH_ACT(dtype, T, (ssd_scan_kernel<T><<<B * H, P * S, smem, st>>>((const T*)x, dt, A, (const T*)Bm, (const T*)Cm, D,
                                                                            (const T*)z, (T*)y, state, L, H, P, G, N, has_init)));
  MLB_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------------------------------
// Gated group RMSNorm of the Mamba-2 mixer: out = rmsnorm_g(y * silu(z)) * w, the mean square taken over each of G
// contiguous channel groups (reference: megatron/core/ssm/mamba_mixer.py:52, the external library's RMSNormGated with
// norm_before_gate=False).  One thread block per row (grid-stride); a thread owns channels tid*8 + it*2048 so its
// weight-gradient partial sums stay in registers across the rows it sees.  y, z and their gradients carry a row
// stride so z can be the slice of the fused input projection it comes from.
namespace mlb {

constexpr int kGnThreads = 256;
constexpr int kGnMaxIt = 8;                 // channels <= 8 * 256 * 8 = 16384
constexpr int kGnMaxGroups = 64;
// the kernels keep a row's NIT x 8 values per thread in registers: NIT = ceil(channels / 2048) is a template
// parameter, so that narrow rows leave registers for more resident blocks
constexpr int gn_blocks_per_sm(int nit) { return nit <= 2 ? 4 : (nit <= 4 ? 2 : 1); }

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

template <typename T, int NIT>
__global__ void __launch_bounds__(kGnThreads, gn_blocks_per_sm(NIT))
gated_rmsnorm_fwd_kernel(const T* __restrict__ y, const T* __restrict__ z, const float* __restrict__ w,
                         T* __restrict__ out, float* __restrict__ rstd, int rows, int C, int G, long long ys,
                         long long zs, float eps) {
  __shared__ float gsum[kGnMaxGroups];
  const int gs = C / G;
  const bool warp_groups = (gs % 256) == 0;          // every warp's channel span stays inside one group
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    if (threadIdx.x < G) gsum[threadIdx.x] = 0.f;
    __syncthreads();
    float u[NIT][8];
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int c = threadIdx.x * 8 + it * kGnThreads * 8;
      float part = 0.f;
      if (c < C) {
        float a[8], b[8];
        load8(y + (size_t)r * ys + c, a);
        load8(z + (size_t)r * zs + c, b);
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) { u[it][k] = a[k] * b[k] * sigmoidf_(b[k]); ss += u[it][k] * u[it][k]; }
        if (!warp_groups) atomicAdd(&gsum[c / gs], ss);
        part = ss;
      }
      if (warp_groups) {
        // a warp's 256 consecutive channels lie in one group: one shared-memory atomic per warp instead of 32
        const float tot = warp_sum(part);
        if ((threadIdx.x & 31) == 0 && c < C) atomicAdd(&gsum[c / gs], tot);
      }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int c = threadIdx.x * 8 + it * kGnThreads * 8;
      if (c < C) {
        const float rs = rsqrtf(gsum[c / gs] / gs + eps);
        float o[8], wv[8];
        load8(w + c, wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = u[it][k] * rs * wv[k];
        store8(out + (size_t)r * C + c, o);
      }
    }
    if (threadIdx.x < G) rstd[(size_t)r * G + threadIdx.x] = rsqrtf(gsum[threadIdx.x] / gs + eps);
    __syncthreads();
  }
}

template <typename T, int NIT>
__global__ void __launch_bounds__(kGnThreads, NIT <= 2 ? 3 : (NIT <= 4 ? 2 : 1))
gated_rmsnorm_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ y, const T* __restrict__ z,
                         const float* __restrict__ w, const float* __restrict__ rstd, T* __restrict__ dy,
                         T* __restrict__ dz, float* __restrict__ dw, int rows, int C, int G, long long ys,
                         long long zs, long long dys, long long dzs) {
  __shared__ float gdot[kGnMaxGroups];
  const int gs = C / G;
  const bool warp_groups = (gs % 256) == 0;
  float wacc[NIT][8];
#pragma unroll
  for (int it = 0; it < NIT; ++it)
#pragma unroll
    for (int k = 0; k < 8; ++k) wacc[it][k] = 0.f;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    if (threadIdx.x < G) gdot[threadIdx.x] = 0.f;
    __syncthreads();
    // pass 1: mean over the group of (dout * w) * n, n = u * rstd
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int c = threadIdx.x * 8 + it * kGnThreads * 8;
      float part = 0.f;
      if (c < C) {
        float a[8], b[8], g[8], wv[8];
        load8(y + (size_t)r * ys + c, a);
        load8(z + (size_t)r * zs + c, b);
        load8(dout + (size_t)r * C + c, g);
        load8(w + c, wv);
        const float rs = rstd[(size_t)r * G + c / gs];
        float dot = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float n = a[k] * b[k] * sigmoidf_(b[k]) * rs;
          dot += g[k] * wv[k] * n;
          wacc[it][k] += g[k] * n;
        }
        if (!warp_groups) atomicAdd(&gdot[c / gs], dot);
        part = dot;
      }
      if (warp_groups) {
        const float tot = warp_sum(part);
        if ((threadIdx.x & 31) == 0 && c < C) atomicAdd(&gdot[c / gs], tot);
      }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int c = threadIdx.x * 8 + it * kGnThreads * 8;
      if (c < C) {
        float a[8], b[8], g[8], wv[8], oy[8], oz[8];
        load8(y + (size_t)r * ys + c, a);
        load8(z + (size_t)r * zs + c, b);
        load8(dout + (size_t)r * C + c, g);
        load8(w + c, wv);
        const float rs = rstd[(size_t)r * G + c / gs];
        const float md = gdot[c / gs] / gs;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float sg = sigmoidf_(b[k]);
          const float sl = b[k] * sg;                                  // silu(z)
          const float n = a[k] * sl * rs;
          const float du = rs * (g[k] * wv[k] - n * md);
          oy[k] = du * sl;
          oz[k] = du * a[k] * sg * (1.f + b[k] * (1.f - sg));
        }
        store8(dy + (size_t)r * dys + c, oy);
        store8(dz + (size_t)r * dzs + c, oz);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int it = 0; it < NIT; ++it) {
    const int c = threadIdx.x * 8 + it * kGnThreads * 8;
    if (c < C) {
#pragma unroll
      for (int k = 0; k < 8; ++k) atomicAdd(dw + c + k, wacc[it][k]);
    }
  }
}

static bool gn_ok(int rows, int C, int G, long long ys, long long zs) {
  return rows > 0 && C > 0 && C % 8 == 0 && C <= kGnThreads * 8 * kGnMaxIt && G >= 1 && G <= kGnMaxGroups &&
         C % G == 0 && (C / G) % 8 == 0 && ys % 8 == 0 && zs % 8 == 0;
}

}  // namespace mlb

MLB_API int mlb_gated_rmsnorm_fwd(int dtype, const void* y, const void* z, const float* w, void* out, float* rstd,
                                  int rows, int C, int G, long long y_stride, long long z_stride, float eps,
                                  cudaStream_t st) {
  using namespace mlb;
  if (!gn_ok(rows, C, G, y_stride, z_stride)) return -3;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  const int nit = (C + kGnThreads * 8 - 1) / (kGnThreads * 8);
#define GN_FWD(N) MLB_DISPATCH_ACT(dtype, T, (gated_rmsnorm_fwd_kernel<T, N><<<grid, kGnThreads, 0, st>>>( \
      (const T*)y, (const T*)z, w, (T*)out, rstd, rows, C, G, y_stride, z_stride, eps)))
  if (nit <= 1) { GN_FWD(1); } else if (nit <= 2) { GN_FWD(2); } else if (nit <= 4) { GN_FWD(4); } else { GN_FWD(8); }
#undef GN_FWD
  MLB_CHECK_LAUNCH();
  return 0;
}

// dw [C] fp32 is accumulated into: zero it (or pass the running gradient) before the call.
MLB_API int mlb_gated_rmsnorm_bwd(int dtype, const void* dout, const void* y, const void* z, const float* w,
                                  const float* rstd, void* dy, void* dz, float* dw, int rows, int C, int G,
                                  long long y_stride, long long z_stride, long long dy_stride, long long dz_stride,
                                  cudaStream_t st) {
  using namespace mlb;
  if (!gn_ok(rows, C, G, y_stride, z_stride) || dy_stride % 8 != 0 || dz_stride % 8 != 0) return -3;
  const int nit = (C + kGnThreads * 8 - 1) / (kGnThreads * 8);
  const int per_sm = nit <= 2 ? 3 : 2;       // every block ends with one atomic per channel into dw: keep the grid small
  const int grid = rows < 148 * per_sm ? rows : 148 * per_sm;
#define GN_BWD(N) MLB_DISPATCH_ACT(dtype, T, (gated_rmsnorm_bwd_kernel<T, N><<<grid, kGnThreads, 0, st>>>( \
      (const T*)dout, (const T*)y, (const T*)z, w, rstd, (T*)dy, (T*)dz, dw, rows, C, G, y_stride, z_stride, \
      dy_stride, dz_stride)))
  if (nit <= 1) { GN_BWD(1); } else if (nit <= 2) { GN_BWD(2); } else if (nit <= 4) { GN_BWD(4); } else { GN_BWD(8); }
#undef GN_BWD
  MLB_CHECK_LAUNCH();
  return 0;
}
