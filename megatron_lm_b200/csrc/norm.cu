// RMSNorm / LayerNorm forward and backward (bandwidth-bound, one pass over x).
//
// Rows are [rows, h] views of [s, b, h] activations.  A block walks rows with a
// grid stride, keeps its slice of the row in registers (h <= 16384), and in the
// backward accumulates its share of dgamma/dbeta in registers; per-block
// partials go to a caller-provided fp32 workspace [grid, 2, h] that a second
// kernel folds into the fp32 gradient (optionally accumulating, for main_grad).
// Replaces the library norms the reference calls at
// megatron/core/extensions/transformer_engine.py:79 and
// megatron/core/fusions/fused_layer_norm.py:137.
#include "common.cuh"

namespace mlb {

constexpr int kNormThreads = 256;

template <typename T, int NV, bool RMS>
__global__ void __launch_bounds__(kNormThreads)
norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                int rows, int h, float eps, int zero_centered) {
  __shared__ float sh[64];
  const int nvec = h >> 3;
  float g[NV][8], b[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      load8(gamma + v * 8, g[i]);
      if (zero_centered) {
#pragma unroll
        for (int k = 0; k < 8; ++k) g[i][k] += 1.f;
      }
      if (!RMS && beta != nullptr) load8(beta + v * 8, b[i]);
      else {
#pragma unroll
        for (int k = 0; k < 8; ++k) b[i][k] = 0.f;
      }
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + (size_t)row * h;
    float xv[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        load8(xr + v * 8, xv[i]);
#pragma unroll
        for (int k = 0; k < 8; ++k) { s1 += xv[i][k]; s2 += xv[i][k] * xv[i][k]; }
      }
    }
    block_sum2(s1, s2, sh);
    float mean = 0.f, rstd;
    if (RMS) {
      rstd = rsqrtf(s2 / h + eps);
    } else {
      mean = s1 / h;
      float var = fmaxf(s2 / h - mean * mean, 0.f);
      rstd = rsqrtf(var + eps);
    }
    if (threadIdx.x == 0) {
      rstd_out[row] = rstd;
      if (!RMS) mean_out[row] = mean;
    }
    T* yr = y + (size_t)row * h;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = (xv[i][k] - mean) * rstd * g[i][k] + b[i][k];
        store8(yr + v * 8, o);
      }
    }
  }
}

template <typename T, int NV, bool RMS>
__global__ void __launch_bounds__(kNormThreads)
norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                T* __restrict__ dx, float* __restrict__ partial /*[grid,2,h]*/,
                int rows, int h, int zero_centered) {
  __shared__ float sh[64];
  const int nvec = h >> 3;
  float g[NV][8], dg[NV][8], db[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
#pragma unroll
    for (int k = 0; k < 8; ++k) { dg[i][k] = 0.f; db[i][k] = 0.f; }
    if (v < nvec) {
      load8(gamma + v * 8, g[i]);
      if (zero_centered) {
#pragma unroll
        for (int k = 0; k < 8; ++k) g[i][k] += 1.f;
      }
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + (size_t)row * h;
    const T* dyr = dy + (size_t)row * h;
    const float rstd = rstd_in[row];
    const float mean = RMS ? 0.f : mean_in[row];
    float xh[NV][8], gy[NV][8];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float d[8];
        load8(xr + v * 8, xh[i]);
        load8(dyr + v * 8, d);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[i][k] = (xh[i][k] - mean) * rstd;
          gy[i][k] = d[k] * g[i][k];
          c1 += gy[i][k];
          c2 += gy[i][k] * xh[i][k];
          dg[i][k] += d[k] * xh[i][k];
          db[i][k] += d[k];
        }
      }
    }
    block_sum2(c1, c2, sh);
    c1 = RMS ? 0.f : c1 / h;
    c2 /= h;
    T* dxr = dx + (size_t)row * h;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rstd * (gy[i][k] - c1 - xh[i][k] * c2);
        store8(dxr + v * 8, o);
      }
    }
  }
  float* pg = partial + (size_t)blockIdx.x * 2 * h;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      store8(pg + v * 8, dg[i]);
      if (!RMS) store8(pg + h + v * 8, db[i]);
    }
  }
}

// Fold [nparts, 2, h] partials into dgamma (and dbeta).  A block owns 32 columns; its 8 warps split the
// partial rows, each lane keeps one column (coalesced 128-byte reads), and shared memory joins the warps.
__global__ void __launch_bounds__(256)
norm_bwd_reduce_kernel(const float* __restrict__ partial, int nparts, int h, float* __restrict__ dgamma,
                       float* __restrict__ dbeta, int accumulate) {
  __shared__ float sa[8][32], sb[8][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float a = 0.f, b = 0.f;
  if (c < h) {
    for (int p = w; p < nparts; p += 8) {
      a += partial[(size_t)p * 2 * h + c];
      if (dbeta) b += partial[(size_t)p * 2 * h + h + c];
    }
  }
  sa[w][lane] = a; sb[w][lane] = b;
  __syncthreads();
  if (w == 0 && c < h) {
#pragma unroll
    for (int k = 1; k < 8; ++k) { a += sa[k][lane]; b += sb[k][lane]; }
    if (accumulate) { dgamma[c] += a; if (dbeta) dbeta[c] += b; }
    else { dgamma[c] = a; if (dbeta) dbeta[c] = b; }
  }
}

static int pick_nv(int h) {
  int nvec = h / 8;
  int nv = (nvec + kNormThreads - 1) / kNormThreads;
  if (nv <= 1) return 1;
  if (nv <= 2) return 2;
  if (nv <= 4) return 4;
  if (nv <= 8) return 8;
  return -1;
}

template <typename T, bool RMS>
static int launch_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                      int rows, int h, float eps, int zc, int grid, cudaStream_t st) {
  const int nv = pick_nv(h);
#define L(NV) norm_fwd_kernel<T, NV, RMS><<<grid, kNormThreads, 0, st>>>((const T*)x, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, h, eps, zc)
  switch (nv) { case 1: L(1); break; case 2: L(2); break; case 4: L(4); break; case 8: L(8); break; default: return -2; }
#undef L
  MLB_CHECK_LAUNCH();
  return 0;
}

template <typename T, bool RMS>
static int launch_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                      void* dx, float* partial, int rows, int h, int zc, int grid, cudaStream_t st) {
  const int nv = pick_nv(h);
#define L(NV) norm_bwd_kernel<T, NV, RMS><<<grid, kNormThreads, 0, st>>>((const T*)dy, (const T*)x, (const T*)gamma, mean, rstd, (T*)dx, partial, rows, h, zc)
  switch (nv) { case 1: L(1); break; case 2: L(2); break; case 4: L(4); break; case 8: L(8); break; default: return -2; }
#undef L
  MLB_CHECK_LAUNCH();
  return 0;
}

}  // namespace mlb

// Number of blocks (and therefore workspace rows) the backward uses.
MLB_API int mlb_norm_bwd_grid(int rows) {
  int g = 148 * 4;
  return rows < g ? (rows > 0 ? rows : 1) : g;
}

MLB_API int mlb_norm_fwd(int dtype, int rms, const void* x, const void* gamma, const void* beta, void* y,
                         float* mean, float* rstd, int rows, int h, float eps, int zero_centered,
                         cudaStream_t st) {
  if (h % 8 != 0 || rows <= 0) return -3;
  int grid = rows < 148 * 8 ? rows : 148 * 8;
  MLB_DISPATCH_ACT(dtype, T, {
    return rms ? mlb::launch_fwd<T, true>(x, gamma, beta, y, mean, rstd, rows, h, eps, zero_centered, grid, st)
               : mlb::launch_fwd<T, false>(x, gamma, beta, y, mean, rstd, rows, h, eps, zero_centered, grid, st);
  });
  return 0;
}

// workspace: fp32 [mlb_norm_bwd_grid(rows), 2, h].  dgamma/dbeta are fp32 [h].
MLB_API int mlb_norm_bwd(int dtype, int rms, const void* dy, const void* x, const void* gamma,
                         const float* mean, const float* rstd, void* dx, float* dgamma, float* dbeta,
                         float* workspace, int rows, int h, int zero_centered, int accumulate,
                         cudaStream_t st) {
  if (h % 8 != 0 || rows <= 0) return -3;
  const int grid = mlb_norm_bwd_grid(rows);
  int rc;
  MLB_DISPATCH_ACT(dtype, T, {
    rc = rms ? mlb::launch_bwd<T, true>(dy, x, gamma, mean, rstd, dx, workspace, rows, h, zero_centered, grid, st)
             : mlb::launch_bwd<T, false>(dy, x, gamma, mean, rstd, dx, workspace, rows, h, zero_centered, grid, st);
  });
  if (rc) return rc;
  mlb::norm_bwd_reduce_kernel<<<(h + 31) / 32, 256, 0, st>>>(workspace, grid, h, dgamma, rms ? nullptr : dbeta,
                                                               accumulate);
  MLB_CHECK_LAUNCH();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant (declared and documented in norm_noalloc.h).
#include "norm_noalloc.h"
#include <mutex>

namespace mlb {
constexpr int kNoAllocBlocks = 148;
constexpr int kNoAllocMaxH = 8192;
// Partial sums [kNoAllocBlocks][2][h].  In host code this name is only a handle for
// cudaGetSymbolAddress; kernels are given the resolved device pointer.
static __device__ __align__(256) float g_norm_noalloc_scratch[kNoAllocBlocks * 2 * kNoAllocMaxH];

constexpr int kMaxDevices = 64;
static float* g_noalloc_ptr[kMaxDevices] = {};
static std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device (resolved on first use per device).
static int noalloc_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return MLB_NOALLOC_NO_SYMBOL;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_norm_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return MLB_NOALLOC_NO_SYMBOL;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace mlb

MLB_API int mlb_norm_bwd_noalloc_max_h(void) { return mlb::kNoAllocMaxH; }

MLB_API int mlb_norm_bwd_noalloc(int dtype, int rms, const void* dy, const void* x, const void* gamma,
                                 const float* mean, const float* rstd, void* dx, float* dgamma, float* dbeta,
                                 int rows, int h, int zero_centered, int accumulate, cudaStream_t st) {
  if (rows < 1 || h < 8 || (h % 8) != 0 || h > mlb::kNoAllocMaxH) return MLB_NOALLOC_BAD_SIZE;
  if (dtype != MLB_F32 && dtype != MLB_BF16 && dtype != MLB_F16) return MLB_NOALLOC_BAD_DTYPE;
  float* scratch = nullptr;
  int rc = mlb::noalloc_scratch(&scratch);
  if (rc) return rc;
  const int grid = rows < mlb::kNoAllocBlocks ? rows : mlb::kNoAllocBlocks;
  MLB_DISPATCH_ACT(dtype, T, {
    rc = rms ? mlb::launch_bwd<T, true>(dy, x, gamma, mean, rstd, dx, scratch, rows, h, zero_centered, grid, st)
             : mlb::launch_bwd<T, false>(dy, x, gamma, mean, rstd, dx, scratch, rows, h, zero_centered, grid, st);
  });
  if (rc) return rc;
  mlb::norm_bwd_reduce_kernel<<<(h + 31) / 32, 256, 0, st>>>(scratch, grid, h, dgamma, rms ? nullptr : dbeta,
                                                             accumulate);
  MLB_CHECK_LAUNCH();
  return 0;
}
