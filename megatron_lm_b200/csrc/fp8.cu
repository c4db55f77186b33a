// FP8 quantisation kernels.
//   mlb_amax            : max |x| of a tensor into a device float (atomic max on the bit pattern)
//   mlb_fp8_cast_transpose : per-tensor ("current") scaling cast to e4m3 / e5m2, producing the row-major copy and,
//                         optionally, its transpose in the same pass (the FP8 GEMM takes K-major operands only,
//                         so dgrad / wgrad read the transposed copies)
//   mlb_mxfp8_quantize  : microscaling format - 32-element blocks along the row (or along the column) share one
//                         power-of-two scale stored as an E8M0 byte
// They cover what the reference obtains from Transformer Engine through megatron/core/fp8_utils.py:413-532
// (recipes "tensorwise" and "mxfp8") and the parameter cast of :394.
#include "common.cuh"
#include <cuda_fp8.h>

namespace mlb {

template <typename T>
__global__ void amax_kernel(const T* __restrict__ x, size_t n, float* __restrict__ amax) {
  __shared__ float sh[32];
  float m = 0.f;
  const size_t stride = (size_t)gridDim.x * blockDim.x * 8;
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
    if (i + 8 <= n) {
      float v[8]; load8(x + i, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(v[k]));
    } else {
      for (size_t k = i; k < n; ++k) m = fmaxf(m, fabsf(to_f(x[k])));
    }
  }
  m = block_max(m, sh);
  if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));
}

__device__ __forceinline__ uint8_t to_fp8(float v, int e5m2) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, e5m2 ? __NV_E5M2 : __NV_E4M3);
}

// 64 x 64 tile per block of 256 threads
template <typename T>
__global__ void cast_transpose_kernel(const T* __restrict__ x, const float* __restrict__ amax, uint8_t* __restrict__ q,
                                      uint8_t* __restrict__ qt, float* __restrict__ scale_inv, int rows, int cols,
                                      int e5m2) {
  __shared__ uint8_t tile[64][64 + 16];
  const float fmax = e5m2 ? 57344.f : 448.f;
  const float a = *amax;
  const float scale = (a > 0.f && isfinite(a)) ? fmax / a : 1.f;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *scale_inv = 1.f / scale;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tr = threadIdx.x >> 2, tc = (threadIdx.x & 3) * 16;
  const int r = r0 + tr, c = c0 + tc;
  uint4 packed = make_uint4(0, 0, 0, 0);
  if (r < rows && c < cols) {
    float v[16];
    load8(x + (size_t)r * cols + c, *reinterpret_cast<float(*)[8]>(v));
    load8(x + (size_t)r * cols + c + 8, *reinterpret_cast<float(*)[8]>(v + 8));
    uint8_t* b = reinterpret_cast<uint8_t*>(&packed);
#pragma unroll
    for (int i = 0; i < 16; ++i) b[i] = to_fp8(v[i] * scale, e5m2);
    *reinterpret_cast<uint4*>(q + (size_t)r * cols + c) = packed;
  }
  if (qt == nullptr) return;
  *reinterpret_cast<uint4*>(&tile[tr][tc]) = packed;
  __syncthreads();
  const int oc = c0 + tr;                  // source column = destination row
  const int orow = r0 + tc;                // first of 16 source rows = destination columns
  if (oc < cols && orow < rows) {
    uint4 o; uint8_t* b = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
    for (int i = 0; i < 16; ++i) b[i] = tile[tc + i][tr];
    *reinterpret_cast<uint4*>(qt + (size_t)oc * rows + orow) = o;
  }
}

__device__ __forceinline__ int e8m0_exponent(float amax) {
  // smallest power of two s.t. amax / 2^e <= 448 (largest e4m3 magnitude)
  if (!(amax > 0.f)) return -127;
  int e = (int)ceilf(log2f(amax / 448.f));
  return max(-127, min(127, e));
}

// row-wise: one thread per 32-element block
template <typename T>
__global__ void mxfp8_row_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sc, int rows,
                                 int cols) {
  const int bpr = cols / 32;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * bpr) return;
  const size_t off = i * 32;
  float v[32];
#pragma unroll
  for (int k = 0; k < 4; ++k) load8(x + off + 8 * k, *reinterpret_cast<float(*)[8]>(v + 8 * k));
  float m = 0.f;
#pragma unroll
  for (int k = 0; k < 32; ++k) m = fmaxf(m, fabsf(v[k]));
  const int e = e8m0_exponent(m);
  const float s = exp2f((float)-e);
  uint4 o[2]; uint8_t* b = reinterpret_cast<uint8_t*>(o);
#pragma unroll
  for (int k = 0; k < 32; ++k) b[k] = to_fp8(v[k] * s, 0);
  reinterpret_cast<uint4*>(q + off)[0] = o[0];
  reinterpret_cast<uint4*>(q + off)[1] = o[1];
  sc[i] = (uint8_t)(e + 127);
}

// column-wise: blocks of 32 consecutive rows of one column; thread per column, coalesced across the warp
template <typename T>
__global__ void mxfp8_col_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sc, int rows,
                                 int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int rb = blockIdx.y;
  if (c >= cols) return;
  float v[32];
  float m = 0.f;
#pragma unroll
  for (int k = 0; k < 32; ++k) { v[k] = to_f(x[(size_t)(rb * 32 + k) * cols + c]); m = fmaxf(m, fabsf(v[k])); }
  const int e = e8m0_exponent(m);
  const float s = exp2f((float)-e);
#pragma unroll
  for (int k = 0; k < 32; ++k) q[(size_t)(rb * 32 + k) * cols + c] = to_fp8(v[k] * s, 0);
  sc[(size_t)rb * cols + c] = (uint8_t)(e + 127);
}

// Scale byte of (row r, K block kb) of a [rows, K] matrix in the "atom" layout the block-scaled GEMM copies to
// tensor memory (gemm_mx.cu): atoms of 128 rows x 4 K blocks, 512 bytes each, row-block major.
__device__ __forceinline__ size_t mx_sf_offset(int r, int kb, int kb4_per_row) {
  return ((size_t)(r >> 7) * kb4_per_row + (kb >> 2)) * 512 + (size_t)(r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3);
}
__device__ __forceinline__ int e8m0_exponent_for(float amax, float fmax) {
  if (!(amax > 0.f)) return -127;
  int e = (int)ceilf(log2f(amax / fmax));
  return max(-127, min(127, e));
}

// One pass over x [rows, cols] for both MXFP8 copies a training GEMM needs:
//   q_row  [rows, cols] : 32-element blocks along the row share a scale (operand with `cols` as reduction dim)
//   q_colT [cols, rows] : x transposed, 32-element blocks along the *source column* share a scale (operand with
//                         `rows` as reduction dim: data gradient of a weight, both weight-gradient operands)
// with their scales in the atom layout.  64 x 128 tile per block of 256 threads.  A thread owns one whole scale
// block in either phase - 32 values of a row (64 contiguous bytes in, 32 out), then 32 values of a column read out
// of the shared tile with consecutive lanes on consecutive columns (conflict free) and written as 32 contiguous
// bytes of the transposed copy - so there is no exchange between lanes and every global access fills its sectors.
__device__ __forceinline__ int e8m0_exponent_bits(float amax, float fmax) {
  // ceil(log2(amax / fmax)) from the bits of the quotient: exponent, plus one when the mantissa is not zero
  if (!(amax > 0.f)) return -127;
  const uint32_t q = __float_as_uint(amax / fmax);
  const int e = (int)(q >> 23) - 127 + ((q & 0x7fffffu) ? 1 : 0);
  return max(-127, min(127, e));
}
template <bool E5M2>
__device__ __forceinline__ void quantize32(const float (&v)[32], float fmax, uint4 (&o)[2], int& e) {
  float m0 = 0.f, m1 = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) { m0 = fmaxf(m0, fabsf(v[2 * i])); m1 = fmaxf(m1, fabsf(v[2 * i + 1])); }
  e = e8m0_exponent_bits(fmaxf(m0, m1), fmax);
  const float sc = exp2f((float)-e);
  uint16_t* h = reinterpret_cast<uint16_t*>(o);
#pragma unroll
  for (int i = 0; i < 16; ++i)
    h[i] = (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(v[2 * i] * sc, v[2 * i + 1] * sc), __NV_SATFINITE,
                                              E5M2 ? __NV_E5M2 : __NV_E4M3);
}
template <typename T, bool E5M2>
__global__ void __launch_bounds__(256)
mxfp8_dual_kernel(const T* __restrict__ x, uint8_t* __restrict__ q_row, uint8_t* __restrict__ sf_row,
                  uint8_t* __restrict__ q_colT, uint8_t* __restrict__ sf_col, int rows, int cols) {
  constexpr int PAD = 16 / sizeof(T);
  __shared__ __align__(16) T tile[64][128 + PAD];
  const float fmax = E5M2 ? 57344.f : 448.f;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 128;
  {
    const int tr = threadIdx.x >> 2, tq = threadIdx.x & 3;          // row of the tile, 32-column quarter
    const int r = r0 + tr, c = c0 + tq * 32;
    float v[32];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (r < rows && c + 8 * k + 8 <= cols) {
        load8(x + (size_t)r * cols + c + 8 * k, *reinterpret_cast<float(*)[8]>(v + 8 * k));
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[8 * k + i] = 0.f;
      }
    }
    if (q_colT != nullptr) {
#pragma unroll
      for (int i = 0; i < 32; ++i) tile[tr][tq * 32 + i] = from_f<T>(v[i]);
    }
    if (q_row != nullptr && r < rows && c < cols) {
      uint4 o[2]; int e;
      quantize32<E5M2>(v, fmax, o, e);
      uint4* dst = reinterpret_cast<uint4*>(q_row + (size_t)r * cols + c);
      dst[0] = o[0]; dst[1] = o[1];
      sf_row[mx_sf_offset(r, c >> 5, (cols + 127) >> 7)] = (uint8_t)(e + 127);
    }
  }
  if (q_colT == nullptr) return;
  __syncthreads();
  {
    const int tc = threadIdx.x & 127, th = threadIdx.x >> 7;        // column of the tile, 32-row half
    const int c = c0 + tc, r = r0 + th * 32;
    if (c < cols && r < rows) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = to_f(tile[th * 32 + i][tc]);
      uint4 o[2]; int e;
      quantize32<E5M2>(v, fmax, o, e);
      uint4* dst = reinterpret_cast<uint4*>(q_colT + (size_t)c * rows + r);
      dst[0] = o[0]; dst[1] = o[1];
      sf_col[mx_sf_offset(c, r >> 5, (rows + 127) >> 7)] = (uint8_t)(e + 127);
    }
  }
}

}  // namespace mlb

using namespace mlb;

// x [rows, cols] -> q_row [rows, cols] + sf_row and/or q_colT [cols, rows] + sf_col (either pair may be null);
// cols a multiple of 32 for the row-wise copy, rows a multiple of 32 for the column-wise one, cols a multiple of 8;
// the scale buffers hold mlb_mx_sf_bytes(rows, cols) resp. (cols, rows) bytes.
MLB_API int mlb_mxfp8_quantize_dual(int dtype, const void* x, void* q_row, void* sf_row, void* q_colT, void* sf_col,
                                    int rows, int cols, int e5m2, cudaStream_t st) {
  if ((cols % 8) || (q_row && (cols % 32)) || (q_colT && (rows % 32))) return -3;
  dim3 grid((cols + 127) / 128, (rows + 63) / 64);
  if (e5m2) {
    MLB_DISPATCH_ACT(dtype, T, (mxfp8_dual_kernel<T, true><<<grid, 256, 0, st>>>(
        (const T*)x, (uint8_t*)q_row, (uint8_t*)sf_row, (uint8_t*)q_colT, (uint8_t*)sf_col, rows, cols)));
  } else {
    MLB_DISPATCH_ACT(dtype, T, (mxfp8_dual_kernel<T, false><<<grid, 256, 0, st>>>(
        (const T*)x, (uint8_t*)q_row, (uint8_t*)sf_row, (uint8_t*)q_colT, (uint8_t*)sf_col, rows, cols)));
  }
  MLB_CHECK_LAUNCH();
  return 0;
}

// amax must be zeroed by the caller (or hold a running maximum to extend)
MLB_API int mlb_amax(int dtype, const void* x, long n, float* amax, cudaStream_t st) {
  if (n <= 0) return 0;
  long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  MLB_DISPATCH_ACT(dtype, T, (amax_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, (size_t)n, amax)));
  MLB_CHECK_LAUNCH();
  return 0;
}

// x [rows, cols] -> q [rows, cols] (and qt [cols, rows] when non-null) as fp8 bytes; scale_inv receives 1/scale
MLB_API int mlb_fp8_cast_transpose(int dtype, const void* x, const float* amax, void* q, void* qt, float* scale_inv,
                                   int rows, int cols, int e5m2, cudaStream_t st) {
  if (rows % 16 || cols % 16) return -3;
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  MLB_DISPATCH_ACT(dtype, T, (cast_transpose_kernel<T><<<grid, 256, 0, st>>>((const T*)x, amax, (uint8_t*)q, (uint8_t*)qt,
                                                                            scale_inv, rows, cols, e5m2)));
  MLB_CHECK_LAUNCH();
  return 0;
}

// along_rows = 1: scales [rows, cols/32]; 0: blocks run down the columns, scales [rows/32, cols]
MLB_API int mlb_mxfp8_quantize(int dtype, const void* x, void* q, void* scales, int rows, int cols, int along_rows,
                               cudaStream_t st) {
  if (along_rows) {
    if (cols % 32) return -3;
    const size_t nb = (size_t)rows * (cols / 32);
    MLB_DISPATCH_ACT(dtype, T, (mxfp8_row_kernel<T><<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(
                                   (const T*)x, (uint8_t*)q, (uint8_t*)scales, rows, cols)));
  } else {
    if (rows % 32) return -3;
    dim3 grid((cols + 127) / 128, rows / 32);
    MLB_DISPATCH_ACT(dtype, T, (mxfp8_col_kernel<T><<<grid, 128, 0, st>>>((const T*)x, (uint8_t*)q, (uint8_t*)scales, rows,
                                                                         cols)));
  }
  MLB_CHECK_LAUNCH();
  return 0;
}
