// Shared device helpers for the sm_100a kernels of this library.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define MLB_API extern "C" __attribute__((visibility("default")))

// dtype codes used across the C ABI
enum : int { MLB_F32 = 0, MLB_BF16 = 1, MLB_F16 = 2 };

#define MLB_CHECK_LAUNCH() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return (int)e__; } while (0)

namespace mlb {

constexpr int kWarp = 32;

template <typename T> struct Vec8 { T v[8]; };

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// 8 consecutive elements -> 8 floats.  Pointer must be aligned to 8*sizeof(T).
template <typename T>
__device__ __forceinline__ void load8(const T* __restrict__ p, float (&o)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 r = *reinterpret_cast<const uint4*>(p);
    const T* h = reinterpret_cast<const T*>(&r);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = to_f(h[i]);
  } else {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* __restrict__ p, const float (&o)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 r;
    T* h = reinterpret_cast<T*>(&r);
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = from_f<T>(o[i]);
    *reinterpret_cast<uint4*>(p) = r;
  } else {
    *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(o[4], o[5], o[6], o[7]);
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum of up to 2 values; every thread gets the result.  `sh` needs 2*32 floats.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* sh) {
  a = warp_sum(a); b = warp_sum(b);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) { sh[w] = a; sh[32 + w] = b; }
  __syncthreads();
  float x = (l < nw) ? sh[l] : 0.f, y = (l < nw) ? sh[32 + l] : 0.f;
  a = warp_sum(x); b = warp_sum(y);
}
__device__ __forceinline__ float block_sum(float a, float* sh) {
  float b = 0.f; block_sum2(a, b, sh); return a;
}
__device__ __forceinline__ float block_max(float a, float* sh) {
  a = warp_max(a);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) sh[w] = a;
  __syncthreads();
  float x = (l < nw) ? sh[l] : -INFINITY;
  return warp_max(x);
}

}  // namespace mlb

// Dispatch a templated launcher on an activation dtype code.
#define MLB_DISPATCH_ACT(code, T, ...)                                   \
  switch (code) {                                                        \
    case MLB_F32:  { using T = float;          __VA_ARGS__; break; }     \
    case MLB_BF16: { using T = __nv_bfloat16;  __VA_ARGS__; break; }     \
    case MLB_F16:  { using T = __half;         __VA_ARGS__; break; }     \
    default: return -1;                                                  \
  }
