// Persistent warp-specialised bf16/fp16 GEMM for sm_100a:
//   D[M,N] (=|+=) A * B  with fp32 accumulation in tensor memory.
//
// * One CTA per SM walks 128 x BN output tiles (BN = 256 or 128).  Warp 0 issues TMA loads
//   into a ring of 128B-swizzled shared-memory stages, warp 1 issues tcgen05.mma (one elected
//   thread) into one of two TMEM accumulators, warps 2-5 drain the other accumulator
//   (tcgen05.ld -> registers -> global), so the epilogue of tile i overlaps the main loop of i+1.
// * Each operand is either K-major (reduction dim contiguous in global memory) or MN-major
//   (output dim contiguous); the same kernel therefore serves forward (X W^T), data gradient
//   (dY W) and weight gradient (dY^T X) without a transpose pass.
// * Output modes: store bf16/fp16, store fp32, or accumulate into fp32 (weight gradients
//   accumulated straight into the main-grad buffer), with an optional row-broadcast bias.
//
// Covers the GEMM call sites of the reference at megatron/core/tensor_parallel/layers.py:480
// (fprop), :523 (dgrad) and :553-598 (wgrad with fp32 accumulation).
#include "tc05.cuh"

namespace mlb {
using namespace tc05;

constexpr int BM = 128, BK = 64, UK = 16;
constexpr int kGemmThreads = 192;   // warp0 TMA, warp1 MMA, warps 2..5 epilogue

enum : int { OUT_LP = 0, OUT_F32 = 1, OUT_F32_ACC = 2 };

struct GemmParams {
  int M, N, K;
  void* D; long ldd;          // output row stride in elements
  const void* bias;           // [N] in the input dtype, or null
  int out_mode;               // OUT_*
  int lp_fmt;                 // 1 = bf16, 0 = fp16 (inputs and OUT_LP output)
  int* status;
  int tiles_m, tiles_n;
  int tma_out;                // 1: epilogue stages tiles in shared memory and stores / add-reduces them by TMA
};

__device__ __forceinline__ float load_bias(const void* bias, int col, int N, int bf) {
  if (col >= N) return 0.f;
  return bf ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[col])
            : __half2float(reinterpret_cast<const __half*>(bias)[col]);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, int bf) {
  if (bf) { __nv_bfloat162 v = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&v); }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int BN> struct GemmSmem {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kEpiBytes = 4 * 2 * 4096;     // per epilogue warp: two 32-row x 128-byte staging buffers
  static constexpr int kBytes = kStages * (kABytes + kBBytes) + kEpiBytes + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmD, const GemmParams p) {
  using S = GemmSmem<BN>;
  constexpr int kStages = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * S::kABytes;
  uint8_t* sEpi = smem + kStages * (S::kABytes + S::kBBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + S::kEpiBytes);
  // bars: full[kStages], empty[kStages], tfull[2], tempty[2]; then tmem slot + abort flag
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
  auto tempty = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull(a), 1); mbar_init(tempty(a), 4); }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB);
    if (p.tma_out) prefetch_tmap(&tmD);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 2 * BN >= 32 ? 2 * BN : 32); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty(stage), phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
          mbar_expect_tx(full(stage), S::kABytes + S::kBBytes);
          const uint32_t a_dst = smem_u32(sA + stage * S::kABytes), b_dst = smem_u32(sB + stage * S::kBBytes);
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d(a_dst, &tmA, full(stage), k0, m0);                 // box [64 k, 128 rows]
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, full(stage), m0 + 64 * j, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &tmB, full(stage), k0, n0);                 // box [64 k, BN rows]
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, full(stage), n0 + 64 * j, k0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {   // let copies already in flight land before the CTA retires
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { __nanosleep(1000); }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BM, BN, p.lp_fmt, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0; uint32_t phase = 0;
      int t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
        const int acc = t & 1;
        const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
        if (!mbar_wait(tempty(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full(stage), phase, abort_flag, p.status, 3)) { ok = false; break; }
          fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * S::kABytes), b_addr = smem_u32(sB + stage * S::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            // K-major: 16 elements = 32 B inside the swizzle row.  MN-major: 16 K-rows = two 1024 B groups.
            const uint64_t da = A_MN ? make_desc(a_addr + k * 2048, 8192, 1024) : make_desc(a_addr + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_desc(b_addr + k * 2048, 8192, 1024) : make_desc(b_addr + k * 32, 16, 1024);
            mma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit(empty(stage));            // stage reusable once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) mma_commit(tfull(acc));        // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may access
    int t = 0;
    int epi_buf = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
      const int acc = t & 1;
      const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
      const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
      if (!mbar_wait(tfull(acc), acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
      fence_after_sync();
      const int row = m0 + quad * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
      if (p.tma_out) {
        // ---- staged epilogue: registers -> 128B-swizzled shared tile -> TMA store / add-reduce.
        // Each warp owns rows [quad*32, quad*32+32) of the tile and two private 4 KB buffers, so no
        // cross-warp synchronisation is needed; out-of-range rows/columns are clipped by the TMA.
        const int cw = (p.out_mode == OUT_LP) ? 64 : 32;          // columns per 128-byte staged row
        uint8_t* my_stage = sEpi + (warp - 2) * 8192;
#pragma unroll 1
        for (int c = 0; c < BN; c += cw) {
          uint32_t r0[32], r1[32];
          tmem_ld32(t_row + (uint32_t)c, r0);
          if (cw == 64) tmem_ld32(t_row + (uint32_t)c + 32, r1);
          tmem_wait_ld();
          if (lane == 0) bulk_wait_read<1>();                      // the buffer used two chunks ago is free
          __syncwarp();
          uint8_t* stage = my_stage + epi_buf * 4096;
          const int col = n0 + c;
          uint32_t w[32];
          if (p.out_mode == OUT_LP) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float a0 = __uint_as_float(r0[2 * i]), a1 = __uint_as_float(r0[2 * i + 1]);
              float b0 = __uint_as_float(r1[2 * i]), b1 = __uint_as_float(r1[2 * i + 1]);
              if (p.bias != nullptr) {
                a0 += load_bias(p.bias, col + 2 * i, p.N, p.lp_fmt); a1 += load_bias(p.bias, col + 2 * i + 1, p.N, p.lp_fmt);
                b0 += load_bias(p.bias, col + 32 + 2 * i, p.N, p.lp_fmt); b1 += load_bias(p.bias, col + 33 + 2 * i, p.N, p.lp_fmt);
              }
              w[i] = pack2(a0, a1, p.lp_fmt);
              w[16 + i] = pack2(b0, b1, p.lp_fmt);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float a = __uint_as_float(r0[i]);
              if (p.bias != nullptr) a += load_bias(p.bias, col + i, p.N, p.lp_fmt);
              w[i] = __float_as_uint(a);
            }
          }
          uint8_t* rowp = stage + lane * 128;
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<uint4*>(rowp + ((q ^ (lane & 7)) << 4)) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0 && col < p.N && (m0 + quad * 32) < p.M) {
            if (p.out_mode == OUT_F32_ACC) tma_reduce_add_2d(&tmD, smem_u32(stage), col, m0 + quad * 32);
            else tma_store_2d(&tmD, smem_u32(stage), col, m0 + quad * 32);
            bulk_commit();
          }
          epi_buf ^= 1;
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(t_row + (uint32_t)c, r);
        tmem_wait_ld();
        const int col = n0 + c;
        if (row < p.M && col < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (col + i < p.N) {
                v[i] += p.lp_fmt ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col + i])
                                 : __half2float(reinterpret_cast<const __half*>(p.bias)[col + i]);
              }
            }
          }
          const bool full_cols = (col + 32 <= p.N);
          if (p.out_mode == OUT_LP) {
            uint16_t* d = reinterpret_cast<uint16_t*>(p.D) + (size_t)row * p.ldd + col;
            if (full_cols && ((reinterpret_cast<uintptr_t>(d) & 15) == 0)) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o; uint16_t* h = reinterpret_cast<uint16_t*>(&o);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  if (p.lp_fmt) { __nv_bfloat16 b = __float2bfloat16_rn(v[q * 8 + i]); h[i] = *reinterpret_cast<uint16_t*>(&b); }
                  else { __half b = __float2half_rn(v[q * 8 + i]); h[i] = *reinterpret_cast<uint16_t*>(&b); }
                }
                reinterpret_cast<uint4*>(d)[q] = o;
              }
            } else {
              for (int i = 0; i < 32 && col + i < p.N; ++i) {
                if (p.lp_fmt) { __nv_bfloat16 b = __float2bfloat16_rn(v[i]); d[i] = *reinterpret_cast<uint16_t*>(&b); }
                else { __half b = __float2half_rn(v[i]); d[i] = *reinterpret_cast<uint16_t*>(&b); }
              }
            }
          } else {
            float* d = reinterpret_cast<float*>(p.D) + (size_t)row * p.ldd + col;
            const bool accum = p.out_mode == OUT_F32_ACC;
            if (full_cols && ((reinterpret_cast<uintptr_t>(d) & 15) == 0)) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                if (accum) { const float4 c4 = reinterpret_cast<const float4*>(d)[q]; o.x += c4.x; o.y += c4.y; o.z += c4.z; o.w += c4.w; }
                reinterpret_cast<float4*>(d)[q] = o;
              }
            } else {
              for (int i = 0; i < 32 && col + i < p.N; ++i) d[i] = accum ? d[i] + v[i] : v[i];
            }
          }
        }
      }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty(acc));
    }
  }
  if (p.tma_out && warp >= 2 && lane == 0) bulk_wait<0>();     // staged stores have landed
  // ---------------------------------------------------------------- teardown
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem_base, 2 * BN >= 32 ? 2 * BN : 32); }
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, GemmParams p,
                       int sm_count, cudaStream_t st) {
  using S = GemmSmem<BN>;
  auto kern = gemm_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count ? tiles : sm_count;
  kern<<<grid, kGemmThreads, S::kBytes, st>>>(tmA, tmB, tmD, p);
  MLB_CHECK_LAUNCH();
  return 0;
}

static int sm_count_cached() {
  static int n = 0;
  if (n == 0) {
    int dev = 0; cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace mlb

using namespace mlb;

// D[M,N] (=|+=) op(A) * op(B) (+ bias).
//   a_mn == 0: A is [M, K] with row stride lda (K contiguous).  a_mn == 1: A is stored [K, M] with row stride lda.
//   b_mn == 0: B is [N, K] with row stride ldb (K contiguous).  b_mn == 1: B is stored [K, N] with row stride ldb.
// lda/ldb/ldd are in elements; operand bases 16-byte aligned and lda, ldb multiples of 8.
// max_ctas > 0 caps the persistent grid (to leave SMs to a concurrent communication kernel).
MLB_API int mlb_gemm(int lp_fmt, const void* A, long lda, int a_mn, const void* B, long ldb, int b_mn, void* D,
                     long ldd, int out_mode, const void* bias, int M, int N, int K, int max_ctas, int* status,
                     cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  const int bn = (N > 128) ? 256 : 128;
  CUtensorMap tmA, tmB;
  int rc;
  {
    uint64_t dims[2], strides[1]; uint32_t box[2];
    if (!a_mn) { dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = BK; box[1] = BM; }
    else       { dims[0] = (uint64_t)M; dims[1] = (uint64_t)K; box[0] = 64; box[1] = BK; }
    strides[0] = (uint64_t)lda * 2;
    if ((rc = make_tmap(&tmA, A, 2, dims, strides, box))) return rc;
    if (!b_mn) { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; box[0] = BK; box[1] = (uint32_t)bn; }
    else       { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; box[0] = 64; box[1] = BK; }
    strides[0] = (uint64_t)ldb * 2;
    if ((rc = make_tmap(&tmB, B, 2, dims, strides, box))) return rc;
  }
  CUtensorMap tmD;
  const int esz = (out_mode == OUT_LP) ? 2 : 4;
  int tma_out = (((size_t)ldd * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(D) & 15) == 0);
  if (tma_out) {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M}, strides[1] = {(uint64_t)ldd * esz};
    uint32_t box[2] = {(uint32_t)(esz == 2 ? 64 : 32), 32};
    if (make_tmap(&tmD, D, 2, dims, strides, box, esz)) tma_out = 0;
  }
  if (!tma_out) tmD = tmA;     // placeholder, unused
  GemmParams p;
  p.tma_out = tma_out;
  p.M = M; p.N = N; p.K = K; p.D = D; p.ldd = ldd; p.bias = bias; p.out_mode = out_mode; p.lp_fmt = lp_fmt;
  p.status = status; p.tiles_m = p.tiles_n = 0;
  int sms = sm_count_cached();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
#define GO(BNv, AM, BMj) return launch_gemm<BNv, AM, BMj>(tmA, tmB, tmD, p, sms, st)
  if (bn == 256) {
    if (!a_mn && !b_mn) GO(256, false, false);
    if (!a_mn && b_mn) GO(256, false, true);
    if (a_mn && !b_mn) GO(256, true, false);
    GO(256, true, true);
  } else {
    if (!a_mn && !b_mn) GO(128, false, false);
    if (!a_mn && b_mn) GO(128, false, true);
    if (a_mn && !b_mn) GO(128, true, false);
    GO(128, true, true);
  }
#undef GO
}
