// Timing probe for the tensor-core instruction stream of one SM: how long one thread needs to get a batch of
// `tcgen05.mma` instructions accepted and how long the batch takes to complete, by instruction width (64 / 128 /
// 256 columns), A operand source (shared or tensor memory) and B layout (K-major or MN-major).  One CTA, operands
// are zeros in shared memory; the figures are SM cycles from clock64().  The kernels of this library are laid
// out around these numbers (an instruction is accepted about every 46 cycles whatever its size, so 64-column
// products cannot keep the tensor core busy); `python -m megatron_lm_b200.ops.microbench tcgen05` prints them.
#include "tc05.cuh"

namespace mlb {
using namespace tc05;

namespace {
__device__ __forceinline__ void probe_mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
               ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
constexpr int kProbeSmem = 196608 + 256;

// out[2 i], out[2 i + 1]: cycles to issue / to complete batch i of 16 instructions (see kNames on the host side)
__global__ void __launch_bounds__(64, 1) tcgen05_probe_kernel(long long* out, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 196608);
  uint32_t* slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = smem_u32(bars);
  for (int i = threadIdx.x; i < 196608 / 4; i += 64) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(bar0, 1); *abort_flag = 0; mbar_fence_init(); }
  if (warp == 1) { tmem_alloc(smem_u32(slot), 512); tmem_relinquish(); }
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *slot;
  if (warp == 1 && lane == 0) {
    const uint32_t sA = smem_u32(smem), sB = smem_u32(smem) + 65536;
    uint32_t ph = 0;
    int o = 0;
    bool ok = true;
    auto finish = [&](long long t0, long long t1) {
      mma_commit(bar0);
      ok = ok && mbar_wait(bar0, ph, abort_flag, status, 90);
      ph ^= 1u;
      out[o++] = t1 - t0; out[o++] = clock64() - t0;
    };
    for (int pass = 0; pass < 2 && ok; ++pass) {          // first pass warms the instruction cache
      o = 0;
      for (int n = 64; n <= 256 && ok; n *= 2) {
        const uint32_t id_k = make_idesc(128, n, 1, 0, 0), id_mn = make_idesc(128, n, 1, 0, 1);
        long long t0 = clock64();
#pragma unroll
        for (int k = 0; k < 16; ++k)                      // A and B in shared memory, both K-major
          mma_f16(tmem, make_desc(sA + (k & 3) * 32, 16, 1024), make_desc(sB + (k & 3) * 32, 16, 1024), id_k, k > 0);
        finish(t0, clock64());
        t0 = clock64();
#pragma unroll
        for (int k = 0; k < 16; ++k)                      // A in tensor memory
          probe_mma_ts(tmem, tmem + 256 + (k & 7) * 8, make_desc(sB + (k & 3) * 32, 16, 1024), id_k, k > 0);
        finish(t0, clock64());
        t0 = clock64();
#pragma unroll
        for (int k = 0; k < 16; ++k)                      // A in tensor memory, B MN-major (16 rows per K step)
          probe_mma_ts(tmem, tmem + 256 + (k & 7) * 8, make_desc(sB + (k & 7) * 2048, 16384, 1024), id_mn, k > 0);
        finish(t0, clock64());
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem, 512); }
}
}  // namespace
}  // namespace mlb

using namespace mlb;

// out: 18 values (9 batches x {issue cycles, completion cycles}) in device memory
MLB_API int mlb_tcgen05_probe(long long* out, int* status, cudaStream_t st) {
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(tcgen05_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem);
    if (e != cudaSuccess) return (int)e;
    set = true;
  }
  tcgen05_probe_kernel<<<1, 64, kProbeSmem, st>>>(out, status);
  MLB_CHECK_LAUNCH();
  return 0;
}
