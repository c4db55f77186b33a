// Erasure-code parity over GF(2^8) (polynomial 0x11d) as a multiply-XOR reduction over up to 16
// source buffers that may live on this GPU or on peers (plain loads through peer-mapped pointers):
//     dst_i = XOR_j coef[i][j] * src_j        i < m <= 4,  j < k <= 16
// Encoding uses the generator rows, decoding the rows of the inverted survivor matrix - same kernel.
// Bytes are processed four to a 32-bit word: multiplication by the constant 2 ("xtime") is
//     ((x & 0x7f7f7f7f) << 1) ^ (((x >> 7) & 0x01010101) * 0x1d)
// and a product by c is the XOR of the x * 2^b for the set bits b of c; the chain of doublings of a
// source word is computed once and shared by all m outputs.  Coefficients are launch parameters,
// so every branch on them is uniform.  The reference has no erasure coding (its in-memory
// checkpoint replicates: megatron/training/checkpointing.py:520-544); this is new functionality.
#include "common.cuh"
#include "tc05.cuh"

namespace mlb {

constexpr int kEcMaxK = 16, kEcMaxM = 4;

struct EcParams {
  const uint4* src[kEcMaxK];
  uint4* dst[kEcMaxM];
  uint8_t coef[kEcMaxM][kEcMaxK];
  int k, m;
  int all_ones;            // every coefficient is 0 or 1: pure XOR, no field multiplications
  size_t nvec;             // 16-byte vectors per buffer
};

__device__ __forceinline__ uint32_t xtime4(uint32_t x) {
  return ((x & 0x7f7f7f7fu) << 1) ^ (((x >> 7) & 0x01010101u) * 0x1du);
}

__global__ void __launch_bounds__(256)
ec_apply_kernel(const EcParams p) {
  for (size_t v = blockIdx.x * (size_t)blockDim.x + threadIdx.x; v < p.nvec; v += (size_t)gridDim.x * blockDim.x) {
    uint32_t acc[kEcMaxM][4];
#pragma unroll
    for (int i = 0; i < kEcMaxM; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0u; }
    for (int j = 0; j < p.k; ++j) {
      const uint4 raw = p.src[j][v];
      uint32_t x[4] = {raw.x, raw.y, raw.z, raw.w};
      if (p.all_ones) {
#pragma unroll
        for (int i = 0; i < kEcMaxM; ++i)
          if (i < p.m && p.coef[i][j]) { acc[i][0] ^= x[0]; acc[i][1] ^= x[1]; acc[i][2] ^= x[2]; acc[i][3] ^= x[3]; }
      } else {
#pragma unroll
        for (int b = 0; b < 8; ++b) {
#pragma unroll
          for (int i = 0; i < kEcMaxM; ++i)
            if (i < p.m && ((p.coef[i][j] >> b) & 1)) {
              acc[i][0] ^= x[0]; acc[i][1] ^= x[1]; acc[i][2] ^= x[2]; acc[i][3] ^= x[3];
            }
          x[0] = xtime4(x[0]); x[1] = xtime4(x[1]); x[2] = xtime4(x[2]); x[3] = xtime4(x[3]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kEcMaxM; ++i)
      if (i < p.m) p.dst[i][v] = make_uint4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
  }
}

// Batched form: a table of jobs in device memory, each with its own sources (local or peer), destinations (local or
// peer: a parity owner may compute all parities of a stripe and store the others' straight into their memory) and
// coefficient rows.  Every job covers `nvec` vectors and is cut into `parts` block-sized pieces.
struct EcJob {
  unsigned long long src[kEcMaxK];
  unsigned long long dst[kEcMaxM];
  uint8_t coef[kEcMaxM][kEcMaxK];
  int k, m, pad0, pad1;
};

__global__ void __launch_bounds__(256, 4)
ec_batch_kernel(const EcJob* __restrict__ jobs, int n_jobs, size_t nvec, int parts) {
  __shared__ EcJob job;
  const size_t per_part = (nvec + parts - 1) / parts;
  for (long w = blockIdx.x; w < (long)n_jobs * parts; w += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < sizeof(EcJob) / 4)
      reinterpret_cast<uint32_t*>(&job)[threadIdx.x] = reinterpret_cast<const uint32_t*>(jobs + w / parts)[threadIdx.x];
    __syncthreads();
    const size_t v0 = (size_t)(w % parts) * per_part;
    const size_t v1 = v0 + per_part < nvec ? v0 + per_part : nvec;
    const int k = job.k, m = job.m;
    for (size_t v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
      uint32_t acc[kEcMaxM][4];
#pragma unroll
      for (int i = 0; i < kEcMaxM; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0u; }
      // sources four at a time: four 16-byte loads in flight per thread, few enough registers for 4 blocks per SM
      for (int j0 = 0; j0 < k; j0 += 4) {
        uint4 raw[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
          if (j0 + jj < k) raw[jj] = reinterpret_cast<const uint4*>(job.src[j0 + jj])[v];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int j = j0 + jj;
          if (j >= k) break;
          uint32_t x[4] = {raw[jj].x, raw[jj].y, raw[jj].z, raw[jj].w};
          uint32_t any = 0;
#pragma unroll
          for (int i = 0; i < kEcMaxM; ++i) any |= (i < m) ? job.coef[i][j] : 0;
#pragma unroll
          for (int b = 0; b < 8; ++b) {
            if ((any >> b) == 0) break;
#pragma unroll
            for (int i = 0; i < kEcMaxM; ++i)
              if (i < m && ((job.coef[i][j] >> b) & 1)) {
                acc[i][0] ^= x[0]; acc[i][1] ^= x[1]; acc[i][2] ^= x[2]; acc[i][3] ^= x[3];
              }
            x[0] = xtime4(x[0]); x[1] = xtime4(x[1]); x[2] = xtime4(x[2]); x[3] = xtime4(x[3]);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < kEcMaxM; ++i)
        if (i < m) reinterpret_cast<uint4*>(job.dst[i])[v] = make_uint4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    }
  }
}

// Staged form of the batched kernel: the sources (mostly peers' memory) are brought into shared memory by bulk
// asynchronous copies - one thread keeps several 4 KB pieces per source in flight, so the NVLink reads are large
// requests that do not depend on how many warps are resident - and the multiply-XOR runs out of shared memory.
// Work item = (job, 4 KB piece); a ring of `stages` stages of k_max pieces each.  Every wait is bounded.
constexpr int kEcPiece = 4096;
__device__ __forceinline__ void ec_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__global__ void __launch_bounds__(288, 2)
ec_staged_kernel(const EcJob* __restrict__ jobs, int n_jobs, size_t nbytes, int k_max, int stages, int* status) {
  using namespace tc05;
  extern __shared__ __align__(128) uint8_t ec_smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(ec_smem);          // full[stages], empty[stages]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 16);
  uint8_t* data = ec_smem + 256;
  const uint32_t bar0 = smem_u32(bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(bar0 + 8u * s, 1); mbar_init(bar0 + 8u * (8 + s), 8); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const long pieces = (long)(nbytes / kEcPiece);
  const long total = (long)n_jobs * pieces;
  const size_t stage_bytes = (size_t)k_max * kEcPiece;
  if (warp == 8) {
    // ---------------------------------------------------------------- producer (one thread)
    if (lane == 0) {
      int st = 0; uint32_t ph = 0;
      for (long w = blockIdx.x; w < total; w += gridDim.x) {
        const EcJob* job = jobs + w / pieces;
        const size_t off = (size_t)(w % pieces) * kEcPiece;
        if (!mbar_wait(bar0 + 8u * (8 + st), ph ^ 1u, abort_flag, status, 71)) break;
        const int k = job->k;
        mbar_expect_tx(bar0 + 8u * st, (uint32_t)k * kEcPiece);
        for (int j = 0; j < k; ++j)
          ec_bulk_g2s(smem_u32(data + st * stage_bytes + (size_t)j * kEcPiece),
                      reinterpret_cast<const uint8_t*>(job->src[j]) + off, kEcPiece, bar0 + 8u * st);
        if (++st == stages) { st = 0; ph ^= 1u; }
      }
    }
  } else {
    // ---------------------------------------------------------------- 256 consumers: one 16-byte vector each
    int st = 0; uint32_t ph = 0;
    const int v = threadIdx.x;                                       // vector index inside the piece
    for (long w = blockIdx.x; w < total; w += gridDim.x) {
      const EcJob* job = jobs + w / pieces;
      const size_t off = (size_t)(w % pieces) * kEcPiece;
      const int k = job->k, m = job->m;
      if (!mbar_wait(bar0 + 8u * st, ph, abort_flag, status, 72)) break;
      uint32_t acc[kEcMaxM][4];
#pragma unroll
      for (int i = 0; i < kEcMaxM; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0u; }
      const uint8_t* base = data + st * stage_bytes;
      for (int j = 0; j < k; ++j) {
        const uint4 raw = reinterpret_cast<const uint4*>(base + (size_t)j * kEcPiece)[v];
        uint32_t x[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t c[kEcMaxM];
        uint32_t any = 0;
#pragma unroll
        for (int i = 0; i < kEcMaxM; ++i) { c[i] = (i < m) ? job->coef[i][j] : 0u; any |= c[i]; }
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          if ((any >> b) == 0) break;
#pragma unroll
          for (int i = 0; i < kEcMaxM; ++i)
            if ((c[i] >> b) & 1u) { acc[i][0] ^= x[0]; acc[i][1] ^= x[1]; acc[i][2] ^= x[2]; acc[i][3] ^= x[3]; }
          x[0] = xtime4(x[0]); x[1] = xtime4(x[1]); x[2] = xtime4(x[2]); x[3] = xtime4(x[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar0 + 8u * (8 + st));              // this warp has read the stage
#pragma unroll
      for (int i = 0; i < kEcMaxM; ++i)
        if (i < m) reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(job->dst[i]) + off)[v] =
            make_uint4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      if (++st == stages) { st = 0; ph ^= 1u; }
    }
  }
}

}  // namespace mlb

using namespace mlb;

MLB_API int mlb_ec_job_bytes() { return (int)sizeof(EcJob); }

// jobs: device array of n_jobs EcJob records (layout: 16 x u64 src, 4 x u64 dst, 4 x 16 coefficient bytes, k, m, 2 pad
// ints); every buffer holds nbytes (multiple of 16).  grid_blocks bounds the SMs used (0 = whole GPU).
// Staged variant (sources through shared memory by bulk copies); nbytes a multiple of 4096, k_max = the largest
// number of sources of any job.  status: optional device word that receives a code if a bounded wait runs out.
MLB_API int mlb_ec_apply_batch_staged(const void* jobs, int n_jobs, long nbytes, int k_max, int grid_blocks,
                                      int* status, cudaStream_t st) {
  if (n_jobs <= 0) return 0;
  if (nbytes <= 0 || (nbytes % kEcPiece) || k_max < 1 || k_max > kEcMaxK) return -3;
  int stages = (96 * 1024) / (k_max * kEcPiece);                     // two blocks per SM when the ring fits 96 KB
  if (stages > 8) stages = 8;
  if (stages < 2) stages = 2;
  const int smem = 256 + stages * k_max * kEcPiece;
  static int smem_set = 0;
  if (smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(ec_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    smem_set = smem;
  }
  const long total = (long)n_jobs * (nbytes / kEcPiece);
  long cap = grid_blocks > 0 ? grid_blocks : 148L * 2;
  unsigned grid = (unsigned)(total < cap ? total : cap);
  ec_staged_kernel<<<grid, 288, smem, st>>>(reinterpret_cast<const EcJob*>(jobs), n_jobs, (size_t)nbytes, k_max, stages,
                                            status);
  MLB_CHECK_LAUNCH();
  return 0;
}

// Copy by a few thread blocks instead of by the copy engine: the destination may be pinned host memory (the second
// tier of the in-memory checkpoint).  A 21 GB cudaMemcpyAsync on a side stream kept the device-to-host copy engine
// busy for a third of a second, and the training stream's own small device-to-host reads (the loss of every step)
// queued behind it: 365 ms lost per save.  Stores from the SMs over PCIe are posted, so a handful of blocks keep
// the link busy and nothing else has to wait.  Fewer blocks disturb the training kernels less: with 16 blocks a save
// cost about 220 ms of training time, with 4 about 55 ms (1.3B GPT on 2 GPUs, 21 GB per rank, a save every 5 steps).
__global__ void __launch_bounds__(256) stream_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t nvec) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) dst[i] = src[i];
}

MLB_API int mlb_stream_copy(void* dst, const void* src, long nbytes, int blocks, cudaStream_t st) {
  if (nbytes <= 0) return 0;
  if ((nbytes % 16) || (reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return -3;
  if (blocks < 1) blocks = 4;
  stream_copy_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<uint4*>(dst), reinterpret_cast<const uint4*>(src),
                                            (size_t)nbytes / 16);
  MLB_CHECK_LAUNCH();
  return 0;
}

MLB_API int mlb_ec_apply_batch(const void* jobs, int n_jobs, long nbytes, int grid_blocks, cudaStream_t st) {
  if (n_jobs <= 0) return 0;
  if (nbytes <= 0 || (nbytes % 16)) return -3;
  const size_t nvec = (size_t)nbytes / 16;
  int parts = (int)((nvec + 256 * 16 - 1) / (256 * 16));      // ~16 vectors per thread per piece
  if (parts < 1) parts = 1;
  long total = (long)n_jobs * parts;
  long cap = grid_blocks > 0 ? grid_blocks : 148L * 8;
  unsigned grid = (unsigned)(total < cap ? total : cap);
  ec_batch_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const EcJob*>(jobs), n_jobs, nvec, parts);
  MLB_CHECK_LAUNCH();
  return 0;
}

// src: host array of k device addresses (16-byte aligned; local or peer-mapped); dst: host array of m local
// addresses; coef: host array [m][k] row-major; nbytes: multiple of 16.
MLB_API int mlb_ec_apply(const void* const* src, void* const* dst, const uint8_t* coef, int k, int m, long nbytes,
                         int max_blocks, cudaStream_t st) {
  if (k < 1 || k > kEcMaxK || m < 1 || m > kEcMaxM || nbytes <= 0 || (nbytes % 16)) return -3;
  EcParams p = {};
  p.k = k; p.m = m; p.nvec = (size_t)nbytes / 16; p.all_ones = 1;
  for (int j = 0; j < k; ++j) {
    if (reinterpret_cast<uintptr_t>(src[j]) & 15) return -3;
    p.src[j] = reinterpret_cast<const uint4*>(src[j]);
  }
  for (int i = 0; i < m; ++i) {
    if (reinterpret_cast<uintptr_t>(dst[i]) & 15) return -3;
    p.dst[i] = reinterpret_cast<uint4*>(dst[i]);
    for (int j = 0; j < k; ++j) { p.coef[i][j] = coef[i * k + j]; if (coef[i * k + j] > 1) p.all_ones = 0; }
  }
  size_t blocks = (p.nvec + 255) / 256;
  size_t cap = max_blocks > 0 ? (size_t)max_blocks : (size_t)148 * 8;
  if (blocks > cap) blocks = cap;
  ec_apply_kernel<<<(unsigned)blocks, 256, 0, st>>>(p);
  MLB_CHECK_LAUNCH();
  return 0;
}
