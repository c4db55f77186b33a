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
// * Communication modes (tensor parallelism with sequence parallelism, one launch per product):
//     AG : the A operand is the all-gather of per-rank row shards.  The first ``n_comm`` CTAs pull the
//          peers' shards over NVLink with bulk async copies (peer global -> shared -> local gathered
//          buffer) and publish a flag per 128-row block; the GEMM CTAs start on this rank's own rows (read
//          in place through a second tensor map), then walk the peers' row blocks in arrival order, their
//          TMA producer waiting on each block's flag.
//     RS : D is reduce-scattered over ranks.  Row blocks owned by other ranks are computed first; the
//          epilogue stages each partial tile in shared memory and TMA-stores it into the owner's receive
//          slot (over NVLink), then bumps the owner's arrival counter.  This rank's own row blocks come last:
//          their epilogue adds the peers' arrived partial rows (+ optional residual) to the accumulator and
//          stores the finished sum, so there is no separate reduction pass.
//   Every cross-rank wait is bounded and reports through the status word.
//
// Covers the GEMM call sites of the reference at megatron/core/tensor_parallel/layers.py:480
// (fprop), :523 (dgrad) and :553-598 (wgrad with fp32 accumulation).
#pragma once
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
  // 8-bit operands (both K-major, 128 elements per 128-byte swizzle row, 32 per MMA): the shared-memory
  // layout in bytes is the same as for 16-bit operands, only the instruction kind and the K step differ
  int fp8, a_fmt, b_fmt;      // formats: 0 = e4m3, 1 = e5m2
  const float* scale_a;       // device scalars: the accumulator is multiplied by (*scale_a) * (*scale_b); may be null
  const float* scale_b;
  // Grouped (ragged) mode for mixture-of-experts: rows of A are sorted by expert; row-tile t covers rows
  // [group_tiles[t].x, group_tiles[t].y) of expert group_tiles[t].z (at most 128 rows, never across two experts).
  // B holds all experts stacked: K-major [E * N, K] or MN-major [E * K, N].  Output rows outside the tile's range
  // are not written, so a short tile may read rows of the next expert without harm.
  const int4* group_tiles;    // device array [tiles_m], or null
  const int* group_count;     // device scalar: number of valid records in group_tiles (tiles_m is then an upper
                              // bound used to size the grid); null = all tiles_m records are valid
  // Grouped weight gradient (one launch for all experts): dW_e [N_out, K_in] (=|+=) dy_e^T x_e, both operands
  // MN-major views of [T, *] activations whose rows are sorted by expert.  Output row blocks are numbered
  // e * wg_mblocks + i; the reduction of expert e runs over rows [group_offsets[e], group_offsets[e + 1]) in steps of
  // BK, and the rows of the last step that belong to the next expert are zeroed in shared memory before the MMA.
  const int* group_offsets;   // device int32 [E + 1], or null
  int wg_mblocks;             // 128-row output blocks per expert (N_out / 128)
  int raster_m;               // row blocks per rasterisation group (plain mode)
};

enum : int { COMM_NONE = 0, COMM_AG = 1, COMM_RS = 2 };
constexpr int kMaxPeers = 8;

struct CommParams {
  int mode, rank, tp, n_comm;
  int bpr;                          // 128-row blocks per rank
  uint32_t seq;                     // call number on this buffer set (flags hold the seq of their last completion)
  // AG
  const void* peer_x[kMaxPeers];    // every rank's [rows_per_rank, K] shard (peer-mapped addresses)
  void* gathered;                   // local [tp * rows_per_rank, K]
  uint32_t* chunk_flags;            // local, one per row block
  uint32_t* peer_sig[kMaxPeers];    // every rank's signal words: ready[tp] then done[tp]
  uint32_t* comm_counter;           // local
  uint32_t comm_target;             // cumulative worker completions that mean "this call's copies are all done"
  long shard_bytes;                 // rows_per_rank * K * 2
  // RS
  void* peer_recv[kMaxPeers];       // every rank's receive buffer [tp][rows_per_rank][N]
  uint32_t* peer_cnt[kMaxPeers];    // every rank's arrival counters [bpr]
  uint32_t cnt_target;              // cumulative arrivals that mean "this call's partials are all here"
  const void* residual; long ld_res;
  void* out; long ld_out;
  // dynamic tile schedule (CTA-pair kernel): two local words, {next tile, pairs that have left}; both are zero
  // between launches.  Null selects the static schedule.
  uint32_t* sched;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// spin until *p >= target (wrap-safe), at most ~2 s; on expiry record `code` and return false
template <bool SYS>
__device__ __forceinline__ bool wait_ge(const uint32_t* p, uint32_t target, int* status, int code) {
  const long long t0 = clock64();
  uint32_t it = 0;
  while (true) {
    const uint32_t v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if ((int32_t)(v - target) >= 0) return true;
    if ((++it & 31u) == 0u) {
      if (clock64() - t0 > kWaitCycles) { if (status) atomicCAS(status, 0, code); return false; }
      // a wait that already ran out on this GPU means the step is lost: do not sit through the limit again
      if ((it & 1023u) == 0u && status && *reinterpret_cast<volatile int*>(status) != 0) return false;
      __nanosleep(64);
    }
  }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}

// Extra tensor maps of the communication modes.  AG: m[0] covers this rank's own [rows_per_rank, K] shard, so its
// rows are multiplied straight from where they are.  RS: m[q] covers, inside rank q's receive buffer, the slot
// [rows_per_rank, N] that belongs to this rank (32-row x 128-byte boxes, stored by the epilogue).
struct ExtraMaps { CUtensorMap m[kMaxPeers]; };

struct TileCoord { int m_blk, n_blk, owner, m_local; };
__device__ __forceinline__ TileCoord map_tile(int tile, const GemmParams& p, const CommParams& c) {
  TileCoord t;
  if (c.mode == COMM_NONE) {
    // Row-block groups of `raster_m`: the ~148 tiles in flight at any time then cover a squarish patch of the
    // output (raster_m row blocks x ~148/raster_m column blocks), so the A and B panels they share stay in L2.
    const int gm = p.raster_m;
    const int per_group = gm * p.tiles_n;
    const int grp = tile / per_group, in_grp = tile % per_group;
    const int first_m = grp * gm;
    const int size_m = (p.tiles_m - first_m) < gm ? (p.tiles_m - first_m) : gm;
    t.m_blk = first_m + in_grp % size_m; t.n_blk = in_grp / size_m; t.owner = 0; t.m_local = t.m_blk;
  } else {
    const int per_group = c.bpr * p.tiles_n;
    const int g = tile / per_group, idx = tile % per_group;
    t.m_local = idx % c.bpr; t.n_blk = idx / c.bpr;
    t.owner = (c.mode == COMM_AG) ? (c.rank + g) % c.tp : (c.rank + 1 + g) % c.tp;
    t.m_blk = t.owner * c.bpr + t.m_local;
  }
  return t;
}

// All-gather worker: one thread streams 32 KB pieces peer -> shared -> local through a ring of stages.
template <int kRing>
__device__ void ag_comm_cta(uint8_t* smem, uint64_t* bars, const GemmParams& p, const CommParams& c) {
  constexpr uint32_t kPiece = 32768;
  if (threadIdx.x != 0) return;
  const uint32_t bar0 = smem_u32(bars);
  for (int s = 0; s < kRing; ++s) mbar_init(bar0 + 8u * s, 1);
  mbar_fence_init();
  volatile int dummy_abort = 0;
  uint32_t* my_sig = c.peer_sig[c.rank];
  if (blockIdx.x == 0)
    for (int q = 0; q < c.tp; ++q) if (q != c.rank) st_release_sys(c.peer_sig[q] + c.rank, c.seq);   // my shard is ready
  const long block_bytes = (long)BM * p.K * 2;
  const int items = c.tp * c.bpr;
  uint32_t base = 0;                     // pieces moved so far in this call (ring position / barrier parity)
  bool ok = true;
  for (int it = blockIdx.x; it < items && ok; it += c.n_comm) {
    // peers in the order the GEMM CTAs want them; the own shard (which the GEMM reads in place) goes last
    const int d = (it / c.bpr + 1) % c.tp, j = it % c.bpr;
    const int q = (c.rank + d) % c.tp;
    if (q != c.rank && !wait_ge<true>(my_sig + q, c.seq, p.status, 41)) { ok = false; break; }
    const uint8_t* src = reinterpret_cast<const uint8_t*>(c.peer_x[q]) + (long)j * block_bytes;
    uint8_t* dst = reinterpret_cast<uint8_t*>(c.gathered) + ((long)q * c.bpr + j) * block_bytes;
    const int pieces = (int)((block_bytes + kPiece - 1) / kPiece);
    auto piece_bytes = [&](int idx) -> uint32_t {
      const long rest = block_bytes - (long)idx * kPiece;
      return (uint32_t)(rest < (long)kPiece ? rest : (long)kPiece);
    };
    auto load_piece = [&](int idx) {
      const uint32_t st = (base + (uint32_t)idx) % kRing;
      mbar_expect_tx(bar0 + 8u * st, piece_bytes(idx));
      bulk_g2s(smem_u32(smem) + st * kPiece, src + (long)idx * kPiece, piece_bytes(idx), bar0 + 8u * st);
    };
    // kRing - 1 loads in flight; piece i + kRing - 1 reuses the stage of piece i - 1, whose store is
    // the second most recent one by the time it is needed
    for (int idx = 0; idx < pieces && idx < kRing - 1; ++idx) load_piece(idx);
    for (int i = 0; i < pieces && ok; ++i) {
      const uint32_t n = base + (uint32_t)i, st = n % kRing;
      if (!mbar_wait(bar0 + 8u * st, (n / kRing) & 1u, &dummy_abort, p.status, 42)) { ok = false; break; }
      bulk_s2g(dst + (long)i * kPiece, smem_u32(smem) + st * kPiece, piece_bytes(i));
      bulk_commit();
      const int nxt = i + kRing - 1;
      if (nxt < pieces) { bulk_wait_read<1>(); load_piece(nxt); }
    }
    base += (uint32_t)pieces;
    if (!ok) break;
    bulk_wait<0>();                      // the block is in local memory
    fence_proxy_async_all();
    __threadfence();
    st_release_gpu(c.chunk_flags + q * c.bpr + j, c.seq);
  }
  // when every worker of this rank is done, tell the peers they may overwrite their shards
  __threadfence();
  const uint32_t prev = atomicAdd(c.comm_counter, 1u);
  if (prev + 1u == c.comm_target)
    for (int q = 0; q < c.tp; ++q) if (q != c.rank) st_release_sys(c.peer_sig[q] + c.tp + c.rank, c.seq);
  if (blockIdx.x == 0)
    for (int q = 0; q < c.tp; ++q) if (q != c.rank) wait_ge<true>(my_sig + c.tp + q, c.seq, p.status, 43);
}

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

// FP8 is a compile-time switch: a run-time choice of the MMA kind inside the issue loop costs the 16-bit path
// more than 15 % (measured), so 8-bit operands get their own instantiations.
template <int BN, bool A_MN, bool B_MN, bool FP8 = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmD, const __grid_constant__ ExtraMaps xm, const GemmParams p_in,
            const CommParams cp) {
  using S = GemmSmem<BN>;
  GemmParams p = p_in;
  if (p.group_count != nullptr) {                        // the number of row tiles is decided on the device
    p.tiles_m = *p.group_count;
    if (p.raster_m > p.tiles_m) p.raster_m = p.tiles_m > 0 ? p.tiles_m : 1;
  }
  const bool gw = p.group_offsets != nullptr;            // grouped weight gradient
  constexpr int kStages = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * S::kABytes;
  uint8_t* sEpi = smem + kStages * (S::kABytes + S::kBBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + S::kEpiBytes);
  // bars: full[kStages], empty[kStages], tfull[2], tempty[2], tail; then tmem slot + abort flag
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
  auto tempty = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };
  const uint32_t tail_bar = bar0 + 8u * (2 * kStages + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (cp.mode == COMM_AG && (int)blockIdx.x < cp.n_comm) {        // communication CTAs take no part in the GEMM
    ag_comm_cta<6>(smem, bars, p, cp);
    return;
  }
  const int cta = (cp.mode == COMM_AG) ? (int)blockIdx.x - cp.n_comm : (int)blockIdx.x;
  const int n_cta = (cp.mode == COMM_AG) ? (int)gridDim.x - cp.n_comm : (int)gridDim.x;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull(a), 1); mbar_init(tempty(a), 4); }
    mbar_init(tail_bar, 1);
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
  constexpr int bk_elems = FP8 ? 2 * BK : BK;                        // elements per 128-byte row of a stage
  const int num_kb = (p.K + bk_elems - 1) / bk_elems;
  // grouped weight gradient: reduction range of the expert that output row block m_blk belongs to
  auto wg_range = [&](int m_blk, int& r0, int& r1) {
    const int e = m_blk / p.wg_mblocks;
    r0 = p.group_offsets[e]; r1 = p.group_offsets[e + 1];
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (gw) {
      // Grouped weight gradient: the whole warp walks the tiles (lane 0 issues the copies); in an expert's last
      // reduction step the rows that belong to the next expert are zeroed by all lanes before the stage is
      // handed to the MMA warp.
      int stage = 0; uint32_t phase = 0, tail_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += n_cta) {
        const TileCoord tc = map_tile(tile, p, cp);
        const int n0 = tc.n_blk * BN;
        const int a_col = (tc.m_blk % p.wg_mblocks) * BM;          // first output row of the block inside its expert
        int r0, r1; wg_range(tc.m_blk, r0, r1);
        const int nkb = (r1 - r0 + BK - 1) / BK;
        for (int kb = 0; kb < nkb && ok; ++kb) {
          const int k0 = r0 + kb * BK;
          const int valid = (r1 - k0) < BK ? (r1 - k0) : BK;       // rows of this step that belong to the expert
          const uint32_t a_dst = smem_u32(sA + stage * S::kABytes), b_dst = smem_u32(sB + stage * S::kBBytes);
          int w_ok = 1;
          if (lane == 0) {
            w_ok = mbar_wait(empty(stage), phase ^ 1u, abort_flag, p.status, 1) ? 1 : 0;
            if (w_ok) {
              const uint32_t bar = valid < BK ? tail_bar : full(stage);
              mbar_expect_tx(bar, S::kABytes + S::kBBytes);
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, bar, a_col + 64 * j, k0);
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, bar, n0 + 64 * j, k0);
              if (valid < BK) w_ok = mbar_wait(tail_bar, tail_phase, abort_flag, p.status, 9) ? 1 : 0;
            }
          }
          w_ok = __shfl_sync(0xffffffffu, w_ok, 0);
          if (!w_ok) { ok = false; break; }
          if (valid < BK) {
            tail_phase ^= 1u;
            // every 64-element chunk of an MN-major tile is BK rows of 128 bytes: rows [valid, BK) are contiguous
            const int n16 = (BK - valid) * 8;                      // 16-byte pieces to clear per chunk
            for (int ch = 0; ch < BM / 64 + BN / 64; ++ch) {
              uint8_t* base = (ch < BM / 64 ? sA + stage * S::kABytes + ch * 8192
                                            : sB + stage * S::kBBytes + (ch - BM / 64) * 8192) + valid * 128;
              for (int i = lane; i < n16; i += 32) reinterpret_cast<uint4*>(base)[i] = make_uint4(0, 0, 0, 0);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(full(stage));
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && lane == 0) { const long long t0 = clock64(); while (clock64() - t0 < 2000000LL) { __nanosleep(1000); } }
    } else if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      int ready_blk = -1;
      for (int tile = cta; tile < num_tiles && ok; tile += n_cta) {
        const TileCoord tc = map_tile(tile, p, cp);
        const int m0 = tc.m_blk * BM, n0 = tc.n_blk * BN;
        const bool own_rows = cp.mode == COMM_AG && tc.owner == cp.rank;
        int a_row = m0, b_row0 = n0, b_k0 = 0;
        if (p.group_tiles != nullptr) {
          const int4 g = p.group_tiles[tc.m_blk];
          a_row = g.x;
          if (B_MN) b_k0 = g.z * p.K; else b_row0 = g.z * p.N + n0;
        }
        if (cp.mode == COMM_AG && !own_rows && tc.m_blk != ready_blk) {
          // rows of this block arrive from a peer: wait for the worker's flag, then order the
          // async-proxy (TMA) reads after the acquired writes
          if (!wait_ge<false>(cp.chunk_flags + tc.m_blk, cp.seq, p.status, 5)) { *abort_flag = 1; ok = false; break; }
          fence_proxy_async_all();
          ready_blk = tc.m_blk;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty(stage), phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
          mbar_expect_tx(full(stage), S::kABytes + S::kBBytes);
          const uint32_t a_dst = smem_u32(sA + stage * S::kABytes), b_dst = smem_u32(sB + stage * S::kBBytes);
          const int k0 = kb * bk_elems;
          if constexpr (!A_MN) {
            if (own_rows) tma_load_2d(a_dst, &xm.m[0], full(stage), k0, tc.m_local * BM);
            else tma_load_2d(a_dst, &tmA, full(stage), k0, a_row);         // box [64 k, 128 rows]
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, full(stage), m0 + 64 * j, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &tmB, full(stage), k0, b_row0);             // box [64 k, BN rows]
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, full(stage), n0 + 64 * j, b_k0 + k0);
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
      const uint32_t idesc = FP8 ? make_idesc_f8(BM, BN, p.a_fmt, p.b_fmt)
                                 : make_idesc(BM, BN, p.lp_fmt, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0; uint32_t phase = 0;
      int t = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += n_cta, ++t) {
        const int acc = t & 1;
        const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
        if (!mbar_wait(tempty(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        int nkb = num_kb;
        if (gw) { int r0, r1; wg_range(map_tile(tile, p, cp).m_blk, r0, r1); nkb = (r1 - r0 + BK - 1) / BK; }
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(full(stage), phase, abort_flag, p.status, 3)) { ok = false; break; }
          fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * S::kABytes), b_addr = smem_u32(sB + stage * S::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            // K-major: 16 elements = 32 B inside the swizzle row.  MN-major: 16 K-rows = two 1024 B groups.
            const uint64_t da = A_MN ? make_desc(a_addr + k * 2048, 8192, 1024) : make_desc(a_addr + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_desc(b_addr + k * 2048, 8192, 1024) : make_desc(b_addr + k * 32, 16, 1024);
            if constexpr (FP8) mma_f8(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else mma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
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
    const float alpha = (p.scale_a ? *p.scale_a : 1.f) * (p.scale_b ? *p.scale_b : 1.f);
    int t = 0;
    int epi_buf = 0;
    int pend_owner = -1, pend_blk = 0;                    // reduce-scatter: tile whose arrival signal is still owed
    bool ok = true;
    for (int tile = cta; tile < num_tiles && ok; tile += n_cta, ++t) {
      const int acc = t & 1;
      const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
      const TileCoord tc = map_tile(tile, p, cp);
      const int m0 = tc.m_blk * BM, n0 = tc.n_blk * BN;
      if (!mbar_wait(tfull(acc), acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
      fence_after_sync();
      int row = m0 + quad * 32 + lane, row_end = p.M;
      bool wg_empty = false;                     // expert without tokens: its gradient tile is zero (no MMA ran)
      if (gw) { int r0, r1; wg_range(tc.m_blk, r0, r1); wg_empty = r1 <= r0; }
      if (p.group_tiles != nullptr) {
        const int4 g = p.group_tiles[tc.m_blk];
        row = g.x + quad * 32 + lane; row_end = g.y;
      }
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
      if (p.tma_out) {
        // ---- staged epilogue: registers -> 128B-swizzled shared tile -> TMA store / add-reduce.
        // Each warp owns rows [quad*32, quad*32+32) of the tile and two private 4 KB buffers, so no
        // cross-warp synchronisation is needed; out-of-range rows/columns are clipped by the TMA.
        // Reduce-scatter: the destination is this rank's slot in the row owner's receive buffer (a TMA store
        // over NVLink unless this rank owns the rows); the owner's arrival counter is bumped once the
        // warp's stores have completed.
        const int cw = (p.out_mode == OUT_LP) ? 64 : 32;          // columns per 128-byte staged row
        uint8_t* my_stage = sEpi + (warp - 2) * 8192;
        // Rows this rank owns are finished here: once the peers' partial tiles of the row block have arrived
        // (they were computed first on every rank), each thread adds their rows and the residual to its
        // accumulator row and the sum goes straight to the output - the own partial never touches memory.
        const bool rs_own = cp.mode == COMM_RS && tc.owner == cp.rank;
        const CUtensorMap* dmap = (cp.mode == COMM_RS && !rs_own) ? &xm.m[tc.owner] : &tmD;
        const int drow = (cp.mode == COMM_RS) ? tc.m_local * BM + quad * 32 : m0 + quad * 32;
        int n_groups = 0;
        if (rs_own && lane == 0 && pend_owner >= 0) {     // last tile sent to a peer: flush its signal
          bulk_wait<0>(); fence_proxy_async_all(); __threadfence_system();
          red_release_sys_add(cp.peer_cnt[pend_owner] + pend_blk, 1u);
          pend_owner = -1;
        }
        if (rs_own) {
          if (lane == 0 && !wait_ge<true>(cp.peer_cnt[cp.rank] + tc.m_local, cp.cnt_target, p.status, 6)) ok = false;
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) { *abort_flag = 1; break; }
          __threadfence_system();              // every lane's loads below are ordered after the acquired counter
        }
#pragma unroll 1
        for (int c = 0; c < BN; c += cw) {
          uint32_t r0[32], r1[32];
          tmem_ld32(t_row + (uint32_t)c, r0);
          if (cw == 64) tmem_ld32(t_row + (uint32_t)c + 32, r1);
          tmem_wait_ld();
          if (wg_empty) {
            if (p.out_mode == OUT_F32_ACC) continue;               // += 0
#pragma unroll
            for (int i = 0; i < 32; ++i) { r0[i] = 0u; r1[i] = 0u; }
          }
          if (lane == 0) bulk_wait_read<1>();                      // the buffer used two chunks ago is free
          __syncwarp();
          uint8_t* stage = my_stage + epi_buf * 4096;
          const int col = n0 + c;
          uint32_t w[32];
          if (p.out_mode == OUT_LP) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float a0 = __uint_as_float(r0[2 * i]) * alpha, a1 = __uint_as_float(r0[2 * i + 1]) * alpha;
              float b0 = __uint_as_float(r1[2 * i]) * alpha, b1 = __uint_as_float(r1[2 * i + 1]) * alpha;
              if (p.bias != nullptr) {
                a0 += load_bias(p.bias, col + 2 * i, p.N, p.lp_fmt); a1 += load_bias(p.bias, col + 2 * i + 1, p.N, p.lp_fmt);
                b0 += load_bias(p.bias, col + 32 + 2 * i, p.N, p.lp_fmt); b1 += load_bias(p.bias, col + 33 + 2 * i, p.N, p.lp_fmt);
              }
              r0[2 * i] = __float_as_uint(a0); r0[2 * i + 1] = __float_as_uint(a1);
              r1[2 * i] = __float_as_uint(b0); r1[2 * i + 1] = __float_as_uint(b1);
            }
            if (rs_own && col < p.N) {
              // 64 columns = 128 bytes of this thread's row in every peer's slot and in the residual
              const size_t rrow = (size_t)(drow + lane);
              auto add_row = [&](const uint16_t* src) {
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  const uint4 raw = *reinterpret_cast<const uint4*>(src + 8 * q);
                  const uint32_t* ww = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
                  for (int k2 = 0; k2 < 4; ++k2) {
                    const float2 f = p.lp_fmt ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ww[k2]))
                                              : __half22float2(*reinterpret_cast<const __half2*>(&ww[k2]));
                    uint32_t* dst = (q < 4) ? &r0[8 * q + 2 * k2] : &r1[8 * (q - 4) + 2 * k2];
                    dst[0] = __float_as_uint(__uint_as_float(dst[0]) + f.x);
                    dst[1] = __float_as_uint(__uint_as_float(dst[1]) + f.y);
                  }
                }
              };
              const uint16_t* recv = reinterpret_cast<const uint16_t*>(cp.peer_recv[cp.rank]);
              const size_t slot_stride = (size_t)cp.bpr * BM * p.N;
              for (int sl = 0; sl < cp.tp; ++sl)
                if (sl != cp.rank) add_row(recv + (size_t)sl * slot_stride + rrow * p.N + col);
              if (cp.residual != nullptr)
                add_row(reinterpret_cast<const uint16_t*>(cp.residual) + rrow * cp.ld_res + col);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              w[i] = pack2(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]), p.lp_fmt);
              w[16 + i] = pack2(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]), p.lp_fmt);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float a = __uint_as_float(r0[i]) * alpha;
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
            if (p.out_mode == OUT_F32_ACC) tma_reduce_add_2d(dmap, smem_u32(stage), col, drow);
            else tma_store_2d(dmap, smem_u32(stage), col, drow);
            bulk_commit();
            ++n_groups;
          }
          epi_buf ^= 1;
        }
      if (cp.mode == COMM_RS && !rs_own && lane == 0) {
        // Signal one tile late: waiting here for this tile's stores to cross NVLink would stall the warp for a
        // round trip per tile.  Everything older than the groups just committed has completed after this wait.
        if (pend_owner >= 0) {
          bulk_wait_upto(n_groups);
          fence_proxy_async_all();
          __threadfence_system();
          red_release_sys_add(cp.peer_cnt[pend_owner] + pend_blk, 1u);
        }
        pend_owner = tc.owner; pend_blk = tc.m_local;
      }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(t_row + (uint32_t)c, r);
        tmem_wait_ld();
        const int col = n0 + c;
        if (row < row_end && col < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
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
    if (lane == 0) {
      if (p.tma_out) bulk_wait<0>();
      if (pend_owner >= 0) {
        fence_proxy_async_all(); __threadfence_system();
        red_release_sys_add(cp.peer_cnt[pend_owner] + pend_blk, 1u);
      }
    }
  }
  // ---------------------------------------------------------------- teardown
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem_base, 2 * BN >= 32 ? 2 * BN : 32); }
}

template <int BN, bool A_MN, bool B_MN, bool FP8 = false>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const ExtraMaps& xm,
                       GemmParams p, const CommParams& cp, int sm_count, cudaStream_t st) {
  using S = GemmSmem<BN>;
  auto kern = gemm_kernel<BN, A_MN, B_MN, FP8>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if (p.group_tiles == nullptr) p.tiles_m = (p.M + BM - 1) / BM;     // grouped mode: set by the caller
  p.tiles_n = (p.N + BN - 1) / BN;
  {
    static int env_gm = -1;
    if (env_gm < 0) { const char* e = getenv("MLB_GEMM_RASTER_M"); env_gm = e ? atoi(e) : 0; }
    p.raster_m = env_gm > 0 ? env_gm : 32;
    if (p.raster_m > p.tiles_m) p.raster_m = p.tiles_m;
    if (p.raster_m < 1) p.raster_m = 1;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  int grid = tiles < sm_count ? tiles : sm_count;
  if (cp.mode == COMM_AG) grid = sm_count;          // workers + GEMM CTAs, all co-resident
  kern<<<grid, kGemmThreads, S::kBytes, st>>>(tmA, tmB, tmD, xm, p, cp);
  MLB_CHECK_LAUNCH();
  return 0;
}

// Tensor maps for A (K- or MN-major), B and, when aligned, the output; then launch.
static int run_gemm(int lp_fmt, const void* A, long lda, int a_mn, const void* B, long ldb, int b_mn, void* D,
                    long ldd, int out_mode, const void* bias, int M, int N, int K, int sms, int* status,
                    const CommParams& cp, cudaStream_t st, const ExtraMaps* xm_in = nullptr);

static int sm_count_cached() {
  static int n = 0;
  if (n == 0) {
    int dev = 0; cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}


static int run_gemm(int lp_fmt, const void* A, long lda, int a_mn, const void* B, long ldb, int b_mn, void* D,
                    long ldd, int out_mode, const void* bias, int M, int N, int K, int sms, int* status,
                    const CommParams& cp, cudaStream_t st, const ExtraMaps* xm_in) {
  static const ExtraMaps kNoMaps = {};
  const ExtraMaps& xm = xm_in ? *xm_in : kNoMaps;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  const int bn = (N > 128) ? 256 : 128;
  CUtensorMap tmA, tmB, tmD;
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
  const int esz = (out_mode == OUT_LP) ? 2 : 4;
  int tma_out = (((size_t)ldd * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(D) & 15) == 0);
  if (cp.mode == COMM_RS) {
    // peers' rows leave through xm; this rank's own rows are stored (already summed) into cp.out through tmD
    tma_out = 1;
    if ((((size_t)cp.ld_out * 2) % 16) || (reinterpret_cast<uintptr_t>(cp.out) & 15)) return -3;
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)(cp.bpr * BM)}, strides[1] = {(uint64_t)cp.ld_out * 2};
    uint32_t box[2] = {64, 32};
    if ((rc = make_tmap(&tmD, cp.out, 2, dims, strides, box, 2))) return rc;
  } else if (tma_out) {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M}, strides[1] = {(uint64_t)ldd * esz};
    uint32_t box[2] = {(uint32_t)(esz == 2 ? 64 : 32), 32};
    if (make_tmap(&tmD, D, 2, dims, strides, box, esz)) tma_out = 0;
  }
  if (!tma_out) tmD = tmA;     // placeholder, unused
  GemmParams p;
  p.tma_out = tma_out;
  p.M = M; p.N = N; p.K = K; p.D = D; p.ldd = ldd; p.bias = bias; p.out_mode = out_mode; p.lp_fmt = lp_fmt;
  p.status = status; p.tiles_m = p.tiles_n = 0;
  p.fp8 = 0; p.a_fmt = p.b_fmt = 0; p.scale_a = p.scale_b = nullptr; p.group_tiles = nullptr;
  p.group_count = nullptr; p.group_offsets = nullptr; p.wg_mblocks = 0;
#define GO(BNv, AM, BMj) return launch_gemm<BNv, AM, BMj>(tmA, tmB, tmD, xm, p, cp, sms, st)
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

// 8-bit operands: A [M, K], B [N, K] bytes, both K-major; D = (A B^T) * (*scale_a) * (*scale_b) (+ bias)
static int run_gemm_fp8(int a_fmt, int b_fmt, const void* A, long lda, const void* B, long ldb, void* D, long ldd,
                        int out_mode, int out_lp_fmt, const void* bias, const float* scale_a, const float* scale_b, int M,
                        int N, int K, int sms, int* status, cudaStream_t st) {
  if ((lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  const int bn = (N > 128) ? 256 : 128;
  CUtensorMap tmA, tmB, tmD;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M}, strides[1] = {(uint64_t)lda};
    uint32_t box[2] = {128, BM};
    if ((rc = make_tmap(&tmA, A, 2, dims, strides, box, 1))) return rc;
    dims[1] = (uint64_t)N; strides[0] = (uint64_t)ldb; box[1] = (uint32_t)bn;
    if ((rc = make_tmap(&tmB, B, 2, dims, strides, box, 1))) return rc;
  }
  const int esz = (out_mode == OUT_LP) ? 2 : 4;
  int tma_out = (((size_t)ldd * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(D) & 15) == 0);
  if (tma_out) {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M}, strides[1] = {(uint64_t)ldd * esz};
    uint32_t box[2] = {(uint32_t)(esz == 2 ? 64 : 32), 32};
    if (make_tmap(&tmD, D, 2, dims, strides, box, esz)) tma_out = 0;
  }
  if (!tma_out) tmD = tmA;
  GemmParams p;
  p.tma_out = tma_out;
  p.M = M; p.N = N; p.K = K; p.D = D; p.ldd = ldd; p.bias = bias; p.out_mode = out_mode; p.lp_fmt = out_lp_fmt;
  p.status = status; p.tiles_m = p.tiles_n = 0;
  p.fp8 = 1; p.a_fmt = a_fmt; p.b_fmt = b_fmt; p.scale_a = scale_a; p.scale_b = scale_b; p.group_tiles = nullptr;
  p.group_count = nullptr; p.group_offsets = nullptr; p.wg_mblocks = 0;
  static const ExtraMaps kNoMaps = {};
  CommParams cp = {};
  if (bn == 256) return launch_gemm<256, false, false, true>(tmA, tmB, tmD, kNoMaps, p, cp, sms, st);
  return launch_gemm<128, false, false, true>(tmA, tmB, tmD, kNoMaps, p, cp, sms, st);
}

// Grouped product over expert-sorted rows (see GemmParams::group_tiles).  A [T, K] K-major; B stacked experts.
static int run_gemm_grouped(int lp_fmt, const void* A, long lda, const void* B, long ldb, int b_mn, void* D, long ldd,
                            const int4* tiles, int n_tiles, int E, int T, int N, int K, int sms, int* status,
                            cudaStream_t st, const int* tile_count = nullptr) {
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (b_mn && (K % BK)) return -3;               // the reduction may not run into the next expert's rows
  const int bn = (N > 128) ? 256 : 128;
  CUtensorMap tmA, tmB;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)T}, strides[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {BK, BM};
    if ((rc = make_tmap(&tmA, A, 2, dims, strides, box))) return rc;
    if (!b_mn) { dims[0] = (uint64_t)K; dims[1] = (uint64_t)E * N; box[0] = BK; box[1] = (uint32_t)bn; }
    else       { dims[0] = (uint64_t)N; dims[1] = (uint64_t)E * K; box[0] = 64; box[1] = BK; }
    strides[0] = (uint64_t)ldb * 2;
    if ((rc = make_tmap(&tmB, B, 2, dims, strides, box))) return rc;
  }
  GemmParams p;
  p.tma_out = 0;
  p.M = T; p.N = N; p.K = K; p.D = D; p.ldd = ldd; p.bias = nullptr; p.out_mode = OUT_LP; p.lp_fmt = lp_fmt;
  p.status = status; p.tiles_m = n_tiles; p.tiles_n = 0;
  p.fp8 = 0; p.a_fmt = p.b_fmt = 0; p.scale_a = p.scale_b = nullptr; p.group_tiles = tiles;
  p.group_count = tile_count; p.group_offsets = nullptr; p.wg_mblocks = 0;
  static const ExtraMaps kNoMaps = {};
  CommParams cp = {};
  if (bn == 256) {
    if (!b_mn) return launch_gemm<256, false, false>(tmA, tmB, tmA, kNoMaps, p, cp, sms, st);
    return launch_gemm<256, false, true>(tmA, tmB, tmA, kNoMaps, p, cp, sms, st);
  }
  if (!b_mn) return launch_gemm<128, false, false>(tmA, tmB, tmA, kNoMaps, p, cp, sms, st);
  return launch_gemm<128, false, true>(tmA, tmB, tmA, kNoMaps, p, cp, sms, st);
}

// Weight gradients of all experts in one launch: dW [E, N_out, K_in] fp32 (=|+=) dy_e^T x_e with dy [T, N_out] and
// x [T, K_in] (rows sorted by expert, expert e = rows [offsets[e], offsets[e + 1])).  N_out a multiple of 128.
static int run_gemm_grouped_wgrad(int lp_fmt, const void* dy, long ld_dy, const void* x, long ld_x, float* dW,
                                  const int* offsets, int E, int T, int N_out, int K_in, int accumulate, int sms,
                                  int* status, cudaStream_t st) {
  if ((ld_dy % 8) || (ld_x % 8) || (reinterpret_cast<uintptr_t>(dy) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return -3;
  if ((N_out % BM) || (K_in % 4) || (reinterpret_cast<uintptr_t>(dW) & 15)) return -3;
  const int bn = (K_in > 128) ? 256 : 128;
  CUtensorMap tmA, tmB, tmD;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)N_out, (uint64_t)T}, strides[1] = {(uint64_t)ld_dy * 2};
    uint32_t box[2] = {64, BK};
    if ((rc = make_tmap(&tmA, dy, 2, dims, strides, box))) return rc;
    dims[0] = (uint64_t)K_in; strides[0] = (uint64_t)ld_x * 2;
    if ((rc = make_tmap(&tmB, x, 2, dims, strides, box))) return rc;
    uint64_t dd[2] = {(uint64_t)K_in, (uint64_t)E * N_out}, ds[1] = {(uint64_t)K_in * 4};
    uint32_t db[2] = {32, 32};
    if ((rc = make_tmap(&tmD, dW, 2, dd, ds, db, 4))) return rc;
  }
  GemmParams p;
  p.tma_out = 1;
  p.M = E * N_out; p.N = K_in; p.K = T; p.D = dW; p.ldd = K_in; p.bias = nullptr;
  p.out_mode = accumulate ? OUT_F32_ACC : OUT_F32; p.lp_fmt = lp_fmt;
  p.status = status; p.tiles_m = 0; p.tiles_n = 0;
  p.fp8 = 0; p.a_fmt = p.b_fmt = 0; p.scale_a = p.scale_b = nullptr; p.group_tiles = nullptr;
  p.group_count = nullptr; p.group_offsets = offsets; p.wg_mblocks = N_out / BM;
  static const ExtraMaps kNoMaps = {};
  CommParams cp = {};
  if (bn == 256) return launch_gemm<256, true, true>(tmA, tmB, tmD, kNoMaps, p, cp, sms, st);
  return launch_gemm<128, true, true>(tmA, tmB, tmD, kNoMaps, p, cp, sms, st);
}

}  // namespace mlb
