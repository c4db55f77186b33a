// CTA-pair variant of the bf16/fp16 GEMM (plain mode): two CTAs of one cluster (one TPC) compute a 256 x 256 output
// tile with `tcgen05.mma.cta_group::2`.  Each CTA stages 128 rows of A and 128 of the 256 B rows per K step, so a
// stage is 32 KB per SM instead of 48 KB - the L2 -> shared traffic per flop drops by a third, which is what
// limits the single-CTA kernel.  Five stages and eight epilogue warps per CTA (two per TMEM lane quadrant, each
// taking half of the tile's columns) fit in shared memory.  The accumulator rows [128 r, 128 r + 128) live in CTA r's
// tensor memory; each CTA drains its own half.
//   * full[s]   lives in the leader (even) CTA: its producer posts the 64 KB expectation, both CTAs' TMA loads
//               complete on it (plain per-CTA loads, the barrier is addressed through the cluster window);
//   * empty[s], tfull[a] exist in both CTAs and are signalled by the leader's commit with a 2-CTA mask;
//   * tempty[a] lives in the leader: the sixteen epilogue warps of the pair arrive on it.
// Every wait is bounded (status word), like in the single-CTA kernel.
#pragma once
#include "gemm_core.cuh"

namespace mlb {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// cluster-scope acquire: pairs with a release.cluster arrive made by the other CTA after it stored data here
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\tselp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// one arrival on the barrier at this shared-memory offset in every CTA of `mask`, once the MMAs issued so far are done
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask) : "memory");
}

constexpr int kGemm2Threads = 320;    // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue (two warps per TMEM lane quadrant)

struct Gemm2Smem {
  static constexpr int kStages = 5;
  static constexpr int kABytes = 128 * BK * 2;          // this CTA's 128 rows of A
  static constexpr int kBBytes = 128 * BK * 2;          // this CTA's 128 of the tile's 256 B rows
  static constexpr int kEpiBytes = 8 * 2 * 4096;        // per epilogue warp: two 32-row x 128-byte staging buffers
  static constexpr int kBytes = kStages * (kABytes + kBBytes) + kEpiBytes + 1024 + 256;
};

// FP8 (both operands K-major bytes, 128 per 128-byte row, 32 per MMA) is a separate instantiation, see gemm_core.cuh.
template <bool A_MN, bool B_MN, bool FP8 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemm2Threads, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
             const __grid_constant__ CUtensorMap tmD, const __grid_constant__ ExtraMaps xm, const GemmParams p,
             const CommParams cp) {
  using S = Gemm2Smem;
  constexpr int kStages = S::kStages;
  constexpr int TN = 256;                                // tile columns
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * S::kABytes;
  uint8_t* sEpi = smem + kStages * (S::kABytes + S::kBBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + S::kEpiBytes);
  constexpr int kSched = 4;                              // depth of the tile-announcement ring (dynamic schedule)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4 + 2 * kSched);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* tile_ring = reinterpret_cast<volatile int*>(tmem_slot + 2);     // [kSched]
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
  auto tempty = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };
  auto sfull = [&](int s) { return bar0 + 8u * (2 * kStages + 4 + s); };              // one per CTA
  auto sempty = [&](int s) { return bar0 + 8u * (2 * kStages + 4 + kSched + s); };    // used in the leader only

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // All-gather mode: the first n_comm CTAs (whole pairs) are copy workers and take no part in the GEMM or in any
  // cluster-wide synchronisation.
  if (cp.mode == COMM_AG && (int)blockIdx.x < cp.n_comm) {
    ag_comm_cta<6>(smem, bars, p, cp);
    return;
  }
  const uint32_t rank = cluster_ctarank();               // 0 = leader
  const bool leader = rank == 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull(a), 1); mbar_init(tempty(a), 16); }
    // a tile announcement is read by 18 parties: the leader's MMA thread, the partner's producer and the
    // 16 epilogue warps of the pair
    for (int q = 0; q < kSched; ++q) { mbar_init(sfull(q), 1); mbar_init(sempty(q), 18); }
    // a wait that ran out earlier on this GPU (this step is lost anyway): drain at once instead of waiting again
    *abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    mbar_fence_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB); prefetch_tmap(&tmD);
  }
  if (warp == 1) { tmem_alloc2(smem_u32(tmem_slot), 512); tmem_relinquish2(); }
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();                                    // the peer's barriers exist before anything signals them
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + 255) / 256, tiles_n = (p.N + TN - 1) / TN;
  const int num_tiles = tiles_m * tiles_n;
  constexpr int bk_elems = FP8 ? 2 * BK : BK;
  const int num_kb = (p.K + bk_elems - 1) / bk_elems;
  const int first_cta = (cp.mode == COMM_AG) ? cp.n_comm : 0;
  const int pair = ((int)blockIdx.x - first_cta) >> 1, n_pairs = ((int)gridDim.x - first_cta) >> 1;
  const int gm = p.raster_m < tiles_m ? (p.raster_m > 0 ? p.raster_m : 1) : tiles_m;
  const int bpr2 = cp.bpr >> 1;                          // 256-row blocks per rank (communication modes)
  // tile -> (256-row block, 256-column block, owner rank of the rows, 256-row block within the owner's rows)
  auto tile_mn = [&](int tile, int& m_blk, int& n_blk, int& owner, int& m_loc) {
    if (cp.mode == COMM_NONE) {
      const int per_group = gm * tiles_n;
      const int grp = tile / per_group, in_grp = tile % per_group;
      const int first_m = grp * gm;
      const int size_m = (tiles_m - first_m) < gm ? (tiles_m - first_m) : gm;
      m_blk = first_m + in_grp % size_m; n_blk = in_grp / size_m; owner = 0; m_loc = m_blk;
    } else {
      const int per_group = bpr2 * tiles_n;
      const int g = tile / per_group, idx = tile % per_group;
      m_loc = idx % bpr2; n_blk = idx / bpr2;
      owner = (cp.mode == COMM_AG) ? (cp.rank + g) % cp.tp : (cp.rank + 1 + g) % cp.tp;
      m_blk = owner * bpr2 + m_loc;
    }
  };

  // Tile schedule.  Static (plain products): pair q takes tiles q, q + n_pairs, ...  Dynamic (cp.sched set; the
  // communication modes): the leader's producer thread draws tile numbers from a global counter and announces
  // them to both CTAs through a small ring, so tiles only ever belong to pairs that are running.  A pair that
  // has not been given an SM yet (other kernels hold it) then owns nothing that a peer GPU or a later tile could
  // wait for: the fused kernels stay deadlock-free whatever share of the grid is resident.
  const bool dyn = cp.sched != nullptr;
  const uint32_t sempty_leader0 = map_to_cta(sempty(0), 0);
  // i-th tile of this pair for a consumer role (-1: no more tiles, -2: a wait ran out)
  auto consumer_tile = [&](int i) -> int {
    if (!dyn) { const int t = pair + i * n_pairs; return t < num_tiles ? t : -1; }
    const int q = i % kSched;
    const uint32_t par = (uint32_t)(i / kSched) & 1u;
    if (!mbar_try_wait_cluster(sfull(q), par)) {
      const long long t0 = clock64();
      uint32_t it = 0;
      while (!mbar_try_wait_cluster(sfull(q), par)) {
        if ((++it & 63u) == 0u) {
          if (*abort_flag) return -2;
          if (clock64() - t0 > kWaitCycles) { *abort_flag = 1; if (p.status) atomicCAS(p.status, 0, 7); return -2; }
        }
      }
    }
    return tile_ring[q];
  };
  auto consumer_release = [&](int i) { mbar_arrive_cluster(sempty_leader0 + 8u * (uint32_t)(i % kSched)); };
  auto draw_tile = [&]() -> int {
    const int t = (int)atomicAdd(cp.sched, 1u);
    return t < num_tiles ? t : -1;
  };
  // leader's producer: publish the i-th tile number (or -1) in both CTAs
  auto announce = [&](int i, int tile) -> bool {
    const int q = i % kSched;
    if (!mbar_wait(sempty(q), ((uint32_t)(i / kSched) & 1u) ^ 1u, abort_flag, p.status, 8)) return false;
    tile_ring[q] = tile;
    st_cluster_u32(map_to_cta(smem_u32(const_cast<int*>(tile_ring + q)), 1), (uint32_t)tile);
    mbar_arrive_cluster(map_to_cta(sfull(q), 0));
    mbar_arrive_cluster(map_to_cta(sfull(q), 1));
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      int ready_blk = -1;
      const bool scheduler = dyn && leader;
      int drawn = scheduler ? draw_tile() : 0;           // the next draw is always in flight behind the current tile
      for (int i = 0; ok; ++i) {
        int tile;
        if (scheduler) {
          tile = drawn;
          if (!announce(i, tile)) { ok = false; break; }
          if (tile >= 0) drawn = draw_tile();
        } else {
          tile = consumer_tile(i);
          if (tile == -2) { ok = false; break; }
          if (dyn) consumer_release(i);
        }
        if (tile < 0) break;
        int mb, nb, owner, mloc; tile_mn(tile, mb, nb, owner, mloc);
        const int m0 = mb * 256 + 128 * (int)rank, n0 = nb * TN + 128 * (int)rank;
        const bool own_rows = cp.mode == COMM_AG && owner == cp.rank;
        if (cp.mode == COMM_AG && !own_rows && (2 * mb + (int)rank) != ready_blk) {
          // this CTA's 128 rows arrive from a peer: wait for the copy worker's flag of that row block
          if (!wait_ge<false>(cp.chunk_flags + 2 * mb + (int)rank, cp.seq, p.status, 5)) { *abort_flag = 1; ok = false; break; }
          fence_proxy_async_all();
          ready_blk = 2 * mb + (int)rank;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty(stage), phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
          if (leader) mbar_expect_tx(full(stage), 2 * (S::kABytes + S::kBBytes));
          const uint32_t fbar = map_to_cta(full(stage), 0);
          const uint32_t a_dst = smem_u32(sA + stage * S::kABytes), b_dst = smem_u32(sB + stage * S::kBBytes);
          const int k0 = kb * bk_elems;
          if constexpr (!A_MN) {
            if (own_rows) tma_load_2d_pair(a_dst, &xm.m[0], fbar, k0, mloc * 256 + 128 * (int)rank);
            else tma_load_2d_pair(a_dst, &tmA, fbar, k0, m0);              // box [64 k, 128 rows]
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(a_dst + j * 8192, &tmA, fbar, m0 + 64 * j, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(b_dst, &tmB, fbar, k0, n0);                   // box [64 k, 128 rows]
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(b_dst + j * 8192, &tmB, fbar, n0 + 64 * j, k0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { const long long t0 = clock64(); while (clock64() - t0 < 2000000LL) { __nanosleep(1000); } }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      const uint32_t idesc = FP8 ? make_idesc_f8(256, TN, p.a_fmt, p.b_fmt)
                                 : make_idesc(256, TN, p.lp_fmt, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0; uint32_t phase = 0;
      int t = 0;
      bool ok = true;
      for (; ok; ++t) {
        const int tile = consumer_tile(t);
        if (tile == -2) { ok = false; break; }
        if (dyn) consumer_release(t);
        if (tile < 0) break;
        const int acc = t & 1;
        const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
        if (!mbar_wait(tempty(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * TN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full(stage), phase, abort_flag, p.status, 3)) { ok = false; break; }
          fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * S::kABytes), b_addr = smem_u32(sB + stage * S::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t da = A_MN ? make_desc(a_addr + k * 2048, 8192, 1024) : make_desc(a_addr + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_desc(b_addr + k * 2048, 8192, 1024) : make_desc(b_addr + k * 32, 16, 1024);
            if constexpr (FP8) mma_f8_pair(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else mma_f16_pair(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit_pair(empty(stage), 3);      // both CTAs may refill this stage once the MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) mma_commit_pair(tfull(acc), 3);  // accumulator complete: wake both CTAs' epilogue warps
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9 of both CTAs): warp w drains
    // TMEM lanes of quadrant w % 4; warps 2..5 take tile columns [0, 128), warps 6..9 columns [128, 256)
    const int quad = warp & 3;
    const int chalf = (warp - 2) >> 2;
    int t = 0, epi_buf = 0;
    // reduce-scatter: the last two tiles stored to a peer still owe their arrival signals (a signal may only go out
    // once the tile's stores have completed at the peer, an NVLink round trip of about two tile times at small K)
    int pend_owner = -1, pend_blk = 0, pend_groups = 0, pend2_owner = -1, pend2_blk = 0;
    bool ok = true;
    const uint32_t tempty_leader0 = map_to_cta(tempty(0), 0);
    for (; ok; ++t) {
      const int tile = consumer_tile(t);                  // every lane reads the announcement
      if (tile == -2) { ok = false; break; }
      if (dyn) { __syncwarp(); if (lane == 0) consumer_release(t); }
      if (tile < 0) break;
      const int acc = t & 1;
      const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
      int mb, nb, owner, mloc; tile_mn(tile, mb, nb, owner, mloc);
      const int m0 = mb * 256 + 128 * (int)rank, n0 = nb * TN;
      // reduce-scatter: rows of other ranks go to this rank's slot in their receive buffer; this rank's own rows
      // (computed last) add the peers' arrived partial rows and the residual and are stored finished
      const bool rs = cp.mode == COMM_RS;
      const bool rs_own = rs && owner == cp.rank;
      if (rs_own && lane == 0 && pend_owner >= 0) {
        // first own tile: the signals still owed to peers go out now, before this tile's accumulator is waited for
        bulk_wait<0>(); fence_proxy_async_all(); __threadfence_system();
        if (pend2_owner >= 0) red_release_sys_add(cp.peer_cnt[pend2_owner] + pend2_blk, 1u);
        red_release_sys_add(cp.peer_cnt[pend_owner] + pend_blk, 1u);
        pend_owner = pend2_owner = -1;
      }
      if (!mbar_wait(tfull(acc), acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
      fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * TN);
      const int cw = (p.out_mode == OUT_LP) ? 64 : 32;
      uint8_t* my_stage = sEpi + (warp - 2) * 8192;
      const int blk_loc = 2 * mloc + (int)rank;            // 128-row block inside the owner's rows
      const CUtensorMap* dmap = (rs && !rs_own) ? &xm.m[owner] : &tmD;
      const int drow = rs ? blk_loc * 128 + quad * 32 : m0 + quad * 32;
      const float alpha = (p.scale_a ? *p.scale_a : 1.f) * (p.scale_b ? *p.scale_b : 1.f);
      int n_groups = 0;
      if (rs_own) {
        if (lane == 0 && !wait_ge<true>(cp.peer_cnt[cp.rank] + blk_loc, cp.cnt_target, p.status, 6)) ok = false;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) { *abort_flag = 1; break; }
        __threadfence_system();
      }
#pragma unroll 1
      for (int c = chalf * 128; c < chalf * 128 + 128; c += cw) {
        uint32_t r0[32], r1[32];
        tmem_ld32(t_row + (uint32_t)c, r0);
        if (cw == 64) tmem_ld32(t_row + (uint32_t)c + 32, r1);
        tmem_wait_ld();
        if (lane == 0) bulk_wait_read<1>();
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
        if (lane == 0 && col < p.N && (rs || drow < p.M)) {
          if (p.out_mode == OUT_F32_ACC) tma_reduce_add_2d(dmap, smem_u32(stage), col, drow);
          else tma_store_2d(dmap, smem_u32(stage), col, drow);
          bulk_commit();
          ++n_groups;
        }
        epi_buf ^= 1;
      }
      if (rs && !rs_own && lane == 0) {
        // Signal two tiles late: waiting here for this tile's stores to cross NVLink would stall the warp for a
        // round trip per tile.  Everything older than the groups of the last two tiles has completed after this wait.
        if (pend2_owner >= 0) {
          bulk_wait_upto(pend_groups + n_groups);
          fence_proxy_async_all();
          __threadfence_system();
          red_release_sys_add(cp.peer_cnt[pend2_owner] + pend2_blk, 1u);
        }
        pend2_owner = pend_owner; pend2_blk = pend_blk;
        pend_owner = owner; pend_blk = blk_loc; pend_groups = n_groups;
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8u * (uint32_t)acc);
    }
    if (lane == 0) {
      bulk_wait<0>();
      if (pend_owner >= 0) {
        fence_proxy_async_all(); __threadfence_system();
        if (pend2_owner >= 0) red_release_sys_add(cp.peer_cnt[pend2_owner] + pend2_blk, 1u);
        red_release_sys_add(cp.peer_cnt[pend_owner] + pend_blk, 1u);
      }
    }
  }
  // ---------------------------------------------------------------- teardown: nobody leaves while the peer may
  // still signal this CTA's barriers or read its operand tiles
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) { fence_after_sync(); tmem_dealloc2(tmem_base, 512); }
  if (dyn && leader && threadIdx.x == 0) {
    // the last pair to leave puts the counters back to zero for the next launch on this buffer set (launches
    // that share a counter pair are ordered on one stream)
    __threadfence();
    if (atomicAdd(cp.sched + 1, 1u) + 1u == (uint32_t)n_pairs) { cp.sched[0] = 0u; cp.sched[1] = 0u; __threadfence(); }
  }
}

template <bool A_MN, bool B_MN, bool FP8 = false>
static int launch_gemm2(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const ExtraMaps& xm,
                        const GemmParams& p, const CommParams& cp, int sm_count, cudaStream_t st) {
  using S = Gemm2Smem;
  auto kern = gemm2_kernel<A_MN, B_MN, FP8>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256);
  int pairs = sm_count / 2;
  if (tiles < pairs && cp.mode != COMM_AG) pairs = tiles;          // all-gather mode: workers + GEMM pairs, all resident
  kern<<<2 * pairs, kGemm2Threads, S::kBytes, st>>>(tmA, tmB, tmD, xm, p, cp);
  MLB_CHECK_LAUNCH();
  return 0;
}

// Same contract as run_gemm (plain mode); the output must be TMA-addressable (16-byte aligned rows).
static int run_gemm2(int lp_fmt, const void* A, long lda, int a_mn, const void* B, long ldb, int b_mn, void* D, long ldd,
                     int out_mode, const void* bias, int M, int N, int K, int sms, int* status, cudaStream_t st,
                     const CommParams* cp_in = nullptr, const ExtraMaps* xm_in = nullptr) {
  static const ExtraMaps kNoMaps = {};
  static const CommParams kNoComm = {};
  const CommParams& cp = cp_in ? *cp_in : kNoComm;
  const ExtraMaps& xm = xm_in ? *xm_in : kNoMaps;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  const int esz = (out_mode == OUT_LP) ? 2 : 4;
  int M_d = M;                                      // rows of the output map
  if (cp.mode == COMM_RS) { D = cp.out; ldd = cp.ld_out; M_d = cp.bpr * BM; }   // only this rank's rows are output
  if ((((size_t)ldd * esz) % 16) || (reinterpret_cast<uintptr_t>(D) & 15)) return -3;
  if (cp.mode != COMM_NONE && ((cp.bpr & 1) || a_mn)) return -7;               // 256-row tiles must not straddle ranks
  CUtensorMap tmA, tmB, tmD;
  int rc;
  uint64_t dims[2], strides[1]; uint32_t box[2];
  if (!a_mn) { dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = BK; box[1] = 128; }
  else       { dims[0] = (uint64_t)M; dims[1] = (uint64_t)K; box[0] = 64; box[1] = BK; }
  strides[0] = (uint64_t)lda * 2;
  if ((rc = make_tmap(&tmA, A, 2, dims, strides, box))) return rc;
  if (!b_mn) { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; box[0] = BK; box[1] = 128; }
  else       { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; box[0] = 64; box[1] = BK; }
  strides[0] = (uint64_t)ldb * 2;
  if ((rc = make_tmap(&tmB, B, 2, dims, strides, box))) return rc;
  {
    uint64_t dd[2] = {(uint64_t)N, (uint64_t)M_d}, ds[1] = {(uint64_t)ldd * esz};
    uint32_t db[2] = {(uint32_t)(esz == 2 ? 64 : 32), 32};
    if ((rc = make_tmap(&tmD, D, 2, dd, ds, db, esz))) return rc;
  }
  GemmParams p = {};
  p.tma_out = 1;
  p.M = M; p.N = N; p.K = K; p.D = D; p.ldd = ldd; p.bias = bias; p.out_mode = out_mode; p.lp_fmt = lp_fmt;
  p.status = status;
  {
    static int env_gm = -1;
    if (env_gm < 0) { const char* e = getenv("MLB_GEMM_RASTER_M"); env_gm = e ? atoi(e) : 0; }
    p.raster_m = env_gm > 0 ? env_gm : 16;
  }
  if (!a_mn && !b_mn) return launch_gemm2<false, false>(tmA, tmB, tmD, xm, p, cp, sms, st);
  if (!a_mn && b_mn) return launch_gemm2<false, true>(tmA, tmB, tmD, xm, p, cp, sms, st);
  if (a_mn && !b_mn) return launch_gemm2<true, false>(tmA, tmB, tmD, xm, p, cp, sms, st);
  return launch_gemm2<true, true>(tmA, tmB, tmD, xm, p, cp, sms, st);
}

// 8-bit operands on the CTA-pair kernel: A [M, K], B [N, K] bytes, K-major; D = (A B^T) * (*scale_a) * (*scale_b) (+ bias)
static int run_gemm2_fp8(int a_fmt, int b_fmt, const void* A, long lda, const void* B, long ldb, void* D, long ldd,
                         int out_mode, int out_lp_fmt, const void* bias, const float* scale_a, const float* scale_b, int M,
                         int N, int K, int sms, int* status, cudaStream_t st) {
  if ((lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  const int esz = (out_mode == OUT_LP) ? 2 : 4;
  if ((((size_t)ldd * esz) % 16) || (reinterpret_cast<uintptr_t>(D) & 15)) return -3;
  CUtensorMap tmA, tmB, tmD;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M}, strides[1] = {(uint64_t)lda};
    uint32_t box[2] = {128, 128};
    if ((rc = make_tmap(&tmA, A, 2, dims, strides, box, 1))) return rc;
    dims[1] = (uint64_t)N; strides[0] = (uint64_t)ldb;
    if ((rc = make_tmap(&tmB, B, 2, dims, strides, box, 1))) return rc;
    uint64_t dd[2] = {(uint64_t)N, (uint64_t)M}, ds[1] = {(uint64_t)ldd * esz};
    uint32_t db[2] = {(uint32_t)(esz == 2 ? 64 : 32), 32};
    if ((rc = make_tmap(&tmD, D, 2, dd, ds, db, esz))) return rc;
  }
  GemmParams p = {};
  p.tma_out = 1;
  p.M = M; p.N = N; p.K = K; p.D = D; p.ldd = ldd; p.bias = bias; p.out_mode = out_mode; p.lp_fmt = out_lp_fmt;
  p.status = status; p.fp8 = 1; p.a_fmt = a_fmt; p.b_fmt = b_fmt; p.scale_a = scale_a; p.scale_b = scale_b;
  p.raster_m = 16;
  static const ExtraMaps kNoMaps = {};
  static const CommParams kNoComm = {};
  return launch_gemm2<false, false, true>(tmA, tmB, tmD, kNoMaps, p, kNoComm, sms, st);
}

}  // namespace mlb
