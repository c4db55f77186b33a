// Block-scaled FP8 (MXFP8: e4m3 / e5m2 elements, one UE8M0 scale per 32 consecutive K elements) GEMM on the
// CTA-pair tensor-core path: D[M,N] (=|+=) A[M,K] * B[N,K]^T with `tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale`.
// Both operands are K-major bytes; the scale factors are applied by the tensor core per 32-element K block, so
// the accumulator needs no dequantisation pass.
//
// Tile: 256 rows (128 per CTA of the pair) x 192 columns.  Two 192-column fp32 accumulators take 384 of the 512
// tensor-memory columns; the scale factors of one K stage need 12 more (4 for this CTA's 128 A rows, 8 for up to
// 256 B rows).  (A 256-column tile would leave no room for them.)
//
// Scale factors travel in chunks of four K stages, on a ring of their own (three 6 KB slots, own barriers): `tcgen05.cp`
// runs in the MMA pipe in issue order, and every switch between products and copies costs the pipe a bubble - three
// copies in front of the four MMAs of every stage kept the tensor pipe 40 % busy (1570 TFLOP/s at 4096 x 11008 x
// 4096; 1890 with the copies left out).  So the MMA thread issues the twelve copies of a chunk back to back into one
// of two 48-column tensor-memory buffers, then the sixteen MMAs of its four stages.  (Writing the scale factors with
// `tcgen05.st` from four extra warps, which keeps them out of the MMA pipe altogether, measured 1060: that path's
// latency per stage is longer than the stage.)
//
// Scale-factor layout in global memory ("atoms"): for a quantised matrix Q[rows, K] the scale of row r and K block
// kb (32 elements) is the byte
//     atom(r / 128, kb / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + (kb % 4)
// with atom(i, j) = i * ceil(K / 128) + j.  One atom (512 bytes = 32 rows x 16 bytes) holds the scales of 128 rows
// x 128 K elements, already in the order `tcgen05.cp.32x128b.warpx4` wants: copied to tensor memory, row r's four
// scales sit in lane r % 32 (replicated to the four lane quadrants), column r / 32, byte kb % 4 - the byte the
// instruction descriptor's scale-factor id selects for each of the four K = 32 MMAs of a 128-byte stage.
// The quantiser (fp8.cu, mlb_mxfp8_quantize_dual) writes this layout directly.
//
// Per stage and CTA: 128 A rows + 96 B rows of 128 bytes (TMA, 128B swizzle), its A atom and the two B atoms that
// cover the tile's 192 columns (TMA, no swizzle).  A 192-column tile starts on a 64-row boundary of an atom, so the
// B scale address handed to the MMA is offset by (n0 % 128) / 32 columns.
//
// Stands in for the MXFP8 recipe the reference reaches through Transformer Engine
// (megatron/core/fp8_utils.py:459-485, megatron/core/extensions/transformer_engine.py:396-427).
#include "gemm2.cuh"

namespace mlb {

constexpr int kMxTN = 192;

__device__ __forceinline__ void mma_mx_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate, uint32_t tsfa, uint32_t tsfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb) : "memory");
}
// shared memory (32 rows x 16 bytes, dense) -> tensor memory, replicated to the four lane quadrants, in both CTAs
// of the pair (each from its own shared memory at this offset)
__device__ __forceinline__ void sf_copy_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// un-swizzled K-major descriptor of a 32 x 16-byte block: 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(128u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
// kind::mxf8f6f4 block-scaled instruction descriptor: UE8M0 scales, fp32 accumulate, both operands K-major
__host__ __device__ constexpr uint32_t make_idesc_mx(int m, int n, int a_fmt, int b_fmt, int sf_id) {
  return ((uint32_t)sf_id << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(n >> 3) << 17) |
         (1u << 23) | ((uint32_t)(m >> 4) << 24) | ((uint32_t)sf_id << 29);
}

struct GemmMxSmem {
  static constexpr int kStages = 5;
  static constexpr int kABytes = 128 * 128;            // this CTA's 128 rows of A, 128 bytes (K elements) each
  static constexpr int kBBytes = 96 * 128;             // this CTA's 96 of the tile's 192 B rows
  static constexpr int kSfSlots = 3;
  static constexpr int kSfBytes = 3 * 2048;            // four K stages of: A atom, two B atoms (atom = 512 bytes)
  static constexpr int kEpiBytes = 8 * 2 * 4096;
  static constexpr int kBytes = kStages * (kABytes + kBBytes) + kSfSlots * kSfBytes + kEpiBytes + 1024 + 256;
};

struct MxParams {
  int M, N, K;
  int out_mode, lp_fmt;
  int a_fmt, b_fmt;
  const void* bias;
  int* status;
  int raster_m;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemm2Threads, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
               const __grid_constant__ CUtensorMap tmD, const MxParams p) {
  using S = GemmMxSmem;
  constexpr int kStages = S::kStages;
  constexpr int TN = kMxTN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * S::kABytes;
  // the epilogue's staging buffers are 128B-swizzled like the operand tiles and must sit on 1024-byte boundaries:
  // they come right after the operand stages, the (un-swizzled) scale-factor stages after them
  uint8_t* sEpi = smem + kStages * (S::kABytes + S::kBBytes);
  uint8_t* sSF = sEpi + S::kEpiBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sSF + S::kSfSlots * S::kSfBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4 + 2 * S::kSfSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
  auto tempty = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };
  auto sf_full = [&](int s) { return bar0 + 8u * (2 * kStages + 4 + s); };
  auto sf_empty = [&](int s) { return bar0 + 8u * (2 * kStages + 4 + S::kSfSlots + s); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull(a), 1); mbar_init(tempty(a), 16); }
    for (int i = 0; i < S::kSfSlots; ++i) { mbar_init(sf_full(i), 1); mbar_init(sf_empty(i), 1); }
    *abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    mbar_fence_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB); prefetch_tmap(&tmSFA); prefetch_tmap(&tmSFB); prefetch_tmap(&tmD);
  }
  if (warp == 1) { tmem_alloc2(smem_u32(tmem_slot), 512); tmem_relinquish2(); }
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sf = tmem_base + 2 * TN;           // 2 chunks x 4 stages x 12 columns behind the accumulators

  const int tiles_m = (p.M + 255) / 256, tiles_n = (p.N + TN - 1) / TN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + 127) / 128;
  const int pair = (int)blockIdx.x >> 1, n_pairs = (int)gridDim.x >> 1;
  const int gm = p.raster_m < tiles_m ? (p.raster_m > 0 ? p.raster_m : 1) : tiles_m;
  auto tile_mn = [&](int tile, int& m_blk, int& n_blk) {
    const int per_group = gm * tiles_n;
    const int grp = tile / per_group, in_grp = tile % per_group;
    const int first_m = grp * gm;
    const int size_m = (tiles_m - first_m) < gm ? (tiles_m - first_m) : gm;
    m_blk = first_m + in_grp % size_m; n_blk = in_grp / size_m;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int slot = 0; uint32_t sphase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int mb, nb; tile_mn(tile, mb, nb);
        const int m0 = mb * 256 + 128 * (int)rank, n0 = nb * TN;
        const int sfa_atom = (m0 >> 7) * num_kb;                  // atom (m0 / 128, 0)
        const int sfb_atom0 = n0 >> 7;
        for (int kb = 0; kb < num_kb; ++kb) {
          if ((kb & 3) == 0) {
            // the scale factors of K stages kb .. kb + 3: three requests of four consecutive atoms each (rows past the
            // end of the buffer are zero-filled and still counted; atoms past this tile's K range are not used)
            if (!mbar_wait(sf_empty(slot), sphase ^ 1u, abort_flag, p.status, 5)) { ok = false; break; }
            if (leader) mbar_expect_tx(sf_full(slot), 2 * S::kSfBytes);
            const uint32_t sbar = map_to_cta(sf_full(slot), 0);
            const uint32_t sf_dst = smem_u32(sSF + slot * S::kSfBytes);
            tma_load_2d_pair(sf_dst, &tmSFA, sbar, 0, sfa_atom + kb);
            tma_load_2d_pair(sf_dst + 2048, &tmSFB, sbar, 0, sfb_atom0 * num_kb + kb);
            tma_load_2d_pair(sf_dst + 4096, &tmSFB, sbar, 0, (sfb_atom0 + 1) * num_kb + kb);
            if (++slot == S::kSfSlots) { slot = 0; sphase ^= 1u; }
          }
          if (!mbar_wait(empty(stage), phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
          if (leader) mbar_expect_tx(full(stage), 2 * (S::kABytes + S::kBBytes));
          const uint32_t fbar = map_to_cta(full(stage), 0);
          const uint32_t a_dst = smem_u32(sA + stage * S::kABytes), b_dst = smem_u32(sB + stage * S::kBBytes);
          tma_load_2d_pair(a_dst, &tmA, fbar, kb * 128, m0);                          // box [128 B, 128 rows]
          tma_load_2d_pair(b_dst, &tmB, fbar, kb * 128, n0 + 96 * (int)rank);         // box [128 B, 96 rows]
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { const long long t0 = clock64(); while (clock64() - t0 < 2000000LL) { __nanosleep(1000); } }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      uint32_t idesc[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) idesc[k] = make_idesc_mx(256, TN, p.a_fmt, p.b_fmt, k);
      int stage = 0; uint32_t phase = 0;
      int t = 0;
      int slot = 0; uint32_t sphase = 0;
      uint32_t chunk = 0;                  // scale-factor chunks consumed so far: picks the tensor-memory buffer
      uint32_t tsf_chunk = tmem_sf;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++t) {
        int mb, nb; tile_mn(tile, mb, nb);
        const uint32_t sfb_col = (uint32_t)(((nb * TN) & 127) >> 5);        // 0 or 2
        const int acc = t & 1;
        const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
        if (!mbar_wait(tempty(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * TN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if ((kb & 3) == 0) {
            if (!mbar_wait(sf_full(slot), sphase, abort_flag, p.status, 6)) { ok = false; break; }
            fence_after_sync();
            tsf_chunk = tmem_sf + (chunk & 1u) * 48u;
            const uint32_t sf_addr = smem_u32(sSF + slot * S::kSfBytes);
            const int n_st = (num_kb - kb) < 4 ? (num_kb - kb) : 4;
            for (int j = 0; j < n_st; ++j) {
              sf_copy_pair(tsf_chunk + j * 12, make_sf_desc(sf_addr + j * 512));
              sf_copy_pair(tsf_chunk + j * 12 + 4, make_sf_desc(sf_addr + 2048 + j * 512));
              sf_copy_pair(tsf_chunk + j * 12 + 8, make_sf_desc(sf_addr + 4096 + j * 512));
            }
            mma_commit_pair(sf_empty(slot), 3);          // the slot may be refilled once these copies have run
            ++chunk;
            if (++slot == S::kSfSlots) { slot = 0; sphase ^= 1u; }
          }
          if (!mbar_wait(full(stage), phase, abort_flag, p.status, 3)) { ok = false; break; }
          fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * S::kABytes), b_addr = smem_u32(sB + stage * S::kBBytes);
          const uint32_t tsf = tsf_chunk + (uint32_t)((kb & 3) * 12);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_mx_pair(d_tmem, make_desc(a_addr + k * 32, 16, 1024), make_desc(b_addr + k * 32, 16, 1024), idesc[k],
                        (kb > 0 || k > 0) ? 1u : 0u, tsf, tsf + 4 + sfb_col);
          mma_commit_pair(empty(stage), 3);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) mma_commit_pair(tfull(acc), 3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9 of both CTAs): TMEM lane
    // quadrant warp % 4; warps 2..5 take tile columns [0, 128), warps 6..9 columns [128, 192)
    const int quad = warp & 3;
    const int chalf = (warp - 2) >> 2;
    const int c_begin = chalf * 128, c_end = chalf ? TN : 128;
    int t = 0, epi_buf = 0;
    bool ok = true;
    const uint32_t tempty_leader0 = map_to_cta(tempty(0), 0);
    for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++t) {
      const int acc = t & 1;
      const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
      int mb, nb; tile_mn(tile, mb, nb);
      const int m0 = mb * 256 + 128 * (int)rank, n0 = nb * TN;
      if (!mbar_wait(tfull(acc), acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
      fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * TN);
      const int cw = (p.out_mode == OUT_LP) ? 64 : 32;
      uint8_t* my_stage = sEpi + (warp - 2) * 8192;
      const int drow = m0 + quad * 32;
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += cw) {
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
        if (lane == 0 && col < p.N && drow < p.M) {
          if (p.out_mode == OUT_F32_ACC) tma_reduce_add_2d(&tmD, smem_u32(stage), col, drow);
          else tma_store_2d(&tmD, smem_u32(stage), col, drow);
          bulk_commit();
        }
        epi_buf ^= 1;
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8u * (uint32_t)acc);
    }
    if (lane == 0) bulk_wait<0>();
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) { fence_after_sync(); tmem_dealloc2(tmem_base, 512); }
}

// tensor map without swizzle over the scale-factor atoms: one row of 128 32-bit words (512 bytes) per atom; a request
// moves four consecutive atoms (four K stages of one 128-row block), each landing in shared memory as the dense
// 32 x 16-byte block tcgen05.cp reads
static int make_sf_tmap(CUtensorMap* out, const void* base, long n_atoms) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t d[2] = {128, (cuuint64_t)n_atoms};
  cuuint64_t s[1] = {512};
  cuuint32_t b[2] = {128, 4};
  cuuint32_t e[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), d, s, b, e,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(1000 + (int)r);
}

}  // namespace mlb

using namespace mlb;

// Bytes of the scale-factor buffer of a quantised [rows, K] matrix (atoms of 128 rows x 128 K elements).
MLB_API long mlb_mx_sf_bytes(long rows, long K) { return ((rows + 127) / 128) * ((K + 127) / 128) * 512; }

// D[M,N] (=|+=) A[M,K] * B[N,K]^T, A / B one byte per element (format 0 = e4m3, 1 = e5m2) with row strides lda / ldb
// (multiples of 16), sfa / sfb in the atom layout described at the top of this file (mlb_mx_sf_bytes bytes each,
// 16-byte aligned).  out_mode: 0 = bf16/fp16 (out_lp_fmt 1/0), 1 = fp32, 2 = fp32 accumulate.  K a multiple of 32.
MLB_API int mlb_gemm_mx(int a_fmt, int b_fmt, const void* A, long lda, const void* sfa, const void* B, long ldb,
                        const void* sfb, void* D, long ldd, int out_mode, int out_lp_fmt, const void* bias, int M, int N,
                        int K, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 32) || (lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15))
    return -3;
  const int esz = (out_mode == OUT_LP) ? 2 : 4;
  if ((((size_t)ldd * esz) % 16) || (reinterpret_cast<uintptr_t>(D) & 15)) return -3;
  CUtensorMap tmA, tmB, tmSFA, tmSFB, tmD;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M}, strides[1] = {(uint64_t)lda};
    uint32_t box[2] = {128, 128};
    if ((rc = make_tmap(&tmA, A, 2, dims, strides, box, 1))) return rc;
    dims[1] = (uint64_t)N; strides[0] = (uint64_t)ldb; box[1] = 96;
    if ((rc = make_tmap(&tmB, B, 2, dims, strides, box, 1))) return rc;
    const long kb4 = (K + 127) / 128;
    if ((rc = make_sf_tmap(&tmSFA, sfa, ((M + 127) / 128) * kb4))) return rc;
    if ((rc = make_sf_tmap(&tmSFB, sfb, ((N + 127) / 128) * kb4))) return rc;
    uint64_t dd[2] = {(uint64_t)N, (uint64_t)M}, ds[1] = {(uint64_t)ldd * esz};
    uint32_t db[2] = {(uint32_t)(esz == 2 ? 64 : 32), 32};
    if ((rc = make_tmap(&tmD, D, 2, dd, ds, db, esz))) return rc;
  }
  MxParams p = {};
  p.M = M; p.N = N; p.K = K; p.out_mode = out_mode; p.lp_fmt = out_lp_fmt; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.bias = bias; p.status = status; p.raster_m = 16;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmMxSmem::kBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int tiles = ((M + 255) / 256) * ((N + kMxTN - 1) / kMxTN);
  int pairs = sm_count_cached() / 2;
  if (tiles < pairs) pairs = tiles;
  gemm_mx_kernel<<<2 * pairs, kGemm2Threads, GemmMxSmem::kBytes, st>>>(tmA, tmB, tmSFA, tmSFB, tmD, p);
  MLB_CHECK_LAUNCH();
  return 0;
}
