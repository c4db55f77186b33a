// Flash attention forward and backward for sm_100a (tcgen05 + TMEM + TMA), causal or full,
// MHA/GQA, head dim 64 or 128, operands addressed in place through 5-d tensor maps
// (head_dim, q-head-in-group, kv-group, batch, sequence) so q/k/v may be views of a fused
// QKV projection and the gradients are written into a fused buffer of the same layout.
//
// Three kernels share one structure - warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 one
// thread per accumulator row (TMEM lane):
//   fwd : per 128 query rows, loop over 64-key tiles.  S = Q K^T lands in TMEM, each thread
//         reads its row, computes exp2 with a lazily updated reference max, writes P (bf16,
//         128B-swizzled) to shared memory, and O += P V accumulates in TMEM; O is rescaled
//         in TMEM only when the row max grows by more than 2^8.
//   dq  : per 128 query rows, loop over 64-key tiles: S and dP = dO V^T in TMEM,
//         dS = P (dP - delta) scale to shared memory, dQ += dS K accumulates in TMEM.
//   dkv : per 128 key rows, loop over query heads of the group and 64-query tiles:
//         S^T = K Q^T and dP^T = V dO^T in TMEM, P^T and dS^T to shared memory,
//         dV += P^T dO and dK += dS^T Q accumulate in TMEM.
// The K/V (resp. Q/dO) tiles are stored once in shared memory and read both as K-major and
// as MN-major operands, which is what removes every transpose.  No atomics: gradients are
// written once, so results are bitwise reproducible.
//
// Replaces the library attention the reference reaches through
// megatron/core/extensions/transformer_engine.py:705-930 and the unfused path of
// megatron/core/transformer/dot_product_attention.py:136-205.
#include "tc05.cuh"

namespace mlb {
using namespace tc05;

constexpr int kAttnThreads = 192;
// backward kernels: warp 0 TMA, warp 1 MMA, warps 2-9 compute - two warps per TMEM lane quadrant, each taking
// one half (32) of the 64 columns of a step, so eight warps instead of four hide the exp2 / TMEM-load latency
constexpr int kAttnBwdThreads = 320;
constexpr int kAttnDqThreads = 576;      // dQ kernel with 128-key steps: warp 0 TMA, warp 1 MMA, 16 compute warps
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct AttnParams {
  int sq, sk, b, ng, qpg, causal, off;     // off = sk - sq (last query sees last key)
  int win;                                 // causal sliding window: query q sees keys [q + off - win, q + off]; 2^30 = none
  float scale, scale_log2;
  int lp_fmt;
  int* status;
  // forward
  void* o; long o_s, o_b, o_g, o_j;
  float* lse;                               // [b, ng, qpg, sq] natural log
  // backward
  const void* q; long q_s, q_b, q_g, q_j;    // raw operands for kernels that read rows themselves
  const void* d_o; long do_s, do_b, do_g, do_j;
  const float* delta;                       // [b, ng, qpg, sq]
  void* dq; long dq_s, dq_b, dq_g, dq_j;
  void* dk; long dk_s, dk_b, dk_g;
  void* dv; long dv_s, dv_b, dv_g;
};

__device__ __forceinline__ uint32_t pack_lp(float a, float b, int bf) {
  if (bf) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// write 64 values of one row (as 32 packed words) into a [rows x 64] K-major 128B-swizzled tile
__device__ __forceinline__ void store_row_sw128(uint8_t* tile, int row, const uint32_t (&w)[32]) {
  uint8_t* base = tile + row * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 v = make_uint4(w[c * 4], w[c * 4 + 1], w[c * 4 + 2], w[c * 4 + 3]);
    *reinterpret_cast<uint4*>(base + ((c ^ (row & 7)) << 4)) = v;
  }
}
// 32 fp32 accumulator values -> low precision -> 64 contiguous bytes in global memory
__device__ __forceinline__ void store_chunk_global(void* dst, const float (&v)[32], int bf) {
  uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int q = 0; q < 4; ++q)
    d[q] = make_uint4(pack_lp(v[q * 8], v[q * 8 + 1], bf), pack_lp(v[q * 8 + 2], v[q * 8 + 3], bf),
                      pack_lp(v[q * 8 + 4], v[q * 8 + 5], bf), pack_lp(v[q * 8 + 6], v[q * 8 + 7], bf));
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (M = 128 rows = lanes, two 16-bit K elements per 32-bit column) comes
// from tensor memory, where the compute warps have just written it - it never goes through shared memory
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp writes row (lane base + t)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void bar_sync_compute() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// half a row (32 values as 16 packed words, columns [32 half, 32 half + 32)) of a [rows x 64] K-major swizzled tile
__device__ __forceinline__ void store_half_row_sw128(uint8_t* tile, int row, int half, const uint32_t (&w)[16]) {
  uint8_t* base = tile + row * 128;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 v = make_uint4(w[c * 4], w[c * 4 + 1], w[c * 4 + 2], w[c * 4 + 3]);
    *reinterpret_cast<uint4*>(base + (((half * 4 + c) ^ (row & 7)) << 4)) = v;
  }
}

// K-major operand inside a [rows x D] tile stored as D/64 column chunks of [rows x 128 B]
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t tile, int kk, int chunk_bytes) {
  return make_desc(tile + (kk >> 2) * chunk_bytes + (kk & 3) * 32, 16, 1024);
}
// MN-major operand: same storage, reduction along rows; 16 rows per step, 64-element chunks LBO apart
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t tile, int kk, int chunk_bytes) {
  return make_desc(tile + kk * 2048, chunk_bytes, 1024);
}

// ============================================================================ forward
template <int D>
__global__ void __launch_bounds__(kAttnThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  constexpr int BM = 128, BN = 64;
  constexpr int QB = D * 256, KVB = D * 128, QC = 16384, KC = 8192;    // tile / chunk bytes
  constexpr uint32_t TCOLS = (64 + D) > 128 ? 256 : 128;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + QB;
  uint8_t* sV = sK + 2 * KVB;
  uint8_t* sP = sV + 2 * KVB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 16384);
  // 0 q_full | 1,2 k_full | 3,4 k_empty | 5 s_full | 6 s_empty | 7 p_full | 8 o_done | 9,10 v_full | 11,12 v_empty
  // K and V tiles have rings of their own: a K tile is free as soon as S = Q K^T of its step has run (early in
  // the step), so the K tile two steps ahead is requested a whole step before it is needed; with one ring for
  // both, the request waited for P V at the end of the step and every step stalled on the copy's latency.
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto B = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int n_qtiles = (p.sq + BM - 1) / BM;
  const int heads = p.ng * p.qpg;
  const int qt = n_qtiles - 1 - (int)(blockIdx.x / (heads * p.b));      // heavy (late) tiles first
  const int hb = blockIdx.x % (heads * p.b);
  const int bb = hb / heads, hh = hb % heads, g = hh / p.qpg, j = hh % p.qpg;
  const int s0 = qt * BM;
  int kv_end = p.sk;
  if (p.causal) { kv_end = s0 + BM + p.off; if (kv_end > p.sk) kv_end = p.sk; }
  const int n_kv = kv_end > 0 ? (kv_end + BN - 1) / BN : 0;

  if (threadIdx.x == 0) {
    mbar_init(B(0), 1);
    mbar_init(B(1), 1); mbar_init(B(2), 1); mbar_init(B(3), 1); mbar_init(B(4), 1);
    mbar_init(B(5), 1); mbar_init(B(6), 4); mbar_init(B(7), 4); mbar_init(B(8), 1);
    mbar_init(B(9), 1); mbar_init(B(10), 1); mbar_init(B(11), 1); mbar_init(B(12), 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TCOLS); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 64;

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      mbar_expect_tx(B(0), QB);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) tma_load_5d(smem_u32(sQ) + c * QC, &tmQ, B(0), c * 64, j, g, bb, s0);
      for (int t = 0; t < n_kv; ++t) {
        const int st = t & 1;
        const uint32_t ph = (((uint32_t)t >> 1) & 1u) ^ 1u;
        if (!mbar_wait(B(3 + st), ph, abort_flag, p.status, 11)) break;
        mbar_expect_tx(B(1 + st), KVB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_5d(smem_u32(sK) + st * KVB + c * KC, &tmK, B(1 + st), c * 64, 0, g, bb, t * BN);
        if (!mbar_wait(B(11 + st), ph, abort_flag, p.status, 11)) break;
        mbar_expect_tx(B(9 + st), KVB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_5d(smem_u32(sV) + st * KVB + c * KC, &tmV, B(9 + st), c * 64, 0, g, bb, t * BN);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, p.lp_fmt, 0, 0);
      const uint32_t idesc_o = make_idesc(BM, D, p.lp_fmt, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP);
      auto issue_s = [&](int t) {
        const uint32_t kb = aK + (t & 1) * KVB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tS, kmajor_desc(aQ, kk, QC), kmajor_desc(kb, kk, KC), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(3 + (t & 1)));            // this K tile may be overwritten once S has been computed
        mma_commit(B(5));
      };
      bool ok = mbar_wait(B(0), 0, abort_flag, p.status, 12) && mbar_wait(B(1), 0, abort_flag, p.status, 13);
      if (ok) { fence_after_sync(); issue_s(0); }
      for (int t = 0; t < n_kv && ok; ++t) {
        if (t + 1 < n_kv) {
          const int st1 = (t + 1) & 1;
          if (!mbar_wait(B(1 + st1), ((uint32_t)(t + 1) >> 1) & 1u, abort_flag, p.status, 14)) { ok = false; break; }
          if (!mbar_wait(B(6), (uint32_t)t & 1u, abort_flag, p.status, 15)) { ok = false; break; }
          fence_after_sync();
          issue_s(t + 1);
        }
        if (!mbar_wait(B(9 + (t & 1)), ((uint32_t)t >> 1) & 1u, abort_flag, p.status, 16)) { ok = false; break; }
        if (!mbar_wait(B(7), (uint32_t)t & 1u, abort_flag, p.status, 16)) { ok = false; break; }
        fence_after_sync();
        const uint32_t vb = aV + (t & 1) * KVB;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16(tO, kmajor_desc(aP, kk, 0), mnmajor_desc(vb, kk, KC), idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
        mma_commit(B(11 + (t & 1)));
        mma_commit(B(8));
      }
    }
  } else if (n_kv > 0) {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int qrow = s0 + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int t = 0; t < n_kv; ++t) {
      const int n0 = t * BN;
      if (!mbar_wait(B(5), (uint32_t)t & 1u, abort_flag, p.status, 17)) { ok = false; break; }
      fence_after_sync();
      uint32_t r0[32], r1[32];
      tmem_ld32(tS + lane_base, r0);
      tmem_ld32(tS + lane_base + 32, r1);
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(6));
      const bool need_mask = (p.causal && (n0 + BN - 1 > s0 + p.off)) || (n0 + BN > p.sk);
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float a = __uint_as_float(r0[c]) * p.scale_log2, bq = __uint_as_float(r1[c]) * p.scale_log2;
        if (need_mask) {
          const int k0 = n0 + c, k1 = n0 + 32 + c;
          if ((p.causal && k0 > qrow + p.off) || k0 >= p.sk) a = -INFINITY;
          if ((p.causal && k1 > qrow + p.off) || k1 >= p.sk) bq = -INFINITY;
        }
        r0[c] = __float_as_uint(a); r1[c] = __float_as_uint(bq);
        mx = fmaxf(mx, fmaxf(a, bq));
      }
      const float m_new = fmaxf(m_ref, mx);
      const bool resc = m_new > m_ref + 8.f;
      float alpha = 1.f;
      if (resc) { alpha = fast_exp2(m_ref - m_new); m_ref = m_new; l *= alpha; }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      uint32_t pw[32];
      float lsum = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float a0 = fast_exp2(__uint_as_float(r0[2 * c]) - m_use), a1 = fast_exp2(__uint_as_float(r0[2 * c + 1]) - m_use);
        const float b0 = fast_exp2(__uint_as_float(r1[2 * c]) - m_use), b1 = fast_exp2(__uint_as_float(r1[2 * c + 1]) - m_use);
        lsum += (a0 + a1) + (b0 + b1);
        pw[c] = pack_lp(a0, a1, p.lp_fmt);
        pw[16 + c] = pack_lp(b0, b1, p.lp_fmt);
      }
      l += lsum;
      if (t > 0) {
        if (!mbar_wait(B(8), (uint32_t)(t - 1) & 1u, abort_flag, p.status, 18)) { ok = false; break; }
        fence_after_sync();
        if (__any_sync(0xffffffffu, resc)) {
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t o[32];
            tmem_ld32(tO + lane_base + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tO + lane_base + c, o);
          }
          tmem_wait_st();
        }
      }
      store_row_sw128(sP, row, pw);
      fence_async_smem();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(7));
    }
    if (ok && mbar_wait(B(8), (uint32_t)(n_kv - 1) & 1u, abort_flag, p.status, 19)) {
      fence_after_sync();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) +
                      2 * ((long)qrow * p.o_s + (long)bb * p.o_b + (long)g * p.o_g + (long)j * p.o_j);
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld32(tO + lane_base + c, o);
        tmem_wait_ld();
        if (qrow < p.sq) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i]) * inv_l;
          store_chunk_global(orow + c * 2, v, p.lp_fmt);
        }
      }
      if (qrow < p.sq)
        p.lse[(((long)bb * p.ng + g) * p.qpg + j) * p.sq + qrow] = l > 0.f ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// ============================================================================ forward, two query tiles per CTA
// One CTA per SM works on 256 query rows as two 128-row tiles that take turns on the tensor core: while the eight
// softmax warps of one tile compute exp2, the products of the other tile run.  Per 128-key step and tile:
//   S = Q K^T (128 x 128, fp32) into tensor memory; one thread per row reads it, writes P (16-bit) over the first
//   64 columns of S, and O += P V takes P as the A operand straight from tensor memory.
// Compared with attn_fwd_kernel (two independent 128-row CTAs per SM, 64-key steps, P through shared memory) a
// K / V tile is copied into shared memory once for 256 rows instead of once per 128, the S product reads 8 KB of
// operands per instruction of 128 x 128 x 16 instead of 6 KB per 128 x 64 x 16, and P is neither stored to nor
// read from shared memory - shared-memory bandwidth, not the tensor core, was what bounded that kernel.
// Tensor memory columns: S0 | S1 (128 each) | O0 | O1 (D each).  The products of one thread run in issue order,
// which is what allows S of step t + 1 to overwrite P of step t right behind the P V product that reads it.
constexpr int kAttnFwd2Threads = 320;
template <int D>
__global__ void __launch_bounds__(kAttnFwd2Threads, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  constexpr int BM = 128, BN = 128;
  constexpr int QB = D * 256, KVB = D * 256, CH = 16384;               // tile bytes; bytes of a 64-column chunk
  constexpr int NSLOT = 5;                                              // ring of K0 V0 K1 V1 K2 ...
  constexpr uint32_t TCOLS = 512;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + 2 * QB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + NSLOT * KVB);
  constexpr int QF = 0, KF = 2, KE = KF + NSLOT, SF = KE + NSLOT, PF = SF + 2, OD = PF + 2, NBAR = OD + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto B = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int n_qtiles = (p.sq + 2 * BM - 1) / (2 * BM);
  const int heads = p.ng * p.qpg;
  const int qt = n_qtiles - 1 - (int)(blockIdx.x / (heads * p.b));      // heavy (late) tiles first
  const int hb = blockIdx.x % (heads * p.b);
  const int bb = hb / heads, hh = hb % heads, g = hh / p.qpg, j = hh % p.qpg;
  const int s0 = qt * 2 * BM;
  auto steps_of = [&](int i) {
    const int s0i = s0 + i * BM;
    int kv_end = p.sk;
    if (p.causal) { kv_end = s0i + BM + p.off; if (kv_end > p.sk) kv_end = p.sk; }
    return (s0i < p.sq && kv_end > 0) ? (kv_end + BN - 1) / BN : 0;
  };
  const int n_t0 = steps_of(0), n_t1 = steps_of(1);
  auto n_of = [&](int i) { return i ? n_t1 : n_t0; };
  const int n_kv = n_t0 > n_t1 ? n_t0 : n_t1;

  if (threadIdx.x == 0) {
    mbar_init(B(QF), 1); mbar_init(B(QF + 1), 1);
    for (int i = 0; i < 2 * NSLOT; ++i) mbar_init(B(KF + i), 1);
    for (int i = 0; i < 2; ++i) { mbar_init(B(SF + i), 1); mbar_init(B(PF + i), 4); mbar_init(B(OD + i), 1); }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TCOLS); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  auto tS = [&](int i) { return tmem + (uint32_t)(128 * i); };
  auto tO = [&](int i) { return tmem + 256u + (uint32_t)(D * i); };

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (n_of(i) > 0) {
          mbar_expect_tx(B(QF + i), QB);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_5d(smem_u32(sQ) + i * QB + c * CH, &tmQ, B(QF + i), c * 64, j, g, bb, s0 + i * BM);
        }
      for (int u = 0; u < 2 * n_kv; ++u) {                              // u = 2 t: K of step t; 2 t + 1: V
        const int slot = u % NSLOT;
        if (!mbar_wait(B(KE + slot), (((uint32_t)(u / NSLOT)) & 1u) ^ 1u, abort_flag, p.status, 11)) break;
        mbar_expect_tx(B(KF + slot), KVB);
        const CUtensorMap* tm = (u & 1) ? &tmV : &tmK;
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_5d(smem_u32(sKV) + slot * KVB + c * CH, tm, B(KF + slot), c * 64, 0, g, bb, (u >> 1) * BN);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, p.lp_fmt, 0, 0);
      const uint32_t idesc_o = make_idesc(BM, D, p.lp_fmt, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aKV = smem_u32(sKV);
      auto kv_ready = [&](int u) {
        return mbar_wait(B(KF + u % NSLOT), ((uint32_t)(u / NSLOT)) & 1u, abort_flag, p.status, 13);
      };
      auto issue_s = [&](int i, int t) {
        const uint32_t kb = aKV + ((2 * t) % NSLOT) * KVB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tS(i), kmajor_desc(aQ + i * QB, kk, CH), kmajor_desc(kb, kk, CH), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(SF + i));
      };
      auto issue_pv = [&](int i, int t) {
        const uint32_t vb = aKV + ((2 * t + 1) % NSLOT) * KVB;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16_ts(tO(i), tS(i) + (uint32_t)(kk * 8), mnmajor_desc(vb, kk, CH), idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
        mma_commit(B(OD + i));
      };
      bool ok = true;
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (ok && n_of(i) > 0) ok = mbar_wait(B(QF + i), 0, abort_flag, p.status, 12);
      if (ok) ok = kv_ready(0);
      if (ok) {
        fence_after_sync();
        if (n_t0 > 0) issue_s(0, 0);
        if (n_t1 > 0) issue_s(1, 0);
        mma_commit(B(KE + 0));
      }
      for (int t = 0; t < n_kv && ok; ++t) {
        bool k_next_ready = false;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (t < n_of(i)) {
            if (i == 0 || !(t < n_t0)) { if (!kv_ready(2 * t + 1)) { ok = false; break; } }
            if (!mbar_wait(B(PF + i), (uint32_t)t & 1u, abort_flag, p.status, 16)) { ok = false; break; }
            fence_after_sync();
            issue_pv(i, t);
          }
          if (t + 1 < n_of(i)) {
            if (!k_next_ready) { if (!kv_ready(2 * t + 2)) { ok = false; break; } k_next_ready = true; fence_after_sync(); }
            issue_s(i, t + 1);
          }
        }
        if (!ok) break;
        mma_commit(B(KE + (2 * t + 1) % NSLOT));                      // V of this step
        if (t + 1 < n_kv) mma_commit(B(KE + (2 * t + 2) % NSLOT));    // K of the next
      }
    }
  } else {
    const int i = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int s0i = s0 + i * BM;
    const int qrow = s0i + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const int n_mine = n_of(i);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int t = 0; t < n_mine; ++t) {
      const int n0 = t * BN;
      if (!mbar_wait(B(SF + i), (uint32_t)t & 1u, abort_flag, p.status, 17)) { ok = false; break; }
      fence_after_sync();
      uint32_t r[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tS(i) + lane_base + c * 32, r[c]);
      tmem_wait_ld();
      const bool need_mask = (p.causal && (n0 + BN - 1 > s0i + p.off)) || (n0 + BN > p.sk);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int kv = n0 + c * 32 + e;
            if ((p.causal && kv > qrow + p.off) || kv >= p.sk) r[c][e] = 0xff800000u;       // -inf
          }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        mx0 = fmaxf(mx0, __uint_as_float(r[0][e])); mx1 = fmaxf(mx1, __uint_as_float(r[1][e]));
        mx2 = fmaxf(mx2, __uint_as_float(r[2][e])); mx3 = fmaxf(mx3, __uint_as_float(r[3][e]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      const float m_new = fmaxf(m_ref, mx);
      const bool resc = m_new > m_ref + 8.f;
      float alpha = 1.f;
      if (resc) { alpha = fast_exp2(m_ref - m_new); m_ref = m_new; l *= alpha; }
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
      float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float a0 = fast_exp2(fmaf(__uint_as_float(r[c][2 * e]), p.scale_log2, neg_m));
          const float a1 = fast_exp2(fmaf(__uint_as_float(r[c][2 * e + 1]), p.scale_log2, neg_m));
          ls0 += a0; ls1 += a1;
          w[e] = pack_lp(a0, a1, p.lp_fmt);
        }
        tmem_st16(tS(i) + lane_base + c * 16, w);                       // keys [32 c, 32 c + 32) -> 16 packed columns
      }
      l += ls0 + ls1;
      if (t > 0 && __any_sync(0xffffffffu, resc)) {
        // O of this tile has to be rescaled: its last product (step t - 1) must have completed
        if (!mbar_wait(B(OD + i), (uint32_t)(t - 1) & 1u, abort_flag, p.status, 18)) { ok = false; break; }
        fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld32(tO(i) + lane_base + c, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(tO(i) + lane_base + c, o);
        }
      }
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(PF + i));
    }
    if (ok && n_mine > 0 && mbar_wait(B(OD + i), (uint32_t)(n_mine - 1) & 1u, abort_flag, p.status, 19)) {
      fence_after_sync();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) +
                      2 * ((long)qrow * p.o_s + (long)bb * p.o_b + (long)g * p.o_g + (long)j * p.o_j);
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld32(tO(i) + lane_base + c, o);
        tmem_wait_ld();
        if (qrow < p.sq) {
          float v[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(o[e]) * inv_l;
          store_chunk_global(orow + c * 2, v, p.lp_fmt);
        }
      }
      if (qrow < p.sq)
        p.lse[(((long)bb * p.ng + g) * p.qpg + j) * p.sq + qrow] = l > 0.f ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// The same kernel with a causal sliding window (query q sees keys [q + off - win, q + off]): a tile starts at the step
// that holds the lowest key its first row sees, rings and barrier phases count from there, and tiles that the window
// cuts get per-element masks.  Kept as a kernel of its own: the forward kernel sits at its register limit, and the
// extra live values of the window logic cost calls without a window a fifth of their speed.
template <int D>
__global__ void __launch_bounds__(kAttnFwd2Threads, 1)
attn_fwd2_win_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  constexpr int BM = 128, BN = 128;
  constexpr int QB = D * 256, KVB = D * 256, CH = 16384;               // tile bytes; bytes of a 64-column chunk
  constexpr int NSLOT = 5;                                              // ring of K0 V0 K1 V1 K2 ...
  constexpr uint32_t TCOLS = 512;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + 2 * QB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + NSLOT * KVB);
  constexpr int QF = 0, KF = 2, KE = KF + NSLOT, SF = KE + NSLOT, PF = SF + 2, OD = PF + 2, NBAR = OD + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto B = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int n_qtiles = (p.sq + 2 * BM - 1) / (2 * BM);
  const int heads = p.ng * p.qpg;
  const int qt = n_qtiles - 1 - (int)(blockIdx.x / (heads * p.b));      // heavy (late) tiles first
  const int hb = blockIdx.x % (heads * p.b);
  const int bb = hb / heads, hh = hb % heads, g = hh / p.qpg, j = hh % p.qpg;
  const int s0 = qt * 2 * BM;
  auto steps_of = [&](int i) {
    const int s0i = s0 + i * BM;
    int kv_end = p.sk;
    if (p.causal) { kv_end = s0i + BM + p.off; if (kv_end > p.sk) kv_end = p.sk; }
    return (s0i < p.sq && kv_end > 0) ? (kv_end + BN - 1) / BN : 0;
  };
  // first step of a tile: the step that holds the lowest key its first row sees (sliding window)
  auto first_of = [&](int i) {
    int lo = p.causal ? s0 + i * BM + p.off - p.win : 0;
    return lo > 0 ? lo / BN : 0;
  };
  const int n_t0 = steps_of(0), n_t1 = steps_of(1);
  const int b_t0 = first_of(0), b_t1 = first_of(1);
  auto n_of = [&](int i) { return i ? n_t1 : n_t0; };
  auto b_of = [&](int i) { return i ? b_t1 : b_t0; };
  const int n_kv = n_t0 > n_t1 ? n_t0 : n_t1;
  const int t_lo = n_t0 > 0 ? b_t0 : b_t1;             // steps [t_lo, n_kv) are loaded; tile i works on [b_of(i), n_of(i))

  if (threadIdx.x == 0) {
    mbar_init(B(QF), 1); mbar_init(B(QF + 1), 1);
    for (int i = 0; i < 2 * NSLOT; ++i) mbar_init(B(KF + i), 1);
    for (int i = 0; i < 2; ++i) { mbar_init(B(SF + i), 1); mbar_init(B(PF + i), 4); mbar_init(B(OD + i), 1); }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TCOLS); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  auto tS = [&](int i) { return tmem + (uint32_t)(128 * i); };
  auto tO = [&](int i) { return tmem + 256u + (uint32_t)(D * i); };

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (n_of(i) > 0) {
          mbar_expect_tx(B(QF + i), QB);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_5d(smem_u32(sQ) + i * QB + c * CH, &tmQ, B(QF + i), c * 64, j, g, bb, s0 + i * BM);
        }
      for (int u = 0; u < 2 * (n_kv - t_lo); ++u) {                     // u = 2 (t - t_lo): K of step t; + 1: V
        const int slot = u % NSLOT;
        if (!mbar_wait(B(KE + slot), (((uint32_t)(u / NSLOT)) & 1u) ^ 1u, abort_flag, p.status, 11)) break;
        mbar_expect_tx(B(KF + slot), KVB);
        const CUtensorMap* tm = (u & 1) ? &tmV : &tmK;
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_5d(smem_u32(sKV) + slot * KVB + c * CH, tm, B(KF + slot), c * 64, 0, g, bb, (t_lo + (u >> 1)) * BN);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, p.lp_fmt, 0, 0);
      const uint32_t idesc_o = make_idesc(BM, D, p.lp_fmt, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aKV = smem_u32(sKV);
      auto kv_ready = [&](int u) {
        return mbar_wait(B(KF + u % NSLOT), ((uint32_t)(u / NSLOT)) & 1u, abort_flag, p.status, 13);
      };
      auto issue_s = [&](int i, int t) {
        const uint32_t kb = aKV + ((2 * (t - t_lo)) % NSLOT) * KVB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tS(i), kmajor_desc(aQ + i * QB, kk, CH), kmajor_desc(kb, kk, CH), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(SF + i));
      };
      auto issue_pv = [&](int i, int t) {
        const uint32_t vb = aKV + ((2 * (t - t_lo) + 1) % NSLOT) * KVB;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16_ts(tO(i), tS(i) + (uint32_t)(kk * 8), mnmajor_desc(vb, kk, CH), idesc_o,
                     (t > b_of(i) || kk > 0) ? 1u : 0u);
        mma_commit(B(OD + i));
      };
      bool ok = true;
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (ok && n_of(i) > 0) ok = mbar_wait(B(QF + i), 0, abort_flag, p.status, 12);
      if (ok) ok = kv_ready(0);
      if (ok) {
        fence_after_sync();
        if (n_t0 > 0 && b_t0 == t_lo) issue_s(0, t_lo);
        if (n_t1 > 0 && b_t1 == t_lo) issue_s(1, t_lo);
        mma_commit(B(KE + 0));
      }
      for (int t = t_lo; t < n_kv && ok; ++t) {
        const int u = 2 * (t - t_lo);
        bool v_ready = false, k_next_ready = false;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (t >= b_of(i) && t < n_of(i)) {
            if (!v_ready) { if (!kv_ready(u + 1)) { ok = false; break; } v_ready = true; }
            if (!mbar_wait(B(PF + i), (uint32_t)(t - b_of(i)) & 1u, abort_flag, p.status, 16)) { ok = false; break; }
            fence_after_sync();
            issue_pv(i, t);
          }
          if (t + 1 >= b_of(i) && t + 1 < n_of(i)) {
            if (!k_next_ready) { if (!kv_ready(u + 2)) { ok = false; break; } k_next_ready = true; fence_after_sync(); }
            issue_s(i, t + 1);
          }
        }
        if (!ok) break;
        if (!v_ready) ok = kv_ready(u + 1);                            // a V tile nobody used is still consumed in order
        if (ok && t + 1 < n_kv && !k_next_ready) ok = kv_ready(u + 2);
        if (!ok) break;
        mma_commit(B(KE + (u + 1) % NSLOT));                          // V of this step
        if (t + 1 < n_kv) mma_commit(B(KE + (u + 2) % NSLOT));        // K of the next
      }
    }
  } else {
    const int i = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int s0i = s0 + i * BM;
    const int qrow = s0i + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const int n_mine = n_of(i), b_mine = b_of(i);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int t = b_mine; t < n_mine; ++t) {
      const int n0 = t * BN;
      const uint32_t par = (uint32_t)(t - b_mine) & 1u;
      if (!mbar_wait(B(SF + i), par, abort_flag, p.status, 17)) { ok = false; break; }
      fence_after_sync();
      uint32_t r[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tS(i) + lane_base + c * 32, r[c]);
      tmem_wait_ld();
      const bool need_mask = (p.causal && (n0 + BN - 1 > s0i + p.off || (n0 + p.win < s0i + BM - 1 + p.off))) ||
                             (n0 + BN > p.sk);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int kv = n0 + c * 32 + e;
            if ((p.causal && (kv > qrow + p.off || (kv + p.win < qrow + p.off))) || kv >= p.sk)
              r[c][e] = 0xff800000u;                                                        // -inf
          }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        mx0 = fmaxf(mx0, __uint_as_float(r[0][e])); mx1 = fmaxf(mx1, __uint_as_float(r[1][e]));
        mx2 = fmaxf(mx2, __uint_as_float(r[2][e])); mx3 = fmaxf(mx3, __uint_as_float(r[3][e]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      const float m_new = fmaxf(m_ref, mx);
      const bool resc = m_new > m_ref + 8.f;
      float alpha = 1.f;
      if (resc) { alpha = fast_exp2(m_ref - m_new); m_ref = m_new; l *= alpha; }
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
      float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float a0 = fast_exp2(fmaf(__uint_as_float(r[c][2 * e]), p.scale_log2, neg_m));
          const float a1 = fast_exp2(fmaf(__uint_as_float(r[c][2 * e + 1]), p.scale_log2, neg_m));
          ls0 += a0; ls1 += a1;
          w[e] = pack_lp(a0, a1, p.lp_fmt);
        }
        tmem_st16(tS(i) + lane_base + c * 16, w);                       // keys [32 c, 32 c + 32) -> 16 packed columns
      }
      l += ls0 + ls1;
      if (t > b_mine && __any_sync(0xffffffffu, resc)) {
        // O of this tile has to be rescaled: its last product (step t - 1) must have completed
        if (!mbar_wait(B(OD + i), par ^ 1u, abort_flag, p.status, 18)) { ok = false; break; }
        fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld32(tO(i) + lane_base + c, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(tO(i) + lane_base + c, o);
        }
      }
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(PF + i));
    }
    if (ok && n_mine > 0 && mbar_wait(B(OD + i), (uint32_t)(n_mine - 1 - b_mine) & 1u, abort_flag, p.status, 19)) {
      fence_after_sync();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) +
                      2 * ((long)qrow * p.o_s + (long)bb * p.o_b + (long)g * p.o_g + (long)j * p.o_j);
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld32(tO(i) + lane_base + c, o);
        tmem_wait_ld();
        if (qrow < p.sq) {
          float v[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(o[e]) * inv_l;
          store_chunk_global(orow + c * 2, v, p.lp_fmt);
        }
      }
      if (qrow < p.sq)
        p.lse[(((long)bb * p.ng + g) * p.qpg + j) * p.sq + qrow] = l > 0.f ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// ============================================================================ delta = rowsum(O * dO)
__global__ void attn_delta_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ d_o, float* __restrict__ delta,
                                  int sq, int b, int ng, int qpg, int D, long o_s, long o_b, long o_g, long o_j,
                                  long do_s, long do_b, long do_g, long do_j, int bf) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long total = (long)sq * b * ng * qpg;
  if (row >= total) return;
  const int lane = threadIdx.x & 31;
  long r = row;
  const int s = (int)(r % sq); r /= sq;
  const int j = (int)(r % qpg); r /= qpg;
  const int g = (int)(r % ng);
  const int bb = (int)(r / ng);
  const uint16_t* op = o + s * o_s + bb * o_b + g * o_g + j * o_j;
  const uint16_t* dp = d_o + s * do_s + bb * do_b + g * do_g + j * do_j;
  float acc = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    const uint32_t a = *reinterpret_cast<const uint32_t*>(op + c), bq = *reinterpret_cast<const uint32_t*>(dp + c);
    if (bf) {
      const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a));
      const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bq));
      acc += x.x * y.x + x.y * y.y;
    } else {
      const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&a));
      const float2 y = __half22float2(*reinterpret_cast<const __half2*>(&bq));
      acc += x.x * y.x + x.y * y.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[row] = acc;      // index order (b, g, j, s) matches the decomposition above
}

// ============================================================================ backward: dQ
template <int D>
__global__ void __launch_bounds__(kAttnBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const AttnParams p) {
  constexpr int BM = 128, BN = 64;
  constexpr int QB = D * 256, KVB = D * 128, QC = 16384, KC = 8192;
  constexpr uint32_t TCOLS = (128 + D) > 128 ? 256 : 128;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + QB;
  // Four K/V stages: a K tile is held until dQ += dS K at the end of its step, so with two stages the tile two
  // steps ahead was requested only when it was already needed and every step waited for the copy.
  constexpr int NST = 4;
  uint8_t* sK = sdO + QB;
  uint8_t* sV = sK + NST * KVB;
  uint8_t* sdS = sV + NST * KVB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 16384);
  // 0 q_full | 1..4 kv_full | 5..8 kv_empty | 9 sdp_full | 10 sdp_empty | 11 ds_full | 12 dq_done
  constexpr int KF = 1, KE = 1 + NST, SF = 1 + 2 * NST, SE = SF + 1, DF = SF + 2, DD = SF + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + DD + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto B = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int n_qtiles = (p.sq + BM - 1) / BM;
  const int heads = p.ng * p.qpg;
  const int qt = n_qtiles - 1 - (int)(blockIdx.x / (heads * p.b));
  const int hb = blockIdx.x % (heads * p.b);
  const int bb = hb / heads, hh = hb % heads, g = hh / p.qpg, j = hh % p.qpg;
  const int s0 = qt * BM;
  int kv_end = p.sk;
  if (p.causal) { kv_end = s0 + BM + p.off; if (kv_end > p.sk) kv_end = p.sk; }
  const int n_kv = kv_end > 0 ? (kv_end + BN - 1) / BN : 0;

  if (threadIdx.x == 0) {
    mbar_init(B(0), 1);
    for (int i = 0; i < 2 * NST; ++i) mbar_init(B(1 + i), 1);
    mbar_init(B(SF), 1); mbar_init(B(SE), 8); mbar_init(B(DF), 8); mbar_init(B(DD), 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmdO);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TCOLS); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 64, tdQ = tmem + 128;

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      mbar_expect_tx(B(0), 2 * QB);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_5d(smem_u32(sQ) + c * QC, &tmQ, B(0), c * 64, j, g, bb, s0);
        tma_load_5d(smem_u32(sdO) + c * QC, &tmdO, B(0), c * 64, j, g, bb, s0);
      }
      for (int t = 0; t < n_kv; ++t) {
        const int st = t % NST;
        if (!mbar_wait(B(KE + st), (((uint32_t)(t / NST)) & 1u) ^ 1u, abort_flag, p.status, 21)) break;
        mbar_expect_tx(B(KF + st), 2 * KVB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_5d(smem_u32(sK) + st * KVB + c * KC, &tmK, B(KF + st), c * 64, 0, g, bb, t * BN);
          tma_load_5d(smem_u32(sV) + st * KVB + c * KC, &tmV, B(KF + st), c * 64, 0, g, bb, t * BN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, p.lp_fmt, 0, 0);       // S, dP: both operands K-major
      const uint32_t idesc_q = make_idesc(BM, D, p.lp_fmt, 0, 1);        // dQ = dS (K-major) x K (MN-major)
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), aK = smem_u32(sK), aV = smem_u32(sV), adS = smem_u32(sdS);
      auto issue_sdp = [&](int t) {
        const uint32_t kb = aK + (t % NST) * KVB, vb = aV + (t % NST) * KVB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tS, kmajor_desc(aQ, kk, QC), kmajor_desc(kb, kk, KC), idesc_s, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tdP, kmajor_desc(adO, kk, QC), kmajor_desc(vb, kk, KC), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(SF));
      };
      bool ok = mbar_wait(B(0), 0, abort_flag, p.status, 22) && mbar_wait(B(KF), 0, abort_flag, p.status, 23);
      if (ok) { fence_after_sync(); issue_sdp(0); }
      for (int t = 0; t < n_kv && ok; ++t) {
        if (t + 1 < n_kv) {
          const int st1 = (t + 1) % NST;
          if (!mbar_wait(B(KF + st1), ((uint32_t)((t + 1) / NST)) & 1u, abort_flag, p.status, 24)) { ok = false; break; }
          if (!mbar_wait(B(SE), (uint32_t)t & 1u, abort_flag, p.status, 25)) { ok = false; break; }
          fence_after_sync();
          issue_sdp(t + 1);
        }
        if (!mbar_wait(B(DF), (uint32_t)t & 1u, abort_flag, p.status, 26)) { ok = false; break; }
        fence_after_sync();
        const uint32_t kb = aK + (t % NST) * KVB;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16(tdQ, kmajor_desc(adS, kk, 0), mnmajor_desc(kb, kk, KC), idesc_q, (t > 0 || kk > 0) ? 1u : 0u);
        mma_commit(B(KE + (t % NST)));
        mma_commit(B(DD));
      }
    }
  } else if (n_kv > 0) {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;                 // which 32 of a step's 64 key columns this warp takes
    const int row = quad * 32 + lane;
    const int qrow = s0 + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const long stat_idx = (((long)bb * p.ng + g) * p.qpg + j) * p.sq + qrow;
    const float lse2 = qrow < p.sq ? p.lse[stat_idx] * kLog2e : 0.f;
    const float dlt = qrow < p.sq ? p.delta[stat_idx] : 0.f;
    bool ok = true;
    for (int t = 0; t < n_kv; ++t) {
      const int n0 = t * BN;
      if (!mbar_wait(B(SF), (uint32_t)t & 1u, abort_flag, p.status, 27)) { ok = false; break; }
      fence_after_sync();
      uint32_t w[16];
      uint32_t rs[32], rp[32];
      tmem_ld32(tS + lane_base + half * 32, rs);
      tmem_ld32(tdP + lane_base + half * 32, rp);
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(SE));              // S / dP are in registers: the next step's products may start
      // only tiles that touch the diagonal, the end of the keys or the end of the queries need per-element masks
      const bool need_mask = (p.causal && (n0 + BN - 1 > s0 + p.off)) || (n0 + BN > p.sk) || (s0 + BM > p.sq);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          float ds[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int kv = n0 + half * 32 + 2 * c + e;
            const bool masked = (p.causal && kv > qrow + p.off) || kv >= p.sk || qrow >= p.sq;
            const float pr = masked ? 0.f : fast_exp2(fmaf(__uint_as_float(rs[2 * c + e]), p.scale_log2, -lse2));
            ds[e] = pr * (__uint_as_float(rp[2 * c + e]) - dlt) * p.scale;
          }
          w[c] = pack_lp(ds[0], ds[1], p.lp_fmt);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(rs[2 * c]), p.scale_log2, -lse2));
          const float p1 = fast_exp2(fmaf(__uint_as_float(rs[2 * c + 1]), p.scale_log2, -lse2));
          w[c] = pack_lp(p0 * (__uint_as_float(rp[2 * c]) - dlt) * p.scale,
                         p1 * (__uint_as_float(rp[2 * c + 1]) - dlt) * p.scale, p.lp_fmt);
        }
      }
      if (t > 0) {
        if (!mbar_wait(B(DD), (uint32_t)(t - 1) & 1u, abort_flag, p.status, 28)) { ok = false; break; }
      }
      store_half_row_sw128(sdS, row, half, w);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(DF));
    }
    if (ok && mbar_wait(B(DD), (uint32_t)(n_kv - 1) & 1u, abort_flag, p.status, 29)) {
      fence_after_sync();
      uint8_t* drow = reinterpret_cast<uint8_t*>(p.dq) +
                      2 * ((long)qrow * p.dq_s + (long)bb * p.dq_b + (long)g * p.dq_g + (long)j * p.dq_j);
#pragma unroll 1
      for (int c = half * (D / 2); c < (half + 1) * (D / 2); c += 32) {
        uint32_t o[32];
        tmem_ld32(tdQ + lane_base + c, o);
        tmem_wait_ld();
        if (qrow < p.sq) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i]);
          store_chunk_global(drow + c * 2, v, p.lp_fmt);
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// ============================================================================ backward: dQ, 128-key steps
// Same product as attn_bwd_dq_kernel, rebuilt around what the tensor core's instruction rate allows: one thread
// gets a `tcgen05.mma` accepted about every 46 cycles whatever its size (measured: 16 instructions of 128 x 64 x 16
// take 740 cycles to issue, 830 to complete - 32 cycles of arithmetic each; of 128 x 128 x 16, 72 cycles each from a
// tensor-memory A operand, 82 from shared memory), so products of 64 columns run the tensor core at two thirds of
// its rate at best and every product here is 128 wide:
//   S = Q K^T and dP = dO V^T (128 x 128 per step) into tensor memory, each behind a barrier of its own so that the
//   exponentials start while dP is still running; dS (16-bit) into tensor-memory columns of its own, from where it is
//   the A operand of dQ += dS K.
// S and dP are single buffers: the compute warps take a step's values into registers and release them at once, so
// S / dP of step t + 1 are issued - ahead of dQ of step t - as soon as step t has been read, and run under its
// arithmetic.  Sixteen compute warps (four per lane quadrant, 32 key columns each): a warp's step is a chain of
// waits, tensor-memory loads, arithmetic and a tensor-memory store that does not overlap with itself.
// Tensor memory columns: S | dP (128 each) | dQ (D) | dS (64).  Shared memory: Q, dO, three K stages (a K tile is
// held until dQ of its step), two V stages.
template <int D>
__global__ void __launch_bounds__(kAttnDqThreads, 1)
attn_bwd_dq_ts_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                      const AttnParams p) {
  constexpr int BM = 128, BN = 128;
  constexpr int TB = D * 256, CH = 16384;              // bytes of a 128-row tile / of one of its 64-column chunks
  constexpr uint32_t TCOLS = 512;
  constexpr int NK = 3, NV = 2;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + TB;
  uint8_t* sK = sdO + TB;
  uint8_t* sV = sK + NK * TB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NV * TB);
  // q_full | k_full[3] | k_empty[3] | v_full[2] | v_empty[2] | s_full | dp_full | s_read | dp_read | ds_full | ds_read | done
  constexpr int KF = 1, KE = KF + NK, VF = KE + NK, VE = VF + NV, SF = VE + NV, PF = SF + 1, SE = PF + 1, PE = SE + 1,
                DF = PE + 1, DR = DF + 1, DN = DR + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + DN + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto B = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int n_qtiles = (p.sq + BM - 1) / BM;
  const int heads = p.ng * p.qpg;
  const int qt = n_qtiles - 1 - (int)(blockIdx.x / (heads * p.b));
  const int hb = blockIdx.x % (heads * p.b);
  const int bb = hb / heads, hh = hb % heads, g = hh / p.qpg, j = hh % p.qpg;
  const int s0 = qt * BM;
  int kv_end = p.sk;
  if (p.causal) { kv_end = s0 + BM + p.off; if (kv_end > p.sk) kv_end = p.sk; }
  const int n_kv = kv_end > 0 ? (kv_end + BN - 1) / BN : 0;

  if (threadIdx.x == 0) {
    mbar_init(B(0), 1);
    for (int i = KF; i < SF; ++i) mbar_init(B(i), 1);
    mbar_init(B(SF), 1); mbar_init(B(PF), 1); mbar_init(B(SE), 16); mbar_init(B(PE), 16); mbar_init(B(DF), 16);
    mbar_init(B(DR), 1); mbar_init(B(DN), 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmdO);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TCOLS); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 128, tdQ = tmem + 256, tdS = tmem + 256 + D;

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      mbar_expect_tx(B(0), 2 * TB);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_5d(smem_u32(sQ) + c * CH, &tmQ, B(0), c * 64, j, g, bb, s0);
        tma_load_5d(smem_u32(sdO) + c * CH, &tmdO, B(0), c * 64, j, g, bb, s0);
      }
      for (int t = 0; t < n_kv; ++t) {
        const int ks = t % NK, vs = t % NV;
        if (!mbar_wait(B(KE + ks), (((uint32_t)(t / NK)) & 1u) ^ 1u, abort_flag, p.status, 21)) break;
        mbar_expect_tx(B(KF + ks), TB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_5d(smem_u32(sK) + ks * TB + c * CH, &tmK, B(KF + ks), c * 64, 0, g, bb, t * BN);
        if (!mbar_wait(B(VE + vs), (((uint32_t)(t / NV)) & 1u) ^ 1u, abort_flag, p.status, 21)) break;
        mbar_expect_tx(B(VF + vs), TB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_5d(smem_u32(sV) + vs * TB + c * CH, &tmV, B(VF + vs), c * 64, 0, g, bb, t * BN);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, p.lp_fmt, 0, 0);
      const uint32_t idesc_q = make_idesc(BM, D, p.lp_fmt, 0, 1);
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), aK = smem_u32(sK), aV = smem_u32(sV);
      // S of step t once its K tile has landed and (t > 0) the compute warps hold S of step t - 1 in registers
      auto issue_s = [&](int t) -> bool {
        if (!mbar_wait(B(KF + t % NK), ((uint32_t)(t / NK)) & 1u, abort_flag, p.status, 24)) return false;
        if (t > 0 && !mbar_wait(B(SE), (uint32_t)(t - 1) & 1u, abort_flag, p.status, 25)) return false;
        fence_after_sync();
        const uint32_t kb = aK + (t % NK) * TB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tS, kmajor_desc(aQ, kk, CH), kmajor_desc(kb, kk, CH), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(SF));
        return true;
      };
      auto issue_dp = [&](int t) -> bool {
        if (!mbar_wait(B(VF + t % NV), ((uint32_t)(t / NV)) & 1u, abort_flag, p.status, 24)) return false;
        if (t > 0 && !mbar_wait(B(PE), (uint32_t)(t - 1) & 1u, abort_flag, p.status, 25)) return false;
        fence_after_sync();
        const uint32_t vb = aV + (t % NV) * TB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tdP, kmajor_desc(adO, kk, CH), kmajor_desc(vb, kk, CH), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(PF));
        mma_commit(B(VE + t % NV));            // this V tile may be overwritten
        return true;
      };
      bool ok = mbar_wait(B(0), 0, abort_flag, p.status, 22);
      if (ok) ok = issue_s(0);
      if (ok) ok = issue_dp(0);
      for (int t = 0; t < n_kv && ok; ++t) {
        if (t + 1 < n_kv) {
          if (!issue_s(t + 1) || !issue_dp(t + 1)) { ok = false; break; }
        }
        if (!mbar_wait(B(DF), (uint32_t)t & 1u, abort_flag, p.status, 26)) { ok = false; break; }
        fence_after_sync();
        const uint32_t kb = aK + (t % NK) * TB;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16_ts(tdQ, tdS + (uint32_t)(kk * 8), mnmajor_desc(kb, kk, CH), idesc_q, (t > 0 || kk > 0) ? 1u : 0u);
        mma_commit(B(KE + t % NK));            // this K tile may be overwritten
        mma_commit(B(DR));                     // and dS rewritten
      }
      if (ok) mma_commit(B(DN));
    }
  } else if (n_kv > 0) {
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;               // which 32 of a step's 128 key columns
    const int row = quad * 32 + lane;
    const int qrow = s0 + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const long stat_idx = (((long)bb * p.ng + g) * p.qpg + j) * p.sq + qrow;
    const float lse2 = qrow < p.sq ? p.lse[stat_idx] * kLog2e : 0.f;
    const float dlt = qrow < p.sq ? p.delta[stat_idx] : 0.f;
    bool ok = true;
    for (int t = 0; t < n_kv; ++t) {
      const int n0 = t * BN + part * 32;            // first key of this warp's columns
      const uint32_t par = (uint32_t)t & 1u;
      uint32_t r[32];
      float pr[32];
      if (!mbar_wait(B(SF), par, abort_flag, p.status, 27)) { ok = false; break; }
      fence_after_sync();
      tmem_ld32(tS + lane_base + part * 32, r);
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(SE));
      const bool need_mask = (p.causal && (n0 + 31 > s0 + p.off)) || (n0 + 32 > p.sk) || (s0 + BM > p.sq);
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int kv = n0 + e;
          const bool masked = (p.causal && kv > qrow + p.off) || kv >= p.sk || qrow >= p.sq;
          pr[e] = masked ? 0.f : fast_exp2(fmaf(__uint_as_float(r[e]), p.scale_log2, -lse2));
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) pr[e] = fast_exp2(fmaf(__uint_as_float(r[e]), p.scale_log2, -lse2));
      }
      if (!mbar_wait(B(PF), par, abort_flag, p.status, 27)) { ok = false; break; }
      fence_after_sync();
      tmem_ld32(tdP + lane_base + part * 32, r);
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(PE));
      uint32_t w[16];
#pragma unroll
      for (int c = 0; c < 16; ++c)
        w[c] = pack_lp(pr[2 * c] * (__uint_as_float(r[2 * c]) - dlt) * p.scale,
                       pr[2 * c + 1] * (__uint_as_float(r[2 * c + 1]) - dlt) * p.scale, p.lp_fmt);
      // dS of the previous step must have been consumed by its dQ product
      if (t > 0 && !mbar_wait(B(DR), (uint32_t)(t - 1) & 1u, abort_flag, p.status, 28)) { ok = false; break; }
      fence_after_sync();
      tmem_st16(tdS + lane_base + part * 16, w);    // keys [32 part, 32 part + 32) = 16 packed columns
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(DF));
    }
    if (ok && mbar_wait(B(DN), 0, abort_flag, p.status, 29)) {
      fence_after_sync();
      uint8_t* drow = reinterpret_cast<uint8_t*>(p.dq) +
                      2 * ((long)qrow * p.dq_s + (long)bb * p.dq_b + (long)g * p.dq_g + (long)j * p.dq_j);
#pragma unroll
      for (int c = part * (D / 4); c < (part + 1) * (D / 4); c += 16) {
        uint32_t o[16];
        tmem_ld16(tdQ + lane_base + c, o);
        tmem_wait_ld();
        if (qrow < p.sq) {
          uint4* d4 = reinterpret_cast<uint4*>(drow + c * 2);
#pragma unroll
          for (int q4 = 0; q4 < 2; ++q4)
            d4[q4] = make_uint4(pack_lp(__uint_as_float(o[q4 * 8]), __uint_as_float(o[q4 * 8 + 1]), p.lp_fmt),
                                pack_lp(__uint_as_float(o[q4 * 8 + 2]), __uint_as_float(o[q4 * 8 + 3]), p.lp_fmt),
                                pack_lp(__uint_as_float(o[q4 * 8 + 4]), __uint_as_float(o[q4 * 8 + 5]), p.lp_fmt),
                                pack_lp(__uint_as_float(o[q4 * 8 + 6]), __uint_as_float(o[q4 * 8 + 7]), p.lp_fmt));
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// The same kernel with a causal sliding window: steps start at the one that holds the lowest key the tile sees.
template <int D>
__global__ void __launch_bounds__(kAttnDqThreads, 1)
attn_bwd_dq_ts_win_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                      const AttnParams p) {
  constexpr int BM = 128, BN = 128;
  constexpr int TB = D * 256, CH = 16384;              // bytes of a 128-row tile / of one of its 64-column chunks
  constexpr uint32_t TCOLS = 512;
  constexpr int NK = 3, NV = 2;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + TB;
  uint8_t* sK = sdO + TB;
  uint8_t* sV = sK + NK * TB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NV * TB);
  // q_full | k_full[3] | k_empty[3] | v_full[2] | v_empty[2] | s_full | dp_full | s_read | dp_read | ds_full | ds_read | done
  constexpr int KF = 1, KE = KF + NK, VF = KE + NK, VE = VF + NV, SF = VE + NV, PF = SF + 1, SE = PF + 1, PE = SE + 1,
                DF = PE + 1, DR = DF + 1, DN = DR + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + DN + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto B = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int n_qtiles = (p.sq + BM - 1) / BM;
  const int heads = p.ng * p.qpg;
  const int qt = n_qtiles - 1 - (int)(blockIdx.x / (heads * p.b));
  const int hb = blockIdx.x % (heads * p.b);
  const int bb = hb / heads, hh = hb % heads, g = hh / p.qpg, j = hh % p.qpg;
  const int s0 = qt * BM;
  int kv_end = p.sk;
  if (p.causal) { kv_end = s0 + BM + p.off; if (kv_end > p.sk) kv_end = p.sk; }
  const int n_kv = kv_end > 0 ? (kv_end + BN - 1) / BN : 0;
  // lowest key the tile's first row sees (sliding window)
  const int kv_lo = (p.causal) ? s0 + p.off - p.win : 0;
  const int t_lo = kv_lo > 0 ? kv_lo / BN : 0;           // steps [t_lo, n_kv); rings and barrier phases count from t_lo

  if (threadIdx.x == 0) {
    mbar_init(B(0), 1);
    for (int i = KF; i < SF; ++i) mbar_init(B(i), 1);
    mbar_init(B(SF), 1); mbar_init(B(PF), 1); mbar_init(B(SE), 16); mbar_init(B(PE), 16); mbar_init(B(DF), 16);
    mbar_init(B(DR), 1); mbar_init(B(DN), 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmdO);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TCOLS); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 128, tdQ = tmem + 256, tdS = tmem + 256 + D;

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      mbar_expect_tx(B(0), 2 * TB);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_5d(smem_u32(sQ) + c * CH, &tmQ, B(0), c * 64, j, g, bb, s0);
        tma_load_5d(smem_u32(sdO) + c * CH, &tmdO, B(0), c * 64, j, g, bb, s0);
      }
      for (int t = t_lo; t < n_kv; ++t) {
        const int u = t - t_lo;
        const int ks = u % NK, vs = u % NV;
        if (!mbar_wait(B(KE + ks), (((uint32_t)(u / NK)) & 1u) ^ 1u, abort_flag, p.status, 21)) break;
        mbar_expect_tx(B(KF + ks), TB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_5d(smem_u32(sK) + ks * TB + c * CH, &tmK, B(KF + ks), c * 64, 0, g, bb, t * BN);
        if (!mbar_wait(B(VE + vs), (((uint32_t)(u / NV)) & 1u) ^ 1u, abort_flag, p.status, 21)) break;
        mbar_expect_tx(B(VF + vs), TB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_5d(smem_u32(sV) + vs * TB + c * CH, &tmV, B(VF + vs), c * 64, 0, g, bb, t * BN);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, p.lp_fmt, 0, 0);
      const uint32_t idesc_q = make_idesc(BM, D, p.lp_fmt, 0, 1);
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), aK = smem_u32(sK), aV = smem_u32(sV);
      // S of step t once its K tile has landed and (t > 0) the compute warps hold S of step t - 1 in registers
      auto issue_s = [&](int u) -> bool {                 // u = step - t_lo
        if (!mbar_wait(B(KF + u % NK), ((uint32_t)(u / NK)) & 1u, abort_flag, p.status, 24)) return false;
        if (u > 0 && !mbar_wait(B(SE), (uint32_t)(u - 1) & 1u, abort_flag, p.status, 25)) return false;
        fence_after_sync();
        const uint32_t kb = aK + (u % NK) * TB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tS, kmajor_desc(aQ, kk, CH), kmajor_desc(kb, kk, CH), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(SF));
        return true;
      };
      auto issue_dp = [&](int u) -> bool {
        if (!mbar_wait(B(VF + u % NV), ((uint32_t)(u / NV)) & 1u, abort_flag, p.status, 24)) return false;
        if (u > 0 && !mbar_wait(B(PE), (uint32_t)(u - 1) & 1u, abort_flag, p.status, 25)) return false;
        fence_after_sync();
        const uint32_t vb = aV + (u % NV) * TB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tdP, kmajor_desc(adO, kk, CH), kmajor_desc(vb, kk, CH), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(PF));
        mma_commit(B(VE + u % NV));            // this V tile may be overwritten
        return true;
      };
      bool ok = mbar_wait(B(0), 0, abort_flag, p.status, 22);
      if (ok) ok = issue_s(0);
      if (ok) ok = issue_dp(0);
      const int n_u = n_kv - t_lo;
      for (int u = 0; u < n_u && ok; ++u) {
        if (u + 1 < n_u) {
          if (!issue_s(u + 1) || !issue_dp(u + 1)) { ok = false; break; }
        }
        if (!mbar_wait(B(DF), (uint32_t)u & 1u, abort_flag, p.status, 26)) { ok = false; break; }
        fence_after_sync();
        const uint32_t kb = aK + (u % NK) * TB;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16_ts(tdQ, tdS + (uint32_t)(kk * 8), mnmajor_desc(kb, kk, CH), idesc_q, (u > 0 || kk > 0) ? 1u : 0u);
        mma_commit(B(KE + u % NK));            // this K tile may be overwritten
        mma_commit(B(DR));                     // and dS rewritten
      }
      if (ok) mma_commit(B(DN));
    }
  } else if (n_kv > 0) {
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;               // which 32 of a step's 128 key columns
    const int row = quad * 32 + lane;
    const int qrow = s0 + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const long stat_idx = (((long)bb * p.ng + g) * p.qpg + j) * p.sq + qrow;
    const float lse2 = qrow < p.sq ? p.lse[stat_idx] * kLog2e : 0.f;
    const float dlt = qrow < p.sq ? p.delta[stat_idx] : 0.f;
    bool ok = true;
    for (int t = t_lo; t < n_kv; ++t) {
      const int n0 = t * BN + part * 32;            // first key of this warp's columns
      const uint32_t par = (uint32_t)(t - t_lo) & 1u;
      uint32_t r[32];
      float pr[32];
      if (!mbar_wait(B(SF), par, abort_flag, p.status, 27)) { ok = false; break; }
      fence_after_sync();
      tmem_ld32(tS + lane_base + part * 32, r);
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(SE));
      const bool need_mask = (p.causal && (n0 + 31 > s0 + p.off || (n0 + p.win < s0 + BM - 1 + p.off))) ||
                             (n0 + 32 > p.sk) || (s0 + BM > p.sq);
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int kv = n0 + e;
          const bool masked = (p.causal && (kv > qrow + p.off || (kv + p.win < qrow + p.off))) || kv >= p.sk || qrow >= p.sq;
          pr[e] = masked ? 0.f : fast_exp2(fmaf(__uint_as_float(r[e]), p.scale_log2, -lse2));
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) pr[e] = fast_exp2(fmaf(__uint_as_float(r[e]), p.scale_log2, -lse2));
      }
      if (!mbar_wait(B(PF), par, abort_flag, p.status, 27)) { ok = false; break; }
      fence_after_sync();
      tmem_ld32(tdP + lane_base + part * 32, r);
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(PE));
      uint32_t w[16];
#pragma unroll
      for (int c = 0; c < 16; ++c)
        w[c] = pack_lp(pr[2 * c] * (__uint_as_float(r[2 * c]) - dlt) * p.scale,
                       pr[2 * c + 1] * (__uint_as_float(r[2 * c + 1]) - dlt) * p.scale, p.lp_fmt);
      // dS of the previous step must have been consumed by its dQ product
      if (t > t_lo && !mbar_wait(B(DR), par ^ 1u, abort_flag, p.status, 28)) { ok = false; break; }
      fence_after_sync();
      tmem_st16(tdS + lane_base + part * 16, w);    // keys [32 part, 32 part + 32) = 16 packed columns
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(DF));
    }
    if (ok && mbar_wait(B(DN), 0, abort_flag, p.status, 29)) {
      fence_after_sync();
      uint8_t* drow = reinterpret_cast<uint8_t*>(p.dq) +
                      2 * ((long)qrow * p.dq_s + (long)bb * p.dq_b + (long)g * p.dq_g + (long)j * p.dq_j);
#pragma unroll
      for (int c = part * (D / 4); c < (part + 1) * (D / 4); c += 16) {
        uint32_t o[16];
        tmem_ld16(tdQ + lane_base + c, o);
        tmem_wait_ld();
        if (qrow < p.sq) {
          uint4* d4 = reinterpret_cast<uint4*>(drow + c * 2);
#pragma unroll
          for (int q4 = 0; q4 < 2; ++q4)
            d4[q4] = make_uint4(pack_lp(__uint_as_float(o[q4 * 8]), __uint_as_float(o[q4 * 8 + 1]), p.lp_fmt),
                                pack_lp(__uint_as_float(o[q4 * 8 + 2]), __uint_as_float(o[q4 * 8 + 3]), p.lp_fmt),
                                pack_lp(__uint_as_float(o[q4 * 8 + 4]), __uint_as_float(o[q4 * 8 + 5]), p.lp_fmt),
                                pack_lp(__uint_as_float(o[q4 * 8 + 6]), __uint_as_float(o[q4 * 8 + 7]), p.lp_fmt));
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// ============================================================================ backward: dK, dV
template <int D>
__global__ void __launch_bounds__(kAttnBwdThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const AttnParams p) {
  constexpr int BM = 128, BN = 64;                 // BM key rows per CTA, BN query rows per step
  constexpr int KB = D * 256, QB = D * 128, KC = 16384, QC = 8192;
  constexpr uint32_t TCOLS = 512;                  // S^T 64 | dP^T 64 | dV D | dK D
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = sK + KB;
  // Three Q / dO stages: a stage is held until dK += dS^T Q at the end of its step; with two, the tile two steps
  // ahead was requested only when it was already needed.
  constexpr int NST = 3;
  uint8_t* sQ = sV + KB;
  uint8_t* sdO = sQ + NST * QB;
  uint8_t* sP = sdO + NST * QB;
  uint8_t* sdS = sP + 16384;
  float* sStat = reinterpret_cast<float*>(sdS + 16384);       // [2][2][64] lse2 / delta per step parity
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + 256);
  // 0 kv_full | 1..3 q_full | 4..6 q_empty | 7 sdp_full | 8 sdp_empty | 9 pds_full | 10 pds_done
  constexpr int QF = 1, QE = 1 + NST, SF = 1 + 2 * NST, SE = SF + 1, PF = SF + 2, PD = SF + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + PD + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto B = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int n_ktiles = (p.sk + BM - 1) / BM;
  const int kt = blockIdx.x / (p.ng * p.b);                    // early key tiles see the most queries
  const int gb = blockIdx.x % (p.ng * p.b);
  const int bb = gb / p.ng, g = gb % p.ng;
  const int n0 = kt * BM;
  (void)n_ktiles;
  // query tiles that can see at least one key of this tile: q + off >= n0
  int q_begin = 0;
  if (p.causal) { q_begin = n0 - p.off; if (q_begin < 0) q_begin = 0; }
  const int qt0 = q_begin / BN;
  const int n_qt = (p.sq + BN - 1) / BN;
  const int per_head = n_qt > qt0 ? n_qt - qt0 : 0;
  const int n_steps = per_head * p.qpg;

  if (threadIdx.x == 0) {
    mbar_init(B(0), 1);
    for (int i = 0; i < 2 * NST; ++i) mbar_init(B(1 + i), 1);
    mbar_init(B(SF), 1); mbar_init(B(SE), 8); mbar_init(B(PF), 8); mbar_init(B(PD), 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmdO);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TCOLS); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 64, tdV = tmem + 128, tdK = tmem + 128 + D;

  if (warp == 0) {
    if (lane == 0 && n_steps > 0) {
      mbar_expect_tx(B(0), 2 * KB);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_5d(smem_u32(sK) + c * KC, &tmK, B(0), c * 64, 0, g, bb, n0);
        tma_load_5d(smem_u32(sV) + c * KC, &tmV, B(0), c * 64, 0, g, bb, n0);
      }
      for (int t = 0; t < n_steps; ++t) {
        const int st = t % NST;
        const int j = t / per_head, q0 = (qt0 + t % per_head) * BN;
        if (!mbar_wait(B(QE + st), (((uint32_t)(t / NST)) & 1u) ^ 1u, abort_flag, p.status, 31)) break;
        mbar_expect_tx(B(QF + st), 2 * QB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_5d(smem_u32(sQ) + st * QB + c * QC, &tmQ, B(QF + st), c * 64, j, g, bb, q0);
          tma_load_5d(smem_u32(sdO) + st * QB + c * QC, &tmdO, B(QF + st), c * 64, j, g, bb, q0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_steps > 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, p.lp_fmt, 0, 0);       // S^T, dP^T
      const uint32_t idesc_g = make_idesc(BM, D, p.lp_fmt, 0, 1);        // dV, dK: A K-major, B MN-major
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO);
      const uint32_t aP = smem_u32(sP), adS = smem_u32(sdS);
      auto issue_sdp = [&](int t) {
        const uint32_t qb = aQ + (t % NST) * QB, ob = adO + (t % NST) * QB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tS, kmajor_desc(aK, kk, KC), kmajor_desc(qb, kk, QC), idesc_s, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tdP, kmajor_desc(aV, kk, KC), kmajor_desc(ob, kk, QC), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(SF));
      };
      bool ok = mbar_wait(B(0), 0, abort_flag, p.status, 32) && mbar_wait(B(QF), 0, abort_flag, p.status, 33);
      if (ok) { fence_after_sync(); issue_sdp(0); }
      for (int t = 0; t < n_steps && ok; ++t) {
        if (t + 1 < n_steps) {
          const int st1 = (t + 1) % NST;
          if (!mbar_wait(B(QF + st1), ((uint32_t)((t + 1) / NST)) & 1u, abort_flag, p.status, 34)) { ok = false; break; }
          if (!mbar_wait(B(SE), (uint32_t)t & 1u, abort_flag, p.status, 35)) { ok = false; break; }
          fence_after_sync();
          issue_sdp(t + 1);
        }
        if (!mbar_wait(B(PF), (uint32_t)t & 1u, abort_flag, p.status, 36)) { ok = false; break; }
        fence_after_sync();
        const uint32_t qb = aQ + (t % NST) * QB, ob = adO + (t % NST) * QB;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16(tdV, kmajor_desc(aP, kk, 0), mnmajor_desc(ob, kk, QC), idesc_g, (t > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16(tdK, kmajor_desc(adS, kk, 0), mnmajor_desc(qb, kk, QC), idesc_g, (t > 0 || kk > 0) ? 1u : 0u);
        mma_commit(B(QE + (t % NST)));
        mma_commit(B(PD));
      }
    }
  } else if (n_steps > 0) {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;                 // which 32 of a step's 64 query columns this warp takes
    const int row = quad * 32 + lane;
    const int ct = threadIdx.x - 64;                 // 0..255 among the compute threads
    const int krow = n0 + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    bool ok = true;
    for (int t = 0; t < n_steps; ++t) {
      const int j = t / per_head, q0 = (qt0 + t % per_head) * BN;
      // stage this step's per-query statistics (64 lse2 + 64 delta) in shared memory
      {
        float* dst = sStat + (t & 1) * 128;
        if (ct < 128) {
          const int qi = q0 + (ct & 63);
          const long idx = (((long)bb * p.ng + g) * p.qpg + j) * p.sq + qi;
          float v = 0.f;
          if (qi < p.sq) v = (ct < 64) ? p.lse[idx] * kLog2e : p.delta[idx];
          dst[ct] = v;
        }
        bar_sync_compute();
      }
      if (!ok) continue;              // a wait gave up: keep meeting the other warps at the barrier above, do no more
      const float* stat = sStat + (t & 1) * 128 + half * 32;
      if (!mbar_wait(B(SF), (uint32_t)t & 1u, abort_flag, p.status, 37)) { ok = false; continue; }
      fence_after_sync();
      uint32_t wp[16], wd[16];
      uint32_t rs[32], rp[32];
      tmem_ld32(tS + lane_base + half * 32, rs);
      tmem_ld32(tdP + lane_base + half * 32, rp);
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(SE));
      // per-element masks only where the step touches the diagonal or the ends of the sequences
      const bool need_mask = (p.causal && (n0 + BM - 1 > q0 + p.off)) || (q0 + BN > p.sq) || (n0 + BM > p.sk);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          float pr[2], ds[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = 2 * c + e;
            const int qi = q0 + half * 32 + col;
            const bool masked = (p.causal && krow > qi + p.off) || qi >= p.sq || krow >= p.sk;
            pr[e] = masked ? 0.f : fast_exp2(fmaf(__uint_as_float(rs[col]), p.scale_log2, -stat[col]));
            ds[e] = pr[e] * (__uint_as_float(rp[col]) - stat[64 + col]) * p.scale;
          }
          wp[c] = pack_lp(pr[0], pr[1], p.lp_fmt);
          wd[c] = pack_lp(ds[0], ds[1], p.lp_fmt);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(rs[2 * c]), p.scale_log2, -stat[2 * c]));
          const float p1 = fast_exp2(fmaf(__uint_as_float(rs[2 * c + 1]), p.scale_log2, -stat[2 * c + 1]));
          wp[c] = pack_lp(p0, p1, p.lp_fmt);
          wd[c] = pack_lp(p0 * (__uint_as_float(rp[2 * c]) - stat[64 + 2 * c]) * p.scale,
                          p1 * (__uint_as_float(rp[2 * c + 1]) - stat[64 + 2 * c + 1]) * p.scale, p.lp_fmt);
        }
      }
      if (t > 0) {
        if (!mbar_wait(B(PD), (uint32_t)(t - 1) & 1u, abort_flag, p.status, 38)) { ok = false; continue; }
      }
      store_half_row_sw128(sP, row, half, wp);
      store_half_row_sw128(sdS, row, half, wd);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(PF));
    }
    if (ok && mbar_wait(B(PD), (uint32_t)(n_steps - 1) & 1u, abort_flag, p.status, 39)) {
      fence_after_sync();
      uint8_t* vrow = reinterpret_cast<uint8_t*>(p.dv) + 2 * ((long)krow * p.dv_s + (long)bb * p.dv_b + (long)g * p.dv_g);
      uint8_t* krow_p = reinterpret_cast<uint8_t*>(p.dk) + 2 * ((long)krow * p.dk_s + (long)bb * p.dk_b + (long)g * p.dk_g);
#pragma unroll 1
      for (int c = half * (D / 2); c < (half + 1) * (D / 2); c += 32) {
        uint32_t o[32];
        float v[32];
        tmem_ld32(tdV + lane_base + c, o);
        tmem_wait_ld();
        if (krow < p.sk) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i]);
          store_chunk_global(vrow + c * 2, v, p.lp_fmt);
        }
        tmem_ld32(tdK + lane_base + c, o);
        tmem_wait_ld();
        if (krow < p.sk) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i]);
          store_chunk_global(krow_p + c * 2, v, p.lp_fmt);
        }
      }
    }
  } else {
    // no query can see this key tile: its gradients are zero
    const int ct = threadIdx.x - 64;
    if (ct >= 0 && ct < 128) {
      const int krow = n0 + ct;
      if (krow < p.sk) {
        uint4 z = make_uint4(0, 0, 0, 0);
        uint4* vrow = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.dv) + 2 * ((long)krow * p.dv_s + (long)bb * p.dv_b + (long)g * p.dv_g));
        uint4* kr = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.dk) + 2 * ((long)krow * p.dk_s + (long)bb * p.dk_b + (long)g * p.dk_g));
        for (int c = 0; c < D / 8; ++c) { vrow[c] = z; kr[c] = z; }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// ============================================================================ backward: dK, dV, 128-query steps
// attn_bwd_dkv_kernel rebuilt like the dQ kernel above: every product 128 wide (one thread gets a `tcgen05.mma`
// accepted about every 46 cycles whatever its size), P^T and dS^T written over the S^T / dP^T columns they were
// computed from and taken from there as the A operands of dV += P^T dO and dK += dS^T Q, sixteen compute warps.
// All 512 tensor-memory columns are taken (dV | dK | S^T | dP^T), so there is no second S^T / dP^T buffer; instead a
// step runs in two phases that alternate on the tensor pipe:
//   phase A: S^T ready -> exponentials -> P^T            | meanwhile the pipe runs dK of step t - 1, dP^T of step t
//   phase B: dP^T ready -> dS^T = P (dP - delta) scale   | meanwhile the pipe runs dV of step t, S^T of step t + 1
// (products of one thread run in issue order, which is what lets S^T of step t + 1 overwrite P^T of step t right
// behind the dV product that reads it, and dP^T of step t + 1 the dS^T that dK reads).
// Shared memory: K, V, two Q / dO stages of 128 rows, per-query statistics of two steps.
template <int D>
__global__ void __launch_bounds__(kAttnDqThreads, 1)
attn_bwd_dkv_ts_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                       const AttnParams p) {
  constexpr int BM = 128, BN = 128;                // BM key rows per CTA, BN query rows per step
  constexpr int TB = D * 256, CH = 16384;          // bytes of a 128-row tile / of one of its 64-column chunks
  constexpr uint32_t TCOLS = 512;
  constexpr int NST = 2;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = sK + TB;
  uint8_t* sQ = sV + TB;
  uint8_t* sdO = sQ + NST * TB;
  float* sStat = reinterpret_cast<float*>(sdO + NST * TB);     // [2][2][128] lse2 / delta per step parity
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + 512);
  // kv_full | q_full[2] | q_empty[2] | s_full | dp_full | p_full | ds_full | done
  constexpr int QF = 1, QE = QF + NST, SF = QE + NST, PF = SF + 1, AF = PF + 1, BF = AF + 1, DN = BF + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + DN + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto B = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int kt = blockIdx.x / (p.ng * p.b);                    // early key tiles see the most queries
  const int gb = blockIdx.x % (p.ng * p.b);
  const int bb = gb / p.ng, g = gb % p.ng;
  const int n0 = kt * BM;
  // query tiles that can see at least one key of this tile: q + off >= n0
  int q_begin = 0;
  if (p.causal) { q_begin = n0 - p.off; if (q_begin < 0) q_begin = 0; }
  const int qt0 = q_begin / BN;
  const int n_qt = (p.sq + BN - 1) / BN;
  const int per_head = n_qt > qt0 ? n_qt - qt0 : 0;
  const int n_steps = per_head * p.qpg;

  if (threadIdx.x == 0) {
    mbar_init(B(0), 1);
    for (int i = 0; i < 2 * NST; ++i) mbar_init(B(QF + i), 1);
    mbar_init(B(SF), 1); mbar_init(B(PF), 1); mbar_init(B(AF), 16); mbar_init(B(BF), 16); mbar_init(B(DN), 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmdO);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TCOLS); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tdV = tmem, tdK = tmem + D, tS = tmem + 2 * D, tdP = tmem + 2 * D + 128;

  if (warp == 0) {
    if (lane == 0 && n_steps > 0) {
      mbar_expect_tx(B(0), 2 * TB);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_5d(smem_u32(sK) + c * CH, &tmK, B(0), c * 64, 0, g, bb, n0);
        tma_load_5d(smem_u32(sV) + c * CH, &tmV, B(0), c * 64, 0, g, bb, n0);
      }
      for (int t = 0; t < n_steps; ++t) {
        const int st = t % NST;
        const int j = t / per_head, q0 = (qt0 + t % per_head) * BN;
        if (!mbar_wait(B(QE + st), (((uint32_t)(t / NST)) & 1u) ^ 1u, abort_flag, p.status, 31)) break;
        mbar_expect_tx(B(QF + st), 2 * TB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_5d(smem_u32(sQ) + st * TB + c * CH, &tmQ, B(QF + st), c * 64, j, g, bb, q0);
          tma_load_5d(smem_u32(sdO) + st * TB + c * CH, &tmdO, B(QF + st), c * 64, j, g, bb, q0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_steps > 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, p.lp_fmt, 0, 0);       // S^T, dP^T
      const uint32_t idesc_g = make_idesc(BM, D, p.lp_fmt, 0, 1);        // dV, dK: A from tensor memory, B MN-major
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO);
      auto issue_s = [&](int t) {
        const uint32_t qb = aQ + (t % NST) * TB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tS, kmajor_desc(aK, kk, CH), kmajor_desc(qb, kk, CH), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(SF));
      };
      auto issue_dp = [&](int t) {
        const uint32_t ob = adO + (t % NST) * TB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tdP, kmajor_desc(aV, kk, CH), kmajor_desc(ob, kk, CH), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(PF));
      };
      bool ok = mbar_wait(B(0), 0, abort_flag, p.status, 32) && mbar_wait(B(QF), 0, abort_flag, p.status, 33);
      if (ok) { fence_after_sync(); issue_s(0); issue_dp(0); }
      for (int t = 0; t < n_steps && ok; ++t) {
        const uint32_t par = (uint32_t)t & 1u;
        const uint32_t qb = aQ + (t % NST) * TB, ob = adO + (t % NST) * TB;
        if (!mbar_wait(B(AF), par, abort_flag, p.status, 36)) { ok = false; break; }
        fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16_ts(tdV, tS + (uint32_t)((kk >> 1) * 32 + (kk & 1) * 8), mnmajor_desc(ob, kk, CH), idesc_g,
                     (t > 0 || kk > 0) ? 1u : 0u);
        if (t + 1 < n_steps) {
          if (!mbar_wait(B(QF + (t + 1) % NST), ((uint32_t)((t + 1) / NST)) & 1u, abort_flag, p.status, 34)) { ok = false; break; }
          fence_after_sync();
          issue_s(t + 1);
        }
        if (!mbar_wait(B(BF), par, abort_flag, p.status, 36)) { ok = false; break; }
        fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16_ts(tdK, tdP + (uint32_t)((kk >> 1) * 32 + (kk & 1) * 8), mnmajor_desc(qb, kk, CH), idesc_g,
                     (t > 0 || kk > 0) ? 1u : 0u);
        mma_commit(B(QE + (t % NST)));         // Q / dO of this step may be overwritten
        if (t + 1 < n_steps) issue_dp(t + 1);
      }
      if (ok) mma_commit(B(DN));
    }
  } else if (n_steps > 0) {
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;                 // which 32 of a step's 128 query columns this warp takes
    const int row = quad * 32 + lane;
    const int ct = threadIdx.x - 64;                 // 0..511 among the compute threads
    const int krow = n0 + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    bool ok = true;
    // per-query statistics of a step (128 lse2 + 128 delta): read from global memory one step ahead
    auto load_stat = [&](int t) -> float {
      const int j = t / per_head, q0 = (qt0 + t % per_head) * BN;
      const int qi = q0 + (ct & 127);
      const long idx = (((long)bb * p.ng + g) * p.qpg + j) * p.sq + qi;
      if (qi >= p.sq) return 0.f;
      return (ct < 128) ? p.lse[idx] * kLog2e : p.delta[idx];
    };
    float stat_next = ct < 256 ? load_stat(0) : 0.f;
    for (int t = 0; t < n_steps; ++t) {
      const int q0 = (qt0 + t % per_head) * BN + part * 32;        // first query of this warp's columns
      const uint32_t par = (uint32_t)t & 1u;
      {
        float* dst = sStat + (t & 1) * 256;
        if (ct < 256) {
          dst[ct] = stat_next;
          if (t + 1 < n_steps) stat_next = load_stat(t + 1);
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
      }
      if (!ok) continue;              // a wait gave up: keep meeting the other warps at the barrier above, do no more
      const float* stat = sStat + (t & 1) * 256 + part * 32;
      uint32_t r[32];
      float pr[32];
      uint32_t w[16];
      // ---- phase A: P^T
      if (!mbar_wait(B(SF), par, abort_flag, p.status, 37)) { ok = false; continue; }
      fence_after_sync();
      tmem_ld32(tS + lane_base + part * 32, r);
      tmem_wait_ld();
      const bool need_mask = (p.causal && (n0 + BM - 1 > q0 + p.off)) || (q0 + 32 > p.sq) || (n0 + BM > p.sk);
#pragma unroll
      for (int e4 = 0; e4 < 8; ++e4) {
        const float4 l4 = *reinterpret_cast<const float4*>(stat + 4 * e4);
        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int e = 4 * e4 + i;
          float v = fast_exp2(fmaf(__uint_as_float(r[e]), p.scale_log2, -ls[i]));
          if (need_mask) {
            const int qi = q0 + e;
            if ((p.causal && krow > qi + p.off) || qi >= p.sq || krow >= p.sk) v = 0.f;
          }
          pr[e] = v;
        }
      }
#pragma unroll
      for (int c = 0; c < 16; ++c) w[c] = pack_lp(pr[2 * c], pr[2 * c + 1], p.lp_fmt);
      // queries [32 part, 32 part + 32) as 16 packed columns over the start of the S^T columns this warp has just read
      tmem_st16(tS + lane_base + part * 32, w);
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(AF));
      // ---- phase B: dS^T
      if (!mbar_wait(B(PF), par, abort_flag, p.status, 38)) { ok = false; continue; }
      fence_after_sync();
      tmem_ld32(tdP + lane_base + part * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int e4 = 0; e4 < 8; ++e4) {
        const float4 d4 = *reinterpret_cast<const float4*>(stat + 128 + 4 * e4);
        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int e = 4 * e4 + i;
          pr[e] = pr[e] * (__uint_as_float(r[e]) - dl[i]) * p.scale;
        }
      }
#pragma unroll
      for (int c = 0; c < 16; ++c) w[c] = pack_lp(pr[2 * c], pr[2 * c + 1], p.lp_fmt);
      tmem_st16(tdP + lane_base + part * 32, w);
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(BF));
    }
    if (ok && mbar_wait(B(DN), 0, abort_flag, p.status, 39)) {
      fence_after_sync();
      uint8_t* vrow = reinterpret_cast<uint8_t*>(p.dv) + 2 * ((long)krow * p.dv_s + (long)bb * p.dv_b + (long)g * p.dv_g);
      uint8_t* krow_p = reinterpret_cast<uint8_t*>(p.dk) + 2 * ((long)krow * p.dk_s + (long)bb * p.dk_b + (long)g * p.dk_g);
#pragma unroll
      for (int c = part * (D / 4); c < (part + 1) * (D / 4); c += 16) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          uint32_t o[16];
          tmem_ld16((which ? tdK : tdV) + lane_base + c, o);
          tmem_wait_ld();
          if (krow < p.sk) {
            uint4* d4 = reinterpret_cast<uint4*>((which ? krow_p : vrow) + c * 2);
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4)
              d4[q4] = make_uint4(pack_lp(__uint_as_float(o[q4 * 8]), __uint_as_float(o[q4 * 8 + 1]), p.lp_fmt),
                                  pack_lp(__uint_as_float(o[q4 * 8 + 2]), __uint_as_float(o[q4 * 8 + 3]), p.lp_fmt),
                                  pack_lp(__uint_as_float(o[q4 * 8 + 4]), __uint_as_float(o[q4 * 8 + 5]), p.lp_fmt),
                                  pack_lp(__uint_as_float(o[q4 * 8 + 6]), __uint_as_float(o[q4 * 8 + 7]), p.lp_fmt));
          }
        }
      }
    }
  } else {
    // no query can see this key tile: its gradients are zero
    const int ct = threadIdx.x - 64;
    if (ct >= 0 && ct < 128) {
      const int krow = n0 + ct;
      if (krow < p.sk) {
        uint4 z = make_uint4(0, 0, 0, 0);
        uint4* vrow = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.dv) + 2 * ((long)krow * p.dv_s + (long)bb * p.dv_b + (long)g * p.dv_g));
        uint4* kr = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.dk) + 2 * ((long)krow * p.dk_s + (long)bb * p.dk_b + (long)g * p.dk_g));
        for (int c = 0; c < D / 8; ++c) { vrow[c] = z; kr[c] = z; }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// The same kernel with a causal sliding window: query tiles end at the last query whose window reaches the key tile.
template <int D>
__global__ void __launch_bounds__(kAttnDqThreads, 1)
attn_bwd_dkv_ts_win_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                       const AttnParams p) {
  constexpr int BM = 128, BN = 128;                // BM key rows per CTA, BN query rows per step
  constexpr int TB = D * 256, CH = 16384;          // bytes of a 128-row tile / of one of its 64-column chunks
  constexpr uint32_t TCOLS = 512;
  constexpr int NST = 2;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = sK + TB;
  uint8_t* sQ = sV + TB;
  uint8_t* sdO = sQ + NST * TB;
  float* sStat = reinterpret_cast<float*>(sdO + NST * TB);     // [2][2][128] lse2 / delta per step parity
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + 512);
  // kv_full | q_full[2] | q_empty[2] | s_full | dp_full | p_full | ds_full | done
  constexpr int QF = 1, QE = QF + NST, SF = QE + NST, PF = SF + 1, AF = PF + 1, BF = AF + 1, DN = BF + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + DN + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto B = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int kt = blockIdx.x / (p.ng * p.b);                    // early key tiles see the most queries
  const int gb = blockIdx.x % (p.ng * p.b);
  const int bb = gb / p.ng, g = gb % p.ng;
  const int n0 = kt * BM;
  // query tiles that can see at least one key of this tile: q + off >= n0
  int q_begin = 0;
  if (p.causal) { q_begin = n0 - p.off; if (q_begin < 0) q_begin = 0; }
  const int qt0 = q_begin / BN;
  // ... and, with a sliding window, at most up to the last query whose window still reaches the tile's last key
  int q_end = p.sq;
  if (p.causal) { const long e = (long)n0 + BM + p.win - p.off; if (e < (long)q_end) q_end = (int)e; }
  const int n_qt = q_end > 0 ? (q_end + BN - 1) / BN : 0;
  const int per_head = n_qt > qt0 ? n_qt - qt0 : 0;
  const int n_steps = per_head * p.qpg;

  if (threadIdx.x == 0) {
    mbar_init(B(0), 1);
    for (int i = 0; i < 2 * NST; ++i) mbar_init(B(QF + i), 1);
    mbar_init(B(SF), 1); mbar_init(B(PF), 1); mbar_init(B(AF), 16); mbar_init(B(BF), 16); mbar_init(B(DN), 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmdO);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TCOLS); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tdV = tmem, tdK = tmem + D, tS = tmem + 2 * D, tdP = tmem + 2 * D + 128;

  if (warp == 0) {
    if (lane == 0 && n_steps > 0) {
      mbar_expect_tx(B(0), 2 * TB);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_5d(smem_u32(sK) + c * CH, &tmK, B(0), c * 64, 0, g, bb, n0);
        tma_load_5d(smem_u32(sV) + c * CH, &tmV, B(0), c * 64, 0, g, bb, n0);
      }
      for (int t = 0; t < n_steps; ++t) {
        const int st = t % NST;
        const int j = t / per_head, q0 = (qt0 + t % per_head) * BN;
        if (!mbar_wait(B(QE + st), (((uint32_t)(t / NST)) & 1u) ^ 1u, abort_flag, p.status, 31)) break;
        mbar_expect_tx(B(QF + st), 2 * TB);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_5d(smem_u32(sQ) + st * TB + c * CH, &tmQ, B(QF + st), c * 64, j, g, bb, q0);
          tma_load_5d(smem_u32(sdO) + st * TB + c * CH, &tmdO, B(QF + st), c * 64, j, g, bb, q0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_steps > 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, p.lp_fmt, 0, 0);       // S^T, dP^T
      const uint32_t idesc_g = make_idesc(BM, D, p.lp_fmt, 0, 1);        // dV, dK: A from tensor memory, B MN-major
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO);
      auto issue_s = [&](int t) {
        const uint32_t qb = aQ + (t % NST) * TB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tS, kmajor_desc(aK, kk, CH), kmajor_desc(qb, kk, CH), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(SF));
      };
      auto issue_dp = [&](int t) {
        const uint32_t ob = adO + (t % NST) * TB;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_f16(tdP, kmajor_desc(aV, kk, CH), kmajor_desc(ob, kk, CH), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(B(PF));
      };
      bool ok = mbar_wait(B(0), 0, abort_flag, p.status, 32) && mbar_wait(B(QF), 0, abort_flag, p.status, 33);
      if (ok) { fence_after_sync(); issue_s(0); issue_dp(0); }
      for (int t = 0; t < n_steps && ok; ++t) {
        const uint32_t par = (uint32_t)t & 1u;
        const uint32_t qb = aQ + (t % NST) * TB, ob = adO + (t % NST) * TB;
        if (!mbar_wait(B(AF), par, abort_flag, p.status, 36)) { ok = false; break; }
        fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16_ts(tdV, tS + (uint32_t)((kk >> 1) * 32 + (kk & 1) * 8), mnmajor_desc(ob, kk, CH), idesc_g,
                     (t > 0 || kk > 0) ? 1u : 0u);
        if (t + 1 < n_steps) {
          if (!mbar_wait(B(QF + (t + 1) % NST), ((uint32_t)((t + 1) / NST)) & 1u, abort_flag, p.status, 34)) { ok = false; break; }
          fence_after_sync();
          issue_s(t + 1);
        }
        if (!mbar_wait(B(BF), par, abort_flag, p.status, 36)) { ok = false; break; }
        fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          mma_f16_ts(tdK, tdP + (uint32_t)((kk >> 1) * 32 + (kk & 1) * 8), mnmajor_desc(qb, kk, CH), idesc_g,
                     (t > 0 || kk > 0) ? 1u : 0u);
        mma_commit(B(QE + (t % NST)));         // Q / dO of this step may be overwritten
        if (t + 1 < n_steps) issue_dp(t + 1);
      }
      if (ok) mma_commit(B(DN));
    }
  } else if (n_steps > 0) {
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;                 // which 32 of a step's 128 query columns this warp takes
    const int row = quad * 32 + lane;
    const int ct = threadIdx.x - 64;                 // 0..511 among the compute threads
    const int krow = n0 + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    bool ok = true;
    // per-query statistics of a step (128 lse2 + 128 delta): read from global memory one step ahead
    auto load_stat = [&](int t) -> float {
      const int j = t / per_head, q0 = (qt0 + t % per_head) * BN;
      const int qi = q0 + (ct & 127);
      const long idx = (((long)bb * p.ng + g) * p.qpg + j) * p.sq + qi;
      if (qi >= p.sq) return 0.f;
      return (ct < 128) ? p.lse[idx] * kLog2e : p.delta[idx];
    };
    float stat_next = ct < 256 ? load_stat(0) : 0.f;
    for (int t = 0; t < n_steps; ++t) {
      const int q0 = (qt0 + t % per_head) * BN + part * 32;        // first query of this warp's columns
      const uint32_t par = (uint32_t)t & 1u;
      {
        float* dst = sStat + (t & 1) * 256;
        if (ct < 256) {
          dst[ct] = stat_next;
          if (t + 1 < n_steps) stat_next = load_stat(t + 1);
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
      }
      if (!ok) continue;              // a wait gave up: keep meeting the other warps at the barrier above, do no more
      const float* stat = sStat + (t & 1) * 256 + part * 32;
      uint32_t r[32];
      float pr[32];
      uint32_t w[16];
      // ---- phase A: P^T
      if (!mbar_wait(B(SF), par, abort_flag, p.status, 37)) { ok = false; continue; }
      fence_after_sync();
      tmem_ld32(tS + lane_base + part * 32, r);
      tmem_wait_ld();
      const bool need_mask = (p.causal && (n0 + BM - 1 > q0 + p.off || (n0 + p.win < q0 + 31 + p.off))) ||
                             (q0 + 32 > p.sq) || (n0 + BM > p.sk);
#pragma unroll
      for (int e4 = 0; e4 < 8; ++e4) {
        const float4 l4 = *reinterpret_cast<const float4*>(stat + 4 * e4);
        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int e = 4 * e4 + i;
          float v = fast_exp2(fmaf(__uint_as_float(r[e]), p.scale_log2, -ls[i]));
          if (need_mask) {
            const int qi = q0 + e;
            if ((p.causal && (krow > qi + p.off || (krow + p.win < qi + p.off))) || qi >= p.sq || krow >= p.sk) v = 0.f;
          }
          pr[e] = v;
        }
      }
#pragma unroll
      for (int c = 0; c < 16; ++c) w[c] = pack_lp(pr[2 * c], pr[2 * c + 1], p.lp_fmt);
      // queries [32 part, 32 part + 32) as 16 packed columns over the start of the S^T columns this warp has just read
      tmem_st16(tS + lane_base + part * 32, w);
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(AF));
      // ---- phase B: dS^T
      if (!mbar_wait(B(PF), par, abort_flag, p.status, 38)) { ok = false; continue; }
      fence_after_sync();
      tmem_ld32(tdP + lane_base + part * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int e4 = 0; e4 < 8; ++e4) {
        const float4 d4 = *reinterpret_cast<const float4*>(stat + 128 + 4 * e4);
        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int e = 4 * e4 + i;
          pr[e] = pr[e] * (__uint_as_float(r[e]) - dl[i]) * p.scale;
        }
      }
#pragma unroll
      for (int c = 0; c < 16; ++c) w[c] = pack_lp(pr[2 * c], pr[2 * c + 1], p.lp_fmt);
      tmem_st16(tdP + lane_base + part * 32, w);
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(B(BF));
    }
    if (ok && mbar_wait(B(DN), 0, abort_flag, p.status, 39)) {
      fence_after_sync();
      uint8_t* vrow = reinterpret_cast<uint8_t*>(p.dv) + 2 * ((long)krow * p.dv_s + (long)bb * p.dv_b + (long)g * p.dv_g);
      uint8_t* krow_p = reinterpret_cast<uint8_t*>(p.dk) + 2 * ((long)krow * p.dk_s + (long)bb * p.dk_b + (long)g * p.dk_g);
#pragma unroll
      for (int c = part * (D / 4); c < (part + 1) * (D / 4); c += 16) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          uint32_t o[16];
          tmem_ld16((which ? tdK : tdV) + lane_base + c, o);
          tmem_wait_ld();
          if (krow < p.sk) {
            uint4* d4 = reinterpret_cast<uint4*>((which ? krow_p : vrow) + c * 2);
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4)
              d4[q4] = make_uint4(pack_lp(__uint_as_float(o[q4 * 8]), __uint_as_float(o[q4 * 8 + 1]), p.lp_fmt),
                                  pack_lp(__uint_as_float(o[q4 * 8 + 2]), __uint_as_float(o[q4 * 8 + 3]), p.lp_fmt),
                                  pack_lp(__uint_as_float(o[q4 * 8 + 4]), __uint_as_float(o[q4 * 8 + 5]), p.lp_fmt),
                                  pack_lp(__uint_as_float(o[q4 * 8 + 6]), __uint_as_float(o[q4 * 8 + 7]), p.lp_fmt));
          }
        }
      }
    }
  } else {
    // no query can see this key tile: its gradients are zero
    const int ct = threadIdx.x - 64;
    if (ct >= 0 && ct < 128) {
      const int krow = n0 + ct;
      if (krow < p.sk) {
        uint4 z = make_uint4(0, 0, 0, 0);
        uint4* vrow = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.dv) + 2 * ((long)krow * p.dv_s + (long)bb * p.dv_b + (long)g * p.dv_g));
        uint4* kr = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.dk) + 2 * ((long)krow * p.dk_s + (long)bb * p.dk_b + (long)g * p.dk_g));
        for (int c = 0; c < D / 8; ++c) { vrow[c] = z; kr[c] = z; }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// ---------------------------------------------------------------------------- host side
static int make_tmap5(CUtensorMap* m, const void* base, int D, int nj, int ng, int b, int s, long st_j, long st_g,
                      long st_b, long st_s, int box_rows) {
  uint64_t dims[5] = {(uint64_t)D, (uint64_t)nj, (uint64_t)ng, (uint64_t)b, (uint64_t)s};
  uint64_t strides[4] = {(uint64_t)st_j * 2, (uint64_t)st_g * 2, (uint64_t)st_b * 2, (uint64_t)st_s * 2};
  uint32_t box[5] = {64, 1, 1, 1, (uint32_t)box_rows};
  for (int i = 0; i < 4; ++i) if (strides[i] % 16) return -3;
  if (reinterpret_cast<uintptr_t>(base) & 15) return -3;
  return make_tmap(m, base, 5, dims, strides, box);
}

template <typename K> static int set_smem(K kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return e == cudaSuccess ? 0 : (int)e;
}

}  // namespace mlb

using namespace mlb;

// strides are in elements; head dim contiguous; D in {64, 128}
MLB_API int mlb_attn_fwd(int lp_fmt, const void* q, const void* k, const void* v, void* o, float* lse,
                         int sq, int sk, int b, int ng, int qpg, int D,
                         long q_s, long q_b, long q_g, long q_j, long k_s, long k_b, long k_g,
                         long v_s, long v_b, long v_g, long o_s, long o_b, long o_g, long o_j,
                         float scale, int causal, int window, int* status, cudaStream_t st) {
  if (D != 64 && D != 128) return -5;
  if (sq <= 0 || sk <= 0 || (causal && sk < sq)) return -6;
  if (window >= 0 && !causal) return -6;              // the sliding window is the causal one: keys [q - window, q]
  if ((o_s % 8) || (o_b % 8) || (o_g % 8) || (o_j % 8) || (reinterpret_cast<uintptr_t>(o) & 15)) return -3;
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  static int use_v2 = -1;                                    // MLB_ATTN_FWD2=0: two independent 128-row CTAs per SM
  if (use_v2 < 0) { const char* e = getenv("MLB_ATTN_FWD2"); use_v2 = (e && e[0] == '0') ? 0 : 1; }
  if ((rc = make_tmap5(&tmQ, q, D, qpg, ng, b, sq, q_j, q_g, q_b, q_s, 128))) return rc;
  if (!use_v2) {
    if ((rc = make_tmap5(&tmK, k, D, 1, ng, b, sk, D, k_g, k_b, k_s, 64))) return rc;
    if ((rc = make_tmap5(&tmV, v, D, 1, ng, b, sk, D, v_g, v_b, v_s, 64))) return rc;
  }
  AttnParams p = {};
  p.sq = sq; p.sk = sk; p.b = b; p.ng = ng; p.qpg = qpg; p.causal = causal; p.off = sk - sq;
  p.scale = scale; p.scale_log2 = scale * kLog2e; p.lp_fmt = lp_fmt; p.status = status;
  p.o = o; p.o_s = o_s; p.o_b = o_b; p.o_g = o_g; p.o_j = o_j; p.lse = lse;
  p.win = window >= 0 ? window : (1 << 30);
  if (window >= 0 && !use_v2) return -7;              // only the two-tile kernel knows windows
  if (use_v2) {
    CUtensorMap tmK2, tmV2;
    if ((rc = make_tmap5(&tmK2, k, D, 1, ng, b, sk, D, k_g, k_b, k_s, 128))) return rc;
    if ((rc = make_tmap5(&tmV2, v, D, 1, ng, b, sk, D, v_g, v_b, v_s, 128))) return rc;
    const int grid2 = ((sq + 255) / 256) * ng * qpg * b;
    const int smem2 = 2 * D * 256 + 5 * D * 256 + 256;
    auto launch = [&](auto kern, bool& set) -> int {
      if (!set) { if (int e = set_smem(kern, smem2)) return e; set = true; }
      kern<<<grid2, kAttnFwd2Threads, smem2, st>>>(tmQ, tmK2, tmV2, p);
      return 0;
    };
    static bool set[4] = {false, false, false, false};
    const bool w = window >= 0;
    if (D == 128) rc = w ? launch(attn_fwd2_win_kernel<128>, set[0]) : launch(attn_fwd2_kernel<128>, set[1]);
    else rc = w ? launch(attn_fwd2_win_kernel<64>, set[2]) : launch(attn_fwd2_kernel<64>, set[3]);
    if (rc) return rc;
    MLB_CHECK_LAUNCH();
    return 0;
  }
  const int grid = ((sq + 127) / 128) * ng * qpg * b;
  const int smem = D * 256 + 4 * D * 128 + 16384 + 128;
  if (D == 128) {
    static bool set = false;
    if (!set) { if ((rc = set_smem(attn_fwd_kernel<128>, smem))) return rc; set = true; }
    attn_fwd_kernel<128><<<grid, kAttnThreads, smem, st>>>(tmQ, tmK, tmV, p);
  } else {
    static bool set = false;
    if (!set) { if ((rc = set_smem(attn_fwd_kernel<64>, smem))) return rc; set = true; }
    attn_fwd_kernel<64><<<grid, kAttnThreads, smem, st>>>(tmQ, tmK, tmV, p);
  }
  MLB_CHECK_LAUNCH();
  return 0;
}

MLB_API int mlb_attn_bwd(int lp_fmt, const void* q, const void* k, const void* v, const void* o, const void* d_o,
                         const float* lse, float* delta, void* dq, void* dk, void* dv,
                         int sq, int sk, int b, int ng, int qpg, int D,
                         long q_s, long q_b, long q_g, long q_j, long k_s, long k_b, long k_g,
                         long v_s, long v_b, long v_g, long o_s, long o_b, long o_g, long o_j,
                         long do_s, long do_b, long do_g, long do_j, long dq_s, long dq_b, long dq_g, long dq_j,
                         long dk_s, long dk_b, long dk_g, long dv_s, long dv_b, long dv_g,
                         float scale, int causal, int window, int* status, cudaStream_t st) {
  if (D != 64 && D != 128) return -5;
  if (sq <= 0 || sk <= 0 || (causal && sk < sq)) return -6;
  const long chk[] = {dq_s, dq_b, dq_g, dq_j, dk_s, dk_b, dk_g, dv_s, dv_b, dv_g};
  for (long x : chk) if (x % 8) return -3;
  if ((reinterpret_cast<uintptr_t>(dq) & 15) || (reinterpret_cast<uintptr_t>(dk) & 15) || (reinterpret_cast<uintptr_t>(dv) & 15)) return -3;
  {
    const long rows = (long)sq * b * ng * qpg;
    attn_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const uint16_t*)o, (const uint16_t*)d_o, delta, sq, b, ng,
                                                                 qpg, D, o_s, o_b, o_g, o_j, do_s, do_b, do_g, do_j, lp_fmt);
    MLB_CHECK_LAUNCH();
  }
  AttnParams p = {};
  p.sq = sq; p.sk = sk; p.b = b; p.ng = ng; p.qpg = qpg; p.causal = causal; p.off = sk - sq;
  p.scale = scale; p.scale_log2 = scale * kLog2e; p.lp_fmt = lp_fmt; p.status = status;
  p.lse = const_cast<float*>(lse); p.delta = delta;
  p.win = window >= 0 ? window : (1 << 30);
  p.q = q; p.q_s = q_s; p.q_b = q_b; p.q_g = q_g; p.q_j = q_j;
  p.d_o = d_o; p.do_s = do_s; p.do_b = do_b; p.do_g = do_g; p.do_j = do_j;
  p.dq = dq; p.dq_s = dq_s; p.dq_b = dq_b; p.dq_g = dq_g; p.dq_j = dq_j;
  p.dk = dk; p.dk_s = dk_s; p.dk_b = dk_b; p.dk_g = dk_g;
  p.dv = dv; p.dv_s = dv_s; p.dv_b = dv_b; p.dv_g = dv_g;
  int rc;
  static int use_ts = -1;                  // MLB_ATTN_TS=0: the kernels with 64-wide steps and P / dS through shared memory
  if (use_ts < 0) { const char* e = getenv("MLB_ATTN_TS"); use_ts = (e && e[0] == '0') ? 0 : 1; }
  if (window >= 0 && (!use_ts || !causal)) return -7;
  // 128-row boxes of all four operands serve both kernels of the default path
  CUtensorMap tmQ, tmdO, tmK128, tmV128;
  if ((rc = make_tmap5(&tmQ, q, D, qpg, ng, b, sq, q_j, q_g, q_b, q_s, 128))) return rc;
  if ((rc = make_tmap5(&tmdO, d_o, D, qpg, ng, b, sq, do_j, do_g, do_b, do_s, 128))) return rc;
  if ((rc = make_tmap5(&tmK128, k, D, 1, ng, b, sk, D, k_g, k_b, k_s, 128))) return rc;
  if ((rc = make_tmap5(&tmV128, v, D, 1, ng, b, sk, D, v_g, v_b, v_s, 128))) return rc;
  {  // dQ: 128-row query tiles
    CUtensorMap tmK, tmV;
    if (!use_ts) {
      if ((rc = make_tmap5(&tmK, k, D, 1, ng, b, sk, D, k_g, k_b, k_s, 64))) return rc;
      if ((rc = make_tmap5(&tmV, v, D, 1, ng, b, sk, D, v_g, v_b, v_s, 64))) return rc;
    }
    const int grid = ((sq + 127) / 128) * ng * qpg * b;
    if (use_ts) {
      const int smem_ts = 7 * D * 256 + 256;                           // Q, dO, three K stages, two V stages
      auto launch = [&](auto kern, bool& set) -> int {
        if (!set) { if (int e = set_smem(kern, smem_ts)) return e; set = true; }
        kern<<<grid, kAttnDqThreads, smem_ts, st>>>(tmQ, tmK128, tmV128, tmdO, p);
        return 0;
      };
      static bool set[4] = {false, false, false, false};
      const bool w = window >= 0;
      if (D == 128) rc = w ? launch(attn_bwd_dq_ts_win_kernel<128>, set[0]) : launch(attn_bwd_dq_ts_kernel<128>, set[1]);
      else rc = w ? launch(attn_bwd_dq_ts_win_kernel<64>, set[2]) : launch(attn_bwd_dq_ts_kernel<64>, set[3]);
      if (rc) return rc;
      MLB_CHECK_LAUNCH();
    } else {
    const int smem = 2 * D * 256 + 8 * D * 128 + 16384 + 128;         // Q, dO, four K/V stages, dS
    if (D == 128) {
      static bool set = false;
      if (!set) { if ((rc = set_smem(attn_bwd_dq_kernel<128>, smem))) return rc; set = true; }
      attn_bwd_dq_kernel<128><<<grid, kAttnBwdThreads, smem, st>>>(tmQ, tmK, tmV, tmdO, p);
    } else {
      static bool set = false;
      if (!set) { if ((rc = set_smem(attn_bwd_dq_kernel<64>, smem))) return rc; set = true; }
      attn_bwd_dq_kernel<64><<<grid, kAttnBwdThreads, smem, st>>>(tmQ, tmK, tmV, tmdO, p);
    }
    MLB_CHECK_LAUNCH();
    }
  }
  {  // dK, dV: 128-row key tiles, 64-row query tiles
    CUtensorMap tmQ64, tmdO64;
    if (!use_ts) {
      if ((rc = make_tmap5(&tmQ64, q, D, qpg, ng, b, sq, q_j, q_g, q_b, q_s, 64))) return rc;
      if ((rc = make_tmap5(&tmdO64, d_o, D, qpg, ng, b, sq, do_j, do_g, do_b, do_s, 64))) return rc;
    }
    const int grid = ((sk + 127) / 128) * ng * b;
    if (use_ts) {
      const int smem_ts = 6 * D * 256 + 2048 + 256;                    // K, V, two Q/dO stages, stats
      auto launch = [&](auto kern, bool& set) -> int {
        if (!set) { if (int e = set_smem(kern, smem_ts)) return e; set = true; }
        kern<<<grid, kAttnDqThreads, smem_ts, st>>>(tmQ, tmK128, tmV128, tmdO, p);
        return 0;
      };
      static bool set[4] = {false, false, false, false};
      const bool w = window >= 0;
      if (D == 128) rc = w ? launch(attn_bwd_dkv_ts_win_kernel<128>, set[0]) : launch(attn_bwd_dkv_ts_kernel<128>, set[1]);
      else rc = w ? launch(attn_bwd_dkv_ts_win_kernel<64>, set[2]) : launch(attn_bwd_dkv_ts_kernel<64>, set[3]);
      if (rc) return rc;
    } else {
      const int smem = 2 * D * 256 + 6 * D * 128 + 2 * 16384 + 1024 + 128;  // K, V, three Q/dO stages, P, dS, stats
      if (D == 128) {
        static bool set = false;
        if (!set) { if ((rc = set_smem(attn_bwd_dkv_kernel<128>, smem))) return rc; set = true; }
        attn_bwd_dkv_kernel<128><<<grid, kAttnBwdThreads, smem, st>>>(tmQ64, tmK128, tmV128, tmdO64, p);
      } else {
        static bool set = false;
        if (!set) { if ((rc = set_smem(attn_bwd_dkv_kernel<64>, smem))) return rc; set = true; }
        attn_bwd_dkv_kernel<64><<<grid, kAttnBwdThreads, smem, st>>>(tmQ64, tmK128, tmV128, tmdO64, p);
      }
    }
    MLB_CHECK_LAUNCH();
  }
  return 0;
}
