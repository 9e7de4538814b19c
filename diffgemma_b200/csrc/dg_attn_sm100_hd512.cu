// Denoise-step canvas attention for head_dim 512 (the reference's full-attention layers:
// src/shaders/attn/cpu.rs:16-28, ARCHITECTURE.md:106-118 of the reference project) on sm_100a.
//
// An fp32 O accumulator of 128 query rows x 512 columns is the whole tensor memory of an SM
// (512 columns), so it cannot live beside S.  The output columns are therefore split over TWO
// CTAs (blockIdx.z = 0 / 1): both compute the same S = Q K^T over the full 512-wide contraction
// and the same softmax, each accumulates O[:, 256 z : 256 z + 256] = P V[:, that half].  The score
// work is done twice (3 units of MMA work for 2 useful); what that buys is a tensor-core path at all.
//
// Per CTA: 128 GQA-stacked query rows x one key split x one half of the value columns.
//   * Q arrives already normed + roped (the stand-alone stage-1 kernel writes it to a staging
//     buffer: full layers use partial proportional RoPE).  Its first 256 elements per row go to
//     TENSOR memory (columns [128, 256): the A operand of the first half of the contraction is read
//     from there, which costs no shared-memory bandwidth), the other 256 into the UMMA K-major
//     128B-swizzled layout in shared memory (4 atoms of 128 rows x 128 B = 64 KB).
//   * key tiles of 64 keys: K 64 x 512 (8 atoms of 64 rows x 128 B = 64 KB) in TWO stages, V 64 x 256
//     (4 atoms, 32 KB) in one; TMA 3-D boxes {64 d, 64 keys}: 224 KB of the 227 KB.
//   * S = 32 x tcgen05.mma M128 N64 K16 (16 with A from tensor memory, 16 with A from shared memory),
//     two S buffers of 64 TMEM columns; P (bf16) overwrites the first 32 columns of its S buffer;
//     O += P V = 4 x tcgen05.mma M128 N256 K16 (A = P from TMEM, B = V MN-major); O in TMEM columns
//     [256, 512).
//   * 8 softmax warps, two threads per query row (32 score columns each), lazy rescale, packed
//     fp32x2 arithmetic; warps 8 / 9 load K / V, one thread of warp 10 issues the MMAs.
//   * key splits meet in the global workspace; the last CTA to arrive at the (query tile, half)
//     counter merges.  Every wait is bounded.
#include <cuda.h>

#include "dg_attn_sm100_common.cuh"
#include "dg_kernels.h"

namespace dg {

using namespace sm100;

namespace h5 {
constexpr uint32_t HDQ = 512;                 // contraction width of S
constexpr uint32_t HDV = 256;                 // value columns per CTA
constexpr uint32_t TN = 64;                   // keys per tile
constexpr uint32_t NTR = 2;                   // threads per query row
constexpr uint32_t SM_WARPS = 4 * NTR;
constexpr uint32_t W_K = SM_WARPS, W_V = SM_WARPS + 1, W_MMA = SM_WARPS + 2;
constexpr uint32_t THREADS = (SM_WARPS + 3) * 32;   // 352
constexpr uint32_t CPT = TN / NTR;            // 32 score columns per thread
constexpr uint32_t OPT = HDV / NTR;           // 128 output columns per thread
constexpr uint32_t Q_ATOM = 128 * 128;        // 128 rows x 128 B
constexpr uint32_t KV_ATOM = 64 * 128;        // 64 rows x 128 B
constexpr uint32_t K_STAGE = 8 * KV_ATOM;             // 64 KB
constexpr uint32_t O_Q = 0;                           // Q[:, 256:512]: 4 atoms = 64 KB
constexpr uint32_t O_K = 4 * Q_ATOM;                  // two K stages = 128 KB
constexpr uint32_t O_V = O_K + 2 * K_STAGE;           // + 32 KB
constexpr uint32_t O_BAR = O_V + 4 * KV_ATOM;         // = 224 KB
constexpr uint32_t O_XCH = O_BAR + 256;               // [2 tile parities][BM][NTR] floats = 2 KB
constexpr uint32_t O_END = O_XCH + 2 * BM * NTR * 4;
constexpr uint32_t SMEM_REQ = 232448;                 // all of the 227 KB a CTA may have
static_assert(O_END <= SMEM_REQ, "shared-memory map does not fit");
constexpr uint32_t T_S = 0, T_Q = 128, T_O = 256;     // TMEM columns: S buffers at 0 and 64, Q[:, 0:256] at 128, O at 256
enum : uint32_t { B_Q = 0, B_K_FULL = 1 /* +stage */, B_V_FULL = 3, B_V_EMPTY = 4 /* +tile&1 */, B_S_FULL = 6 /* +buffer */,
                  B_P_FULL = 8 /* +buffer */, B_O_FINAL = 10, B_COUNT = 11 };

__host__ __device__ inline TileSched tile_sched64(const MaskParams& mk, uint32_t row_first, uint32_t row_last) {
  TileSched t{0, 0, 0, 0};
  const uint32_t lo = mask_row_lo(mk, row_first);
  if (mk.pre_hi > lo) {
    t.a0 = lo / TN;
    t.nA = (mk.pre_hi + TN - 1) / TN - t.a0;
  }
  const uint32_t can_hi = mask_can_hi_rows(mk, row_last);
  if (can_hi > mk.kv_len) {
    const uint32_t b0 = mk.kv_len / TN, b1 = (can_hi + TN - 1) / TN;
    if (t.nA > 0 && b0 < t.a0 + t.nA) {
      const uint32_t a1 = (t.a0 + t.nA) > b1 ? (t.a0 + t.nA) : b1;
      t.nA = a1 - t.a0;
    } else {
      t.b0 = b0;
      t.nB = b1 - b0;
    }
  }
  return t;
}
}  // namespace h5

__device__ __forceinline__ void row_pair_sync(uint32_t smw) {
  asm volatile("bar.sync %0, %1;" ::"r"(smw + 1u), "n"(h5::NTR * 32) : "memory");
}

__global__ void __launch_bounds__(h5::THREADS, 1)
dg_attn_sm100_hd512_kernel(const AttnParams p, const __grid_constant__ CUtensorMap tm_k,
                           const __grid_constant__ CUtensorMap tm_v) {
  using namespace h5;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // the map above needs a 1024-byte aligned base and leaves 768 bytes of slack for it
  if (smem_base - smem_u32(smem_raw) + O_END > SMEM_REQ) {
    if (tid == 0) dev_status_set(p.status, DG_DEV_SMEM_LAYOUT, KID_SM100, blockIdx.x, smem_base - smem_u32(smem_raw));
    return;
  }
  const uint32_t sQ = smem_base + O_Q, sK = smem_base + O_K, sV = smem_base + O_V;
  const uint32_t bar_base = smem_base + O_BAR;
  volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + O_BAR + B_COUNT * 8);
  float* xch_max = reinterpret_cast<float*>(smem + O_XCH);   // [2][BM][NTR]

  const uint32_t tiles_per_head = (p.C * p.G + BM - 1) / BM;
  const uint32_t kvh = blockIdx.x / tiles_per_head;
  const uint32_t mt = blockIdx.x % tiles_per_head;
  const uint32_t split = blockIdx.y;
  const uint32_t dh = blockIdx.z;                  // which half of the value columns
  const uint32_t rows_per_head = p.C * p.G;
  const uint32_t rows_total = p.C * p.Hq;
  const MaskParams mk = p.mask;

  const uint32_t row_first = (mt * BM) / p.G;
  const uint32_t row_last = ((mt + 1u) * BM - 1u) / p.G;
  const TileSched ts = tile_sched64(mk, row_first < p.C ? row_first : p.C - 1, row_last < p.C ? row_last : p.C - 1);
  const uint32_t n_tiles = ts.nA + ts.nB;
  const uint32_t v_begin = uint32_t((uint64_t(split) * n_tiles) / p.n_splits);
  const uint32_t v_end = uint32_t((uint64_t(split + 1) * n_tiles) / p.n_splits);
  const uint32_t n_local = v_end - v_begin;

  // ------------------------------------------------------------------ set-up
  if (tid == 0) {
    mbar_init(bar_addr(bar_base, B_Q), SM_WARPS);
    mbar_init(bar_addr(bar_base, B_V_FULL), 1);
    for (uint32_t s = 0; s < 2; ++s) {
      mbar_init(bar_addr(bar_base, B_K_FULL + s), 1);
      mbar_init(bar_addr(bar_base, B_V_EMPTY + s), 1);
      mbar_init(bar_addr(bar_base, B_S_FULL + s), 1);
      mbar_init(bar_addr(bar_base, B_P_FULL + s), SM_WARPS);
    }
    mbar_init(bar_addr(bar_base, B_O_FINAL), 1);
    ctl[1] = 0u;
    ctl[2] = 0u;
    fence_mbar_init();
  }
  if (warp == W_MMA) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(&ctl[0])), TMEM_COLS);
    tmem_relinquish();
  }
  if ((warp == W_K || warp == W_V) && lane == 0) tma_prefetch_desc(warp == W_K ? &tm_k : &tm_v);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl[0];
  // everything this kernel reads was written by kernels launched before it on the stream
  asm volatile("griddepcontrol.wait;" ::: "memory");
  volatile uint32_t* abort_flag = &ctl[1];

  const uint32_t smw = warp & 3u, half = (warp >> 2) & 1u;
  const uint32_t r = smw * 32 + lane;
  float m_used = -INFINITY, l_run = 0.f;

  if (warp < SM_WARPS) {
    // ---------------------------------------------------------------- Q tile: copy (two threads per row)
    {
      const uint32_t R = mt * BM + r;
      const bool valid = R < rows_per_head;
      const uint32_t i = valid ? R / p.G : 0u;
      const uint32_t h = kvh * p.G + (valid ? R % p.G : 0u);
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t(i) * p.Hq + h) * HDQ);
      if (half == 0) {
        // elements [0, 256) of the row -> tensor memory: 16-byte chunk c = columns [4c, 4c + 4) of lane r,
        // so that the 16 elements of contraction step kk sit in columns [8 kk, 8 kk + 8) (the layout P uses)
        const uint32_t t_row = tmem + ((smw * 32u) << 16) + T_Q;
#pragma unroll 1
        for (uint32_t g8 = 0; g8 < 4; ++g8) {
          uint32_t w[32];
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j) {
            const uint4 v4 = valid ? src[g8 * 8 + j] : make_uint4(0u, 0u, 0u, 0u);
            w[4 * j] = v4.x; w[4 * j + 1] = v4.y; w[4 * j + 2] = v4.z; w[4 * j + 3] = v4.w;
          }
          tmem_st32(t_row + g8 * 32u, w);
        }
        tmem_wait_st();
        tc_fence_before();
      } else {
        // elements [256, 512) -> shared memory, K-major 128-byte-swizzled: atom = 64-element column block,
        // 16-byte chunk index XOR (row & 7)
#pragma unroll 4
        for (uint32_t j = 0; j < 32; ++j) {
          const uint4 v4 = valid ? src[32 + j] : make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(smem + O_Q + (j >> 3) * Q_ATOM + r * 128u + (((j & 7u) ^ (r & 7u)) << 4)) = v4;
        }
        fence_proxy_async_smem();
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_addr(bar_base, B_Q));

    // ---------------------------------------------------------------- softmax main loop
    const uint32_t R = mt * BM + r;
    const uint32_t i_row = (R < rows_per_head) ? R / p.G : p.C - 1;
    const RowVis rv = mask_row(mk, i_row);
    const uint32_t t_lane = tmem + ((smw * 32u) << 16);
    const float sc = p.scale_log2;

    for (uint32_t n = 0; n < n_local; ++n) {
      const uint32_t v = v_begin + n;
      const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
      const uint32_t k0 = jt * TN;
      const uint32_t b = n & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, B_S_FULL + b), (n >> 1) & 1u, abort_flag))) break;
      tc_fence_after();
      uint32_t sraw[32];
      tmem_ld32(t_lane + T_S + b * TN + half * CPT, sraw);
      tmem_wait_ld();
      if (!mask_range_full(mk, rv, k0, TN)) {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (!mask_visible_row(mk, rv, k0 + half * CPT + e)) sraw[e] = 0xff800000u;  // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 32; e += 2)
        mx4[(e >> 1) & 3] = max3_f32(mx4[(e >> 1) & 3], __uint_as_float(sraw[e]), __uint_as_float(sraw[e + 1]));
      const float mx_part = max3_f32(max3_f32(mx4[0], mx4[1], mx4[2]), mx4[3], -INFINITY);
      // the two threads of a row agree on the row maximum through shared memory; after this barrier
      // both have their S columns in registers, so P may overwrite any S column
      xch_max[(b * BM + r) * NTR + half] = mx_part;
      row_pair_sync(smw);
      const float mx = fmaxf(mx_part, xch_max[(b * BM + r) * NTR + (half ^ 1u)]);
      const float m_new = mx * sc;
      const bool first = (n == 0);
      const bool need = first || (m_new > m_used + RESCALE_THRESHOLD);
      if (!first && __any_sync(0xffffffffu, need)) {
        // PV(n - 1) must be complete before O is touched
        if (!__all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, B_V_EMPTY + ((n - 1) & 1u)), ((n - 1) >> 1) & 1u, abort_flag))) break;
        tc_fence_after();
        const float alpha = need ? fast_exp2(m_used - m_new) : 1.0f;
#pragma unroll 1
        for (uint32_t c = 0; c < OPT / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(t_lane + T_O + half * OPT + c * 32u, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(t_lane + T_O + half * OPT + c * 32u, o);
        }
        tmem_wait_st();
        l_run *= alpha;
      }
      if (need) m_used = m_new;
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      const float neg_m = -m_eff;
      const uint64_t sc2 = pack_f32x2(sc, sc), nm2 = pack_f32x2(neg_m, neg_m);
      uint64_t ls2[2] = {0ull, 0ull};
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        float x0, x1;
        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[e]), __uint_as_float(sraw[e + 1])), sc2, nm2), x0, x1);
        const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
        ls2[(e >> 1) & 1] = add_f32x2(ls2[(e >> 1) & 1], pack_f32x2(p0, p1));
        pk[e >> 1] = pack_bf16x2(p0, p1);
      }
      {
        float s0, s1;
        unpack_f32x2(add_f32x2(ls2[0], ls2[1]), s0, s1);
        l_run += s0 + s1;
      }
      // P column j = keys (2j, 2j+1): this thread's 32 keys are 16 columns
      tmem_st16(t_lane + T_S + b * TN + half * (CPT / 2), pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_addr(bar_base, B_P_FULL + b));
    }
  } else if (warp == W_K) {
    // ---------------------------------------------------------------- K loader: 8 boxes {64 d, 64 keys}
    if (lane == 0) {
      for (uint32_t n = 0; n < n_local; ++n) {
        const uint32_t v = v_begin + n;
        const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
        // K stage n & 1 is free once QK(n - 2) has completed
        const uint32_t st = n & 1u;
        if (n > 1 && !mbar_wait(bar_addr(bar_base, B_S_FULL + st), ((n - 2) >> 1) & 1u, abort_flag)) break;
        const uint32_t full = bar_addr(bar_base, B_K_FULL + st);
        mbar_expect_tx(full, K_STAGE);
#pragma unroll
        for (uint32_t a = 0; a < 8; ++a)
          tma_load_3d(sK + st * K_STAGE + a * KV_ATOM, &tm_k, full, int32_t(a * 64), int32_t((jt * TN - p.pos_base) & p.ring_mask),
                      int32_t(kvh));
      }
    }
  } else if (warp == W_V) {
    // ---------------------------------------------------------------- V loader: this half's 4 boxes
    if (lane == 0) {
      for (uint32_t n = 0; n < n_local; ++n) {
        const uint32_t v = v_begin + n;
        const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
        if (n > 0 && !mbar_wait(bar_addr(bar_base, B_V_EMPTY + ((n - 1) & 1u)), ((n - 1) >> 1) & 1u, abort_flag)) break;
        const uint32_t full = bar_addr(bar_base, B_V_FULL);
        mbar_expect_tx(full, 4 * KV_ATOM);
#pragma unroll
        for (uint32_t a = 0; a < 4; ++a)
          tma_load_3d(sV + a * KV_ATOM, &tm_v, full, int32_t(dh * HDV + a * 64), int32_t((jt * TN - p.pos_base) & p.ring_mask),
                      int32_t(kvh));
      }
    }
  } else {
    // ---------------------------------------------------------------- MMA issuer (one thread)
    if (lane == 0 && n_local > 0) {
      constexpr uint32_t IDESC_QK = umma_idesc_bf16(BM, TN, 0, 0);    // A, B K-major
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(BM, HDV, 0, 1);   // B (= V) MN-major
      constexpr uint32_t HI = (1024u >> 4) | (1u << 14) | (2u << 29); // SBO 1024, version 1, 128B swizzle
      const uint32_t q_lo = ((sQ >> 4) & 0x3FFFu) | ((16u >> 4) << 16);
      const uint32_t k_lo = ((sK >> 4) & 0x3FFFu) | ((16u >> 4) << 16);
      const uint32_t v_lo = ((sV >> 4) & 0x3FFFu) | ((KV_ATOM >> 4) << 16);   // LBO = 64-column chunk stride
      auto mkdesc = [](uint32_t lo, uint32_t hi) { return (uint64_t(hi) << 32) | uint64_t(lo); };
      bool ok = mbar_wait(bar_addr(bar_base, B_Q), 0u, abort_flag);
      auto issue_qk = [&](uint32_t n) -> bool {
        const uint32_t st = n & 1u;
        if (!mbar_wait(bar_addr(bar_base, B_K_FULL + st), (n >> 1) & 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t d_tmem = tmem + T_S + (n & 1u) * TN;
        uint32_t kb = k_lo + st * (K_STAGE >> 4);
        // contraction steps 0-15: Q[:, 0:256] from tensor memory
        uint32_t qt = tmem + T_Q;
#pragma unroll 1
        for (uint32_t a = 0; a < 4; ++a) {
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk)
            umma_ts(d_tmem, qt + kk * 8u, mkdesc(kb + kk * 2u, HI), IDESC_QK, (a | kk) != 0u);
          qt += 32u;
          kb += KV_ATOM >> 4;
        }
        // contraction steps 16-31: Q[:, 256:512] from shared memory
        uint32_t qa = q_lo;
#pragma unroll 1
        for (uint32_t a = 0; a < 4; ++a) {
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk)
            umma_ss(d_tmem, mkdesc(qa + kk * 2u, HI), mkdesc(kb + kk * 2u, HI), IDESC_QK, 1u);
          qa += Q_ATOM >> 4;
          kb += KV_ATOM >> 4;
        }
        umma_commit(bar_addr(bar_base, B_S_FULL + (n & 1u)));   // S ready; this K stage is free
        return true;
      };
      ok = ok && issue_qk(0);
      for (uint32_t n = 0; ok && n < n_local; ++n) {
        if (n + 1 < n_local) {
          ok = issue_qk(n + 1);
          if (!ok) break;
        }
        if (!mbar_wait(bar_addr(bar_base, B_P_FULL + (n & 1u)), (n >> 1) & 1u, abort_flag)) break;
        if (!mbar_wait(bar_addr(bar_base, B_V_FULL), n & 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t p_tmem = tmem + T_S + (n & 1u) * TN;
#pragma unroll
        for (uint32_t ks = 0; ks < TN / 16; ++ks)
          umma_ts(tmem + T_O, p_tmem + ks * 8u, mkdesc(v_lo + ks * (2048u >> 4), HI), IDESC_PV, (n | ks) != 0u);
        umma_commit(bar_addr(bar_base, B_V_EMPTY + (n & 1u)));  // PV done; the V tile is free
        if (n + 1 == n_local) umma_commit(bar_addr(bar_base, B_O_FINAL));
      }
    }
  }

  // ------------------------------------------------------------------ epilogue (softmax warps)
  if (warp < SM_WARPS) {
    bool have_o = __all_sync(0xffffffffu, n_local > 0 && !*abort_flag);
    if (have_o) {
      have_o = __all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, B_O_FINAL), 0u, abort_flag));
      tc_fence_after();
    }
    const uint32_t R = mt * BM + r;
    const bool valid = R < rows_per_head;
    const uint32_t i_row = valid ? R / p.G : 0u;
    const uint32_t h = kvh * p.G + (valid ? R % p.G : 0u);
    const size_t orow = size_t(i_row) * p.Hq + h;
    const uint32_t t_lane = tmem + ((smw * 32u) << 16);
    // the row's denominator is the sum of its two threads' partial sums (slot of parity 0 is free now)
    __syncwarp();
    row_pair_sync(smw);
    xch_max[r * NTR + half] = l_run;
    row_pair_sync(smw);
    const float l_tot = xch_max[r * NTR] + xch_max[r * NTR + 1];
    const bool direct = (p.n_splits == 1);
    const bool to_bf16 = direct && p.out != nullptr;
    const float inv_l = l_tot > 0.f ? 1.0f / l_tot : 0.f;
    const float mul = to_bf16 ? inv_l : 1.0f;
    float* dst_o = direct ? p.out_o : p.ws_o + size_t(split) * rows_total * HDQ;
    // 32 x 32 chunks go through a padded per-warp tile in shared memory (the Q tile is dead) so that
    // every store instruction of the warp writes whole 128-byte lines
    float* tile = reinterpret_cast<float*>(smem + O_Q) + warp * (32 * 36);
    size_t orow_k[8];
    bool valid_k[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t Rk = mt * BM + smw * 32 + k * 4 + (lane >> 3);
      valid_k[k] = Rk < rows_per_head;
      const uint32_t Rc = valid_k[k] ? Rk : 0u;
      orow_k[k] = size_t(Rc / p.G) * p.Hq + kvh * p.G + Rc % p.G;
    }
#pragma unroll 1
    for (uint32_t c = 0; c < OPT / 32; ++c) {
      const uint32_t col0 = half * OPT + c * 32u;
      uint32_t o[32];
      if (have_o) {
        tmem_ld32(t_lane + T_O + col0, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = 0u;
      }
#pragma unroll
      for (int q4 = 0; q4 < 8; ++q4)
        *reinterpret_cast<float4*>(tile + lane * 36 + q4 * 4) =
            make_float4(__uint_as_float(o[q4 * 4]) * mul, __uint_as_float(o[q4 * 4 + 1]) * mul,
                        __uint_as_float(o[q4 * 4 + 2]) * mul, __uint_as_float(o[q4 * 4 + 3]) * mul);
      __syncwarp();
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 v4 = *reinterpret_cast<const float4*>(tile + (k * 4 + (lane >> 3)) * 36 + (lane & 7) * 4);
        if (!valid_k[k]) continue;
        const size_t off = orow_k[k] * HDQ + dh * HDV + col0 + (lane & 7) * 4;
        if (to_bf16) {
          uint2 w2;
          w2.x = pack_bf16x2(v4.x, v4.y);
          w2.y = pack_bf16x2(v4.z, v4.w);
          *reinterpret_cast<uint2*>(p.out + off) = w2;
        } else {
          *reinterpret_cast<float4*>(dst_o + off) = v4;
        }
      }
      __syncwarp();
    }
    if (valid && !to_bf16 && half == 0) {
      if (direct) {
        if (dh == 0) {   // both halves hold the same (m, l)
          p.out_m[orow] = m_used * 0.6931471805599453f;
          p.out_l[orow] = l_tot;
        }
      } else {
        float2* ml = reinterpret_cast<float2*>(p.ws_ml) + (size_t(split) * 2 + dh) * rows_total + orow;
        *ml = make_float2(m_used, l_tot);
      }
    }
    if (!direct) __threadfence();
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    if (tid == 0) dev_status_set(p.status, DG_DEV_WAIT_TIMEOUT, KID_SM100, blockIdx.x + gridDim.x * blockIdx.y, n_local);
    if (warp == W_K && lane == 0 && n_local > 0) {
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000ll) {}   // ~1 ms: far longer than any tile load in flight
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == W_MMA) tmem_dealloc(tmem, TMEM_COLS);

  // ------------------------------------------------------------------ split merge by the last CTA to arrive
  if (p.n_splits > 1) {
    const uint32_t S = p.n_splits;
    uint32_t* counter = p.ws_counters + blockIdx.x * 2 + dh;
    if (tid == 0) {
      __threadfence();
      const uint32_t old = atomicAdd(counter, 1u);
      ctl[2] = (old == S - 1u) ? 1u : 0u;
    }
    __syncthreads();
    if (ctl[2]) {
      __threadfence();
      const float2* ml_all = reinterpret_cast<const float2*>(p.ws_ml);
      for (uint32_t rr = warp; rr < BM; rr += THREADS / 32) {
        const uint32_t R = mt * BM + rr;
        if (R >= rows_per_head) break;
        const size_t orow = size_t(R / p.G) * p.Hq + kvh * p.G + R % p.G;
        float2 ml = make_float2(-INFINITY, 0.f);
        if (lane < S) ml = ml_all[(size_t(lane) * 2 + dh) * rows_total + orow];
        float mg = ml.x;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, o));
        const float w_mine = (ml.x == -INFINITY) ? 0.f : fast_exp2(ml.x - mg);
        float lg = w_mine * ml.y;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lg += __shfl_xor_sync(0xffffffffu, lg, o);
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (uint32_t s = 0; s < S; ++s) {
          const float w = __shfl_sync(0xffffffffu, w_mine, int(s));
          const float4* src = reinterpret_cast<const float4*>(p.ws_o + (size_t(s) * rows_total + orow) * HDQ + dh * HDV + lane * 8);
          const float4 a = src[0], bq = src[1];
          acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * a.z; acc[3] += w * a.w;
          acc[4] += w * bq.x; acc[5] += w * bq.y; acc[6] += w * bq.z; acc[7] += w * bq.w;
        }
        const size_t off = orow * HDQ + dh * HDV + lane * 8;
        if (p.out) {
          const float inv = lg > 0.f ? 1.0f / lg : 0.f;
          uint4 w4;
          w4.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
          w4.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
          w4.z = pack_bf16x2(acc[4] * inv, acc[5] * inv);
          w4.w = pack_bf16x2(acc[6] * inv, acc[7] * inv);
          *reinterpret_cast<uint4*>(p.out + off) = w4;
        } else {
          float4* dst = reinterpret_cast<float4*>(p.out_o + off);
          dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
          dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
          if (lane == 0 && dh == 0) {
            p.out_m[orow] = mg * 0.6931471805599453f;
            p.out_l[orow] = lg;
          }
        }
      }
      if (tid == 0) *counter = 0u;   // ready for the next launch
    }
  }
}

cudaError_t sm100_hd512_configure() {
  return cudaFuncSetAttribute(dg_attn_sm100_hd512_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(h5::SMEM_REQ));
}

uint32_t sm100_hd512_key_tiles(const MaskParams& mk) {
  const TileSched t = h5::tile_sched64(mk, 0, kMaxCanvas - 1);
  return t.nA + t.nB;
}

// tm_k, tm_v: 3-D tensor maps {512, cap, Hkv} with boxes {64 d, 64 keys, 1}
cudaError_t launch_attn_sm100_hd512(const AttnParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                                    cudaStream_t st) {
  const dim3 grid(sm100_query_tiles(p.C, p.G, p.Hkv), p.n_splits, 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(h5::THREADS);
  cfg.dynamicSmemBytes = h5::SMEM_REQ;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, dg_attn_sm100_hd512_kernel, p, tm_k, tm_v);
}

}  // namespace dg
