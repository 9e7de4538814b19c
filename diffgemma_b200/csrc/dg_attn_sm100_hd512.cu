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

#include "dg_attn_sm100_hd512.cuh"
#include "dg_kernels.h"

namespace dg {

namespace h5 {
constexpr uint32_t NTR = 2;                   // threads per query row
constexpr uint32_t SM_WARPS = 4 * NTR;
constexpr uint32_t W_K = SM_WARPS, W_V = SM_WARPS + 1, W_MMA = SM_WARPS + 2;
constexpr uint32_t THREADS = (SM_WARPS + 3) * 32;   // 352
constexpr uint32_t CPT = TN / NTR;            // 32 score columns per thread
constexpr uint32_t K_STAGE = 8 * KV_ATOM;             // 64 KB
constexpr uint32_t O_Q = 0;                           // Q[:, 256:512]: 4 atoms = 64 KB
constexpr uint32_t O_K = 4 * Q_ATOM;                  // two K stages = 128 KB
constexpr uint32_t O_V = O_K + 2 * K_STAGE;           // + 32 KB
constexpr uint32_t O_BAR = O_V + 4 * KV_ATOM;         // = 224 KB
constexpr uint32_t O_XCH = O_BAR + 256;               // [2 tile parities][BM][NTR] floats = 2 KB
constexpr uint32_t O_END = O_XCH + 2 * BM * NTR * 4;
static_assert(O_END <= SMEM_REQ, "shared-memory map does not fit");
enum : uint32_t { B_Q = 0, B_K_FULL = 1 /* +stage */, B_V_FULL = 3, B_V_EMPTY = 4 /* +tile&1 */, B_S_FULL = 6 /* +buffer */,
                  B_P_FULL = 8 /* +buffer */, B_O_FINAL = 10, B_COUNT = 11 };
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
    copy_q_tile(p, smem + O_Q, tmem, kvh, mt, smw, lane, half);
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
    // the row's denominator is the sum of its two threads' partial sums (slot of parity 0 is free now)
    __syncwarp();
    row_pair_sync(smw);
    xch_max[r * NTR + half] = l_run;
    row_pair_sync(smw);
    const float l_tot = xch_max[r * NTR] + xch_max[r * NTR + 1];
    // the Q tile is dead: its shared memory stages the stores
    store_o_half(p, smem + O_Q, tmem, kvh, mt, split, dh, smw, lane, half, have_o, m_used, l_tot);
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
  if (p.n_splits > 1) merge_splits_last(p, &ctl[2], kvh, mt, dh, THREADS);
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
