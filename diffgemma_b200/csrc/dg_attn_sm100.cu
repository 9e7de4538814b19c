// Denoise-step canvas attention for head_dim 256 on sm_100a: one fused flash-style kernel.
//
//   * Q prologue in the kernel: per-head RMSNorm(+weight) + split-half RoPE on the CTA's 128
//     query rows, rounded to bf16 and written straight into the UMMA shared-memory layout.
//   * K/V tiles of 128 keys are TMA-staged (3-D tiled loads, 128-byte swizzle, no multicast) from
//     the head-major bf16 cache K[Hkv][cap][256], V[Hkv][cap][256].
//   * S = Q K^T and O += P V run on tcgen05.mma with fp32 accumulators in tensor memory:
//     TMEM columns [0,128) and [128,256) double-buffer S, [256,512) hold O; P (bf16) overwrites
//     the first 64 columns of its S buffer and is consumed from TMEM as the A operand.
//   * online softmax in registers, two threads per query row (64 key columns each, so that every
//     scheduler has two softmax warps to hide instruction latency), with lazy rescaling of O (only
//     when the running maximum grows by more than 2^8).
//   * intra-GPU split-KV: grid.y CTAs share one query tile.  For 2, 4 or 8 splits they form a
//     thread-block cluster: each keeps its (O, m, l) partial in shared memory and, after a cluster
//     barrier, merges its share of the rows by reading the peers' partials through distributed
//     shared memory.  Other split counts write partials to a global workspace and the last CTA to
//     finish merges them.  Either way there is no second launch.
//
// Query rows are the GQA-stacked rows of one KV head: stacked row R -> canvas row R / G, query
// head kvh*G + R % G, so all 128 rows of a CTA reuse the same K/V tiles.
//
// Semantics restated from the reference (paths relative to the reference project):
//   src/shaders/attn/attention/attention.metal:22-133 (denoise mask, online softmax),
//   src/shaders/attn/attention/attention_mma2.metal:53-307 (tiled variant, p = 0 for masked keys,
//   fully masked row -> 0), src/shaders/include/attention_device.metal:154-165 ((m, l, O) state).
#include <cuda.h>

#include "dg_attn_sm100_common.cuh"
#include "dg_kernels.h"

namespace dg {

using namespace sm100;

// Single-CTA kernel: four softmax warpgroups.  Warps w, w+4, w+8, w+12 share the 32 query rows of
// TMEM quadrant w & 3; warpgroup q = w >> 2 handles key columns [32 q, 32 q + 32) of every tile, so
// each scheduler has four softmax warps in flight to hide TMEM, MUFU and barrier latency.
namespace one {
constexpr uint32_t NTR = 4;                       // threads per query row
constexpr uint32_t SM_WARPS = 4 * NTR;            // 16 softmax warps
constexpr uint32_t W_K = SM_WARPS, W_V = SM_WARPS + 1, W_MMA = SM_WARPS + 2;
constexpr uint32_t THREADS = (SM_WARPS + 3) * 32;   // 608
constexpr uint32_t CPT = BN / NTR;                // 32 key columns per thread
constexpr uint32_t OPT = HD / NTR;                // 64 output columns per thread
}  // namespace one

// named barrier of the NTR warps that own the same 32 query rows
__device__ __forceinline__ void row_group_sync(uint32_t smw) {
  asm volatile("bar.sync %0, %1;" ::"r"(smw + 1u), "n"(one::NTR * 32) : "memory");
}

__global__ void __launch_bounds__(one::THREADS, 1)
dg_attn_sm100_kernel(const AttnParams p, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v) {
  using namespace one;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + OFF_Q, sK = smem_base + OFF_K, sV = smem_base + OFF_V;
  const uint32_t bar_base = smem_base + OFF_BAR;
  volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + OFF_BAR + N_BARS * 8);
  // ctl[0] = TMEM base address, ctl[1] = abort flag, ctl[2] = "this CTA merges" flag
  float* xch_max = reinterpret_cast<float*>(smem + OFF_XCH);   // [2 tile parities][BM][NTR]
  float* xch_misc = xch_max + 2 * BM * NTR;                     // [BM][NTR]: prologue sums of squares
  float* xch_l = xch_misc + BM * NTR;                           // [BM][NTR]: final softmax denominators

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t tiles_per_head = (p.C * p.G + BM - 1) / BM;
  const uint32_t kvh = blockIdx.x / tiles_per_head;
  const uint32_t mt = blockIdx.x % tiles_per_head;
  const uint32_t split = blockIdx.y;
  const uint32_t rows_per_head = p.C * p.G;
  const MaskParams mk = p.mask;

  const uint32_t row_first = (mt * BM) / p.G;
  const TileSched ts = tile_sched(mk, row_first < p.C ? row_first : p.C - 1);
  const uint32_t n_tiles = ts.nA + ts.nB;
  const uint32_t v_begin = uint32_t((uint64_t(split) * n_tiles) / p.n_splits);
  const uint32_t v_end = uint32_t((uint64_t(split + 1) * n_tiles) / p.n_splits);
  const uint32_t n_local = v_end - v_begin;

  stamp(p, 0);
  // ------------------------------------------------------------------ set-up
  if (tid == 0) {
    mbar_init(bar_addr(bar_base, BAR_Q), SM_WARPS);          // one arrival per softmax warp
    mbar_init(bar_addr(bar_base, BAR_K_FULL), 1);
    mbar_init(bar_addr(bar_base, BAR_K_EMPTY), 1);
    mbar_init(bar_addr(bar_base, BAR_V_FULL), 1);
    mbar_init(bar_addr(bar_base, BAR_V_EMPTY), 1);
    mbar_init(bar_addr(bar_base, BAR_S_FULL0), 1);
    mbar_init(bar_addr(bar_base, BAR_S_FULL0 + 1), 1);
    mbar_init(bar_addr(bar_base, BAR_P_FULL0), SM_WARPS);
    mbar_init(bar_addr(bar_base, BAR_P_FULL0 + 1), SM_WARPS);
    mbar_init(bar_addr(bar_base, BAR_PV_DONE), 1);
    mbar_init(bar_addr(bar_base, BAR_O_FINAL), 1);
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
  // Programmatic dependent launch: everything above overlapped the tail of the preceding kernel
  // on the stream (the canvas K/V append, which also writes the RoPE table); its results are
  // needed from here on.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  stamp(p, 1);
  volatile uint32_t* abort_flag = &ctl[1];

  // softmax-thread geometry: TMEM quadrant smw, row r of the query tile, column quarter qd
  const uint32_t smw = warp & 3u, qd = (warp >> 2) & (NTR - 1u);
  const uint32_t r = smw * 32 + lane;
  // per-row softmax state (identical in every thread of a row, except l_run which is per quarter)
  float m_used = -INFINITY, l_run = 0.f;

  if (warp < SM_WARPS) {
    // ---------------------------------------------------------------- Q prologue (four threads per row)
    // Thread (row, qd) owns the RoPE pairs (d, d+128) with d in [32 qd, 32 qd + 32): four 16-byte
    // chunks from each half of the row.  No shuffles; the partial sums of squares meet through
    // shared memory.
    {
      constexpr int NJ = 16 / NTR;
      const uint32_t R = mt * BM + r;
      const bool valid = R < rows_per_head;
      const uint32_t i = valid ? R / p.G : 0u;
      const uint32_t h = kvh * p.G + (valid ? R % p.G : 0u);
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t(i) * p.Hq + h) * HD);
      const bool do_norm = !p.q_prenormed;
      uint4 lo[NJ], hi[NJ];
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        lo[j] = src[qd * NJ + j];
        hi[j] = src[16 + qd * NJ + j];
      }
      if (!valid) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) lo[j] = hi[j] = make_uint4(0u, 0u, 0u, 0u);
      }
      // RoPE-table entries of this thread's pairs: issued now so that they arrive while the sums of
      // squares are reduced
      float4 tabv[NJ * 4];
      if (do_norm) {
        const float4* tab = reinterpret_cast<const float4*>(p.rope_table + size_t(i) * 128 + qd * (8 * NJ));
#pragma unroll
        for (int t = 0; t < NJ * 4; ++t) tabv[t] = tab[t];
      }
      float inv = 1.0f;
      if (do_norm) {
        float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          const uint32_t a[4] = {lo[j].x, lo[j].y, lo[j].z, lo[j].w};
          const uint32_t b[4] = {hi[j].x, hi[j].y, hi[j].z, hi[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float a0 = __uint_as_float(a[e] << 16), a1 = __uint_as_float(a[e] & 0xffff0000u);
            const float b0 = __uint_as_float(b[e] << 16), b1 = __uint_as_float(b[e] & 0xffff0000u);
            ss0 += a0 * a0 + a1 * a1;
            ss1 += b0 * b0 + b1 * b1;
          }
        }
        xch_misc[r * NTR + qd] = ss0 + ss1;
        row_group_sync(smw);
        float ss = 0.f;
#pragma unroll
        for (uint32_t k = 0; k < NTR; ++k) ss += xch_misc[r * NTR + k];   // same order in every thread
        inv = 1.0f / sqrtf(ss / float(HD) + p.eps);
      }
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const uint32_t c_lo = qd * NJ + j, c_hi = c_lo + 16;
        uint4 out_lo = lo[j], out_hi = hi[j];
        if (do_norm) {
          uint4 wl4 = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u), wh4 = wl4;   // bf16 1.0
          if (p.qw) {
            wl4 = reinterpret_cast<const uint4*>(p.qw)[c_lo];
            wh4 = reinterpret_cast<const uint4*>(p.qw)[c_hi];
          }
          const uint32_t a[4] = {lo[j].x, lo[j].y, lo[j].z, lo[j].w};
          const uint32_t b[4] = {hi[j].x, hi[j].y, hi[j].z, hi[j].w};
          const uint32_t wa[4] = {wl4.x, wl4.y, wl4.z, wl4.w};
          const uint32_t wb[4] = {wh4.x, wh4.y, wh4.z, wh4.w};
          uint32_t ya[4], yb[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float4 cs = tabv[j * 4 + e];   // (cos, sin) of pairs 8*c_lo + 2e and + 2e + 1
            const float a0 = __uint_as_float(a[e] << 16) * (inv * __uint_as_float(wa[e] << 16));
            const float a1 = __uint_as_float(a[e] & 0xffff0000u) * (inv * __uint_as_float(wa[e] & 0xffff0000u));
            const float b0 = __uint_as_float(b[e] << 16) * (inv * __uint_as_float(wb[e] << 16));
            const float b1 = __uint_as_float(b[e] & 0xffff0000u) * (inv * __uint_as_float(wb[e] & 0xffff0000u));
            ya[e] = pack_bf16x2(a0 * cs.x - b0 * cs.y, a1 * cs.z - b1 * cs.w);
            yb[e] = pack_bf16x2(a0 * cs.y + b0 * cs.x, a1 * cs.w + b1 * cs.z);
          }
          out_lo = make_uint4(ya[0], ya[1], ya[2], ya[3]);
          out_hi = make_uint4(yb[0], yb[1], yb[2], yb[3]);
        }
        // K-major 128-byte-swizzled layout: atom = 64-element column block, 16-byte chunk index
        // XORed with (row & 7)
        *reinterpret_cast<uint4*>(smem + OFF_Q + (c_lo >> 3) * ATOM_BYTES + r * 128u + (((c_lo & 7u) ^ (r & 7u)) << 4)) = out_lo;
        *reinterpret_cast<uint4*>(smem + OFF_Q + (c_hi >> 3) * ATOM_BYTES + r * 128u + (((c_hi & 7u) ^ (r & 7u)) << 4)) = out_hi;
      }
    }
    // every lane publishes its own stores, then one lane arrives for the warp
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_addr(bar_base, BAR_Q));
    stamp(p, 2);

    // ---------------------------------------------------------------- softmax main loop
    const uint32_t R = mt * BM + r;
    const uint32_t i_row = (R < rows_per_head) ? R / p.G : p.C - 1;
    const uint32_t row_lo = mask_row_lo(mk, i_row);
    const uint32_t t_lane = tmem + ((smw * 32u) << 16);
    const bool contiguous = (mk.pre_hi == mk.kv_len) && (mk.can_hi > mk.kv_len);
    const float sc = p.scale_log2;

    for (uint32_t n = 0; n < n_local; ++n) {
      const uint32_t v = v_begin + n;
      const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
      const uint32_t k0 = jt * BN;
      const uint32_t b = n & 1u;
      // warp-uniform outcome: the TMEM instructions below need the whole warp
      if (!__all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, BAR_S_FULL0 + b), (n >> 1) & 1u, abort_flag))) break;
      tc_fence_after();
      uint32_t sraw[32];
      tmem_ld32(t_lane + TM_S + b * 128u + qd * CPT, sraw);
      tmem_wait_ld();

      const bool full = (k0 >= row_lo && k0 + BN <= mk.pre_hi) || (k0 >= mk.kv_len && k0 + BN <= mk.can_hi) ||
                        (contiguous && k0 >= row_lo && k0 + BN <= mk.can_hi);
      if (!full) {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (!mask_visible_lo(mk, row_lo, k0 + qd * CPT + e)) sraw[e] = 0xff800000u;  // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sraw[e]));
      const float mx_part = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // the threads of a row agree on the row maximum through shared memory; after this barrier
      // all of them have their S columns in registers, so P may overwrite any S column
      xch_max[(b * BM + r) * NTR + qd] = mx_part;
      row_group_sync(smw);
      float mx = mx_part;
#pragma unroll
      for (uint32_t k = 0; k < NTR; ++k) mx = fmaxf(mx, xch_max[(b * BM + r) * NTR + k]);
      const float m_new = mx * sc;   // sc > 0; -inf stays -inf
      const bool first = (n == 0);
      const bool need = first || (m_new > m_used + RESCALE_THRESHOLD);
      if (!first && __any_sync(0xffffffffu, need)) {
        // O holds sum p v relative to m_used: bring it to the new reference point (each thread of
        // the row rescales its own 64 columns of O)
        if (!__all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, BAR_PV_DONE), (n - 1) & 1u, abort_flag))) break;
        tc_fence_after();
        const float alpha = need ? fast_exp2(m_used - m_new) : 1.0f;
#pragma unroll 1
        for (uint32_t c = 0; c < OPT / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(t_lane + TM_O + qd * OPT + c * 32u, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(t_lane + TM_O + qd * OPT + c * 32u, o);
        }
        tmem_wait_st();
        l_run *= alpha;
      }
      if (need) m_used = m_new;
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      const float neg_m = -m_eff;
      float ls0 = 0.f, ls1 = 0.f;
      // P column j (32 bit) = keys (2j, 2j+1) as bf16x2: this thread's 32 keys are 16 columns
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(sraw[e]), sc, neg_m));
        const float p1 = fast_exp2(fmaf(__uint_as_float(sraw[e + 1]), sc, neg_m));
        ls0 += p0;
        ls1 += p1;
        pk[e >> 1] = pack_bf16x2(p0, p1);
      }
      l_run += ls0 + ls1;
      tmem_st16(t_lane + TM_S + b * 128u + qd * (CPT / 2), pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_addr(bar_base, BAR_P_FULL0 + b));
    }
  } else if (warp == W_K) {
    // ---------------------------------------------------------------- K loader
    if (lane == 0) {
      for (uint32_t n = 0; n < n_local; ++n) {
        const uint32_t v = v_begin + n;
        const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
        if (n > 0 && !mbar_wait(bar_addr(bar_base, BAR_K_EMPTY), (n - 1) & 1u, abort_flag)) break;
        const uint32_t full = bar_addr(bar_base, BAR_K_FULL);
        mbar_expect_tx(full, TILE_BYTES);
#pragma unroll
        for (uint32_t a = 0; a < 4; ++a)
          tma_load_3d(sK + a * ATOM_BYTES, &tm_k, full, int32_t(a * 64), int32_t(jt * BN), int32_t(kvh));
      }
    }
  } else if (warp == W_V) {
    // ---------------------------------------------------------------- V loader
    if (lane == 0) {
      for (uint32_t n = 0; n < n_local; ++n) {
        const uint32_t v = v_begin + n;
        const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
        if (n > 0 && !mbar_wait(bar_addr(bar_base, BAR_V_EMPTY), (n - 1) & 1u, abort_flag)) break;
        const uint32_t full = bar_addr(bar_base, BAR_V_FULL);
        mbar_expect_tx(full, TILE_BYTES);
#pragma unroll
        for (uint32_t a = 0; a < 4; ++a)
          tma_load_3d(sV + a * ATOM_BYTES, &tm_v, full, int32_t(a * 64), int32_t(jt * BN), int32_t(kvh));
      }
    }
  } else {
    // ---------------------------------------------------------------- MMA issuer (one thread)
    if (lane == 0 && n_local > 0) {
      constexpr uint32_t IDESC_QK = umma_idesc_bf16(BM, BN, 0, 0);   // A, B K-major
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(BM, HD, 0, 1);   // B (= V) MN-major
      bool ok = mbar_wait(bar_addr(bar_base, BAR_Q), 0u, abort_flag);
      auto issue_qk = [&](uint32_t n) -> bool {
        if (!mbar_wait(bar_addr(bar_base, BAR_K_FULL), n & 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t d_tmem = tmem + TM_S + (n & 1u) * 128u;
#pragma unroll
        for (uint32_t a = 0; a < 4; ++a)
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk) {
            const uint64_t da = umma_smem_desc(sQ + a * ATOM_BYTES + kk * 32u, 16u, 1024u);
            const uint64_t db = umma_smem_desc(sK + a * ATOM_BYTES + kk * 32u, 16u, 1024u);
            umma_ss(d_tmem, da, db, IDESC_QK, (a | kk) != 0u);
          }
        umma_commit(bar_addr(bar_base, BAR_K_EMPTY));
        umma_commit(bar_addr(bar_base, BAR_S_FULL0 + (n & 1u)));
        return true;
      };
      ok = ok && issue_qk(0);
      for (uint32_t n = 0; ok && n < n_local; ++n) {
        if (n + 1 < n_local) {
          ok = issue_qk(n + 1);
          if (!ok) break;
        }
        if (!mbar_wait(bar_addr(bar_base, BAR_P_FULL0 + (n & 1u)), (n >> 1) & 1u, abort_flag)) break;
        if (!mbar_wait(bar_addr(bar_base, BAR_V_FULL), n & 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t p_tmem = tmem + TM_S + (n & 1u) * 128u;
#pragma unroll
        for (uint32_t ks = 0; ks < 8; ++ks) {
          const uint64_t db = umma_smem_desc(sV + ks * 2048u, ATOM_BYTES, 1024u);
          umma_ts(tmem + TM_O, p_tmem + ks * 8u, db, IDESC_PV, (n | ks) != 0u);
        }
        umma_commit(bar_addr(bar_base, BAR_V_EMPTY));
        umma_commit(bar_addr(bar_base, BAR_PV_DONE));
        // The epilogue must not reuse BAR_PV_DONE: when the last S tile is ready only PV(n-3) is
        // known to be complete, so a parity wait on that barrier could alias by two phases.
        if (n + 1 == n_local) umma_commit(bar_addr(bar_base, BAR_O_FINAL));
      }
    }
  }

  stamp(p, 3);
  // ------------------------------------------------------------------ epilogue (softmax warps)
  const uint32_t rows_total = p.C * p.Hq;
  bool have_o = false;
  if (warp < SM_WARPS) {
    have_o = __all_sync(0xffffffffu, n_local > 0 && !*abort_flag);
    if (have_o) {
      have_o = __all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, BAR_O_FINAL), 0u, abort_flag));
      tc_fence_after();
    }
  }
  // Cluster merge: partial rows are pushed into the owner CTA's Q/K/V region, which must be dead
  // in EVERY CTA of the cluster first - all of this CTA's MMAs are complete once its softmax
  // warps have seen O_FINAL, and this barrier collects that from all CTAs.
  if (p.cluster_merge && p.n_splits > 1) cluster_sync_all();
  if (warp < SM_WARPS) {
    const uint32_t R = mt * BM + r;
    const bool valid = R < rows_per_head;
    const uint32_t i_row = valid ? R / p.G : 0u;
    const uint32_t h = kvh * p.G + (valid ? R % p.G : 0u);
    const size_t orow = size_t(i_row) * p.Hq + h;
    const uint32_t t_lane = tmem + ((smw * 32u) << 16);
    // the row's denominator is the sum of its threads' partial sums
    xch_l[r * NTR + qd] = l_run;
    row_group_sync(smw);
    float l_tot = 0.f;
#pragma unroll
    for (uint32_t k = 0; k < NTR; ++k) l_tot += xch_l[r * NTR + k];
    const bool direct = (p.n_splits == 1);
    const bool via_dsmem = (p.cluster_merge != 0u) && !direct;
    if (via_dsmem) {
      // The partial stays on chip.  Row r of the query tile is merged by CTA r / (BM / S) of the
      // cluster, so each thread pushes its columns of the un-normalised O row (and one thread the
      // (m, l) pair) straight into that CTA's receive buffer with remote shared-memory stores:
      // recv[source CTA][row within the owner's share][OBUF_LD floats] in the dead Q/K/V region.
      const uint32_t S = p.n_splits;
      const uint32_t rpc = BM / S;
      const uint32_t src_rank = cluster_ctarank();
      const uint32_t owner = r / rpc, rl = r % rpc;
      const uint32_t dst_row = dsmem_addr(smem_base + OFF_Q + ((src_rank * rpc + rl) * OBUF_LD) * 4u, owner);
#pragma unroll 1
      for (uint32_t c = 0; c < OPT / 32; ++c) {
        const uint32_t col0 = qd * OPT + c * 32u;
        uint32_t o[32];
        if (have_o) {
          tmem_ld32(t_lane + TM_O + col0, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0u;
        }
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4)
          dsmem_st_u4(dst_row + (col0 + q4 * 4) * 4u, make_uint4(o[q4 * 4], o[q4 * 4 + 1], o[q4 * 4 + 2], o[q4 * 4 + 3]));
      }
      if (qd == 0) dsmem_st_f2(dsmem_addr(smem_base + OFF_ML + (src_rank * rpc + rl) * 8u, owner), make_float2(m_used, l_tot));
    } else {
    const bool to_bf16 = direct && p.out != nullptr;
    const float inv_l = l_tot > 0.f ? 1.0f / l_tot : 0.f;
    const float mul = to_bf16 ? inv_l : 1.0f;
    float* dst_o = direct ? p.out_o : p.ws_o + size_t(split) * rows_total * HD;
    // Each thread owns a quarter of one row in TMEM, but rows are 1 KB apart in memory.  A 32 x 32
    // chunk goes through a padded per-warp tile in shared memory (the Q tile is dead by now) so that
    // every store instruction of the warp writes four full 128-byte lines (64-byte for bf16).
    float* tile = reinterpret_cast<float*>(smem + OFF_Q) + warp * (32 * 36);
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
      const uint32_t col0 = qd * OPT + c * 32u;
      uint32_t o[32];
      if (have_o) {
        tmem_ld32(t_lane + TM_O + col0, o);
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
        if (to_bf16) {
          uint2 w2;
          w2.x = pack_bf16x2(v4.x, v4.y);
          w2.y = pack_bf16x2(v4.z, v4.w);
          *reinterpret_cast<uint2*>(p.out + orow_k[k] * HD + col0 + (lane & 7) * 4) = w2;
        } else {
          *reinterpret_cast<float4*>(dst_o + orow_k[k] * HD + col0 + (lane & 7) * 4) = v4;
        }
      }
      __syncwarp();
    }
    if (valid && !to_bf16 && qd == 0) {
      if (direct) {
        p.out_m[orow] = m_used * 0.6931471805599453f;   // log2 units -> natural units
        p.out_l[orow] = l_tot;
      } else {
        float2* ml = reinterpret_cast<float2*>(p.ws_ml) + size_t(split) * rows_total + orow;
        *ml = make_float2(m_used, l_tot);   // log2 units inside the workspace
      }
    }
    if (!direct) __threadfence();
    }   // !via_dsmem
  }

  stamp(p, 4);
  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    // a bounded wait gave up: report, let our own TMA traffic land, then leave
    if (tid == 0) dev_status_set(p.status, DG_DEV_WAIT_TIMEOUT, KID_SM100, blockIdx.x + gridDim.x * blockIdx.y, n_local);
    if (warp == W_K && lane == 0 && n_local > 0) {
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000ll) {}   // ~1 ms: far longer than any tile load in flight
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == W_MMA) tmem_dealloc(tmem, TMEM_COLS);

  // ------------------------------------------------------------------ split merge inside the cluster
  if (p.n_splits > 1 && p.cluster_merge) {
    // The n_splits CTAs of this query tile are one thread-block cluster (cluster dims (1, S, 1)).
    // Every CTA has pushed each partial row to the CTA that owns it; after the cluster barrier CTA k
    // holds all S partials of rows [k*BM/S, (k+1)*BM/S) in its own shared memory and merges them.
    // Nothing touches remote shared memory after the barrier, so no second barrier is needed.
    const uint32_t S = p.n_splits;
    cluster_sync_all();
    const uint32_t rank = cluster_ctarank();
    const uint32_t rpc = BM / S;
    const float* recv = reinterpret_cast<const float*>(smem + OFF_Q);        // [S][rpc][OBUF_LD]
    const float2* recv_ml = reinterpret_cast<const float2*>(smem + OFF_ML);  // [S][rpc]
    for (uint32_t rl = warp; rl < rpc; rl += THREADS / 32) {
      const uint32_t rr = rank * rpc + rl;
      const uint32_t R = mt * BM + rr;
      if (R >= rows_per_head) continue;
      const size_t orow = size_t(R / p.G) * p.Hq + kvh * p.G + R % p.G;
      float2 ml = make_float2(-INFINITY, 0.f);
      if (lane < S) ml = recv_ml[lane * rpc + rl];
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
      for (uint32_t s2 = 0; s2 < S; ++s2) {
        const float w = __shfl_sync(0xffffffffu, w_mine, int(s2));
        const float4* src = reinterpret_cast<const float4*>(recv + (s2 * rpc + rl) * OBUF_LD + lane * 8);
        const float4 a = src[0], bq = src[1];
        acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * a.z; acc[3] += w * a.w;
        acc[4] += w * bq.x; acc[5] += w * bq.y; acc[6] += w * bq.z; acc[7] += w * bq.w;
      }
      if (p.out) {
        const float inv = lg > 0.f ? 1.0f / lg : 0.f;
        uint4 w4;
        w4.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
        w4.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
        w4.z = pack_bf16x2(acc[4] * inv, acc[5] * inv);
        w4.w = pack_bf16x2(acc[6] * inv, acc[7] * inv);
        *reinterpret_cast<uint4*>(p.out + orow * HD + lane * 8) = w4;
      } else {
        float4* dst = reinterpret_cast<float4*>(p.out_o + orow * HD + lane * 8);
        dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        if (lane == 0) {
          p.out_m[orow] = mg * 0.6931471805599453f;
          p.out_l[orow] = lg;
        }
      }
    }
  } else if (p.n_splits > 1) {
    // ---------------------------------------------------------------- split merge by the last CTA
    if (tid == 0) {
      __threadfence();
      const uint32_t old = atomicAdd(p.ws_counters + blockIdx.x, 1u);
      ctl[2] = (old == p.n_splits - 1u) ? 1u : 0u;
    }
    __syncthreads();
    if (ctl[2]) {
      __threadfence();
      const uint32_t S = p.n_splits;
      const float2* ml_all = reinterpret_cast<const float2*>(p.ws_ml);
      // Phase A: one thread per row turns the S (m, l) pairs into merge weights, kept in shared
      // memory (the Q tile is dead): wsm[row][s] = 2^(m_s - m_g), plus m_g and l_g per row.
      float* wsm = reinterpret_cast<float*>(smem + OFF_Q);            // [BM][32]
      float* wl = wsm + BM * 32;                                        // [BM][32]
      float* row_mg = wl + BM * 32;                                     // [BM]
      float* row_lg = row_mg + BM;                                      // [BM]
      if (tid < BM) {
        const uint32_t R = mt * BM + tid;
        const bool live = R < rows_per_head;
        const uint32_t Rc = live ? R : mt * BM;
        const size_t orow = size_t(Rc / p.G) * p.Hq + kvh * p.G + Rc % p.G;
        float mg = -INFINITY;
        for (uint32_t s0 = 0; s0 < S; s0 += 8) {
          float2 v[8];
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j) {
            const uint32_t sidx = (s0 + j < S) ? s0 + j : S - 1;
            v[j] = ml_all[size_t(sidx) * rows_total + orow];
          }
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j)
            if (s0 + j < S) {
              wsm[tid * 32 + s0 + j] = v[j].x;                          // m_s for now
              wl[tid * 32 + s0 + j] = v[j].y;
              mg = fmaxf(mg, v[j].x);
            }
        }
        float lg = 0.f;
        for (uint32_t s = 0; s < S; ++s) {
          const float ms = wsm[tid * 32 + s];
          const float w = (ms == -INFINITY) ? 0.f : fast_exp2(ms - mg);
          wsm[tid * 32 + s] = w;
          lg += w * wl[tid * 32 + s];
        }
        row_mg[tid] = mg;
        row_lg[tid] = lg;
      }
      __syncthreads();
      // Phase B: each warp merges four rows per iteration with up to 4 x 4 x 2 16-byte loads in
      // flight, so the pass is bound by L2 bandwidth rather than by a round trip per row and split.
      constexpr uint32_t NW = THREADS / 32;
      constexpr uint32_t RK = 2;
      for (uint32_t r0 = warp * RK; r0 < BM; r0 += NW * RK) {
        size_t orow[RK];
        bool live[RK];
        float acc[RK][8];
#pragma unroll
        for (uint32_t k = 0; k < RK; ++k) {
          const uint32_t R = mt * BM + r0 + k;
          live[k] = (r0 + k < BM) && (R < rows_per_head);
          const uint32_t Rc = live[k] ? R : mt * BM;
          orow[k] = size_t(Rc / p.G) * p.Hq + kvh * p.G + Rc % p.G;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[k][e] = 0.f;
        }
        for (uint32_t s0 = 0; s0 < S; s0 += 4) {
          float4 a[RK][4], bq[RK][4];
#pragma unroll
          for (uint32_t k = 0; k < RK; ++k)
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
              const uint32_t sidx = (s0 + j < S) ? s0 + j : S - 1;   // clamped; its weight is zeroed below
              const float4* src = reinterpret_cast<const float4*>(p.ws_o + (size_t(sidx) * rows_total + orow[k]) * HD + lane * 8);
              a[k][j] = src[0];
              bq[k][j] = src[1];
            }
#pragma unroll
          for (uint32_t k = 0; k < RK; ++k)
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
              const uint32_t rr = (r0 + k < BM) ? r0 + k : BM - 1;
              const float w = (s0 + j < S) ? wsm[rr * 32 + s0 + j] : 0.f;
              acc[k][0] += w * a[k][j].x; acc[k][1] += w * a[k][j].y; acc[k][2] += w * a[k][j].z; acc[k][3] += w * a[k][j].w;
              acc[k][4] += w * bq[k][j].x; acc[k][5] += w * bq[k][j].y; acc[k][6] += w * bq[k][j].z; acc[k][7] += w * bq[k][j].w;
            }
        }
#pragma unroll
        for (uint32_t k = 0; k < RK; ++k) {
          if (!live[k]) continue;
          const float lg = row_lg[r0 + k], mg = row_mg[r0 + k];
          if (p.out) {
            const float inv = lg > 0.f ? 1.0f / lg : 0.f;
            uint4 w4;
            w4.x = pack_bf16x2(acc[k][0] * inv, acc[k][1] * inv);
            w4.y = pack_bf16x2(acc[k][2] * inv, acc[k][3] * inv);
            w4.z = pack_bf16x2(acc[k][4] * inv, acc[k][5] * inv);
            w4.w = pack_bf16x2(acc[k][6] * inv, acc[k][7] * inv);
            *reinterpret_cast<uint4*>(p.out + orow[k] * HD + lane * 8) = w4;
          } else {
            float4* dst = reinterpret_cast<float4*>(p.out_o + orow[k] * HD + lane * 8);
            dst[0] = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
            dst[1] = make_float4(acc[k][4], acc[k][5], acc[k][6], acc[k][7]);
            if (lane == 0) {
              p.out_m[orow[k]] = mg * 0.6931471805599453f;
              p.out_l[orow[k]] = lg;
            }
          }
        }
      }
      if (tid == 0) p.ws_counters[blockIdx.x] = 0u;   // ready for the next launch
    }
  }
  stamp(p, 5);
}

cudaError_t sm100_attn_configure() {
  return cudaFuncSetAttribute(dg_attn_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES));
}

// How many clusters of (1, cluster_y, 1) CTAs of the single-CTA kernel the device can hold at once.
int sm100_max_active_clusters(uint32_t cluster_y) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, cluster_y, 148);
  cfg.blockDim = dim3(one::THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = cluster_y;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, dg_attn_sm100_kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return n;
}

uint32_t sm100_query_tiles(uint32_t C, uint32_t G, uint32_t Hkv) { return Hkv * ((C * G + BM - 1) / BM); }

uint32_t sm100_key_tiles(const MaskParams& mk) {
  const TileSched t = tile_sched(mk, 0);
  return t.nA + t.nB;
}

cudaError_t launch_attn_sm100(const AttnParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                              cudaStream_t st) {
  const dim3 grid(sm100_query_tiles(p.C, p.G, p.Hkv), p.n_splits);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(one::THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  unsigned n_attr = 0;
  // start while the preceding kernel on the stream drains; the kernel waits (griddepcontrol.wait)
  // before it touches anything that kernel wrote
  attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
  ++n_attr;
  if (p.cluster_merge && p.n_splits > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = p.n_splits;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  return cudaLaunchKernelEx(&cfg, dg_attn_sm100_kernel, p, tm_k, tm_v);
}

}  // namespace dg
