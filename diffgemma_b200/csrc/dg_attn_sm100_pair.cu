// CTA-pair variant of the head_dim-256 canvas-attention kernel (sm_100a, tcgen05 cta_group::2).
//
// Two CTAs on the two SMs of one TPC own two adjacent query tiles of the same KV head.  One thread
// of the pair's leader issues M = 256 MMAs that span both CTAs: each CTA supplies its own 128 query
// rows (Q from shared memory, P from tensor memory) and HALF of every K/V tile from its own shared
// memory - 64 of the 128 keys for S = Q K^T, 128 of the 256 value columns for O += P V.  Every K/V
// byte therefore crosses L2 -> SM once per pair instead of once per query tile, and the halved
// tiles leave room for two stages of K and of V, so tile loads overlap the MMAs of the previous
// tile.  No TMA load uses multicast; each CTA loads its own halves and the byte counts of both land
// on the leader's barrier.
//
// Everything else (Q prologue, two-threads-per-row online softmax with lazy rescale, cluster /
// DSMEM split merge or global-workspace merge, bounded waits) is as in dg_attn_sm100.cu.
#include <cuda.h>

#include "dg_attn_sm100_common.cuh"
#include "dg_kernels.h"

namespace dg {

using namespace sm100;

namespace pr {
constexpr uint32_t K_STAGE = 32768;      // 64 keys x 256 d bf16: 4 atoms of 64 rows x 128 B
constexpr uint32_t K_ATOM = 8192;
constexpr uint32_t V_STAGE = 32768;      // 128 keys x 128 d bf16: 2 atoms of 128 rows x 128 B
constexpr uint32_t P_OFF_Q = 0;
constexpr uint32_t P_OFF_K = TILE_BYTES;                 // 2 stages
constexpr uint32_t P_OFF_V = TILE_BYTES + 2 * K_STAGE;   // 2 stages
constexpr uint32_t P_OFF_BAR = TILE_BYTES + 2 * K_STAGE + 2 * V_STAGE;   // 192 KB
constexpr uint32_t P_OFF_XCH = P_OFF_BAR + 256;
constexpr uint32_t P_SMEM_BYTES = P_OFF_XCH + 4096 + 1024;
enum : uint32_t {
  PB_Q = 0,          // leader: 16 arrivals (one per softmax warp of both CTAs)
  PB_K_FULL0 = 1,    // leader: +1 for stage 1; expect_tx of 64 KB (32 KB from each CTA)
  PB_V_FULL0 = 3,    // leader
  PB_P_FULL0 = 5,    // leader: 16 arrivals, +1 for buffer 1
  PB_K_EMPTY0 = 7,   // each CTA, +1 for stage 1
  PB_V_EMPTY0 = 9,   // each CTA
  PB_S_FULL0 = 11,   // each CTA, +1 for buffer 1
  PB_PV_DONE = 13,   // each CTA
  PB_O_FINAL = 14,   // each CTA
  PN_BARS = 15
};
}  // namespace pr

__global__ void __launch_bounds__(N_THREADS, 1)
dg_attn_sm100_pair_kernel(const AttnParams p, const __grid_constant__ CUtensorMap tm_k64,
                          const __grid_constant__ CUtensorMap tm_v) {
  using namespace pr;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + P_OFF_Q, sK = smem_base + P_OFF_K, sV = smem_base + P_OFF_V;
  const uint32_t bar_base = smem_base + P_OFF_BAR;
  volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + P_OFF_BAR + PN_BARS * 8);
  // ctl[0] = TMEM base address, ctl[1] = abort flag, ctl[2] = "this CTA merges" flag
  float* xch_max = reinterpret_cast<float*>(smem + P_OFF_XCH);   // [2 tile parities][BM][2 halves]
  float* xch_misc = xch_max + 2 * BM * 2;                         // [BM][2]
  float* xch_l = xch_misc + BM * 2;                               // [BM][2]

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t tiles_per_head = (p.C * p.G + BM - 1) / BM;
  const uint32_t tph2 = (tiles_per_head + 1u) & ~1u;   // tiles per head rounded up to whole pairs
  const uint32_t kvh = blockIdx.x / tph2;
  const uint32_t mt = blockIdx.x % tph2;                // may be a padding tile (every row invalid)
  const uint32_t split = blockIdx.y;
  const uint32_t rows_per_head = p.C * p.G;
  const MaskParams mk = p.mask;

  const uint32_t rank = cluster_ctarank();
  const uint32_t xi = rank & 1u;                        // position inside the pair
  const uint32_t leader = rank & ~1u;
  const bool is_leader = xi == 0u;

  // both CTAs of a pair walk the same key tiles: schedule from the pair's first canvas row
  const uint32_t row_first = ((mt & ~1u) * BM) / p.G;
  const TileSched ts = tile_sched(mk, row_first < p.C ? row_first : p.C - 1);
  const uint32_t n_tiles = ts.nA + ts.nB;
  const uint32_t v_begin = uint32_t((uint64_t(split) * n_tiles) / p.n_splits);
  const uint32_t v_end = uint32_t((uint64_t(split + 1) * n_tiles) / p.n_splits);
  const uint32_t n_local = v_end - v_begin;

  // cluster addresses of the leader's barriers (also valid when this CTA is the leader)
  auto lead_bar = [&](uint32_t idx) { return dsmem_addr(bar_addr(bar_base, idx), leader); };
  auto peer_bar = [&](uint32_t idx) { return dsmem_addr(bar_addr(bar_base, idx), leader | 1u); };

  stamp(p, 0);
  // ------------------------------------------------------------------ set-up
  if (tid == 0) {
    mbar_init(bar_addr(bar_base, PB_Q), 2 * N_SM_WARPS);   // one arrival per softmax warp of either CTA
    for (uint32_t s = 0; s < 2; ++s) {
      mbar_init(bar_addr(bar_base, PB_K_FULL0 + s), 1);
      mbar_init(bar_addr(bar_base, PB_V_FULL0 + s), 1);
      mbar_init(bar_addr(bar_base, PB_P_FULL0 + s), 2 * N_SM_WARPS);
      mbar_init(bar_addr(bar_base, PB_K_EMPTY0 + s), 1);
      mbar_init(bar_addr(bar_base, PB_V_EMPTY0 + s), 1);
      mbar_init(bar_addr(bar_base, PB_S_FULL0 + s), 1);
    }
    mbar_init(bar_addr(bar_base, PB_PV_DONE), 1);
    mbar_init(bar_addr(bar_base, PB_O_FINAL), 1);
    ctl[1] = 0u;
    ctl[2] = 0u;
    fence_mbar_init();
  }
  if (warp == WARP_MMA) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(&ctl[0])), TMEM_COLS);
    tmem_relinquish_pair();
  }
  if ((warp == WARP_K || warp == WARP_V) && lane == 0) tma_prefetch_desc(warp == WARP_K ? &tm_k64 : &tm_v);
  tc_fence_before();
  __syncthreads();
  // the peer's barriers must exist before anything of ours can signal them
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = ctl[0];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  stamp(p, 1);
  volatile uint32_t* abort_flag = &ctl[1];

  const uint32_t smw = warp & 3u, half = (warp >> 2) & 1u;
  const uint32_t r = smw * 32 + lane;
  float m_used = -INFINITY, l_run = 0.f;

  if (warp < N_SM_WARPS) {
    // ---------------------------------------------------------------- Q prologue (two threads per row)
    {
      const uint32_t R = mt * BM + r;
      const bool valid = mt < tiles_per_head && R < rows_per_head;
      const uint32_t i = valid ? R / p.G : 0u;
      const uint32_t h = kvh * p.G + (valid ? R % p.G : 0u);
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t(i) * p.Hq + h) * HD);
      const bool do_norm = !p.q_prenormed;
      uint4 lo[8], hi[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        lo[j] = src[half * 8 + j];
        hi[j] = src[16 + half * 8 + j];
      }
      if (!valid) {
#pragma unroll
        for (int j = 0; j < 8; ++j) lo[j] = hi[j] = make_uint4(0u, 0u, 0u, 0u);
      }
      float inv = 1.0f;
      if (do_norm) {
        float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
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
        xch_misc[r * 2 + half] = ss0 + ss1;
        pair_sync(smw);
        const float ss = xch_misc[r * 2 + 0] + xch_misc[r * 2 + 1];
        inv = 1.0f / sqrtf(ss / float(HD) + p.eps);
      }
      const float4* tab = reinterpret_cast<const float4*>(p.rope_table + size_t(i) * 128 + half * 64);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t c_lo = half * 8 + j, c_hi = c_lo + 16;
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
            const float4 cs = tab[j * 4 + e];
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
        *reinterpret_cast<uint4*>(smem + P_OFF_Q + (c_lo >> 3) * ATOM_BYTES + r * 128u + (((c_lo & 7u) ^ (r & 7u)) << 4)) = out_lo;
        *reinterpret_cast<uint4*>(smem + P_OFF_Q + (c_hi >> 3) * ATOM_BYTES + r * 128u + (((c_hi & 7u) ^ (r & 7u)) << 4)) = out_hi;
      }
    }
    // the leader's MMA thread reads this tile through the async proxy, possibly from the other SM
    fence_proxy_async_all();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(lead_bar(PB_Q));
    stamp(p, 2);

    // ---------------------------------------------------------------- softmax main loop
    const uint32_t R = mt * BM + r;
    const uint32_t i_row = (mt < tiles_per_head && R < rows_per_head) ? R / p.G : p.C - 1;
    const uint32_t row_lo = mask_row_lo(mk, i_row);
    const uint32_t t_lane = tmem + ((smw * 32u) << 16);
    const bool contiguous = (mk.pre_hi == mk.kv_len) && (mk.can_hi > mk.kv_len);
    const float sc = p.scale_log2;
    const uint32_t p_full0 = lead_bar(PB_P_FULL0), p_full1 = lead_bar(PB_P_FULL0 + 1);

    for (uint32_t n = 0; n < n_local; ++n) {
      const uint32_t v = v_begin + n;
      const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
      const uint32_t k0 = jt * BN;
      const uint32_t b = n & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait_cluster(bar_addr(bar_base, PB_S_FULL0 + b), (n >> 1) & 1u, abort_flag))) break;
      tc_fence_after();
      uint32_t sraw[2][32];
      tmem_ld32(t_lane + TM_S + b * 128u + half * 64u, sraw[0]);
      tmem_ld32(t_lane + TM_S + b * 128u + half * 64u + 32u, sraw[1]);
      tmem_wait_ld();

      const bool full = (k0 >= row_lo && k0 + BN <= mk.pre_hi) || (k0 >= mk.kv_len && k0 + BN <= mk.can_hi) ||
                        (contiguous && k0 >= row_lo && k0 + BN <= mk.can_hi);
      if (!full) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (!mask_visible_lo(mk, row_lo, k0 + half * 64 + c * 32 + e)) sraw[c][e] = 0xff800000u;  // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sraw[c][e]));
      const float mx_half = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      xch_max[(b * BM + r) * 2 + half] = mx_half;
      pair_sync(smw);
      const float mx = fmaxf(mx_half, xch_max[(b * BM + r) * 2 + (half ^ 1u)]);
      const float m_new = mx * sc;
      const bool first = (n == 0);
      const bool need = first || (m_new > m_used + RESCALE_THRESHOLD);
      if (!first && __any_sync(0xffffffffu, need)) {
        if (!__all_sync(0xffffffffu, mbar_wait_cluster(bar_addr(bar_base, PB_PV_DONE), (n - 1) & 1u, abort_flag))) break;
        tc_fence_after();
        const float alpha = need ? fast_exp2(m_used - m_new) : 1.0f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(t_lane + TM_O + half * 128u + c * 32u, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(t_lane + TM_O + half * 128u + c * 32u, o);
        }
        tmem_wait_st();
        l_run *= alpha;
      }
      if (need) m_used = m_new;
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      const float neg_m = -m_eff;
      float ls0 = 0.f, ls1 = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(sraw[c][e]), sc, neg_m));
          const float p1 = fast_exp2(fmaf(__uint_as_float(sraw[c][e + 1]), sc, neg_m));
          ls0 += p0;
          ls1 += p1;
          pk[c * 16 + (e >> 1)] = pack_bf16x2(p0, p1);
        }
      l_run += ls0 + ls1;
      tmem_st32(t_lane + TM_S + b * 128u + half * 32u, pk);
      tmem_wait_st();
      tc_fence_before();
      // one (possibly remote) arrival per warp instead of one per thread
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(b ? p_full1 : p_full0);
    }
  } else if (warp == WARP_K) {
    // ---------------------------------------------------------------- K loader: this CTA's 64 keys
    if (lane == 0) {
      for (uint32_t n = 0; n < n_local; ++n) {
        const uint32_t v = v_begin + n;
        const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
        const uint32_t s = n & 1u, u = n >> 1;
        if (u > 0 && !mbar_wait_cluster(bar_addr(bar_base, PB_K_EMPTY0 + s), (u - 1) & 1u, abort_flag)) break;
        if (is_leader) mbar_expect_tx(bar_addr(bar_base, PB_K_FULL0 + s), 2 * K_STAGE);
        const uint32_t full = lead_bar(PB_K_FULL0 + s);
#pragma unroll
        for (uint32_t a = 0; a < 4; ++a)
          tma_load_3d_pair(sK + s * K_STAGE + a * K_ATOM, &tm_k64, full, int32_t(a * 64),
                           int32_t(jt * BN + xi * 64), int32_t(kvh));
      }
    }
  } else if (warp == WARP_V) {
    // ---------------------------------------------------------------- V loader: this CTA's 128 value columns
    if (lane == 0) {
      for (uint32_t n = 0; n < n_local; ++n) {
        const uint32_t v = v_begin + n;
        const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
        const uint32_t s = n & 1u, u = n >> 1;
        if (u > 0 && !mbar_wait_cluster(bar_addr(bar_base, PB_V_EMPTY0 + s), (u - 1) & 1u, abort_flag)) break;
        if (is_leader) mbar_expect_tx(bar_addr(bar_base, PB_V_FULL0 + s), 2 * V_STAGE);
        const uint32_t full = lead_bar(PB_V_FULL0 + s);
#pragma unroll
        for (uint32_t a = 0; a < 2; ++a)
          tma_load_3d_pair(sV + s * V_STAGE + a * ATOM_BYTES, &tm_v, full, int32_t(xi * 128 + a * 64),
                           int32_t(jt * BN), int32_t(kvh));
      }
    }
  } else {
    // ---------------------------------------------------------------- MMA issuer (one thread of the leader)
    if (is_leader && lane == 0 && n_local > 0) {
      constexpr uint32_t IDESC_QK = umma_idesc_bf16(2 * BM, BN, 0, 0);   // M = 256 over the pair
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(2 * BM, HD, 0, 1);   // B (= V) MN-major
      // completion signals go to the same barrier slot in both CTAs
      auto commit_both = [&](uint32_t idx) {
        umma_commit_pair(lead_bar(idx));
        umma_commit_pair(peer_bar(idx));
      };
      bool ok = mbar_wait_cluster(bar_addr(bar_base, PB_Q), 0u, abort_flag);
      auto issue_qk = [&](uint32_t n) -> bool {
        const uint32_t s = n & 1u, u = n >> 1;
        if (!mbar_wait_cluster(bar_addr(bar_base, PB_K_FULL0 + s), u & 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t d_tmem = tmem + TM_S + s * 128u;
#pragma unroll
        for (uint32_t a = 0; a < 4; ++a)
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk) {
            const uint64_t da = umma_smem_desc(sQ + a * ATOM_BYTES + kk * 32u, 16u, 1024u);
            const uint64_t db = umma_smem_desc(sK + s * K_STAGE + a * K_ATOM + kk * 32u, 16u, 1024u);
            umma_ss_pair(d_tmem, da, db, IDESC_QK, (a | kk) != 0u);
          }
        commit_both(PB_K_EMPTY0 + s);
        commit_both(PB_S_FULL0 + s);
        return true;
      };
      ok = ok && issue_qk(0);
      for (uint32_t n = 0; ok && n < n_local; ++n) {
        if (n + 1 < n_local) {
          ok = issue_qk(n + 1);
          if (!ok) break;
        }
        const uint32_t s = n & 1u, u = n >> 1;
        if (!mbar_wait_cluster(bar_addr(bar_base, PB_P_FULL0 + s), u & 1u, abort_flag)) break;
        if (!mbar_wait_cluster(bar_addr(bar_base, PB_V_FULL0 + s), u & 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t p_tmem = tmem + TM_S + s * 128u;
#pragma unroll
        for (uint32_t ks = 0; ks < 8; ++ks) {
          const uint64_t db = umma_smem_desc(sV + s * V_STAGE + ks * 2048u, ATOM_BYTES, 1024u);
          umma_ts_pair(tmem + TM_O, p_tmem + ks * 8u, db, IDESC_PV, (n | ks) != 0u);
        }
        commit_both(PB_V_EMPTY0 + s);
        commit_both(PB_PV_DONE);
        if (n + 1 == n_local) commit_both(PB_O_FINAL);
      }
    }
  }

  stamp(p, 3);
  // ------------------------------------------------------------------ epilogue (softmax warps)
  const uint32_t rows_total = p.C * p.Hq;
  const bool tile_real = mt < tiles_per_head;
  if (warp < N_SM_WARPS) {
    const uint32_t R = mt * BM + r;
    const bool valid = tile_real && R < rows_per_head;
    const uint32_t i_row = valid ? R / p.G : 0u;
    const uint32_t h = kvh * p.G + (valid ? R % p.G : 0u);
    const size_t orow = size_t(i_row) * p.Hq + h;
    const uint32_t t_lane = tmem + ((smw * 32u) << 16);
    bool have_o = __all_sync(0xffffffffu, n_local > 0 && !*abort_flag);
    if (have_o) {
      have_o = __all_sync(0xffffffffu, mbar_wait_cluster(bar_addr(bar_base, PB_O_FINAL), 0u, abort_flag));
      tc_fence_after();
    }
    xch_l[r * 2 + half] = l_run;
    pair_sync(smw);
    const float l_tot = xch_l[r * 2 + 0] + xch_l[r * 2 + 1];
    const bool direct = (p.n_splits == 1);
    const bool via_dsmem = (p.cluster_merge != 0u) && !direct;
    if (via_dsmem) {
      float* obuf = reinterpret_cast<float*>(smem + P_OFF_Q);
      float2* mlbuf = reinterpret_cast<float2*>(smem + P_OFF_XCH);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        const uint32_t col0 = half * 128u + c * 32u;
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
          *reinterpret_cast<uint4*>(obuf + r * OBUF_LD + col0 + q4 * 4) = make_uint4(o[q4 * 4], o[q4 * 4 + 1], o[q4 * 4 + 2], o[q4 * 4 + 3]);
      }
      if (half == 0) mlbuf[r] = make_float2(m_used, l_tot);
    } else {
      const bool to_bf16 = direct && p.out != nullptr;
      const float inv_l = l_tot > 0.f ? 1.0f / l_tot : 0.f;
      const float mul = to_bf16 ? inv_l : 1.0f;
      float* dst_o = direct ? p.out_o : p.ws_o + size_t(split) * rows_total * HD;
      float* tile = reinterpret_cast<float*>(smem + P_OFF_Q) + warp * (32 * 36);
      size_t orow_k[8];
      bool valid_k[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t Rk = mt * BM + smw * 32 + k * 4 + (lane >> 3);
        valid_k[k] = tile_real && Rk < rows_per_head;
        const uint32_t Rc = valid_k[k] ? Rk : 0u;
        orow_k[k] = size_t(Rc / p.G) * p.Hq + kvh * p.G + Rc % p.G;
      }
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        const uint32_t col0 = half * 128u + c * 32u;
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
      if (valid && !to_bf16 && half == 0) {
        if (direct) {
          p.out_m[orow] = m_used * 0.6931471805599453f;
          p.out_l[orow] = l_tot;
        } else {
          float2* ml = reinterpret_cast<float2*>(p.ws_ml) + size_t(split) * rows_total + orow;
          *ml = make_float2(m_used, l_tot);
        }
      }
      if (!direct) __threadfence();
    }
  }

  stamp(p, 4);
  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    if (tid == 0) dev_status_set(p.status, DG_DEV_WAIT_TIMEOUT, KID_SM100, blockIdx.x + gridDim.x * blockIdx.y, n_local);
    if (warp == WARP_K && lane == 0 && n_local > 0) {
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000ll) {}   // ~1 ms: far longer than any tile load in flight
    }
  }
  tc_fence_before();
  __syncthreads();
  // Neither CTA of the pair may free tensor memory or leave while the other can still be the
  // target of a pair-wide MMA, commit or DSMEM read: one cluster barrier covers all of these.
  cluster_sync_all();
  if (warp == WARP_MMA) tmem_dealloc_pair(tmem, TMEM_COLS);

  if (p.n_splits > 1 && p.cluster_merge) {
    // ---------------------------------------------------------------- split merge inside the cluster
    // cluster dims (2, S, 1): the CTAs holding this query tile's partials have ranks xi + 2 s.
    // (the cluster barrier above already ordered every partial before these reads)
    const uint32_t S = p.n_splits;
    const uint32_t yk = rank >> 1;           // this CTA's share of the rows
    const uint32_t rpc = BM / S;
    const uint32_t obuf_s = smem_base + P_OFF_Q, ml_s = smem_base + P_OFF_XCH;
    for (uint32_t rl = warp; rl < rpc; rl += N_THREADS / 32) {
      const uint32_t rr = yk * rpc + rl;
      const uint32_t R = mt * BM + rr;
      if (!tile_real || R >= rows_per_head) continue;
      const size_t orow = size_t(R / p.G) * p.Hq + kvh * p.G + R % p.G;
      float2 ml = make_float2(-INFINITY, 0.f);
      if (lane < S) ml = dsmem_ld_f2(dsmem_addr(ml_s + rr * 8u, xi + 2u * lane));
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
      const uint32_t row_off = obuf_s + (rr * OBUF_LD + lane * 8u) * 4u;
      for (uint32_t s0 = 0; s0 < S; s0 += 4) {
        float4 a[4], bq[4];
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
          const uint32_t src = (s0 + j < S) ? s0 + j : S - 1;
          const uint32_t ra = dsmem_addr(row_off, xi + 2u * src);
          a[j] = dsmem_ld_f4(ra);
          bq[j] = dsmem_ld_f4(ra + 16u);
        }
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
          float w = __shfl_sync(0xffffffffu, w_mine, int((s0 + j) & 31u));
          if (s0 + j >= S) w = 0.f;
          acc[0] += w * a[j].x; acc[1] += w * a[j].y; acc[2] += w * a[j].z; acc[3] += w * a[j].w;
          acc[4] += w * bq[j].x; acc[5] += w * bq[j].y; acc[6] += w * bq[j].z; acc[7] += w * bq[j].w;
        }
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
    cluster_sync_all();
  } else if (p.n_splits > 1) {
    // ---------------------------------------------------------------- split merge by the last CTA
    if (tid == 0) {
      __threadfence();
      const uint32_t old = atomicAdd(p.ws_counters + blockIdx.x, 1u);
      ctl[2] = (old == p.n_splits - 1u) ? 1u : 0u;
    }
    __syncthreads();
    if (ctl[2] && tile_real) {
      __threadfence();
      const uint32_t S = p.n_splits;
      const float2* ml_all = reinterpret_cast<const float2*>(p.ws_ml);
      for (uint32_t rr = warp; rr < BM; rr += N_THREADS / 32) {
        const uint32_t R = mt * BM + rr;
        if (R >= rows_per_head) break;
        const size_t orow = size_t(R / p.G) * p.Hq + kvh * p.G + R % p.G;
        float2 ml = make_float2(-INFINITY, 0.f);
        if (lane < S) ml = ml_all[size_t(lane) * rows_total + orow];
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
          const float4* src = reinterpret_cast<const float4*>(p.ws_o + (size_t(s) * rows_total + orow) * HD + lane * 8);
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
    }
    if (ctl[2] && tid == 0) p.ws_counters[blockIdx.x] = 0u;   // ready for the next launch
  }
  stamp(p, 5);
}

cudaError_t sm100_pair_configure() {
  return cudaFuncSetAttribute(dg_attn_sm100_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              int(pr::P_SMEM_BYTES));
}

// How many clusters of (2, cluster_y, 1) CTAs of the pair kernel the device can hold at once.
int sm100_pair_max_active_clusters(uint32_t cluster_y) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, cluster_y, 148);
  cfg.blockDim = dim3(N_THREADS);
  cfg.dynamicSmemBytes = pr::P_SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = cluster_y;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, dg_attn_sm100_pair_kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return n;
}

uint32_t sm100_pair_query_tiles(uint32_t C, uint32_t G, uint32_t Hkv) {
  const uint32_t tph = (C * G + BM - 1) / BM;
  return Hkv * ((tph + 1u) & ~1u);
}

// tm_k64: K tensor map with box {64 d, 64 keys, 1}; tm_v: V tensor map with box {64 d, 128 keys, 1}.
cudaError_t launch_attn_sm100_pair(const AttnParams& p, const CUtensorMap& tm_k64, const CUtensorMap& tm_v,
                                   cudaStream_t st) {
  const dim3 grid(sm100_pair_query_tiles(p.C, p.G, p.Hkv), p.n_splits);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(N_THREADS);
  cfg.dynamicSmemBytes = pr::P_SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = (p.cluster_merge && p.n_splits > 1) ? p.n_splits : 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, dg_attn_sm100_pair_kernel, p, tm_k64, tm_v);
}

}  // namespace dg
