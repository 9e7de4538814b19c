// Denoise-step canvas attention for head_dim 512 on sm_100a, four CTAs per cluster: the P exchange of
// dg_attn_sm100_hd512x.cu between the two value-column halves of a query tile, and on top of it tcgen05
// cta_group::2 MMAs over TWO query tiles of one KV head, so that K and V are staged once per pair of tiles.
//
// Cluster (2, 1, 2), rank = x + 2 z: x = which of the two query tiles, z = which half of the value columns
// (and which 64-key tile of a step).  The CTAs (0, z) and (1, z) are a cta_group::2 pair: one lane of the
// leader's (x = 0) MMA warp issues M = 256 MMAs over both, each CTA supplies its own 128 query rows (Q, P) and
// half of the N extent of B from its own shared memory: 32 of the 64 keys of its K tile, 128 of this half's 256
// value columns.  The CTAs (x, 0) and (x, 1) exchange row maxima and P exactly as in the two-CTA form.
// Per CTA and step of 128 keys: 64 KB of Q operand reads, 32 KB of K and 32 KB of V operand reads, 64 KB of TMA
// writes, 32 KB for the relay of the peer's P = 224 KB (the two-CTA form: 352 KB), and K and V have two stages
// each.  Needs an even number of query tiles per KV head.
#include <cuda.h>

#include "dg_attn_sm100_hd512.cuh"
#include "dg_kernels.h"

namespace dg {

namespace h5q {
using namespace h5;
constexpr uint32_t SM_WARPS = 8;
constexpr uint32_t W_K = SM_WARPS, W_V = SM_WARPS + 1, W_MMA = SM_WARPS + 2;
constexpr uint32_t THREADS = (SM_WARPS + 3) * 32;   // 352
constexpr uint32_t K_ATOM = 32 * 128;                 // this CTA's 32 keys of a tile x 64 contraction elements = 4 KB
constexpr uint32_t K_STAGE = 8 * K_ATOM;              // 32 keys x 512 = 32 KB
constexpr uint32_t V_TILE = 2 * KV_ATOM;              // 64 keys x this CTA's 128 value columns = 16 KB
constexpr uint32_t V_STAGE = 2 * V_TILE;              // both tiles of a step = 32 KB
constexpr uint32_t P_BUF = Q_ATOM;                    // 128 rows x 64 keys bf16 = 16 KB
constexpr uint32_t O_Q = 0;                           // Q[:, 256:512]: 4 atoms = 64 KB
constexpr uint32_t O_K = 4 * Q_ATOM;                  // 2 stages = 64 KB
constexpr uint32_t O_V = O_K + 2 * K_STAGE;           // 2 stages = 64 KB
constexpr uint32_t O_PR = O_V + 2 * V_STAGE;          // the peer's P, 2 buffers = 32 KB
constexpr uint32_t O_BAR = O_PR + 2 * P_BUF;          // = 224 KB
constexpr uint32_t O_MX = O_BAR + 256;                // the peer's row maxima, [2 buffers][BM] floats
constexpr uint32_t O_REF = O_MX + 2 * BM * 4;         // reference maximum of every row, handed between the warpgroups
constexpr uint32_t O_END = O_REF + BM * 4;
static_assert(O_END + 1024 <= SMEM_REQ + 256, "shared-memory map does not fit");
// after the key loop the K region is dead: row sums of the two warpgroups and of the peer
constexpr uint32_t O_LSUM = O_K;                      // [2][BM] floats
constexpr uint32_t O_LPEER = O_K + 2 * BM * 4;        // [BM] floats
enum : uint32_t {
  B_Q = 0,          // leader: the Q tiles of both CTAs are in place
  B_K_FULL = 1,     // + stage; leader: both CTAs' halves of the K tile have landed
  B_K_EMPTY = 5,    // + stage
  B_V_FULL = 9,     // + stage; leader
  B_V_EMPTY = 11,   // + stage
  B_S_FULL = 13,    // + buffer
  B_P_FULL = 15,    // + buffer; leader: own P of both CTAs in tensor memory
  B_PR_FULL = 17,   // + buffer: the peer's P has landed in shared memory (bytes counted)
  B_P2_FULL = 19,   // + buffer; leader: the peers' P of both CTAs in tensor memory
  B_MX = 21,        // + buffer: the peer's row maxima have landed (bytes counted)
  B_REF = 23,       // + warpgroup that published the reference
  B_O_FINAL = 25,
  B_COUNT = 26
};
static_assert(B_COUNT * 8 + 16 <= 256, "barrier block");
}  // namespace h5q

__global__ void __launch_bounds__(h5q::THREADS, 1)
dg_attn_sm100_hd512q_kernel(const AttnParams p, const __grid_constant__ CUtensorMap tm_k,
                            const __grid_constant__ CUtensorMap tm_v) {
  using namespace h5q;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t crank = cluster_ctarank();        // x + 2 z
  const uint32_t xi = crank & 1u;                  // which query tile of the pair
  const uint32_t dh = crank >> 1;                  // which half of the value columns, and which tile of a step
  const uint32_t peer = dh ^ 1u;                   // the other value half (tile), as an index
  const uint32_t peer_rank = crank ^ 2u;           // the CTA with the same query tile and the other value half
  const uint32_t leader = crank & ~1u;             // the CTA of this cta_group::2 pair whose MMA warp issues
  const bool is_leader = xi == 0u;
  // The two CTAs of the cluster take the same branch here: the dynamic shared memory of a kernel starts at
  // the same offset in every CTA.
  if (smem_base - smem_u32(smem_raw) + O_END > SMEM_REQ) {
    if (tid == 0) dev_status_set(p.status, DG_DEV_SMEM_LAYOUT, KID_SM100, blockIdx.x, smem_base - smem_u32(smem_raw));
    return;
  }
  const uint32_t sQ = smem_base + O_Q, sK = smem_base + O_K, sV = smem_base + O_V, sPR = smem_base + O_PR;
  const uint32_t bar_base = smem_base + O_BAR;
  auto lead_bar = [&](uint32_t idx) { return dsmem_addr(bar_addr(bar_base, idx), leader); };
  auto pair_bar = [&](uint32_t idx) { return dsmem_addr(bar_addr(bar_base, idx), leader | 1u); };
  volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + O_BAR + B_COUNT * 8);
  volatile float* mx_peer = reinterpret_cast<volatile float*>(smem + O_MX);   // [2][BM]
  volatile float* m_ref = reinterpret_cast<volatile float*>(smem + O_REF);    // [BM]

  const uint32_t tiles_per_head = (p.C * p.G + BM - 1) / BM;
  const uint32_t kvh = blockIdx.x / tiles_per_head;
  const uint32_t mt = blockIdx.x % tiles_per_head;
  const uint32_t split = blockIdx.y;
  const uint32_t rows_per_head = p.C * p.G;
  const MaskParams mk = p.mask;

  // the two query tiles of a pair walk the same key tiles: schedule from the pair's first and last canvas row
  const uint32_t row_first = ((mt & ~1u) * BM) / p.G;
  const uint32_t row_last = (((mt | 1u) + 1u) * BM - 1u) / p.G;
  const TileSched ts = tile_sched64(mk, row_first < p.C ? row_first : p.C - 1, row_last < p.C ? row_last : p.C - 1);
  const uint32_t n_tiles = ts.nA + ts.nB;            // 64-key tiles
  const uint32_t n_steps = (n_tiles + 1u) / 2u;      // pairs of tiles
  const uint32_t u_begin = uint32_t((uint64_t(split) * n_steps) / p.n_splits);
  const uint32_t u_end = uint32_t((uint64_t(split + 1) * n_steps) / p.n_splits);
  const uint32_t n_local = u_end - u_begin;
  // absolute 64-key tile of virtual tile v; a step's second tile may not exist (odd count): it is loaded
  // from the last tile and wholly masked
  auto tile_of = [&](uint32_t v) -> uint32_t {
    const uint32_t vc = v < n_tiles ? v : n_tiles - 1u;
    return vc < ts.nA ? ts.a0 + vc : ts.b0 + (vc - ts.nA);
  };

  // ------------------------------------------------------------------ set-up
  if (tid == 0) {
    mbar_init(bar_addr(bar_base, B_Q), 2 * SM_WARPS);
    for (uint32_t s = 0; s < 2; ++s) {
      mbar_init(bar_addr(bar_base, B_K_FULL + s), 1);
      mbar_init(bar_addr(bar_base, B_K_EMPTY + s), 1);
      mbar_init(bar_addr(bar_base, B_V_FULL + s), 1);
      mbar_init(bar_addr(bar_base, B_V_EMPTY + s), 1);
      mbar_init(bar_addr(bar_base, B_S_FULL + s), 1);
      mbar_init(bar_addr(bar_base, B_P_FULL + s), 2 * 4);
      mbar_init(bar_addr(bar_base, B_PR_FULL + s), 1);
      mbar_init(bar_addr(bar_base, B_P2_FULL + s), 2 * 4);
      mbar_init(bar_addr(bar_base, B_MX + s), 1);
      mbar_init(bar_addr(bar_base, B_REF + s), 4);
    }
    mbar_init(bar_addr(bar_base, B_O_FINAL), 1);
    ctl[1] = 0u;
    ctl[2] = 0u;
    fence_mbar_init();
  }
  if (warp == W_MMA) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(&ctl[0])), TMEM_COLS);
    tmem_relinquish_pair();
  }
  if ((warp == W_K || warp == W_V) && lane == 0) tma_prefetch_desc(warp == W_K ? &tm_k : &tm_v);
  tc_fence_before();
  // the peer must not signal a barrier of this CTA before it is initialised
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = ctl[0];
  // everything this kernel reads was written by kernels launched before it on the stream
  asm volatile("griddepcontrol.wait;" ::: "memory");
  volatile uint32_t* abort_flag = &ctl[1];

  stamp(p, 0);
  const uint32_t smw = warp & 3u, grp = (warp >> 2) & 1u;
  const uint32_t r = smw * 32 + lane;
  float m_seen = -INFINITY, l_part = 0.f;

  if (warp < SM_WARPS) {
    // ---------------------------------------------------------------- Q tile: copy (two threads per row)
    copy_q_tile(p, smem + O_Q, tmem, kvh, mt, smw, lane, grp);
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(lead_bar(B_Q));      // the Q tile's shared-memory half is ordinary stores

    // ---------------------------------------------------------------- softmax: this warpgroup's steps
    const uint32_t R = mt * BM + r;
    const uint32_t i_row = (R < rows_per_head) ? R / p.G : p.C - 1;
    const RowVis rv = mask_row(mk, i_row);
    const uint32_t t_lane = tmem + ((smw * 32u) << 16);
    const float sc = p.scale_log2;
    const uint32_t b = grp;
    const uint32_t peer_mx = dsmem_addr(smem_base + O_MX + (b * BM + r) * 4u, peer_rank);
    const uint32_t peer_pr = dsmem_addr(sPR + b * P_BUF + r * 128u, peer_rank);
    const uint32_t peer_bar_mx = dsmem_addr(bar_addr(bar_base, B_MX + b), peer_rank);
    const uint32_t peer_bar_pr = dsmem_addr(bar_addr(bar_base, B_PR_FULL + b), peer_rank);
    const uint32_t lead_p_full = lead_bar(B_P_FULL + b), lead_p2_full = lead_bar(B_P2_FULL + b);
    // cycles thread 0 spends in the waits and exchanges of its steps (only with a stamp buffer)
    const bool prof = p.stamps != nullptr && tid == 0;
    long long w_s = 0, w_ref = 0, w_mx = 0, w_free = 0, c_send = 0, c_deliver = 0, c_exp = 0, n_resc = 0;
    stamp(p, 1);

    for (uint32_t n = grp; n < n_local; n += 2) {
      const uint32_t k = n >> 1;                      // this buffer's use count
      const uint32_t v = 2u * (u_begin + n) + dh;
      const bool phantom = v >= n_tiles;
      const uint32_t k0 = tile_of(v) * TN;
      // this step's bytes from the peer: 128 row maxima and 128 rows of P
      if (smw == 0 && lane == 0) {
        mbar_expect_tx(bar_addr(bar_base, B_MX + b), BM * 4u);
        mbar_expect_tx(bar_addr(bar_base, B_PR_FULL + b), P_BUF);
      }
      if (!__all_sync(0xffffffffu, timed_wait(prof, w_s, [&] { return mbar_wait(bar_addr(bar_base, B_S_FULL + b), k & 1u, abort_flag); }))) break;
      tc_fence_after();
      uint32_t sraw[64];
      tmem_ld32(t_lane + T_S + b * TN, *reinterpret_cast<uint32_t(*)[32]>(&sraw[0]));
      tmem_ld32(t_lane + T_S + b * TN + 32u, *reinterpret_cast<uint32_t(*)[32]>(&sraw[32]));
      tmem_wait_ld();
      if (phantom) {
#pragma unroll
        for (int e = 0; e < 64; ++e) sraw[e] = 0xff800000u;
      } else if (!mask_range_full(mk, rv, k0, TN)) {
#pragma unroll
        for (int e = 0; e < 64; ++e)
          if (!mask_visible_row(mk, rv, k0 + e)) sraw[e] = 0xff800000u;  // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 64; e += 2)
        mx4[(e >> 1) & 3] = max3_f32(mx4[(e >> 1) & 3], __uint_as_float(sraw[e]), __uint_as_float(sraw[e + 1]));
      const float mx_own = max3_f32(max3_f32(mx4[0], mx4[1], mx4[2]), mx4[3], -INFINITY);
      // this tile's row maximum to the peer
      long long t_a = prof ? clock64() : 0;
      dsmem_st_async_f32(peer_mx, mx_own, peer_bar_mx);
      if (prof) c_send += clock64() - t_a;
      // the reference maximum the other warpgroup left after the step before
      if (n > 0) {
        if (!__all_sync(0xffffffffu, timed_wait(prof, w_ref, [&] { return mbar_wait(bar_addr(bar_base, B_REF + (grp ^ 1u)), ((n - 1u) >> 1) & 1u, abort_flag); }))) break;
        const float m_cur = m_ref[r];
        if (m_cur != m_seen) {
          l_part *= (m_seen == -INFINITY) ? 0.f : fast_exp2(m_seen - m_cur);
          m_seen = m_cur;
        }
      }
      if (!__all_sync(0xffffffffu, timed_wait(prof, w_mx, [&] { return mbar_wait_cluster(bar_addr(bar_base, B_MX + b), k & 1u, abort_flag); }))) break;
      const float mx = fmaxf(mx_own, mx_peer[b * BM + r]);
      const float m_new = mx * sc;
      const bool first = (n == 0);
      const bool need = first || (m_new > m_seen + RESCALE_THRESHOLD);
      if (!first && __any_sync(0xffffffffu, need)) {
        // PV(n - 1) must be complete before O is touched
        if (!__all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, B_V_EMPTY + ((n - 1u) & 1u)), ((n - 1u) >> 1) & 1u, abort_flag))) break;
        tc_fence_after();
        const float alpha = need ? ((m_seen == -INFINITY) ? 0.f : fast_exp2(m_seen - m_new)) : 1.0f;
#pragma unroll 1
        for (uint32_t c = 0; c < HDV / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(t_lane + T_O + c * 32u, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(t_lane + T_O + c * 32u, o);
        }
        tmem_wait_st();
        l_part *= alpha;
        ++n_resc;
      }
      if (need) m_seen = m_new;
      if (n + 1u < n_local) {
        m_ref[r] = m_seen;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_addr(bar_base, B_REF + grp));
      }
      t_a = prof ? clock64() : 0;
      const float m_eff = (m_seen == -INFINITY) ? 0.f : m_seen;
      const float neg_m = -m_eff;
      const uint64_t sc2 = pack_f32x2(sc, sc), nm2 = pack_f32x2(neg_m, neg_m);
      uint64_t ls2[2] = {0ull, 0ull};
      uint32_t pk[32];
      // Every 8 keys (one 16-byte chunk of the row) leave for the peer as soon as they are computed, so that the
      // transfer of the row runs under the exponentials of its later keys: chunk j = keys [8j, 8j + 8) at chunk
      // position j ^ (r & 7).  The buffer is free: the peer read its step n - 2 before it sent the row maxima of step
      // n, which this thread has waited for.
#pragma unroll
      for (uint32_t j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = int(j) * 8; e < int(j) * 8 + 8; e += 2) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[e]), __uint_as_float(sraw[e + 1])), sc2, nm2), x0, x1);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          ls2[(e >> 1) & 1] = add_f32x2(ls2[(e >> 1) & 1], pack_f32x2(p0, p1));
          pk[e >> 1] = pack_bf16x2(p0, p1);
        }
        dsmem_st_async_u4(peer_pr + ((j ^ (r & 7u)) << 4), make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]),
                          peer_bar_pr);
      }
      {
        float s0, s1;
        unpack_f32x2(add_f32x2(ls2[0], ls2[1]), s0, s1);
        l_part += s0 + s1;
      }
      if (prof) {
        const long long t_b = clock64();
        c_exp += t_b - t_a;
        t_a = t_b;
      }
      // own copy: P column j = keys (2j, 2j + 1), over the first 32 columns of the S buffer
      tmem_st32(t_lane + T_S + b * TN, pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(lead_p_full);
      // the peer's P of this step: from shared memory into columns [32, 64) of the S buffer
      if (!__all_sync(0xffffffffu, timed_wait(prof, w_free, [&] { return mbar_wait_cluster(bar_addr(bar_base, B_PR_FULL + b), k & 1u, abort_flag); }))) break;
      {
        const uint32_t row = sPR + b * P_BUF + r * 128u;
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
          uint4 v4;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v4.x), "=r"(v4.y), "=r"(v4.z), "=r"(v4.w)
                       : "r"(row + ((j ^ (r & 7u)) << 4)) : "memory");
          pk[4 * j] = v4.x; pk[4 * j + 1] = v4.y; pk[4 * j + 2] = v4.z; pk[4 * j + 3] = v4.w;
        }
      }
      tmem_st32(t_lane + T_S + b * TN + 32u, pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(lead_p2_full);
      if (prof) c_deliver += clock64() - t_a;
    }
    stamp(p, 2);
    if (prof) {
      stamp_cycles(p, 11, w_s);
      stamp_cycles(p, 12, w_ref);
      stamp_cycles(p, 13, w_mx);
      stamp_cycles(p, 14, w_free);
      stamp_cycles(p, 15, c_send);
      stamp_cycles(p, 3, c_deliver);
      stamp_cycles(p, 4, n_resc);
      stamp_cycles(p, 5, c_exp);
    }
  } else if (warp == W_K) {
    // ---------------------------------------------------------------- K loader: this CTA's 32 keys of the pair's tile, 8 boxes {64 d, 32 keys}
    if (lane == 0) {
      for (uint32_t n = 0; n < n_local; ++n) {
        const uint32_t jt = tile_of(2u * (u_begin + n) + dh);
        const int32_t key0 = int32_t((jt * TN + xi * 32u - p.pos_base) & p.ring_mask);
        const uint32_t st = n & 1u, use = n >> 1;
        // the stage is free once the MMAs of step n - 2 have completed
        if (use > 0 && !mbar_wait(bar_addr(bar_base, B_K_EMPTY + st), (use - 1u) & 1u, abort_flag)) break;
        if (is_leader) mbar_expect_tx(bar_addr(bar_base, B_K_FULL + st), 2 * K_STAGE);
        const uint32_t full = lead_bar(B_K_FULL + st);
#pragma unroll
        for (uint32_t a = 0; a < 8; ++a)
          tma_load_3d_pair(sK + st * K_STAGE + a * K_ATOM, &tm_k, full, int32_t(a * 64u), key0, int32_t(kvh));
      }
    }
  } else if (warp == W_V) {
    // ---------------------------------------------------------------- V loader: both tiles of a step, this CTA's 128 of the half's 256 columns
    if (lane == 0) {
      for (uint32_t n = 0; n < n_local; ++n) {
        const uint32_t st = n & 1u, use = n >> 1;
        if (use > 0 && !mbar_wait(bar_addr(bar_base, B_V_EMPTY + st), (use - 1u) & 1u, abort_flag)) break;
        if (is_leader) mbar_expect_tx(bar_addr(bar_base, B_V_FULL + st), 2 * V_STAGE);
        const uint32_t full = lead_bar(B_V_FULL + st);
#pragma unroll
        for (uint32_t t = 0; t < 2; ++t) {
          const uint32_t jt = tile_of(2u * (u_begin + n) + t);
#pragma unroll
          for (uint32_t a = 0; a < 2; ++a)
            tma_load_3d_pair(sV + st * V_STAGE + t * V_TILE + a * KV_ATOM, &tm_v, full, int32_t(dh * HDV + xi * 128u + a * 64u),
                             int32_t((jt * TN - p.pos_base) & p.ring_mask), int32_t(kvh));
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- MMA issuer: the leader's warp, for both CTAs of the pair
    // The whole warp runs the loop and its waits and one elected lane issues.
    if (n_local > 0 && is_leader) {
      auto lead = [&]() -> bool { return elect_one(); };
      // a wait of the whole warp has one outcome for all its lanes
      auto uni = [&](bool ok1) -> bool { return __all_sync(0xffffffffu, ok1); };
      // completion signal to the same barrier in both CTAs
      auto commit2 = [&](uint32_t idx) {
        umma_commit_pair(lead_bar(idx));
        umma_commit_pair(pair_bar(idx));
      };
      constexpr uint32_t IDESC_QK = umma_idesc_bf16(2 * BM, TN, 0, 0);    // M = 256 over the pair; A, B K-major
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(2 * BM, HDV, 0, 1);   // B (= V) MN-major, 128 of its 256 columns per CTA
      constexpr uint32_t HI = (1024u >> 4) | (1u << 14) | (2u << 29);     // SBO 1024, version 1, 128B swizzle
      const uint32_t q_lo = ((sQ >> 4) & 0x3FFFu) | ((16u >> 4) << 16);
      const uint32_t k_lo = ((sK >> 4) & 0x3FFFu) | ((16u >> 4) << 16);
      const uint32_t v_lo = ((sV >> 4) & 0x3FFFu) | ((KV_ATOM >> 4) << 16);   // LBO = 64-column chunk stride
      auto mkdesc = [](uint32_t lo, uint32_t hi) { return (uint64_t(hi) << 32) | uint64_t(lo); };
      const bool prof = p.stamps != nullptr;
      long long w_k = 0, w_v = 0, w_p = 0, w_pr = 0;
      const long long t_loop = clock64();
      // the other CTA's Q tile half in shared memory is ordinary stores of its threads: cluster scope
      bool ok = uni(mbar_wait_cluster(bar_addr(bar_base, B_Q), 0u, abort_flag));
      auto issue_qk = [&](uint32_t n) -> bool {
        const uint32_t st = n & 1u;
        if (!uni(timed_wait(prof, w_k, [&] { return mbar_wait(bar_addr(bar_base, B_K_FULL + st), (n >> 1) & 1u, abort_flag); }))) return false;
        tc_fence_after();
        if (lead()) {
          const uint32_t d_tmem = tmem + T_S + (n & 1u) * TN;
#pragma unroll 1
          for (uint32_t a = 0; a < 4; ++a) {
            // contraction steps 0-15: Q[:, 0:256] from tensor memory
            const uint32_t kb = k_lo + st * (K_STAGE >> 4) + a * (K_ATOM >> 4);
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk)
              umma_ts_pair(d_tmem, tmem + T_Q + a * 32u + kk * 8u, mkdesc(kb + kk * 2u, HI), IDESC_QK, (a | kk) != 0u);
          }
#pragma unroll 1
          for (uint32_t a = 4; a < 8; ++a) {
            // contraction steps 16-31: Q[:, 256:512] from shared memory
            const uint32_t kb = k_lo + st * (K_STAGE >> 4) + a * (K_ATOM >> 4);
            const uint32_t qa = q_lo + (a - 4u) * (Q_ATOM >> 4);
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk)
              umma_ss_pair(d_tmem, mkdesc(qa + kk * 2u, HI), mkdesc(kb + kk * 2u, HI), IDESC_QK, 1u);
          }
          commit2(B_K_EMPTY + st);          // the K stage may be refilled, in both CTAs
          commit2(B_S_FULL + (n & 1u));     // S ready, in both CTAs
        }
        __syncwarp();
        return true;
      };
      ok = ok && issue_qk(0);
      for (uint32_t n = 0; ok && n < n_local; ++n) {
        if (n + 1 < n_local) {
          ok = issue_qk(n + 1);
          if (!ok) break;
        }
        const uint32_t b = n & 1u, k = n >> 1, st = n & 1u;
        // the pair's own tile (tile dh of the step): P of both CTAs in tensor memory
        if (!uni(timed_wait(prof, w_p, [&] { return mbar_wait(bar_addr(bar_base, B_P_FULL + b), k & 1u, abort_flag); }))) break;
        if (!uni(timed_wait(prof, w_v, [&] { return mbar_wait(bar_addr(bar_base, B_V_FULL + st), k & 1u, abort_flag); }))) break;
        tc_fence_after();
        const uint32_t p_tmem = tmem + T_S + b * TN;
        const uint32_t vb = v_lo + st * (V_STAGE >> 4);
        if (lead()) {
#pragma unroll
          for (uint32_t ks = 0; ks < TN / 16; ++ks)
            umma_ts_pair(tmem + T_O, p_tmem + ks * 8u, mkdesc(vb + dh * (V_TILE >> 4) + ks * (2048u >> 4), HI), IDESC_PV,
                         (n | ks) != 0u);
        }
        __syncwarp();
        // the other tile of the step: its P, relayed into columns [32, 64) of the same buffer in both CTAs
        if (!uni(timed_wait(prof, w_pr, [&] { return mbar_wait(bar_addr(bar_base, B_P2_FULL + b), k & 1u, abort_flag); }))) break;
        tc_fence_after();
        if (lead()) {
#pragma unroll
          for (uint32_t ks = 0; ks < TN / 16; ++ks)
            umma_ts_pair(tmem + T_O, p_tmem + 32u + ks * 8u, mkdesc(vb + peer * (V_TILE >> 4) + ks * (2048u >> 4), HI), IDESC_PV, 1u);
          commit2(B_V_EMPTY + st);          // PV of this step done: the V stage is free, O may be rescaled
          if (n + 1 == n_local) commit2(B_O_FINAL);
        }
        __syncwarp();
      }
      if (prof && lane == 0) {
        stamp_cycles(p, 6, w_k);
        stamp_cycles(p, 7, w_v);
        stamp_cycles(p, 8, w_p);
        stamp_cycles(p, 9, clock64() - t_loop);
        stamp_cycles(p, 10, w_pr);
      }
    }
  }

  // ------------------------------------------------------------------ row sums: two warpgroups, two CTAs
  bool have_o = false;
  if (warp < SM_WARPS) {
    have_o = __all_sync(0xffffffffu, n_local > 0 && !*abort_flag);
    if (have_o) {
      have_o = __all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, B_O_FINAL), 0u, abort_flag));
      tc_fence_after();
    }
    // all MMAs and loads of this CTA have completed (or it gave up): the K region is free.  The warpgroup that
    // took the last step holds the final reference maximum.
    float* lsum = reinterpret_cast<float*>(smem + O_LSUM);
    const uint32_t last_grp = (n_local > 0) ? ((n_local - 1u) & 1u) : 0u;
    if (grp == last_grp) m_ref[r] = m_seen;
    asm volatile("bar.sync 9, %0;" ::"n"(SM_WARPS * 32) : "memory");
    const float m_fin = m_ref[r];
    if (m_fin != m_seen) {
      l_part *= (m_seen == -INFINITY) ? 0.f : fast_exp2(m_seen - m_fin);
      m_seen = m_fin;
    }
    lsum[grp * BM + r] = l_part;
    asm volatile("bar.sync 9, %0;" ::"n"(SM_WARPS * 32) : "memory");
    if (grp == 0) {
      const float l_cta = lsum[r] + lsum[BM + r];
      lsum[r] = l_cta;
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dsmem_addr(smem_base + O_LPEER + r * 4u, peer_rank)), "f"(l_cta) : "memory");
    }
  }
  // every remote store and arrival of both CTAs lies before this barrier; neither CTA leaves before the other
  // has passed it
  cluster_sync_all();

  // ------------------------------------------------------------------ epilogue (softmax warps)
  if (warp < SM_WARPS) {
    const float* lsum = reinterpret_cast<const float*>(smem + O_LSUM);
    const float* lpeer = reinterpret_cast<const float*>(smem + O_LPEER);
    const float l_tot = lsum[r] + lpeer[r];
    // the Q tile is dead: its shared memory stages the stores
    store_o_half(p, smem + O_Q, tmem, kvh, mt, split, dh, smw, lane, grp, have_o, m_seen, l_tot);
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
  // neither CTA of a pair frees tensor memory while the other still reads its O
  cluster_sync_all();
  if (warp == W_MMA) tmem_dealloc_pair(tmem, TMEM_COLS);

  // ------------------------------------------------------------------ split merge by the last CTA to arrive
  if (p.n_splits > 1) merge_splits_last(p, &ctl[2], kvh, mt, dh, THREADS);
}

cudaError_t sm100_hd512q_configure() {
  return cudaFuncSetAttribute(dg_attn_sm100_hd512q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(h5::SMEM_REQ));
}

// tm_k, tm_v: 3-D tensor maps {512, cap, Hkv} with boxes {64 d, 64 keys, 1}
cudaError_t launch_attn_sm100_hd512q(const AttnParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                                     cudaStream_t st) {
  const dim3 grid(sm100_query_tiles(p.C, p.G, p.Hkv), p.n_splits, 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(h5q::THREADS);
  cfg.dynamicSmemBytes = h5::SMEM_REQ;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 2;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, dg_attn_sm100_hd512q_kernel, p, tm_k, tm_v);
}

}  // namespace dg
