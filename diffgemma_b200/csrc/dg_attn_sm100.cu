// Denoise-step canvas attention for head_dim 256 on sm_100a: one fused flash-style kernel.
//
//   * Q prologue in the kernel: per-head RMSNorm(+weight) + split-half RoPE on the CTA's 128
//     query rows, rounded to bf16 and written straight into the UMMA shared-memory layout (one warp
//     per row, the raw rows copied asynchronously into place before the set-up barrier).
//   * K/V tiles of 128 keys are TMA-staged (3-D tiled loads, 128-byte swizzle, no multicast) from
//     the head-major bf16 cache K[Hkv][cap][256], V[Hkv][cap][256]; a ring cache (sliding layers) keeps
//     key position t in slot t & ring_mask, and because the ring is a multiple of 128 slots a key
//     tile stays one contiguous box.
//   * S = Q K^T and O += P V run on tcgen05.mma with fp32 accumulators in tensor memory:
//     TMEM columns [0,128) and [128,256) double-buffer S, [256,512) hold O; P (bf16) overwrites
//     the first 64 columns of its S buffer and is consumed from TMEM as the A operand.
//   * online softmax in registers, four threads per query row (32 key columns each), packed
//     fp32x2 arithmetic, lazy rescaling of O (only when the running maximum grows by more than 2^8).
//   * two forms of the same kernel (template parameter PAIR): one CTA per query tile, or CTA pairs
//     (tcgen05 cta_group::2, M = 256) where every CTA stages only half of each K/V tile in two
//     stages.  The single-CTA form is bound by shared-memory bandwidth (per 128-key tile it reads
//     Q 64 KB + K 64 KB + V 64 KB as MMA operands and takes 128 KB of TMA writes = 320 KB against
//     128 B/clk = 2,560 cycles, the MMAs alone need 2,048); the pair form moves 192 KB per tile.
//   * intra-GPU split-KV: grid.y CTAs share one query tile.  Consecutive splits form a thread-block
//     cluster (2 / 4 / 8 in the single-CTA form, 2 pairs in the pair form): every CTA pushes its partial
//     rows into the shared memory of the CTA that owns them - as fp16 with a power-of-two scale per
//     row, because an SM moves only about 16 B/clk into another SM - and merges the rows it owns.
//     Groups that are left meet in a global workspace, per warp: the warp of the last group to
//     arrive at a four-row counter folds the others into the rows it still holds.  Split counts
//     that form no cluster write whole partials to the workspace and the last CTA to arrive merges.
//     Either way there is no second launch, and the result does not depend on arrival order.
//   * the MMA-issuing thread is the critical resource: it shares a scheduler with four softmax
//     warps, so its instruction stream is kept short (rolled loops, descriptor adds, one commit per
//     MMA group - S_FULL doubles as "K stage free", V_EMPTY as "PV done") and nothing is polled.
//
// Query rows are the GQA-stacked rows of one KV head: stacked row R -> canvas row R / G, query
// head kvh*G + R % G, so all 128 rows of a CTA reuse the same K/V tiles.
//
// Semantics restated from the reference (paths relative to the reference project):
//   src/shaders/attn/attention/attention.metal:22-133 (denoise mask, online softmax),
//   src/shaders/attn/attention/attention_mma2.metal:53-307 (tiled variant, p = 0 for masked keys,
//   fully masked row -> 0), src/shaders/include/attention_device.metal:154-165 ((m, l, O) state).
#include <cuda.h>

#include "dg_append_vec.cuh"
#include "dg_attn_sm100_common.cuh"
#include "dg_kernels.h"

namespace dg {

using namespace sm100;

// Four softmax warpgroups.  Warps w, w+4, w+8, w+12 share the 32 query rows of
// TMEM quadrant w & 3; warpgroup q = w >> 2 handles key columns [32 q, 32 q + 32) of every tile, so
// each scheduler has four softmax warps in flight to hide TMEM, MUFU and barrier latency.
namespace one {
constexpr uint32_t NTR = 4;                       // threads per query row
constexpr uint32_t SM_WARPS = 4 * NTR;            // 16 softmax warps
constexpr uint32_t W_K = SM_WARPS, W_V = SM_WARPS + 1, W_MMA = SM_WARPS + 2;
constexpr uint32_t THREADS = (SM_WARPS + 3) * 32;   // 608
constexpr uint32_t CPT = BN / NTR;                // 32 key columns per thread
constexpr uint32_t OPT = HD / NTR;                // 64 output columns per thread
// CTA-pair form: every CTA stages half of each tile - 64 keys of K (4 atoms of 64 rows x 128 B),
// 128 value columns of V (2 atoms of 128 rows x 128 B) - in two stages each
constexpr uint32_t K_STAGE = 32768, K_ATOM = 8192, V_STAGE = 32768;
// barrier slots.  In the pair form Q, K_FULL, V_FULL and P_FULL are used in the pair's leader only
// (arrivals and byte counts of both CTAs land there); the others exist in both CTAs.
enum : uint32_t {
  B_Q = 0,
  B_K_FULL = 1,    // +stage
  B_V_FULL = 3,    // +stage
  B_V_EMPTY = 7,   // +(tile & 1): PV of the tile complete -> its V stage is free, O may be rescaled
  B_S_FULL = 9,    // +(tile & 1): QK of the tile complete -> S is ready, its K stage is free
  B_P_FULL = 11,   // +buffer: P of the tile's keys [0, 64)
  B_O_FINAL = 14,  // single phase: every PV of this CTA has completed
  B_P2_FULL = 15,  // +buffer: P of the tile's keys [64, 128)
  B_COUNT = 17
};
}  // namespace one

// named barrier of the NTR warps that own the same 32 query rows
__device__ __forceinline__ void row_group_sync(uint32_t smw) {
  asm volatile("bar.sync %0, %1;" ::"r"(smw + 1u), "n"(one::NTR * 32) : "memory");
}

// PAIR = false: one CTA per (query tile, key split), tm_k / tm_v with boxes {64 d, 128 keys}.
// PAIR = true: two CTAs on the two SMs of a TPC own two adjacent query tiles of one KV head; one
// thread of the pair's leader issues M = 256 MMAs (cta_group::2) that span both: each CTA supplies
// its own 128 query rows and HALF of every K/V tile from its own shared memory (64 of the 128 keys
// for S, 128 of the 256 value columns for O), so every K/V byte enters an SM's shared memory once
// per pair and is read from it half as often.  tm_k then has boxes {64 d, 64 keys}.  No load uses
// multicast.
// blockIdx.z selects one of the independent canvases of the launch: its parameters and tensor maps.
template <bool PAIR>
__global__ void __launch_bounds__(one::THREADS, 1)
dg_attn_sm100_kernel(const __grid_constant__ AttnBatch bat) {
  using namespace one;
  const AttnParams& p = bat.p[blockIdx.z];
  const CUtensorMap& tm_k = bat.tm_k[blockIdx.z];
  const CUtensorMap& tm_v = bat.tm_v[blockIdx.z];
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + OFF_Q, sK = smem_base + OFF_K, sV = smem_base + OFF_V;
  const uint32_t bar_base = smem_base + OFF_BAR;
  volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + OFF_BAR + B_COUNT * 8);
  // ctl[0] = TMEM base address, ctl[1] = abort flag, ctl[2] = "this CTA merges" flag
  float* xch_max = reinterpret_cast<float*>(smem + OFF_XCH);   // [2 tile parities][BM][NTR]
  float* xch_misc = xch_max + 2 * BM * NTR;                     // [BM][NTR]: row maxima of |O| for the fp16 exchange
  float* xch_l = xch_misc + BM * NTR;                           // [BM][NTR]: final softmax denominators

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t tiles_per_head = (p.C * p.G + BM - 1) / BM;
  // pair form: tiles per head rounded up to whole pairs; a padding tile has only invalid rows
  const uint32_t tiles_x = PAIR ? ((tiles_per_head + 1u) & ~1u) : tiles_per_head;
  const uint32_t kvh = blockIdx.x / tiles_x;
  const uint32_t mt = blockIdx.x % tiles_x;
  const uint32_t split = blockIdx.y;
  const uint32_t rows_per_head = p.C * p.G;
  const MaskParams mk = p.mask;

  // position in the cluster: (1, S, 1) or, in the pair form, (2, S, 1) with x fastest
  const uint32_t crank = (PAIR || p.cluster_splits > 1) ? cluster_ctarank() : 0u;
  // split merge, level 1: cs consecutive splits form a cluster and merge through shared memory;
  // level 2: the n_splits / cs groups meet in the global workspace
  const uint32_t cs = p.cluster_splits, n_groups = p.n_splits / cs, grp = split / cs;
  const uint32_t xi = PAIR ? (crank & 1u) : 0u;          // position inside the pair
  const uint32_t leader = crank & ~1u;                    // pair form: cluster rank of the pair's leader
  const bool is_leader = xi == 0u;
  auto lead_bar = [&](uint32_t idx) { return dsmem_addr(bar_addr(bar_base, idx), leader); };
  auto peer_bar = [&](uint32_t idx) { return dsmem_addr(bar_addr(bar_base, idx), leader | 1u); };
  // bounded wait on one of this CTA's own barriers.  Only the Q barrier orders ordinary shared
  // memory written by the other CTA of a pair and needs cluster scope; the others order TMA bytes
  // or tensor-memory contents, which carry their own fences.
  auto wait_bar = [&](uint32_t idx, uint32_t parity, volatile uint32_t* flag) -> bool {
    return (PAIR && idx == B_Q) ? mbar_wait_cluster(bar_addr(bar_base, idx), parity, flag)
                                : mbar_wait(bar_addr(bar_base, idx), parity, flag);
  };

  // both CTAs of a pair walk the same key tiles: schedule from the pair's first canvas row
  const uint32_t row_first = ((PAIR ? (mt & ~1u) : mt) * BM) / p.G;
  const uint32_t row_last = (((PAIR ? (mt | 1u) : mt) + 1u) * BM - 1u) / p.G;
  const TileSched ts = tile_sched(mk, row_first < p.C ? row_first : p.C - 1, row_last < p.C ? row_last : p.C - 1);
  const uint32_t n_tiles = ts.nA + ts.nB;
  const uint32_t v_begin = uint32_t((uint64_t(split) * n_tiles) / p.n_splits);
  const uint32_t v_end = uint32_t((uint64_t(split + 1) * n_tiles) / p.n_splits);
  const uint32_t n_local = v_end - v_begin;

  // Q prologue, first half: a warp copies its eight raw query rows asynchronously into their final
  // (swizzled) place, lane c the 16-byte chunk c of each row.  When Q does not come from the kernel
  // that precedes this one on the stream, the copies are issued before the set-up barrier and fly
  // during it.
  auto issue_q_rows = [&]() {
    constexpr uint32_t RPW = BM / SM_WARPS;
    const uint32_t c = lane, R0 = mt * BM + warp * RPW;
    uint8_t* q_own = smem + OFF_Q + (c >> 3) * ATOM_BYTES + warp * RPW * 128u;
    uint32_t i = R0 / p.G, g = R0 % p.G;
#pragma unroll
    for (uint32_t it = 0; it < RPW; ++it) {
      const bool valid = R0 + it < rows_per_head;   // warp-uniform; rows past the end are zero-filled
      const __nv_bfloat16* src = valid ? p.q + (size_t(i) * p.Hq + kvh * p.G + g) * HD + c * 8u : p.q;
      cp_async_16(smem_u32(q_own + it * 128u + (((c & 7u) ^ it) << 4)), src, valid ? 16u : 0u);
      if (++g == p.G) { g = 0; ++i; }
    }
  };
  // Let the kernel that follows this one on the stream be scheduled as soon as SMs free up, if it was
  // launched to allow that (the library's own append, attention and merge kernels are; each of them waits
  // for this grid's completion before it touches anything this grid reads or writes).  Every CTA of this
  // grid has started by the time the last one executes this, so a waiting successor never keeps a CTA of
  // this grid off the device.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (p.early_q && warp < SM_WARPS) issue_q_rows();
  stamp(p, 0);
  // ------------------------------------------------------------------ set-up
  if (tid == 0) {
    mbar_init(bar_addr(bar_base, B_Q), (PAIR ? 2u : 1u) * SM_WARPS);   // one arrival per softmax warp
    for (uint32_t st = 0; st < 2; ++st) {
      mbar_init(bar_addr(bar_base, B_K_FULL + st), 1);
      mbar_init(bar_addr(bar_base, B_V_FULL + st), 1);
      mbar_init(bar_addr(bar_base, B_V_EMPTY + st), 1);
      mbar_init(bar_addr(bar_base, B_S_FULL + st), 1);
      mbar_init(bar_addr(bar_base, B_P_FULL + st), (PAIR ? 2u : 1u) * SM_WARPS);
      mbar_init(bar_addr(bar_base, B_P2_FULL + st), (PAIR ? 2u : 1u) * SM_WARPS);
    }
    mbar_init(bar_addr(bar_base, B_O_FINAL), 1);
    ctl[1] = 0u;
    ctl[2] = 0u;
    fence_mbar_init();
  }
  if (warp == W_MMA) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(&ctl[0])), TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(const_cast<uint32_t*>(&ctl[0])), TMEM_COLS);
      tmem_relinquish();
    }
  }
  if ((warp == W_K || warp == W_V) && lane == 0) tma_prefetch_desc(warp == W_K ? &tm_k : &tm_v);
  tc_fence_before();
  __syncthreads();
  // pair form: the peer's barriers must exist before anything of ours can signal them
  if (PAIR) cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = ctl[0];
  // Programmatic dependent launch: everything above overlapped the tail of the preceding kernel
  // on the stream (the canvas K/V append, which also writes the RoPE table); its results are
  // needed from here on.
  // The softmax warps read Q, its norm weight and the RoPE table: when none of those comes from
  // that kernel (the table is cached across steps at the same positions) they skip the wait, so the
  // whole Q prologue overlaps the append; the loaders always wait before they touch the cache.
  if (!(p.early_q && warp < SM_WARPS)) asm volatile("griddepcontrol.wait;" ::: "memory");
  stamp(p, 1);
  volatile uint32_t* abort_flag = &ctl[1];
  const bool prof = p.stamps != nullptr;
  long long w_s = 0, w_r = 0;

  // softmax-thread geometry: TMEM quadrant smw, row r of the query tile, column quarter qd
  const uint32_t smw = warp & 3u, qd = (warp >> 2) & (NTR - 1u);
  const uint32_t r = smw * 32 + lane;
  // per-row softmax state (identical in every thread of a row, except l_run which is per quarter)
  float m_used = -INFINITY, l_run = 0.f;

  if (warp < SM_WARPS) {
    // ---------------------------------------------------------------- Q prologue (one warp per row)
    // A warp takes eight rows of the tile; lane c owns the 16-byte chunk c of a row, so every global
    // access is one contiguous 512-byte row.  The raw rows are copied asynchronously straight into
    // their final (swizzled) place; each lane then reads back its own chunk and its RoPE partner,
    // chunk c ^ 16, and overwrites its own chunk with
    //     rsqrt(mean(x^2) + eps) * (x * (w cos) -/+ partner * (w_partner sin)),
    // in packed fp32 pairs.  The prologue is bound by instruction issue (sixteen warps on four
    // schedulers), so the per-row work is kept to the reads, one butterfly and four packed products.
    // Consecutive stacked rows share their canvas row, hence their table entries, G at a time.
    {
      constexpr uint32_t RPW = BM / SM_WARPS;
      const bool do_norm = !p.q_prenormed;
      const uint32_t c = lane, c16 = lane & 15u;
      const uint32_t R0 = mt * BM + warp * RPW;
      const uint32_t i0 = R0 / p.G, g0 = R0 % p.G;
      // byte offset of (row it of this warp, chunk c): (c ^ 16) has the same low three bits, so the
      // partner sits at the same place two swizzle atoms away
      uint8_t* q_own = smem + OFF_Q + (c >> 3) * ATOM_BYTES + warp * RPW * 128u;
      uint8_t* q_par = smem + OFF_Q + ((c ^ 16u) >> 3) * ATOM_BYTES + warp * RPW * 128u;
      if (!p.early_q) issue_q_rows();
      if (do_norm) {
        uint4 w4 = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u), wp4 = w4;   // bf16 1.0
        if (p.qw) {
          w4 = reinterpret_cast<const uint4*>(p.qw)[c];
          wp4 = reinterpret_cast<const uint4*>(p.qw)[c ^ 16u];
        }
        // low half of a row: x cos - partner sin; high half: x cos + partner sin
        const float sgn = lane < 16u ? -1.0f : 1.0f;
        const uint64_t sgn2 = pack_f32x2(sgn, sgn);
        const uint32_t wm[4] = {w4.x, w4.y, w4.z, w4.w};
        const uint32_t wq[4] = {wp4.x, wp4.y, wp4.z, wp4.w};
        uint64_t wm2[4], wq2[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          wm2[e] = bf16x2_to_f32x2(wm[e]);
          wq2[e] = mul_f32x2(bf16x2_to_f32x2(wq[e]), sgn2);
        }
        uint64_t A[4], B[4];   // w cos and -/+ w_partner sin of this lane's eight pairs
        float4 raw[4];         // the table entries of the NEXT canvas row, requested one canvas row ahead
        auto fetch_table = [&](uint32_t i) {
          // (cos, sin) of the pairs 8 c16 .. 8 c16 + 7 of canvas row i
          const float4* tab = reinterpret_cast<const float4*>(p.rope_table + size_t(i < p.C ? i : p.C - 1u) * 128 + c16 * 8u);
#pragma unroll
          for (int e = 0; e < 4; ++e) raw[e] = tab[e];
        };
        auto use_table = [&]() {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            A[e] = mul_f32x2(wm2[e], pack_f32x2(raw[e].x, raw[e].z));
            B[e] = mul_f32x2(wq2[e], pack_f32x2(raw[e].y, raw[e].w));
          }
        };
        if (R0 < rows_per_head) fetch_table(i0);
        cp_async_wait_all();
        __syncwarp();
        uint32_t i = i0, g = g0;
        if (R0 < rows_per_head) {
          use_table();
          fetch_table(i0 + 1u);   // in flight while the rows of canvas row i0 are worked on
        }
#pragma unroll
        for (uint32_t it = 0; it < RPW; ++it) {
          if (R0 + it >= rows_per_head) break;   // warp-uniform
          if (it != 0 && g == 0) {
            use_table();
            fetch_table(i + 1u);
          }
          const uint32_t off = it * 128u + (((c & 7u) ^ it) << 4);
          const uint4 xm = *reinterpret_cast<const uint4*>(q_own + off);
          const uint4 xq = *reinterpret_cast<const uint4*>(q_par + off);
          const uint32_t m[4] = {xm.x, xm.y, xm.z, xm.w};
          const uint32_t q[4] = {xq.x, xq.y, xq.z, xq.w};
          uint64_t m2[4];
          uint64_t acc = 0ull;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            m2[e] = bf16x2_to_f32x2(m[e]);
            acc = fma_f32x2(m2[e], m2[e], acc);
          }
          float s0, s1;
          unpack_f32x2(acc, s0, s1);
          float ss = s0 + s1;
#pragma unroll
          for (uint32_t o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // identical in every lane
          const float inv = rsqrtf(ss * (1.0f / float(HD)) + p.eps);
          const uint64_t inv2 = pack_f32x2(inv, inv);
          uint32_t y[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint64_t t = fma_f32x2(m2[e], A[e], mul_f32x2(bf16x2_to_f32x2(q[e]), B[e]));
            float y0, y1;
            unpack_f32x2(mul_f32x2(t, inv2), y0, y1);
            y[e] = pack_bf16x2(y0, y1);
          }
          __syncwarp();   // the partner has read this chunk
          *reinterpret_cast<uint4*>(q_own + off) = make_uint4(y[0], y[1], y[2], y[3]);
          if (++g == p.G) { g = 0; ++i; }
        }
      } else {
        cp_async_wait_all();
      }
    }
    if (PAIR) fence_proxy_async_all(); else fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (PAIR) mbar_arrive_cluster(lead_bar(B_Q)); else mbar_arrive(bar_addr(bar_base, B_Q));
    }
    stamp(p, 2);

    // ---------------------------------------------------------------- canvas append inside the launch
    // The 2 C Hkv head vectors of canvas K / V are cut into units of up to four heads of one token's K or V (the
    // token's rotation is prepared once per unit) and the units into shares of one unit per softmax warp.  Every CTA
    // that gets here keeps taking shares from a counter until none is left, so all shares are taken by CTAs
    // that are running - also when part of the grid has not been scheduled yet (more clusters than fit) - and
    // none of them needs anything from anybody to finish its shares.  Whoever waits for the append (the
    // loaders, before a key tile that holds canvas positions) therefore never waits for a CTA that has not
    // started.  The window between "Q is ready" and the first score tile is otherwise idle for these warps.
    // The last CTA to leave the kernel puts the counters back to zero.
    if (p.ap_vectors != 0u) {
      if (p.early_q) asm volatile("griddepcontrol.wait;" ::: "memory");   // the cache may still be in use ahead of us
      AppendVecArgs av;
      av.k_in = p.ap_k;
      av.v_in = p.ap_v;
      av.kw = p.ap_kw;
      av.table = p.rope_table;
      av.cache_k = p.ap_cache_k;
      av.cache_v = p.ap_cache_v;
      av.cap = p.cap;
      av.pos0 = mk.kv_len;
      av.Hkv = p.Hkv;
      av.v_norm = p.ap_v_norm;
      av.ring_mask = p.ring_mask;
      av.write_end = p.ap_write_end;
      av.pos_base = p.pos_base;
      av.eps = p.eps;
      // a share = one unit (up to four heads of one token's K or V) for every softmax warp
      const uint32_t n_units = append_unit_count(p.ap_vectors / (2u * p.Hkv), p.Hkv);
      const uint32_t n_shares = (n_units + SM_WARPS - 1u) / SM_WARPS;
      uint4 kw_own, kw_partner;
      append_norm_weight(av, lane, kw_own, kw_partner);
      // In a share the K units (norm, rotation) and the V units (a copy unless V is normed) of a token alternate
      // in runs of `groups`; odd shares shift the warps by one run, so that no warp gets the K units every time.
      const uint32_t groups = (p.Hkv + APPEND_UNIT_HEADS - 1u) / APPEND_UNIT_HEADS;
      uint32_t mine = 0;
      // the next share number is asked for before the work on this one starts: its round trip through the counter
      // (about 500 cycles) then runs beside the work
      if (tid == 0) ctl[3u] = atomicAdd(p.ap_ctl, 1u);
      for (uint32_t it = 0;; ++it) {
        // two slots in turn: a slot is rewritten only after the barrier that follows everybody's read of it
        asm volatile("bar.sync 5, %0;" ::"n"(SM_WARPS * 32) : "memory");
        const uint32_t share = ctl[3u + (it & 1u)];
        if (share >= n_shares) break;
        uint32_t next = 0;
        if (tid == 0) next = atomicAdd(p.ap_ctl, 1u);
        const uint32_t u = share * SM_WARPS + ((warp + (share & 1u) * groups) % SM_WARPS);
        if (u < n_units) mine += append_table_unit(av, u, lane, kw_own, kw_partner);
        if (tid == 0) ctl[3u + ((it + 1u) & 1u)] = next;
      }
      if (mine != 0u) {
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(p.ap_ctl + 1, mine);
      }
    }

    // ---------------------------------------------------------------- softmax main loop
    const uint32_t R = mt * BM + r;
    const uint32_t i_row = (R < rows_per_head) ? R / p.G : p.C - 1;
    const RowVis rv = mask_row(mk, i_row);
    const uint32_t t_lane = tmem + ((smw * 32u) << 16);
    const float sc = p.scale_log2;
    const uint32_t p_full0 = PAIR ? lead_bar(B_P_FULL) : bar_addr(bar_base, B_P_FULL);
    const uint32_t p_full1 = PAIR ? lead_bar(B_P_FULL + 1) : bar_addr(bar_base, B_P_FULL + 1);
    const uint32_t p2_full0 = PAIR ? lead_bar(B_P2_FULL) : bar_addr(bar_base, B_P2_FULL);
    const uint32_t p2_full1 = PAIR ? lead_bar(B_P2_FULL + 1) : bar_addr(bar_base, B_P2_FULL + 1);

    for (uint32_t n = 0; n < n_local; ++n) {
      const uint32_t v = v_begin + n;
      const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
      const uint32_t k0 = jt * BN;
      const uint32_t b = n & 1u;
      // warp-uniform outcome: the TMEM instructions below need the whole warp
      if (!__all_sync(0xffffffffu, timed_wait(prof, w_s, [&] { return wait_bar(B_S_FULL + b, (n >> 1) & 1u, abort_flag); }))) break;
      tc_fence_after();
      // This thread's 32 score columns are keys [16 qd, 16 qd + 16) and [64 + 16 qd, 64 + 16 qd + 16) of the tile:
      // every thread then finishes its share of the tile's first 64 keys first, and the PV MMAs over those keys
      // run while the exponentials of the other 64 are still being computed.
      uint32_t sraw[32];
      tmem_ld16(t_lane + TM_S + b * 128u + qd * (CPT / 2), *reinterpret_cast<uint32_t(*)[16]>(&sraw[0]));
      tmem_ld16(t_lane + TM_S + b * 128u + 64u + qd * (CPT / 2), *reinterpret_cast<uint32_t(*)[16]>(&sraw[16]));
      tmem_wait_ld();

      if (!mask_range_full(mk, rv, k0, BN)) {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (!mask_visible_row(mk, rv, k0 + (e < 16 ? 0u : 48u) + qd * (CPT / 2) + e)) sraw[e] = 0xff800000u;  // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 32; e += 2)
        mx4[(e >> 1) & 3] = max3_f32(mx4[(e >> 1) & 3], __uint_as_float(sraw[e]), __uint_as_float(sraw[e + 1]));
      const float mx_part = max3_f32(max3_f32(mx4[0], mx4[1], mx4[2]), mx4[3], -INFINITY);
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
        if (!__all_sync(0xffffffffu, timed_wait(prof, w_r, [&] { return wait_bar(B_V_EMPTY + ((n - 1) & 1u), ((n - 1) >> 1) & 1u, abort_flag); }))) break;
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
      // P column j (32 bit) = keys (2j, 2j+1) as bf16x2: each run of 16 keys is 8 columns.
      // Scale/shift and row sums run on packed fp32 pairs.
      const uint64_t sc2 = pack_f32x2(sc, sc), nm2 = pack_f32x2(neg_m, neg_m);
      uint64_t ls2[2] = {0ull, 0ull};   // (0.f, 0.f)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t pk[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[hf * 16 + e]), __uint_as_float(sraw[hf * 16 + e + 1])), sc2, nm2), x0, x1);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          ls2[(e >> 1) & 1] = add_f32x2(ls2[(e >> 1) & 1], pack_f32x2(p0, p1));
          pk[e >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st8(t_lane + TM_S + b * 128u + uint32_t(hf) * 32u + qd * (CPT / 4), pk);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          const uint32_t bar = hf == 0 ? (b ? p_full1 : p_full0) : (b ? p2_full1 : p2_full0);
          if (PAIR) mbar_arrive_remote(bar); else mbar_arrive(bar);
        }
      }
      {
        float s0, s1;
        unpack_f32x2(add_f32x2(ls2[0], ls2[1]), s0, s1);
        l_run += s0 + s1;
      }
    }
    if (prof && tid == 0) {
      stamp_cycles(p, 10, w_s);
      stamp_cycles(p, 11, w_r);
    }
  } else if (warp == W_K) {
    // ---------------------------------------------------------------- K loader
    if (lane == 0) {
      bool canvas_ready = p.ap_vectors == 0u || mk.can_hi <= mk.kv_len;
      for (uint32_t n = 0; n < n_local; ++n) {
        const uint32_t v = v_begin + n;
        const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
        if (!canvas_ready && jt * BN + BN > mk.kv_len) {
          if (!wait_counter_gpu(p.ap_ctl + 1, p.ap_vectors, abort_flag)) break;
          canvas_ready = true;
        }
        if (PAIR) {
          // this CTA's 64 keys of the tile into stage n & 1
          const uint32_t st = n & 1u, u = n >> 1;
          if (u > 0 && !wait_bar(B_S_FULL + st, (u - 1) & 1u, abort_flag)) break;   // QK(n - 2) complete
          if (is_leader) mbar_expect_tx(bar_addr(bar_base, B_K_FULL + st), 2 * K_STAGE);
          const uint32_t full = lead_bar(B_K_FULL + st);
#pragma unroll
          for (uint32_t a = 0; a < 4; ++a)
            tma_load_3d_pair(sK + st * K_STAGE + a * K_ATOM, &tm_k, full, int32_t(a * 64), int32_t((jt * BN + xi * 64 - p.pos_base) & p.ring_mask),
                             int32_t(kvh));
        } else {
          if (n > 0 && !wait_bar(B_S_FULL + ((n - 1) & 1u), ((n - 1) >> 1) & 1u, abort_flag)) break;   // QK(n - 1) complete
          const uint32_t full = bar_addr(bar_base, B_K_FULL);
          mbar_expect_tx(full, TILE_BYTES);
#pragma unroll
          for (uint32_t a = 0; a < 4; ++a)
            tma_load_3d(sK + a * ATOM_BYTES, &tm_k, full, int32_t(a * 64), int32_t((jt * BN - p.pos_base) & p.ring_mask), int32_t(kvh));
        }
      }
    }
  } else if (warp == W_V) {
    // ---------------------------------------------------------------- V loader
    if (lane == 0) {
      bool canvas_ready = p.ap_vectors == 0u || mk.can_hi <= mk.kv_len;
      for (uint32_t n = 0; n < n_local; ++n) {
        const uint32_t v = v_begin + n;
        const uint32_t jt = v < ts.nA ? ts.a0 + v : ts.b0 + (v - ts.nA);
        if (!canvas_ready && jt * BN + BN > mk.kv_len) {
          if (!wait_counter_gpu(p.ap_ctl + 1, p.ap_vectors, abort_flag)) break;
          canvas_ready = true;
        }
        if (PAIR) {
          // this CTA's 128 value columns of the tile into stage n & 1
          const uint32_t st = n & 1u, u = n >> 1;
          if (u > 0 && !wait_bar(B_V_EMPTY + st, (u - 1) & 1u, abort_flag)) break;
          if (is_leader) mbar_expect_tx(bar_addr(bar_base, B_V_FULL + st), 2 * V_STAGE);
          const uint32_t full = lead_bar(B_V_FULL + st);
#pragma unroll
          for (uint32_t a = 0; a < 2; ++a)
            tma_load_3d_pair(sV + st * V_STAGE + a * ATOM_BYTES, &tm_v, full, int32_t(xi * 128 + a * 64),
                             int32_t((jt * BN - p.pos_base) & p.ring_mask), int32_t(kvh));
        } else {
          if (n > 0 && !wait_bar(B_V_EMPTY + ((n - 1) & 1u), ((n - 1) >> 1) & 1u, abort_flag)) break;   // PV(n - 1) complete
          const uint32_t full = bar_addr(bar_base, B_V_FULL);
          mbar_expect_tx(full, TILE_BYTES);
#pragma unroll
          for (uint32_t a = 0; a < 4; ++a)
            tma_load_3d(sV + a * ATOM_BYTES, &tm_v, full, int32_t(a * 64), int32_t((jt * BN - p.pos_base) & p.ring_mask), int32_t(kvh));
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- MMA issuer (pair form: of the leader)
    // The whole warp runs the loop and its waits; one lane, chosen by elect.sync, issues.  With the issuing
    // branch under elect.sync the instruction stream of an MMA is shorter than under a lane == 0 test
    // (measured on the head_dim-512 kernel: a quarter less time per step with the tensor pipe free-running).
    if (n_local > 0 && is_leader) {
      auto uni = [&](bool ok1) -> bool { return __all_sync(0xffffffffu, ok1); };
      constexpr uint32_t IDESC_QK = umma_idesc_bf16(PAIR ? 2 * BM : BM, BN, 0, 0);   // A, B K-major
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(PAIR ? 2 * BM : BM, HD, 0, 1);   // B (= V) MN-major
      // completion signal: pair form -> the same barrier slot in both CTAs
      auto commit = [&](uint32_t idx) {
        if (PAIR) {
          umma_commit_pair(lead_bar(idx));
          umma_commit_pair(peer_bar(idx));
        } else {
          umma_commit(bar_addr(bar_base, idx));
        }
      };
      bool ok = uni(wait_bar(B_Q, 0u, abort_flag));
      long long w_k = 0, w_v = 0, w_p = 0;
      const long long t_loop = prof ? clock64() : 0;
      // Descriptors are advanced with adds on their low word (start address >> 4; every operand
      // lives below 256 KB, so the 14-bit field cannot carry), and the MMA loops are kept rolled: the
      // issuing thread shares its scheduler with four softmax warps, so its instruction stream must
      // stay short to keep the tensor pipe fed.
      constexpr uint32_t HI_KMAJ = (1024u >> 4) | (1u << 14) | (2u << 29);          // SBO 1024, version 1, 128B swizzle
      constexpr uint32_t HI_MNMAJ = HI_KMAJ;                                          // same SBO for V
      const uint32_t q_lo = ((sQ >> 4) & 0x3FFFu) | ((16u >> 4) << 16);              // LBO 16 (unused for K-major)
      const uint32_t k_lo0 = ((sK >> 4) & 0x3FFFu) | ((16u >> 4) << 16);
      const uint32_t v_lo0 = ((sV >> 4) & 0x3FFFu) | ((ATOM_BYTES >> 4) << 16);      // LBO = 64-column chunk stride
      auto mkdesc = [](uint32_t lo, uint32_t hi) { return (uint64_t(hi) << 32) | uint64_t(lo); };
      // The issuing thread polls (without blocking) for what the NEXT group of MMAs needs while the
      // tensor pipe still has queued work, so that the blocking wait in front of that group normally
      // finds the phase complete and the pipe does not drain at the S / O hand-over.
      //   issue_qk(n, pv): S(n) = Q K(n)^T; polls P_FULL / V_FULL of tile pv (the PV issued next)
      bool p_ready = false, v_ready = false, k_ready = false;
      auto issue_qk = [&](uint32_t n, uint32_t pv, bool poll) -> bool {
        // stage and phase of tile n: pair form two stages, else one
        const uint32_t st = PAIR ? (n & 1u) : 0u, ph = PAIR ? ((n >> 1) & 1u) : (n & 1u);
        if (!k_ready && !uni(timed_wait(prof, w_k, [&] { return wait_bar(B_K_FULL + st, ph, abort_flag); }))) return false;
        k_ready = false;
        tc_fence_after();
        if (elect_one()) {
          const uint32_t d_tmem = tmem + TM_S + (n & 1u) * 128u;
          uint32_t qa = q_lo, kb = k_lo0 + (PAIR ? st * (K_STAGE >> 4) : 0u);
          constexpr uint32_t k_atom16 = (PAIR ? K_ATOM : ATOM_BYTES) >> 4;
#pragma unroll 1
          for (uint32_t a = 0; a < 4; ++a) {
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk) {
              const uint64_t da = mkdesc(qa + kk * 2u, HI_KMAJ), db = mkdesc(kb + kk * 2u, HI_KMAJ);
              if (PAIR) umma_ss_pair(d_tmem, da, db, IDESC_QK, (a | kk) != 0u);
              else umma_ss(d_tmem, da, db, IDESC_QK, (a | kk) != 0u);
            }
            qa += ATOM_BYTES >> 4;
            kb += k_atom16;
          }
          commit(B_S_FULL + (n & 1u));
        }
        __syncwarp();
        return true;
      };
      ok = ok && issue_qk(0, 0, false);
      for (uint32_t n = 0; ok && n < n_local; ++n) {
        if (n + 1 < n_local) {
          ok = issue_qk(n + 1, n, true);
          if (!ok) break;
        }
        const uint32_t st = PAIR ? (n & 1u) : 0u, ph = PAIR ? ((n >> 1) & 1u) : (n & 1u);
        if (!p_ready && !uni(timed_wait(prof, w_p, [&] { return wait_bar(B_P_FULL + (n & 1u), (n >> 1) & 1u, abort_flag); }))) break;
        if (!v_ready && !uni(timed_wait(prof, w_v, [&] { return wait_bar(B_V_FULL + st, ph, abort_flag); }))) break;
        p_ready = v_ready = false;
        tc_fence_after();
        uint32_t p_tmem = tmem + TM_S + (n & 1u) * 128u;
        uint32_t vb = v_lo0 + (PAIR ? st * (V_STAGE >> 4) : 0u);
        // keys [0, 64) of the tile, then, once the rest of P is there, keys [64, 128)
#pragma unroll 1
        for (uint32_t hf = 0; hf < 2; ++hf) {
          if (hf == 1) {
            if (!uni(timed_wait(prof, w_p, [&] { return wait_bar(B_P2_FULL + (n & 1u), (n >> 1) & 1u, abort_flag); }))) { ok = false; break; }
            tc_fence_after();
          }
          if (elect_one()) {
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
              const uint64_t db = mkdesc(vb + j * (2048u >> 4), HI_MNMAJ);
              if (PAIR) umma_ts_pair(tmem + TM_O, p_tmem + j * 8u, db, IDESC_PV, (n | hf | j) != 0u);
              else umma_ts(tmem + TM_O, p_tmem + j * 8u, db, IDESC_PV, (n | hf | j) != 0u);
            }
            if (hf == 1) {
              commit(B_V_EMPTY + (n & 1u));
              // The epilogue must not reuse B_V_EMPTY: when the last S tile is ready only PV(n-3) is
              // known to be complete, so a parity wait on that barrier could alias by two phases.
              if (n + 1 == n_local) commit(B_O_FINAL);
            }
          }
          __syncwarp();
          vb += 4u * (2048u >> 4);
          p_tmem += 32u;
        }
        if (!ok) break;
      }
      if (prof && lane == 0) {
        stamp_cycles(p, 6, w_k);
        stamp_cycles(p, 7, w_v);
        stamp_cycles(p, 8, w_p);
        stamp_cycles(p, 9, clock64() - t_loop);
      }
    }
  }

  stamp(p, 3);
  // ------------------------------------------------------------------ epilogue (softmax warps)
  const uint32_t rows_total = p.C * p.Hq;
  bool have_o = false;
  if (warp < SM_WARPS) {
    // the warps that skipped the wait at the top must not write anything (output, workspace) that the
    // kernels ahead of this one on the stream may still use; normally long satisfied by now
    if (p.early_q) asm volatile("griddepcontrol.wait;" ::: "memory");
    have_o = __all_sync(0xffffffffu, n_local > 0 && !*abort_flag);
    if (have_o) {
      have_o = __all_sync(0xffffffffu, wait_bar(B_O_FINAL, 0u, abort_flag));
      tc_fence_after();
    }
  }
  stamp(p, 12);
  // Cluster merge: partial rows are pushed into the owner CTA's Q/K/V region, which must be dead
  // in EVERY CTA of the cluster first - all of this CTA's MMAs are complete once its softmax
  // warps have seen O_FINAL, and this barrier collects that from all CTAs.
  if (cs > 1) cluster_sync_all();
  stamp(p, 13);
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
    const bool via_dsmem = cs > 1;
    if (via_dsmem) {
      // The partial stays on chip.  Row r of the query tile is merged by CTA r / (BM / S) of the
      // cluster, so each thread pushes its columns of the un-normalised O row (and one thread the
      // row's (m, l, 1 / scale)) straight into that CTA's receive buffer with remote shared-memory
      // stores: recv[source CTA][row within the owner's share][HBUF_LD halves] in the dead Q/K/V
      // region.  An SM moves only about 16 B/clk into another SM's shared memory, so the rows travel
      // as fp16 with one power-of-two scale per row that puts the row's largest magnitude into
      // [2^14, 2^15): 11 significant bits relative to the row maximum whatever the range of V, against
      // the 8 bits of the bf16 output, and half the bytes.
      const uint32_t rpc = BM / cs;
      // split index of this CTA inside the cluster and cluster rank of the CTA that owns row r
      // (pair form: the CTA with the same position in its pair)
      const uint32_t src_rank = PAIR ? (crank >> 1) : crank;
      const uint32_t owner_split = r / rpc, rl = r % rpc;
      const uint32_t owner = PAIR ? ((owner_split << 1) | xi) : owner_split;
      // rows this CTA owns itself stay in its own shared memory (plain stores): only the others' rows
      // take the SM-to-SM path
      const bool own = owner == crank;
      const uint32_t row_local = smem_base + OFF_Q + ((src_rank * rpc + rl) * HBUF_LD) * 2u;
      const uint32_t dst_row = own ? row_local : dsmem_addr(row_local, owner);
      uint32_t oa[32], ob[32];
      if (have_o) {
        tmem_ld32(t_lane + TM_O + qd * OPT, oa);
        tmem_ld32(t_lane + TM_O + qd * OPT + 32u, ob);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (uint32_t e = 0; e < 32; ++e) oa[e] = ob[e] = 0u;
      }
      float amax = 0.f;
#pragma unroll
      for (uint32_t e = 0; e < 32; e += 2) {
        amax = max3_f32(amax, fabsf(__uint_as_float(oa[e])), fabsf(__uint_as_float(oa[e + 1])));
        amax = max3_f32(amax, fabsf(__uint_as_float(ob[e])), fabsf(__uint_as_float(ob[e + 1])));
      }
      xch_misc[r * NTR + qd] = amax;
      row_group_sync(smw);
      float rmax = 0.f;
#pragma unroll
      for (uint32_t k = 0; k < NTR; ++k) rmax = fmaxf(rmax, xch_misc[r * NTR + k]);
      // biased exponent of the row maximum; tiny, zero, infinite or NaN maxima travel unscaled
      const uint32_t eb = (__float_as_uint(rmax) >> 23) & 0xffu;
      const bool scaled = eb >= 15u && eb < 255u;
      const float sc = scaled ? __uint_as_float((268u - eb) << 23) : 1.0f;       // 2^(14 - exponent)
      const float inv_sc = scaled ? __uint_as_float((eb - 14u) << 23) : 1.0f;
#pragma unroll
      for (uint32_t q4 = 0; q4 < 4; ++q4) {
        uint32_t ha[4], hb[4];
#pragma unroll
        for (uint32_t e = 0; e < 4; ++e) {
          ha[e] = pack_f16x2(__uint_as_float(oa[q4 * 8 + 2 * e]) * sc, __uint_as_float(oa[q4 * 8 + 2 * e + 1]) * sc);
          hb[e] = pack_f16x2(__uint_as_float(ob[q4 * 8 + 2 * e]) * sc, __uint_as_float(ob[q4 * 8 + 2 * e + 1]) * sc);
        }
        if (own) {
          smem_st_u4(dst_row + (qd * OPT + q4 * 8u) * 2u, make_uint4(ha[0], ha[1], ha[2], ha[3]));
          smem_st_u4(dst_row + (qd * OPT + 32u + q4 * 8u) * 2u, make_uint4(hb[0], hb[1], hb[2], hb[3]));
        } else {
          dsmem_st_u4(dst_row + (qd * OPT + q4 * 8u) * 2u, make_uint4(ha[0], ha[1], ha[2], ha[3]));
          dsmem_st_u4(dst_row + (qd * OPT + 32u + q4 * 8u) * 2u, make_uint4(hb[0], hb[1], hb[2], hb[3]));
        }
      }
      if (qd == 0) {
        const uint32_t ml_local = smem_base + OFF_ML + (src_rank * rpc + rl) * 16u;
        const uint4 rec = make_uint4(__float_as_uint(m_used), __float_as_uint(l_tot), __float_as_uint(inv_sc), 0u);
        if (own) smem_st_u4(ml_local, rec); else dsmem_st_u4(dsmem_addr(ml_local, owner), rec);
      }
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
  if (PAIR) {
    // Neither CTA of the pair may free tensor memory or leave while the other can still be the
    // target of a pair-wide MMA or commit; in cluster-merge mode this barrier also closes the
    // exchange of partial rows.
    cluster_sync_all();
    if (warp == W_MMA) tmem_dealloc_pair(tmem, TMEM_COLS);
  } else if (warp == W_MMA) {
    tmem_dealloc(tmem, TMEM_COLS);
  }

  // ------------------------------------------------------------------ split merge, level 1: inside the cluster
  if (cs > 1) {
    // The cs CTAs that hold consecutive splits of this query tile are one thread-block cluster
    // (cluster dims (1, cs, 1), pair form (2, cs, 1)).  Every CTA has pushed each partial row to the
    // CTA that owns it; after the cluster barrier CTA k holds all cs partials of rows
    // [k*BM/cs, (k+1)*BM/cs) in its own shared memory and merges them.  Nothing touches remote
    // shared memory after the barrier, so no second barrier is needed.
    if (!PAIR) cluster_sync_all();
    stamp(p, 14);
    const uint32_t rank = PAIR ? (crank >> 1) : crank;
    const uint32_t rpc = BM / cs;
    const __half* recv = reinterpret_cast<const __half*>(smem + OFF_Q);      // [cs][rpc][HBUF_LD], scaled
    const float4* recv_ml = reinterpret_cast<const float4*>(smem + OFF_ML);  // [cs][rpc]: m, l, 1 / scale
    // A warp merges four rows at a time (lane = eight columns), every lane reading the cs (m, l)
    // pairs itself: no shuffles and four independent chains, because this pass is bound by latency
    constexpr uint32_t RK1 = 4;
    for (uint32_t rl0 = warp * RK1; rl0 < rpc; rl0 += (THREADS / 32) * RK1) {
      float mg[RK1], lg[RK1], acc[RK1][8];
#pragma unroll
      for (uint32_t k = 0; k < RK1; ++k) {
        const uint32_t rl = rl0 + k < rpc ? rl0 + k : rpc - 1;
        mg[k] = -INFINITY;
        for (uint32_t s2 = 0; s2 < cs; ++s2) mg[k] = fmaxf(mg[k], recv_ml[s2 * rpc + rl].x);
        lg[k] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[k][e] = 0.f;
      }
      for (uint32_t s2 = 0; s2 < cs; ++s2) {
#pragma unroll
        for (uint32_t k = 0; k < RK1; ++k) {
          const uint32_t rl = rl0 + k < rpc ? rl0 + k : rpc - 1;
          const float4 ml = recv_ml[s2 * rpc + rl];
          const float w = (ml.x == -INFINITY) ? 0.f : fast_exp2(ml.x - mg[k]);
          lg[k] += w * ml.y;
          const float ws = w * ml.z;   // the row's scale folded into its weight
          const uint4 x = *reinterpret_cast<const uint4*>(recv + (s2 * rpc + rl) * HBUF_LD + lane * 8);
          const float2 x0 = unpack_f16x2(x.x), x1 = unpack_f16x2(x.y), x2 = unpack_f16x2(x.z), x3 = unpack_f16x2(x.w);
          acc[k][0] += ws * x0.x; acc[k][1] += ws * x0.y; acc[k][2] += ws * x1.x; acc[k][3] += ws * x1.y;
          acc[k][4] += ws * x2.x; acc[k][5] += ws * x2.y; acc[k][6] += ws * x3.x; acc[k][7] += ws * x3.y;
        }
      }
      size_t orow[RK1];
      bool live[RK1];
#pragma unroll
      for (uint32_t k = 0; k < RK1; ++k) {
        const uint32_t R = mt * BM + rank * rpc + rl0 + k;
        live[k] = rl0 + k < rpc && R < rows_per_head;
        const uint32_t Rc = live[k] ? R : mt * BM;
        orow[k] = size_t(Rc / p.G) * p.Hq + kvh * p.G + Rc % p.G;
      }
      if (n_groups > 1) {
        // Level 2, per warp: the group's merged rows (un-normalised, relative to mg) go to the
        // workspace, the warp counts itself in on the arrival counter of these four rows, and the
        // warp of the LAST group to arrive folds the other groups' rows into the ones it still holds
        // in registers.  No CTA-wide barrier, and nobody reads its own partial back.
#pragma unroll
        for (uint32_t k = 0; k < RK1; ++k) {
          if (!live[k]) continue;
          float4* dst = reinterpret_cast<float4*>(p.ws_o + (size_t(grp) * rows_total + orow[k]) * HD + lane * 8);
          dst[0] = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
          dst[1] = make_float4(acc[k][4], acc[k][5], acc[k][6], acc[k][7]);
          if (lane == 0) reinterpret_cast<float2*>(p.ws_ml)[size_t(grp) * rows_total + orow[k]] = make_float2(mg[k], lg[k]);
        }
        __threadfence();
        __syncwarp();
        uint32_t* cnt = p.ws_counters + blockIdx.x * (BM / RK1) + (rank * rpc + rl0) / RK1;
        uint32_t old = 0;
        if (lane == 0) old = atomicAdd(cnt, 1u);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old != n_groups - 1u) continue;   // warp-uniform
        __threadfence();
        if (lane == 0) *cnt = 0u;             // ready for the next launch
        // The result must not depend on which group happened to arrive last.  With two groups the
        // fold is written symmetrically (separately rounded products, one addition), so folding the
        // other group into the rows held in registers gives the same bits either way round; with
        // more groups the rows are re-read and folded in group order.
        const bool two = n_groups == 2;
        for (uint32_t g2 = 0; g2 < n_groups; ++g2) {
          if (two && g2 == grp) continue;
          float2 ml2[RK1];
          float4 a2[RK1], b2[RK1];
#pragma unroll
          for (uint32_t k = 0; k < RK1; ++k) {
            const size_t slot = size_t(g2) * rows_total + orow[k];
            ml2[k] = __ldcg(reinterpret_cast<const float2*>(p.ws_ml) + slot);
            const float4* src = reinterpret_cast<const float4*>(p.ws_o + slot * HD + lane * 8);
            a2[k] = __ldcg(src);
            b2[k] = __ldcg(src + 1);
          }
#pragma unroll
          for (uint32_t k = 0; k < RK1; ++k) {
            if (!two && g2 == 0) {   // group order: start from group 0 as it is in the workspace
              mg[k] = ml2[k].x;
              lg[k] = ml2[k].y;
              acc[k][0] = a2[k].x; acc[k][1] = a2[k].y; acc[k][2] = a2[k].z; acc[k][3] = a2[k].w;
              acc[k][4] = b2[k].x; acc[k][5] = b2[k].y; acc[k][6] = b2[k].z; acc[k][7] = b2[k].w;
              continue;
            }
            const float mn = fmaxf(mg[k], ml2[k].x);
            const float wa = (mg[k] == -INFINITY) ? 0.f : fast_exp2(mg[k] - mn);
            const float wb = (ml2[k].x == -INFINITY) ? 0.f : fast_exp2(ml2[k].x - mn);
            lg[k] = __fadd_rn(__fmul_rn(wa, lg[k]), __fmul_rn(wb, ml2[k].y));
            mg[k] = mn;
            const float x2[8] = {a2[k].x, a2[k].y, a2[k].z, a2[k].w, b2[k].x, b2[k].y, b2[k].z, b2[k].w};
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[k][e] = __fadd_rn(__fmul_rn(wa, acc[k][e]), __fmul_rn(wb, x2[e]));
          }
        }
      }
#pragma unroll
      for (uint32_t k = 0; k < RK1; ++k) {
        if (!live[k]) continue;
        if (p.out) {
          const float inv = lg[k] > 0.f ? 1.0f / lg[k] : 0.f;
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
            p.out_m[orow[k]] = mg[k] * 0.6931471805599453f;
            p.out_l[orow[k]] = lg[k];
          }
        }
      }
    }
  }
  if (n_groups > 1 && cs == 1) {
    // ---------------------------------------------------------------- splits without clusters
    // (odd split counts, the fixed-scratch entry point): every CTA wrote its whole partial to the
    // workspace in the epilogue; one arrival counter per query tile, the last CTA to arrive merges
    const uint32_t row0 = 0, n_rows = BM;
    const uint32_t S = n_groups;
    uint32_t* counter = p.ws_counters + blockIdx.x;
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      const uint32_t old = atomicAdd(counter, 1u);
      ctl[2] = (old == S - 1u) ? 1u : 0u;
    }
    __syncthreads();
    if (ctl[2]) {
      __threadfence();
      const float2* ml_all = reinterpret_cast<const float2*>(p.ws_ml);
      if (S == 2) {
        // Two splits: one round trip.  A warp takes four rows, every lane loads
        // both (m, l) pairs and its eight columns of both partials at once.
        constexpr uint32_t RK2 = 4;
        for (uint32_t r0 = warp * RK2; r0 < n_rows; r0 += (THREADS / 32) * RK2) {
          size_t orow[RK2];
          bool live[RK2];
          float2 ml[RK2][2];
          float4 a[RK2][2], bq[RK2][2];
#pragma unroll
          for (uint32_t k = 0; k < RK2; ++k) {
            const uint32_t R = mt * BM + row0 + r0 + k;
            live[k] = (r0 + k < n_rows) && (R < rows_per_head);
            const uint32_t Rc = live[k] ? R : mt * BM;
            orow[k] = size_t(Rc / p.G) * p.Hq + kvh * p.G + Rc % p.G;
#pragma unroll
            for (uint32_t j = 0; j < 2; ++j) {
              ml[k][j] = ml_all[size_t(j) * rows_total + orow[k]];
              const float4* src = reinterpret_cast<const float4*>(p.ws_o + (size_t(j) * rows_total + orow[k]) * HD + lane * 8);
              a[k][j] = src[0];
              bq[k][j] = src[1];
            }
          }
#pragma unroll
          for (uint32_t k = 0; k < RK2; ++k) {
            if (!live[k]) continue;
            const float mg = fmaxf(ml[k][0].x, ml[k][1].x);
            const float w0 = (ml[k][0].x == -INFINITY) ? 0.f : fast_exp2(ml[k][0].x - mg);
            const float w1 = (ml[k][1].x == -INFINITY) ? 0.f : fast_exp2(ml[k][1].x - mg);
            const float lg = w0 * ml[k][0].y + w1 * ml[k][1].y;
            float acc[8];
            acc[0] = w0 * a[k][0].x + w1 * a[k][1].x; acc[1] = w0 * a[k][0].y + w1 * a[k][1].y;
            acc[2] = w0 * a[k][0].z + w1 * a[k][1].z; acc[3] = w0 * a[k][0].w + w1 * a[k][1].w;
            acc[4] = w0 * bq[k][0].x + w1 * bq[k][1].x; acc[5] = w0 * bq[k][0].y + w1 * bq[k][1].y;
            acc[6] = w0 * bq[k][0].z + w1 * bq[k][1].z; acc[7] = w0 * bq[k][0].w + w1 * bq[k][1].w;
            if (p.out) {
              const float inv = lg > 0.f ? 1.0f / lg : 0.f;
              uint4 w4;
              w4.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
              w4.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
              w4.z = pack_bf16x2(acc[4] * inv, acc[5] * inv);
              w4.w = pack_bf16x2(acc[6] * inv, acc[7] * inv);
              *reinterpret_cast<uint4*>(p.out + orow[k] * HD + lane * 8) = w4;
            } else {
              float4* dst = reinterpret_cast<float4*>(p.out_o + orow[k] * HD + lane * 8);
              dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
              dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
              if (lane == 0) {
                p.out_m[orow[k]] = mg * 0.6931471805599453f;
                p.out_l[orow[k]] = lg;
              }
            }
          }
        }
      } else {
      // Phase A: one thread per row turns the S (m, l) pairs into merge weights, kept in shared
      // memory (the Q tile is dead): wsm[row][s] = 2^(m_s - m_g), plus m_g and l_g per row.
      float* wsm = reinterpret_cast<float*>(smem + OFF_Q);            // [BM][32]
      float* wl = wsm + BM * 32;                                        // [BM][32]
      float* row_mg = wl + BM * 32;                                     // [BM]
      float* row_lg = row_mg + BM;                                      // [BM]
      if (tid < n_rows) {
        const uint32_t R = mt * BM + row0 + tid;
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
      for (uint32_t r0 = warp * RK; r0 < n_rows; r0 += NW * RK) {
        size_t orow[RK];
        bool live[RK];
        float acc[RK][8];
#pragma unroll
        for (uint32_t k = 0; k < RK; ++k) {
          const uint32_t R = mt * BM + row0 + r0 + k;
          live[k] = (r0 + k < n_rows) && (R < rows_per_head);
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
              const uint32_t rr = (r0 + k < n_rows) ? r0 + k : n_rows - 1;
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
      }   // S > 2
      if (tid == 0) *counter = 0u;   // ready for the next launch
    }
  }
  stamp(p, 5);
  if (p.ap_vectors != 0u && tid == 0) {
    // every CTA is past its own share taking and its waits on the append counters by now; the last one to
    // get here puts the share counter and the done counter back to zero for the next launch
    const uint32_t n_ctas = gridDim.x * gridDim.y;
    if (atomicInc(p.ap_ctl + 2, n_ctas - 1u) == n_ctas - 1u) {
      p.ap_ctl[0] = 0u;
      p.ap_ctl[1] = 0u;
      __threadfence();
    }
  }
}

cudaError_t sm100_attn_configure() {
  return cudaFuncSetAttribute(dg_attn_sm100_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES));
}
cudaError_t sm100_pair_configure() {
  return cudaFuncSetAttribute(dg_attn_sm100_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES));
}

// How many clusters of (cluster_x, cluster_y, 1) CTAs of the kernel the device can hold at once.
template <bool PAIR>
static int max_active_clusters(uint32_t cluster_y) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(PAIR ? 2 : 1, cluster_y, 148);
  cfg.blockDim = dim3(one::THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = cluster_y;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, dg_attn_sm100_kernel<PAIR>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return n;
}
int sm100_max_active_clusters(uint32_t cluster_y) { return max_active_clusters<false>(cluster_y); }
int sm100_pair_max_active_clusters(uint32_t cluster_y) { return max_active_clusters<true>(cluster_y); }

uint32_t sm100_query_tiles(uint32_t C, uint32_t G, uint32_t Hkv) { return Hkv * ((C * G + BM - 1) / BM); }
uint32_t sm100_pair_query_tiles(uint32_t C, uint32_t G, uint32_t Hkv) {
  const uint32_t tph = (C * G + BM - 1) / BM;
  return Hkv * ((tph + 1u) & ~1u);
}

uint32_t sm100_key_tiles(const MaskParams& mk) {
  const TileSched t = tile_sched(mk, 0, kMaxCanvas - 1);
  return t.nA + t.nB;
}

template <bool PAIR>
static cudaError_t launch(const AttnParams* ps, const CUtensorMap* const* tm_k, const CUtensorMap* const* tm_v, uint32_t n,
                          cudaStream_t st) {
  if (n == 0 || n > kMaxBatchLaunch) return cudaErrorInvalidValue;
  AttnBatch bat;
  for (uint32_t b = 0; b < kMaxBatchLaunch; ++b) {
    const uint32_t src = b < n ? b : 0;   // unused entries repeat the first canvas
    bat.p[b] = ps[src];
    bat.tm_k[b] = *tm_k[src];
    bat.tm_v[b] = *tm_v[src];
  }
  const AttnParams& p = ps[0];          // grid shape, split counts and cluster shape are the same for every canvas
  const dim3 grid(PAIR ? sm100_pair_query_tiles(p.C, p.G, p.Hkv) : sm100_query_tiles(p.C, p.G, p.Hkv), p.n_splits, n);
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
  const bool clustered_splits = p.cluster_splits > 1;
  if (PAIR || clustered_splits) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = PAIR ? 2 : 1;
    attr[n_attr].val.clusterDim.y = p.cluster_splits;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  return cudaLaunchKernelEx(&cfg, dg_attn_sm100_kernel<PAIR>, bat);
}

cudaError_t launch_attn_sm100(const AttnParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                              cudaStream_t st) {
  const CUtensorMap* k = &tm_k;
  const CUtensorMap* v = &tm_v;
  return launch<false>(&p, &k, &v, 1, st);
}
// tm_k64: K tensor map with boxes {64 d, 64 keys, 1}
cudaError_t launch_attn_sm100_pair(const AttnParams& p, const CUtensorMap& tm_k64, const CUtensorMap& tm_v,
                                   cudaStream_t st) {
  const CUtensorMap* k = &tm_k64;
  const CUtensorMap* v = &tm_v;
  return launch<true>(&p, &k, &v, 1, st);
}
// n <= kMaxBatchLaunch independent canvases in one launch (same geometry, split count and kernel form)
cudaError_t launch_attn_sm100_batch(const AttnParams* p, const CUtensorMap* const* tm_k, const CUtensorMap* const* tm_v,
                                    uint32_t n, bool pair, cudaStream_t st) {
  return pair ? launch<true>(p, tm_k, tm_v, n, st) : launch<false>(p, tm_k, tm_v, n, st);
}

}  // namespace dg
