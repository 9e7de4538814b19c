// Denoise-step canvas attention for head_dim 256 on sm_100a: one fused flash-style kernel.
//
//   * Q prologue in the kernel: per-head RMSNorm(+weight) + split-half RoPE on the CTA's 128
//     query rows, rounded to bf16 and written straight into the UMMA shared-memory layout.
//   * K/V tiles of 128 keys are TMA-staged (3-D tiled loads, 128-byte swizzle, no multicast) from
//     the head-major bf16 cache K[Hkv][cap][256], V[Hkv][cap][256].
//   * S = Q K^T and O += P V run on tcgen05.mma with fp32 accumulators in tensor memory:
//     TMEM columns [0,128) and [128,256) double-buffer S, [256,512) hold O; P (bf16) overwrites
//     the first 64 columns of its S buffer and is consumed from TMEM as the A operand.
//   * online softmax in registers, one thread per query row, with lazy rescaling of O (only when
//     the running maximum grows by more than 2^8).
//   * intra-GPU split-KV: grid.y CTAs share one query tile, each writes an (O, m, l) partial and
//     the last one to finish merges them (log-sum-exp) - no second launch.
//
// Query rows are the GQA-stacked rows of one KV head: stacked row R -> canvas row R / G, query
// head kvh*G + R % G, so all 128 rows of a CTA reuse the same K/V tiles.
//
// Semantics restated from the reference (paths relative to the reference project):
//   src/shaders/attn/attention/attention.metal:22-133 (denoise mask, online softmax),
//   src/shaders/attn/attention/attention_mma2.metal:53-307 (tiled variant, p = 0 for masked keys,
//   fully masked row -> 0), src/shaders/include/attention_device.metal:154-165 ((m, l, O) state).
#include <cuda.h>

#include "dg_common.cuh"
#include "dg_kernels.h"
#include "sm100_ptx.cuh"

namespace dg {

namespace {

constexpr uint32_t BM = 128;            // query rows per CTA
constexpr uint32_t BN = 128;            // keys per tile
constexpr uint32_t HD = 256;            // head_dim
constexpr uint32_t ATOM_BYTES = 128 * 128;        // 128 rows x 128 B (64 bf16): one swizzle-atom column
constexpr uint32_t TILE_BYTES = 4 * ATOM_BYTES;   // 128 rows x 256 bf16
constexpr uint32_t OFF_Q = 0;
constexpr uint32_t OFF_K = TILE_BYTES;
constexpr uint32_t OFF_V = 2 * TILE_BYTES;
constexpr uint32_t OFF_BAR = 3 * TILE_BYTES;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 256 + 1024;   // + barrier block + alignment slack
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_S = 0;            // two S buffers of 128 columns
constexpr uint32_t TM_O = 256;          // O accumulator, 256 columns
constexpr uint32_t N_THREADS = 224;     // warps 0-3 softmax, 4 K loader, 5 V loader, 6 MMA issuer
constexpr float RESCALE_THRESHOLD = 8.0f;   // log2 units

// barrier slots (8 bytes each) inside the barrier block
enum : uint32_t {
  BAR_Q = 0,
  BAR_K_FULL = 1,
  BAR_K_EMPTY = 2,
  BAR_V_FULL = 3,
  BAR_V_EMPTY = 4,
  BAR_S_FULL0 = 5,   // +1 for buffer 1
  BAR_P_FULL0 = 7,   // +1 for buffer 1
  BAR_PV_DONE = 9,   // one phase per key tile; only waited on when O must be rescaled
  BAR_O_FINAL = 10,  // single phase: every PV of this CTA has completed
  N_BARS = 11
};

struct TileSched {
  uint32_t a0, nA, b0, nB;
};
// Key tiles (absolute index = key / 128) a CTA whose first canvas row is `row_first` must visit:
// the prefix interval [lo, pre_hi) and the canvas interval [kv_len, can_hi), merged when they touch.
__host__ __device__ inline TileSched tile_sched(const MaskParams& mk, uint32_t row_first) {
  TileSched t{0, 0, 0, 0};
  const uint32_t lo = mask_row_lo(mk, row_first);
  if (mk.pre_hi > lo) {
    t.a0 = lo / BN;
    t.nA = (mk.pre_hi + BN - 1) / BN - t.a0;
  }
  if (mk.can_hi > mk.kv_len) {
    const uint32_t b0 = mk.kv_len / BN, b1 = (mk.can_hi + BN - 1) / BN;
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

__device__ __forceinline__ uint32_t bar_addr(uint32_t bar_base, uint32_t idx) { return bar_base + idx * 8u; }

}  // namespace

__global__ void __launch_bounds__(N_THREADS, 1)
dg_attn_sm100_kernel(const AttnParams p, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + OFF_Q, sK = smem_base + OFF_K, sV = smem_base + OFF_V;
  const uint32_t bar_base = smem_base + OFF_BAR;
  volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + OFF_BAR + N_BARS * 8);
  // ctl[0] = TMEM base address, ctl[1] = abort flag, ctl[2] = "this CTA merges" flag

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

  // ------------------------------------------------------------------ set-up
  if (tid == 0) {
    mbar_init(bar_addr(bar_base, BAR_Q), 128);
    mbar_init(bar_addr(bar_base, BAR_K_FULL), 1);
    mbar_init(bar_addr(bar_base, BAR_K_EMPTY), 1);
    mbar_init(bar_addr(bar_base, BAR_V_FULL), 1);
    mbar_init(bar_addr(bar_base, BAR_V_EMPTY), 1);
    mbar_init(bar_addr(bar_base, BAR_S_FULL0), 1);
    mbar_init(bar_addr(bar_base, BAR_S_FULL0 + 1), 1);
    mbar_init(bar_addr(bar_base, BAR_P_FULL0), 128);
    mbar_init(bar_addr(bar_base, BAR_P_FULL0 + 1), 128);
    mbar_init(bar_addr(bar_base, BAR_PV_DONE), 1);
    mbar_init(bar_addr(bar_base, BAR_O_FINAL), 1);
    ctl[1] = 0u;
    ctl[2] = 0u;
    fence_mbar_init();
  }
  if (warp == 6) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(&ctl[0])), TMEM_COLS);
    tmem_relinquish();
  }
  if ((warp == 4 || warp == 5) && lane == 0) tma_prefetch_desc(warp == 4 ? &tm_k : &tm_v);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl[0];
  volatile uint32_t* abort_flag = &ctl[1];

  // per-row softmax state lives in the softmax threads across the main loop and the epilogue
  float m_used = -INFINITY, l_run = 0.f;

  if (warp < 4) {
    // ---------------------------------------------------------------- Q prologue (warp per row)
    // Rows are processed in batches of QB with every global load of a batch (raw row chunk and
    // RoPE table entries) issued before the first use, so a warp pays one memory round trip per
    // batch instead of one per row.
    constexpr int QB = 4;
    float wq[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) wq[e] = 1.0f;
    if (!p.q_prenormed && p.qw) {
      const uint4 wr = *reinterpret_cast<const uint4*>(p.qw + lane * 8);
      const uint32_t w[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        wq[2 * e] = __uint_as_float(w[e] << 16);
        wq[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
      }
    }
#pragma unroll 1
    for (uint32_t batch = 0; batch < 32 / QB; ++batch) {
      uint4 raw[QB];
      float2 cs[QB][8];
#pragma unroll
      for (int b = 0; b < QB; ++b) {
        const uint32_t r = warp * 32 + batch * QB + b;
        const uint32_t R = mt * BM + r;
        const bool valid = R < rows_per_head;
        const uint32_t i = valid ? R / p.G : 0u;
        const uint32_t h = kvh * p.G + (valid ? R % p.G : 0u);
        raw[b] = valid ? *reinterpret_cast<const uint4*>(p.q + (size_t(i) * p.Hq + h) * HD + lane * 8)
                       : make_uint4(0u, 0u, 0u, 0u);
        if (!p.q_prenormed) {
          const float4* tab = reinterpret_cast<const float4*>(p.rope_table + size_t(i) * 128 + (lane & 15) * 8);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float4 t4 = tab[e];
            cs[b][2 * e] = make_float2(t4.x, t4.y);
            cs[b][2 * e + 1] = make_float2(t4.z, t4.w);
          }
        }
      }
#pragma unroll
      for (int b = 0; b < QB; ++b) {
        const uint32_t r = warp * 32 + batch * QB + b;
        float x[8];
        const uint32_t w[4] = {raw[b].x, raw[b].y, raw[b].z, raw[b].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          x[2 * e] = __uint_as_float(w[e] << 16);
          x[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        }
        if (!p.q_prenormed) {
          float ss = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          const float inv = 1.0f / sqrtf(ss / float(HD) + p.eps);
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] *= inv * wq[e];
          // split-half RoPE: element d pairs with d + 128, i.e. lane l pairs with lane l ^ 16
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
            const float2 c2 = cs[b][e];
            x[e] = (lane < 16) ? (x[e] * c2.x - other * c2.y) : (other * c2.y + x[e] * c2.x);
          }
        }
        uint4 packed;
        packed.x = pack_bf16x2(x[0], x[1]);
        packed.y = pack_bf16x2(x[2], x[3]);
        packed.z = pack_bf16x2(x[4], x[5]);
        packed.w = pack_bf16x2(x[6], x[7]);
        // K-major 128-byte-swizzled layout: atom = 64-element column block, 16-byte chunk index
        // XORed with (row & 7)
        const uint32_t atom = lane >> 3, cc = lane & 7;
        const uint32_t off = OFF_Q + atom * ATOM_BYTES + r * 128u + ((cc ^ (r & 7u)) << 4);
        *reinterpret_cast<uint4*>(smem + off) = packed;
      }
    }
    fence_proxy_async_smem();
    mbar_arrive(bar_addr(bar_base, BAR_Q));

    // ---------------------------------------------------------------- softmax main loop
    const uint32_t r = warp * 32 + lane;
    const uint32_t R = mt * BM + r;
    const uint32_t i_row = (R < rows_per_head) ? R / p.G : p.C - 1;
    const uint32_t row_lo = mask_row_lo(mk, i_row);
    const uint32_t t_lane = tmem + ((warp * 32u) << 16);
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
      uint32_t sraw[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(t_lane + TM_S + b * 128u + c * 32u, sraw[c]);
      tmem_wait_ld();

      const bool full = (k0 >= row_lo && k0 + BN <= mk.pre_hi) || (k0 >= mk.kv_len && k0 + BN <= mk.can_hi) ||
                        (contiguous && k0 >= row_lo && k0 + BN <= mk.can_hi);
      if (!full) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (!mask_visible_lo(mk, row_lo, k0 + c * 32 + e)) sraw[c][e] = 0xff800000u;  // -inf
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(sraw[c][e]));
      const float m_new = mx * sc;   // sc > 0; -inf stays -inf
      const bool first = (n == 0);
      const bool need = first || (m_new > m_used + RESCALE_THRESHOLD);
      if (!first && __any_sync(0xffffffffu, need)) {
        // O holds sum p v relative to m_used: bring it to the new reference point
        if (!__all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, BAR_PV_DONE), (n - 1) & 1u, abort_flag))) break;
        tc_fence_after();
        const float alpha = need ? fast_exp2(m_used - m_new) : 1.0f;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[32];
          tmem_ld32(t_lane + TM_O + c * 32u, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(t_lane + TM_O + c * 32u, o);
        }
        tmem_wait_st();
        l_run *= alpha;
      }
      if (need) m_used = m_new;
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      const float neg_m = -m_eff;
      float lsum = 0.f;
      // P column j (32 bit) = keys (2j, 2j+1) as bf16x2; 64 columns overwrite the head of S
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t pk[32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc)
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const int c = hf * 2 + cc;
            const float p0 = fast_exp2(fmaf(__uint_as_float(sraw[c][e]), sc, neg_m));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sraw[c][e + 1]), sc, neg_m));
            lsum += p0 + p1;
            pk[cc * 16 + (e >> 1)] = pack_bf16x2(p0, p1);
          }
        tmem_st32(t_lane + TM_S + b * 128u + hf * 32u, pk);
      }
      l_run += lsum;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_addr(bar_base, BAR_P_FULL0 + b));
    }
  } else if (warp == 4) {
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
  } else if (warp == 5) {
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

  // ------------------------------------------------------------------ epilogue (softmax warps)
  const uint32_t rows_total = p.C * p.Hq;
  if (warp < 4) {
    const uint32_t r = warp * 32 + lane;
    const uint32_t R = mt * BM + r;
    const bool valid = R < rows_per_head;
    const uint32_t i_row = valid ? R / p.G : 0u;
    const uint32_t h = kvh * p.G + (valid ? R % p.G : 0u);
    const size_t orow = size_t(i_row) * p.Hq + h;
    const uint32_t t_lane = tmem + ((warp * 32u) << 16);
    bool have_o = __all_sync(0xffffffffu, n_local > 0 && !*abort_flag);
    if (have_o) {
      have_o = __all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, BAR_O_FINAL), 0u, abort_flag));
      tc_fence_after();
    }
    const bool direct = (p.n_splits == 1);
    const bool to_bf16 = direct && p.out != nullptr;
    const float inv_l = l_run > 0.f ? 1.0f / l_run : 0.f;
    const float mul = to_bf16 ? inv_l : 1.0f;
    float* dst_o = direct ? p.out_o : p.ws_o + size_t(split) * rows_total * HD;
#pragma unroll 1
    for (int c = 0; c < 8; ++c) {
      uint32_t o[32];
      if (have_o) {
        tmem_ld32(t_lane + TM_O + c * 32u, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = 0u;
      }
      if (!valid) continue;
      if (to_bf16) {
        uint4* d4 = reinterpret_cast<uint4*>(p.out + orow * HD + c * 32);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[q4 * 8 + 0]) * mul, __uint_as_float(o[q4 * 8 + 1]) * mul);
          w.y = pack_bf16x2(__uint_as_float(o[q4 * 8 + 2]) * mul, __uint_as_float(o[q4 * 8 + 3]) * mul);
          w.z = pack_bf16x2(__uint_as_float(o[q4 * 8 + 4]) * mul, __uint_as_float(o[q4 * 8 + 5]) * mul);
          w.w = pack_bf16x2(__uint_as_float(o[q4 * 8 + 6]) * mul, __uint_as_float(o[q4 * 8 + 7]) * mul);
          d4[q4] = w;
        }
      } else {
        uint4* d4 = reinterpret_cast<uint4*>(dst_o + orow * HD + c * 32);
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4) d4[q4] = make_uint4(o[q4 * 4], o[q4 * 4 + 1], o[q4 * 4 + 2], o[q4 * 4 + 3]);
      }
    }
    if (valid && !to_bf16) {
      if (direct) {
        p.out_m[orow] = m_used * 0.6931471805599453f;   // log2 units -> natural units
        p.out_l[orow] = l_run;
      } else {
        float2* ml = reinterpret_cast<float2*>(p.ws_ml) + size_t(split) * rows_total + orow;
        *ml = make_float2(m_used, l_run);   // log2 units inside the workspace
      }
    }
    if (!direct) __threadfence();
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    // a bounded wait gave up: report, let our own TMA traffic land, then leave
    if (tid == 0) dev_status_set(p.status, DG_DEV_WAIT_TIMEOUT, KID_SM100, blockIdx.x + gridDim.x * blockIdx.y, n_local);
    if (warp == 4 && lane == 0 && n_local > 0) {
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000ll) {}   // ~1 ms: far longer than any tile load in flight
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 6) tmem_dealloc(tmem, TMEM_COLS);

  // ------------------------------------------------------------------ split merge by the last CTA
  if (p.n_splits > 1) {
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
      // Each warp merges two rows per iteration and keeps up to 2 x 4 x 2 16-byte loads in flight,
      // so the merge is bound by L2 bandwidth rather than by one round trip per row and split.
      constexpr uint32_t NW = N_THREADS / 32;
      for (uint32_t r0 = warp * 2; r0 < BM; r0 += NW * 2) {
        size_t orow[2];
        bool live[2];
        float2 ml[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint32_t R = mt * BM + r0 + k;
          live[k] = (r0 + k < BM) && (R < rows_per_head);
          const uint32_t Rc = live[k] ? R : mt * BM;
          orow[k] = size_t(Rc / p.G) * p.Hq + kvh * p.G + Rc % p.G;
          ml[k] = make_float2(-INFINITY, 0.f);
          if (lane < S) ml[k] = ml_all[size_t(lane) * rows_total + orow[k]];
        }
        float mg[2], lg[2], w_mine[2], acc[2][8];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          mg[k] = ml[k].x;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) mg[k] = fmaxf(mg[k], __shfl_xor_sync(0xffffffffu, mg[k], o));
          w_mine[k] = (ml[k].x == -INFINITY) ? 0.f : fast_exp2(ml[k].x - mg[k]);
          lg[k] = w_mine[k] * ml[k].y;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) lg[k] += __shfl_xor_sync(0xffffffffu, lg[k], o);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[k][e] = 0.f;
        }
        for (uint32_t s0 = 0; s0 < S; s0 += 4) {
          float4 a[2][4], bq[2][4];
#pragma unroll
          for (int k = 0; k < 2; ++k)
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
              const uint32_t sidx = (s0 + j < S) ? s0 + j : S - 1;   // clamped; its weight is zeroed below
              const float4* src = reinterpret_cast<const float4*>(p.ws_o + (size_t(sidx) * rows_total + orow[k]) * HD + lane * 8);
              a[k][j] = src[0];
              bq[k][j] = src[1];
            }
#pragma unroll
          for (int k = 0; k < 2; ++k)
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
              float w = __shfl_sync(0xffffffffu, w_mine[k], int((s0 + j) & 31u));
              if (s0 + j >= S) w = 0.f;
              acc[k][0] += w * a[k][j].x; acc[k][1] += w * a[k][j].y; acc[k][2] += w * a[k][j].z; acc[k][3] += w * a[k][j].w;
              acc[k][4] += w * bq[k][j].x; acc[k][5] += w * bq[k][j].y; acc[k][6] += w * bq[k][j].z; acc[k][7] += w * bq[k][j].w;
            }
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
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
      if (tid == 0) p.ws_counters[blockIdx.x] = 0u;   // ready for the next launch
    }
  }
}

cudaError_t sm100_attn_configure() {
  return cudaFuncSetAttribute(dg_attn_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES));
}

uint32_t sm100_query_tiles(uint32_t C, uint32_t G, uint32_t Hkv) { return Hkv * ((C * G + BM - 1) / BM); }

uint32_t sm100_key_tiles(const MaskParams& mk) {
  const TileSched t = tile_sched(mk, 0);
  return t.nA + t.nB;
}

cudaError_t launch_attn_sm100(const AttnParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                              cudaStream_t st) {
  const dim3 grid(sm100_query_tiles(p.C, p.G, p.Hkv), p.n_splits);
  dg_attn_sm100_kernel<<<grid, N_THREADS, SMEM_BYTES, st>>>(p, tm_k, tm_v);
  return cudaGetLastError();
}

}  // namespace dg
