// Shared host/device definitions for the canvas-attention kernels: the mask predicate (one
// definition used by every kernel and by the visibility dump, so the mask is bit-exact by
// construction), launch parameter blocks and the device status word.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/dg_attn.h"

namespace dg {

constexpr uint32_t kMaxHeadDim = 512;
constexpr uint32_t kMaxCanvas = 256;
constexpr uint32_t kMaxRotHalf = 256;   // rotary_dim / 2 <= 256

// Which keys a canvas row may attend (src/shaders/attn/attention/attention.metal:51-63 for the
// window and causal rules; split-KV shards intersect the prefix interval with [t0, t1)).
//   prefix key t (t < kv_len) visible  iff  max(lo(row), t0) <= t < pre_hi
//   canvas key t (kv_len <= t < can_hi) visible iff include_canvas, and in the causal mode only
//   for lo(row) <= t <= kv_len + row (the query's own position)
struct MaskParams {
  uint32_t kv_len;    // first canvas position = number of prefix keys
  uint32_t t0;        // shard lower bound (0 when unsharded)
  uint32_t pre_hi;    // min(t1, kv_len)
  uint32_t can_hi;    // kv_len + canvas when canvas keys are included, else kv_len
  uint32_t mode;      // DG_MASK_*
  uint32_t wm1;       // window - 1 (unused when mode == NONE or window == 0)
  uint32_t windowed;  // 1 when a window applies
  uint32_t pad_;
};

__host__ __device__ inline MaskParams make_mask(const dg_layer_desc& d, uint32_t kv_len, uint32_t t0, uint32_t t1,
                                                int include_canvas) {
  MaskParams m;
  m.kv_len = kv_len;
  m.t0 = t0;
  m.pre_hi = t1 < kv_len ? t1 : kv_len;
  m.can_hi = include_canvas ? kv_len + d.canvas : kv_len;
  m.mode = d.mask_mode;
  m.windowed = (d.mask_mode != DG_MASK_NONE && d.window != 0) ? 1u : 0u;
  m.wm1 = m.windowed ? d.window - 1u : 0u;
  m.pad_ = 0;
  return m;
}

// lower end of the window of canvas row `row` (0 without a window), before any shard bound
__host__ __device__ inline uint32_t mask_window_lo(const MaskParams& m, uint32_t row) {
  if (!m.windowed) return 0u;
  const uint32_t qpos = (m.mode == DG_MASK_WINDOW_UNIFORM) ? m.kv_len : m.kv_len + row;
  return qpos > m.wm1 ? qpos - m.wm1 : 0u;
}

// lowest visible prefix key of canvas row `row`
__host__ __device__ inline uint32_t mask_row_lo(const MaskParams& m, uint32_t row) {
  const uint32_t lo = mask_window_lo(m, row);
  return lo > m.t0 ? lo : m.t0;
}

// What one canvas row sees: prefix keys [lo, pre_hi) and canvas keys [can_lo, can_hi).
struct RowVis {
  uint32_t lo, can_lo, can_hi;
};
__host__ __device__ inline RowVis mask_row(const MaskParams& m, uint32_t row) {
  RowVis v;
  v.lo = mask_row_lo(m, row);
  v.can_lo = m.kv_len;
  v.can_hi = m.can_hi;
  if (m.mode == DG_MASK_CAUSAL) {
    const uint32_t wlo = mask_window_lo(m, row);
    const uint32_t own = m.kv_len + row + 1u;             // one past the query's own position
    if (wlo > v.can_lo) v.can_lo = wlo;
    if (own < v.can_hi) v.can_hi = own;
    if (v.can_hi < v.can_lo) v.can_hi = v.can_lo;         // nothing of the canvas
  }
  return v;
}

__host__ __device__ inline bool mask_visible_row(const MaskParams& m, const RowVis& v, uint32_t t) {
  return (t >= v.lo && t < m.pre_hi) || (t >= v.can_lo && t < v.can_hi);
}
__host__ __device__ inline bool mask_visible(const MaskParams& m, uint32_t row, uint32_t t) {
  return mask_visible_row(m, mask_row(m, row), t);
}
// whole key range [k0, k0 + n) visible to the row
__host__ __device__ inline bool mask_range_full(const MaskParams& m, const RowVis& v, uint32_t k0, uint32_t n) {
  const bool joined = m.pre_hi == m.kv_len && v.can_lo == m.kv_len && v.can_hi > m.kv_len;
  return (k0 >= v.lo && k0 + n <= m.pre_hi) || (k0 >= v.can_lo && k0 + n <= v.can_hi) ||
         (joined && k0 >= v.lo && k0 + n <= v.can_hi);
}
// one past the last canvas key any of the canvas rows [row_first, row_last] sees
__host__ __device__ inline uint32_t mask_can_hi_rows(const MaskParams& m, uint32_t row_last) {
  if (m.mode != DG_MASK_CAUSAL) return m.can_hi;
  const uint32_t own = m.kv_len + row_last + 1u;
  return own < m.can_hi ? own : m.can_hi;
}

// Device status word {code, kernel_id, cta, value}: first writer wins.
struct DevStatus {
  uint32_t code, kernel_id, cta, value;
};
__device__ inline void dev_status_set(DevStatus* s, uint32_t code, uint32_t kernel_id, uint32_t cta,
                                      uint32_t value) {
  if (s == nullptr) return;
  if (atomicCAS(&s->code, 0u, code) == 0u) {
    s->kernel_id = kernel_id;
    s->cta = cta;
    s->value = value;
  }
}

enum : uint32_t { KID_APPEND = 1, KID_GENERAL = 2, KID_SM100 = 3, KID_MERGE = 4, KID_VIS = 5, KID_SELFTEST = 6, KID_GEMM = 7 };

// ----------------------------------------------------------------------------------------
// Launch parameter blocks
// ----------------------------------------------------------------------------------------
struct RopeParams {
  uint32_t rot_half;     // rotary_dim / 2
  uint32_t pair_off;     // offset of the partner element: rot_half (split-half) or D/2 (proportional)
  float inv_freq[kMaxRotHalf];
};

// qk_rope_kv / append kernel
struct AppendParams {
  const __nv_bfloat16* q_in;   // [n][Hq][D] or null
  __nv_bfloat16* q_out;        // normed + roped Q (may alias q_in) or null
  const __nv_bfloat16* k_in;   // [n][Hkv][D]
  __nv_bfloat16* k_out;        // normed + roped K written back (may alias k_in) or null
  const __nv_bfloat16* v_in;   // [n][Hkv][D]
  __nv_bfloat16* v_out;        // normed V written back or null
  const __nv_bfloat16* qw;     // [D] or null
  const __nv_bfloat16* kw;     // [D] or null
  __nv_bfloat16* cache_k;      // K[Hkv][cap][D]
  __nv_bfloat16* cache_v;
  float2* rope_table;          // [n][rot_half] (cos, sin) of positions pos0 + i, or null
  const float2* rope_table_in; // the same table, already written by an earlier launch for these positions, or null
  uint64_t cap;
  uint32_t pos0, n;
  uint32_t Hq, Hkv, D;
  uint32_t v_norm;
  float eps;
  uint32_t ring_mask;          // cache slot of position pos = (pos - pos_base) & ring_mask (0xffffffff: linear cache)
  uint32_t write_end;          // positions >= write_end are not written to the cache (0xffffffff: none)
  uint32_t pos_base;           // first position the cache holds (a shard of a long prefix; 0 otherwise)
};

// attention kernels (general and sm100)
struct AttnParams {
  const __nv_bfloat16* q;        // [C][Hq][D]
  const __nv_bfloat16* qw;       // [D] or null (unit)
  const float2* rope_table;      // [C][rot_half]; only read when q_prenormed == 0
  const __nv_bfloat16* cache_k;  // K[Hkv][cap][D]
  const __nv_bfloat16* cache_v;
  const uint8_t* attend;         // optional bitmap [C][kv_len+C] (general kernel only)
  __nv_bfloat16* out;            // [C][Hq][D] or null when partial output is requested
  float* out_o;                  // partial: [C][Hq][D] fp32 un-normalised
  float* out_m;                  // partial: [C][Hq]
  float* out_l;                  // partial: [C][Hq]
  float* ws_o;                   // split workspace [n_splits][C*Hq][D]
  float* ws_ml;                  // split workspace [n_splits][C*Hq][2]
  uint32_t* ws_counters;         // one per query tile, zero between launches
  DevStatus* status;
  unsigned long long* stamps;    // optional per-CTA phase time stamps [CTAs][8] (ns), null = off
  uint64_t cap;
  MaskParams mask;
  uint32_t C, Hq, Hkv, G, D;
  uint32_t q_prenormed;
  uint32_t ring_mask;            // cache slot of key position t = (t - pos_base) & ring_mask (0xffffffff: linear cache)
  uint32_t pos_base;             // first position the cache holds (multiple of 128; 0 unless the cache is a shard)
  uint32_t early_q;              // 1: nothing the Q prologue reads is written by the preceding kernel on the stream
  uint32_t n_splits;
  uint32_t cluster_splits;       // consecutive splits per thread-block cluster (divides n_splits; 1 = no cluster merge)
  uint32_t rot_half, pair_off;
  float scale_log2;              // softmax_scale * log2(e)
  float eps;
  // Canvas append folded into the attention launch (head_dim-256 tensor kernel, RoPE table already in
  // memory): ap_vectors = canvas * 2 * Hkv head vectors of raw canvas K / V are normed, rotated and
  // written to the cache by the launch's own CTAs before any of them loads a key tile that holds canvas
  // positions.  0 = the cache already holds the canvas K / V.
  const __nv_bfloat16* ap_k;     // [C][Hkv][256]
  const __nv_bfloat16* ap_v;
  const __nv_bfloat16* ap_kw;    // [256] or null
  __nv_bfloat16* ap_cache_k;     // the cache, writable
  __nv_bfloat16* ap_cache_v;
  uint32_t* ap_ctl;              // {next share, vectors done, CTAs finished}: zero between launches
  uint32_t ap_vectors;
  uint32_t ap_v_norm;
  uint32_t ap_write_end;         // positions >= this are not stored (0xffffffff: none)
};

// Up to kMaxBatchLaunch independent canvases served by ONE launch of the head_dim-256 tensor kernel
// (blockIdx.z = canvas): the kernel's whole parameter block, tensor maps first (64-byte aligned).
constexpr uint32_t kMaxBatchLaunch = 4;
struct alignas(64) AttnBatch {
  CUtensorMap tm_k[kMaxBatchLaunch];
  CUtensorMap tm_v[kMaxBatchLaunch];
  AttnParams p[kMaxBatchLaunch];
};

// peer-to-peer split-KV merge (dg_p2p_merge.cu)
struct P2pParams {
  uint8_t* peer[8];        // exchange buffer of every rank, as mapped into this process
  size_t off_o[2], off_m[2], off_l[2], off_res[2];   // per parity
  size_t off_pflag, off_rflag, off_done;             // u32 pflag[2][8], rflag[2][8], done[2]
  // push form: per slot (step mod 3) a receive area [world][slice_cap][D] fp16 rows, their [world][slice_cap]
  // (m, l, 1 / scale, -) records, and one arrival counter (rows received since the last reset)
  size_t off_recv[3], off_rml[3], off_cnt;
  // shared query staging of the host pipeline: per pipe slot a full [rows][D] bf16 query block that every rank
  // fills with its own row slice (copied from host memory) and its peers' slices (pushed over NVLink), and one
  // arrival counter per slot (rows received from peers since the last reset)
  size_t off_qstage[8], off_qcnt;
  DevStatus* status;
  long long wait_limit;    // cycles
  uint32_t world, rank, rows, D, step, parity;
  uint32_t all_rows;       // 1: every rank merges every row itself (no result scatter, no second flag round)
  uint32_t slice_cap;      // rows of the largest row slice: ceil(rows / world)
  // push form: which step's rows this launch sends (phase A) and which step's slice it merges (phase B).  The
  // plain form does both for the current step, A then B; the pipelined form merges the PREVIOUS step first and
  // then sends the current one, so that nobody ever waits for rows that are still on their way.
  uint32_t send_slot, send_on;       // receive slot of the step whose rows are sent; 0: nothing to send
  uint32_t merge_slot, merge_uses, merge_on;   // slot and use count of the step whose slice is merged; 0: none
  uint32_t merge_first;              // 1: phase B runs before phase A
  unsigned long long* stamps;   // optional [8] globaltimer stamps of CTA 0 (measurement aid), null = off
};

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }

// D[M][N] = A[M][K] . W[N][K]^T of the projections either side of the attention stage (csrc/dg_gemm_sm100.cu).
// Output columns [col_begin, next segment's col_begin) go to dst with row stride ld (elements).
struct GemmSeg {
  void* dst;
  uint32_t col_begin;
  uint32_t ld;
};
struct GemmParams {
  uint32_t M, N, K, n_seg;
  GemmSeg seg[3];
  float* rowsq;        // optional [M][N / tile width]: sum of squares of each row's rounded outputs per tile
  float* part;         // split-K: fp32 partial sums [k_slices][M][N] instead of the bf16 output
  uint32_t k_slices;
  uint32_t a_inner;    // 0: A is a {K, M} map.  G > 0: A is a {K, G, M / G} map (rows (i, g) of one KV head of a
                       // [C][Hq][D] tensor) with boxes {64, G, 128 / G}
  uint32_t w_z;        // third coordinate of the W map (the KV head of a cache map), else 0
  DevStatus* status;
};

// top-k selection + gathered PV over a plane of 16-bit scores (csrc/dg_topk.cu)
struct TopkParams {
  const uint16_t* scores;        // bf16 [Hkv][head_rows][ld]: row i * G + g of KV head h, key t
  uint32_t ld, head_rows;        // head_rows = C * G rounded up to whole 128-row tiles
  const __nv_bfloat16* q;        // normed + roped Q [C][Hq][D]
  const __nv_bfloat16* k;        // caches [Hkv][cap][D]
  const __nv_bfloat16* v;
  __nv_bfloat16* out;            // [C][Hq][D]
  uint32_t C, Hq, G, D;
  uint64_t cap;
  MaskParams mask;
  uint32_t k_fixed, k_div, k_min, k_max;   // k = k_div ? clamp(n_visible / k_div, k_min, k_max) : k_fixed, at most n_visible
  float scale_log2;
};

}  // namespace dg
