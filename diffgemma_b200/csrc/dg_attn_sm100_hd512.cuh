// Parts shared by the two head_dim-512 attention kernels (one CTA per value-column half with the score
// work done by both, and the CTA-pair form whose halves exchange P): tile geometry, the 64-key tile
// schedule, the epilogue that stores a CTA's 128 rows x 256 columns, and the merge of the key splits.
#pragma once
#include <cuda.h>

#include "dg_attn_sm100_common.cuh"

namespace dg {

using namespace sm100;

namespace h5 {
constexpr uint32_t HDQ = 512;                 // contraction width of S
constexpr uint32_t HDV = 256;                 // value columns per CTA
constexpr uint32_t TN = 64;                   // keys per tile
constexpr uint32_t Q_ATOM = 128 * 128;        // 128 rows x 128 B
constexpr uint32_t KV_ATOM = 64 * 128;        // 64 rows x 128 B
constexpr uint32_t SMEM_REQ = 232448;         // all of the 227 KB a CTA may have
constexpr uint32_t T_S = 0, T_Q = 128, T_O = 256;     // TMEM columns: S buffers at 0 and 64, Q[:, 0:256] at 128, O at 256
constexpr uint32_t OPT = 128;                 // output columns per epilogue thread (two threads per row)

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

// Copies a query tile into the CTA: elements [0, 256) of every row into tensor memory (by the threads with
// half == 0), elements [256, 512) into the K-major 128-byte-swizzled shared-memory atoms at q_smem (half == 1).
// Thread (smw, lane) owns row r = smw * 32 + lane; the caller signals the barrier afterwards.
__device__ __forceinline__ void copy_q_tile(const AttnParams& p, uint8_t* q_smem, uint32_t tmem, uint32_t kvh, uint32_t mt,
                                            uint32_t smw, uint32_t lane, uint32_t half) {
  const uint32_t r = smw * 32 + lane;
  const uint32_t R = mt * BM + r;
  const bool valid = R < p.C * p.G;
  const uint32_t i = valid ? R / p.G : 0u;
  const uint32_t h = kvh * p.G + (valid ? R % p.G : 0u);
  const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t(i) * p.Hq + h) * HDQ);
  if (half == 0) {
    // 16-byte chunk c = columns [4c, 4c + 4) of lane r, so that the 16 elements of contraction step kk sit in
    // columns [8 kk, 8 kk + 8) (the layout P uses)
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
    // atom = 64-element column block, 16-byte chunk index XOR (row & 7)
#pragma unroll 4
    for (uint32_t j = 0; j < 32; ++j) {
      const uint4 v4 = valid ? src[32 + j] : make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(q_smem + (j >> 3) * Q_ATOM + r * 128u + (((j & 7u) ^ (r & 7u)) << 4)) = v4;
    }
    fence_proxy_async_smem();
  }
}

// Stores this CTA's O (TMEM columns [T_O, T_O + 256), rows = lanes) for value-column half dh: bf16 rows of the
// output when there is one split and an output tensor, else fp32 partial rows plus the row's (m, l).  Two
// threads per row (`half` = which 128 columns); `tile_smem` is dead shared memory of at least 8 x 4,608 bytes.
__device__ __forceinline__ void store_o_half(const AttnParams& p, uint8_t* tile_smem, uint32_t tmem, uint32_t kvh, uint32_t mt,
                                             uint32_t split, uint32_t dh, uint32_t smw, uint32_t lane, uint32_t half,
                                             bool have_o, float m_used, float l_tot) {
  const uint32_t rows_per_head = p.C * p.G;
  const uint32_t rows_total = p.C * p.Hq;
  const uint32_t r = smw * 32 + lane;
  const uint32_t R = mt * BM + r;
  const bool valid = R < rows_per_head;
  const uint32_t i_row = valid ? R / p.G : 0u;
  const uint32_t h = kvh * p.G + (valid ? R % p.G : 0u);
  const size_t orow = size_t(i_row) * p.Hq + h;
  const uint32_t t_lane = tmem + ((smw * 32u) << 16);
  const bool direct = (p.n_splits == 1);
  const bool to_bf16 = direct && p.out != nullptr;
  const float inv_l = l_tot > 0.f ? 1.0f / l_tot : 0.f;
  const float mul = to_bf16 ? inv_l : 1.0f;
  float* dst_o = direct ? p.out_o : p.ws_o + size_t(split) * rows_total * HDQ;
  // 32 x 32 chunks go through a padded per-warp tile in shared memory so that every store instruction of the
  // warp writes whole 128-byte lines
  float* tile = reinterpret_cast<float*>(tile_smem) + (half * 4u + smw) * (32 * 36);
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

// Key splits meet in the global workspace: the last CTA to arrive at the (query tile, half) counter merges the
// partial rows of all splits.  Called by every thread of the CTA after its partial rows are stored;
// `is_last` is one word of shared memory.
__device__ __forceinline__ void merge_splits_last(const AttnParams& p, volatile uint32_t* is_last, uint32_t kvh, uint32_t mt,
                                                  uint32_t dh, uint32_t n_threads) {
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rows_per_head = p.C * p.G;
  const uint32_t rows_total = p.C * p.Hq;
  const uint32_t S = p.n_splits;
  uint32_t* counter = p.ws_counters + blockIdx.x * 2 + dh;
  if (tid == 0) {
    __threadfence();
    const uint32_t old = atomicAdd(counter, 1u);
    *is_last = (old == S - 1u) ? 1u : 0u;
  }
  __syncthreads();
  if (!*is_last) return;
  __threadfence();
  const float2* ml_all = reinterpret_cast<const float2*>(p.ws_ml);
  for (uint32_t rr = warp; rr < BM; rr += n_threads / 32) {
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

}  // namespace h5
}  // namespace dg
