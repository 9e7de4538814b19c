// One head vector of the canvas append when the RoPE table of its position is already in memory:
// head_dim 256, full split-half rotary.  A warp handles one (token, K or V head) vector, lane c owns the
// 16-byte chunk c, the RoPE partner of a chunk is chunk c ^ 16 (one shuffle away).  Shared by the
// stand-alone append kernel and by the attention kernel's in-launch append, so that both write the same
// bits (and the same bits as the general append kernel, which follows the same order of operations).  Semantics: src/shaders/attn/qk_rope_kv/qk_rope_kv.metal:58-149 of the reference (norm, weight,
// rotation, cache write with the ring slot and the kv_write_end guard).
#pragma once
#include "dg_common.cuh"

namespace dg {

__device__ __forceinline__ float rope_rotate_lo(float x0, float x1, float c, float s) {
  return __fmaf_rn(x0, c, -__fmul_rn(x1, s));
}
__device__ __forceinline__ float rope_rotate_hi(float x0, float x1, float c, float s) {
  return __fmaf_rn(x0, s, __fmul_rn(x1, c));
}
// K rotation with the norm folded in, one element: m = this element, q = its RoPE partner, both as loaded;
// a = w_own * cos, b = -(w_partner * sin) for the low element of a pair and +(w_partner * sin) for the high one;
// inv = 1 / rms.  Every kernel that writes K to a cache goes through these three functions, in this order of
// operations, so that they all write the same bits (the reference multiplies by inv and w first and rotates after:
// the same value up to fp32 rounding, far below the bf16 rounding of the stored result).
__device__ __forceinline__ float rope_coef_a(float w_own, float c) { return __fmul_rn(w_own, c); }
__device__ __forceinline__ float rope_coef_b(float w_partner, float s, bool low) {
  const float t = __fmul_rn(w_partner, s);
  return low ? -t : t;
}
__device__ __forceinline__ float rope_norm_rotate(float m, float q, float a, float b, float inv) {
  return __fmul_rn(__fmaf_rn(m, a, __fmul_rn(q, b)), inv);
}
__device__ __forceinline__ float warp_sum_xor(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct AppendVecArgs {
  const __nv_bfloat16* k_in;    // [n][Hkv][256]
  const __nv_bfloat16* v_in;
  const __nv_bfloat16* kw;      // [256] or null
  const float2* table;          // [n][128] (cos, sin) of positions pos0 + tok
  __nv_bfloat16* cache_k;       // K[Hkv][cap][256]
  __nv_bfloat16* cache_v;
  uint64_t cap;
  uint32_t pos0, Hkv, v_norm, ring_mask, write_end, pos_base;
  float eps;
};

// What a lane needs of one token to rotate that token's K vectors: a and b of its eight elements.
struct AppendRot {
  float a[8], b[8];
};
// kw_own / kw_partner: the K norm weight's chunk of this lane and of lane ^ 16 (bf16 1.0 without a weight)
__device__ __forceinline__ void append_norm_weight(const AppendVecArgs& p, uint32_t lane, uint4& kw_own, uint4& kw_partner) {
  kw_own = kw_partner = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
  if (p.kw) {
    kw_own = reinterpret_cast<const uint4*>(p.kw)[lane];
    kw_partner = reinterpret_cast<const uint4*>(p.kw)[lane ^ 16u];
  }
}
__device__ __forceinline__ void append_token_rot(const AppendVecArgs& p, uint32_t tok, uint32_t lane, const uint4 kw_own,
                                                 const uint4 kw_partner, AppendRot& r) {
  const float4* tab = reinterpret_cast<const float4*>(p.table + size_t(tok) * 128u + (lane & 15u) * 8u);
  const uint32_t wm[4] = {kw_own.x, kw_own.y, kw_own.z, kw_own.w};
  const uint32_t wq[4] = {kw_partner.x, kw_partner.y, kw_partner.z, kw_partner.w};
  const bool low = lane < 16u;   // this lane holds element i (low) or its partner i + 128 (high) of each pair
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float4 cs = tab[e];   // (cos, sin) of pairs 8 (lane & 15) + 2e and + 2e + 1
    r.a[2 * e] = rope_coef_a(__uint_as_float(wm[e] << 16), cs.x);
    r.a[2 * e + 1] = rope_coef_a(__uint_as_float(wm[e] & 0xffff0000u), cs.z);
    r.b[2 * e] = rope_coef_b(__uint_as_float(wq[e] << 16), cs.y, low);
    r.b[2 * e + 1] = rope_coef_b(__uint_as_float(wq[e] & 0xffff0000u), cs.w, low);
  }
}
// One vector whose 16 bytes x this lane already holds: norm, rotation (K) and the cache write.  Whole warp.
__device__ __forceinline__ void append_vector_finish(const AppendVecArgs& p, bool is_k, uint32_t h, uint32_t pos, uint32_t lane,
                                                     const uint4 x, const AppendRot& rot) {
  uint4 y = x;
  if (is_k || p.v_norm) {
    const uint32_t m[4] = {x.x, x.y, x.z, x.w};
    float f[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      f[2 * e] = __uint_as_float(m[e] << 16);
      f[2 * e + 1] = __uint_as_float(m[e] & 0xffff0000u);
    }
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = __fmaf_rn(f[e], f[e], ss);
    ss = warp_sum_xor(ss);   // butterfly: identical in every lane
    const float inv = 1.0f / sqrtf(ss / 256.0f + p.eps);
    float r[8];
    if (is_k) {
      const uint32_t q[4] = {__shfl_xor_sync(0xffffffffu, m[0], 16), __shfl_xor_sync(0xffffffffu, m[1], 16),
                             __shfl_xor_sync(0xffffffffu, m[2], 16), __shfl_xor_sync(0xffffffffu, m[3], 16)};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        r[2 * e] = rope_norm_rotate(f[2 * e], __uint_as_float(q[e] << 16), rot.a[2 * e], rot.b[2 * e], inv);
        r[2 * e + 1] = rope_norm_rotate(f[2 * e + 1], __uint_as_float(q[e] & 0xffff0000u), rot.a[2 * e + 1], rot.b[2 * e + 1], inv);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) r[e] = f[e] * inv;
    }
    __nv_bfloat162 b[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) b[e] = __floats2bfloat162_rn(r[2 * e], r[2 * e + 1]);
    y = make_uint4(*reinterpret_cast<uint32_t*>(&b[0]), *reinterpret_cast<uint32_t*>(&b[1]),
                   *reinterpret_cast<uint32_t*>(&b[2]), *reinterpret_cast<uint32_t*>(&b[3]));
  }
  __nv_bfloat16* cache = (is_k ? p.cache_k : p.cache_v) + (size_t(h) * p.cap + ((pos - p.pos_base) & p.ring_mask)) * 256u;
  reinterpret_cast<uint4*>(cache)[lane] = y;
}

// vector index w = tok * 2 Hkv + slot, slot < Hkv: K head slot, else V head slot - Hkv.  Whole warp.
__device__ __forceinline__ void append_table_vector(const AppendVecArgs& p, uint32_t w, uint32_t lane) {
  const uint32_t per_tok = 2u * p.Hkv;
  const uint32_t tok = w / per_tok, slot = w % per_tok;
  const bool is_k = slot < p.Hkv;
  const uint32_t h = is_k ? slot : slot - p.Hkv;
  const uint32_t pos = p.pos0 + tok;
  // zero-padded tail of a chunk: must not wrap onto live ring slots; positions below a shard's base have no slot
  if (pos >= p.write_end || pos < p.pos_base) return;
  const uint4 x = reinterpret_cast<const uint4*>((is_k ? p.k_in : p.v_in) + (size_t(tok) * p.Hkv + h) * 256u)[lane];
  AppendRot rot;
  if (is_k) {
    uint4 kw_own, kw_partner;
    append_norm_weight(p, lane, kw_own, kw_partner);
    append_token_rot(p, tok, lane, kw_own, kw_partner, rot);
  }
  append_vector_finish(p, is_k, h, pos, lane, x, rot);
}

// The same work cut into units of up to APPEND_UNIT_HEADS heads of one token's K or V: a warp loads the vectors of
// its unit together and prepares the token's rotation once.  Unit u = (tok * 2 + kv) * groups + grp with
// groups = ceil(Hkv / APPEND_UNIT_HEADS); returns how many vectors the unit stands for (written or not).
constexpr uint32_t APPEND_UNIT_HEADS = 4;
__host__ __device__ inline uint32_t append_unit_count(uint32_t n_tok, uint32_t Hkv) {
  return n_tok * 2u * ((Hkv + APPEND_UNIT_HEADS - 1u) / APPEND_UNIT_HEADS);
}
__device__ __forceinline__ uint32_t append_table_unit(const AppendVecArgs& p, uint32_t u, uint32_t lane, const uint4 kw_own,
                                                      const uint4 kw_partner) {
  const uint32_t groups = (p.Hkv + APPEND_UNIT_HEADS - 1u) / APPEND_UNIT_HEADS;
  const uint32_t tok = u / (2u * groups), rem = u % (2u * groups);
  const bool is_k = rem < groups;
  const uint32_t h0 = (is_k ? rem : rem - groups) * APPEND_UNIT_HEADS;
  const uint32_t nh = p.Hkv - h0 < APPEND_UNIT_HEADS ? p.Hkv - h0 : APPEND_UNIT_HEADS;
  const uint32_t pos = p.pos0 + tok;
  if (pos >= p.write_end || pos < p.pos_base) return nh;
  const uint4* src = reinterpret_cast<const uint4*>((is_k ? p.k_in : p.v_in) + (size_t(tok) * p.Hkv + h0) * 256u) + lane;
  uint4 x[APPEND_UNIT_HEADS];
#pragma unroll
  for (uint32_t j = 0; j < APPEND_UNIT_HEADS; ++j)
    if (j < nh) x[j] = src[j * 32u];
  AppendRot rot;
  if (is_k) append_token_rot(p, tok, lane, kw_own, kw_partner, rot);
#pragma unroll
  for (uint32_t j = 0; j < APPEND_UNIT_HEADS; ++j)
    if (j < nh) append_vector_finish(p, is_k, h0 + j, pos, lane, x[j], rot);
  return nh;
}

}  // namespace dg
