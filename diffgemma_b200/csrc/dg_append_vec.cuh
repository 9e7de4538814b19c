// One head vector of the canvas append when the RoPE table of its position is already in memory:
// head_dim 256, full split-half rotary.  A warp handles one (token, K or V head) vector, lane c owns the
// 16-byte chunk c, the RoPE partner of a chunk is chunk c ^ 16 (one shuffle away).  Shared by the
// stand-alone append kernel and by the attention kernel's in-launch append, so that both write the same
// bits.  Semantics: src/shaders/attn/qk_rope_kv/qk_rope_kv.metal:58-149 of the reference (norm, weight,
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
      uint4 w4 = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u), wp4 = w4;   // bf16 1.0
      if (p.kw) {
        w4 = reinterpret_cast<const uint4*>(p.kw)[lane];
        wp4 = reinterpret_cast<const uint4*>(p.kw)[lane ^ 16u];
      }
      const float4* tab = reinterpret_cast<const float4*>(p.table + size_t(tok) * 128u + (lane & 15u) * 8u);
      const uint32_t q[4] = {__shfl_xor_sync(0xffffffffu, m[0], 16), __shfl_xor_sync(0xffffffffu, m[1], 16),
                             __shfl_xor_sync(0xffffffffu, m[2], 16), __shfl_xor_sync(0xffffffffu, m[3], 16)};
      const uint32_t wm[4] = {w4.x, w4.y, w4.z, w4.w};
      const uint32_t wq[4] = {wp4.x, wp4.y, wp4.z, wp4.w};
      const bool low = lane < 16u;   // this lane holds element i (low) or its partner i + 128 (high) of each pair
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float4 cs = tab[e];   // (cos, sin) of pairs 8 (lane & 15) + 2e and + 2e + 1
        const float m0 = f[2 * e] * (inv * __uint_as_float(wm[e] << 16));
        const float m1 = f[2 * e + 1] * (inv * __uint_as_float(wm[e] & 0xffff0000u));
        const float q0 = __uint_as_float(q[e] << 16) * (inv * __uint_as_float(wq[e] << 16));
        const float q1 = __uint_as_float(q[e] & 0xffff0000u) * (inv * __uint_as_float(wq[e] & 0xffff0000u));
        r[2 * e] = low ? rope_rotate_lo(m0, q0, cs.x, cs.y) : rope_rotate_hi(q0, m0, cs.x, cs.y);
        r[2 * e + 1] = low ? rope_rotate_lo(m1, q1, cs.z, cs.w) : rope_rotate_hi(q1, m1, cs.z, cs.w);
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

}  // namespace dg
