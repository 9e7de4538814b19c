// Test infrastructure only.  Compiles the reference's own stage-1 shader
// (src/shaders/attn/qk_rope_kv/qk_rope_kv.metal, read where it lies in the reference tree) as C++
// through the stand-in in ref_shim/ and runs it on the CPU, one call per (token, head) grid point.
#include "metal_shim.h"

namespace ref_qk {
using namespace metal;
#include "fc_axes.metal"
#include "debug_status.metal"
#include "arena.metal"
#include "attention_device.metal"
#include "sampler_device.metal"
#include "qk_rope_kv.metal"
}  // namespace ref_qk

// q: [canvas][n_q][hd], k, v: [canvas][n_kv][hd] bf16 bit patterns, normed / roped IN PLACE as the
// shader does; kv: the cache region (f16 bit patterns, slot-major, see ref_attention.cpp), written at
// the slots of positions kv_len + tok; q_norm / k_norm: [hd] bf16 bit patterns of the norm weights.
// v_aliases_k != 0 runs the full-layer form without a v_proj (V is the raw K input, normed without
// a weight).
extern "C" int ref_qk_rope_kv(uint16_t* q, uint16_t* k, uint16_t* v, uint16_t* kv, const uint16_t* q_norm,
                              const uint16_t* k_norm, uint32_t canvas, uint32_t n_q_heads, uint32_t n_kv_heads,
                              uint32_t hd, uint32_t is_full, uint32_t v_aliases_k, uint32_t kv_len,
                              uint32_t kv_write_end, uint32_t ring_mask) {
  ref_qk::LayerOffsets L;
  ref_qk::StepParams P;
  ref_qk::AttnDims dims;
  std::memset(&L, 0, sizeof(L));
  std::memset(&P, 0, sizeof(P));
  // weight blob: [q_norm | k_norm] as bytes
  static uint16_t blob[2 * 512];
  if (hd > 512) return -1;
  std::memcpy(blob, q_norm, hd * 2);
  std::memcpy(blob + 512, k_norm, hd * 2);
  L.q_norm = 0;
  L.k_norm = 512 * 2;
  L.v_proj = v_aliases_k ? 0ul : 1ul;
  L.head_dim = hd;
  L.n_kv_heads = n_kv_heads;
  L.is_full = is_full;
  L.kv_ring_mask = ring_mask;
  L.kv_region = 0;
  P.kv_len = kv_len;
  P.kv_write_end = kv_write_end;
  dims.canvas = canvas;
  dims.n_q_heads = n_q_heads;
  dims.causal = 0;
  dims.window = 0;
  const uint32_t slots = n_q_heads + 2 * n_kv_heads;
  for (uint32_t tok = 0; tok < canvas; ++tok)
    for (uint32_t h = 0; h < slots; ++h) {
      const uint2 gid = {tok, h};
      ref_qk::qk_rope_kv(q, k, v, kv, reinterpret_cast<const uchar*>(blob), &L, P, dims, nullptr, nullptr, gid);
    }
  return 0;
}
