// Test infrastructure only.  Compiles the reference's own attention shader
// (src/shaders/attn/attention/attention.metal, with the headers it includes, read where they lie in
// the reference tree - nothing is copied) as C++ through the stand-in in ref_shim/, and runs it on the
// CPU: one threadgroup per (canvas token, query head), lanes as fibers.  Used to pin the numpy / C++
// oracle's mask rule (window, causal), ring mapping and online softmax against the reference itself.
#include "metal_shim.h"

namespace ref_attn {
using namespace metal;
// headers first, while `threadgroup` is still an empty qualifier (they use it on pointers) ...
#include "fc_axes.metal"
#include "debug_status.metal"
#include "common.metal"
#include "attention_device.metal"
#include "arena.metal"
#include "sampler_device.metal"
// ... then the kernel, where `threadgroup float red[8];` must be one array for all lanes
#undef threadgroup
#define threadgroup static
#include "attention.metal"
#undef threadgroup
#define threadgroup
}  // namespace ref_attn

namespace {
struct Launch {
  const ushort* q;
  const ushort* kv;
  ushort* out;
  ref_attn::LayerOffsets L;
  ref_attn::StepParams P;
  ref_attn::AttnDims dims;
  uint3 tgid, tpg;
} g_launch;

void lane_body(int lane) {
  const uint3 lid = {uint(lane), 0u, 0u};
  ref_attn::attention(g_launch.q, g_launch.kv, g_launch.out, &g_launch.L, g_launch.P, g_launch.dims, nullptr,
                      g_launch.tgid, lid, g_launch.tpg);
}
}  // namespace

// q, out: [canvas][n_q_heads][hd] bf16 bit patterns (the reference's activation arena).
// kv: the layer's cache region, f16 bit patterns, slot-major: slot s = [K: n_kv x hd][V: n_kv x hd];
//     slot of position t is t (ring_mask = 0) or t & ring_mask.
// lanes: threads per threadgroup (32 for hd <= 256, 64 for hd = 512: the shader needs hd / lanes <= 8).
extern "C" int ref_attention(const uint16_t* q, const uint16_t* kv, uint16_t* out, uint32_t canvas, uint32_t n_q_heads,
                             uint32_t n_kv_heads, uint32_t hd, uint32_t kv_len, uint32_t window, uint32_t causal,
                             uint32_t ring_mask, uint32_t lanes) {
  if (lanes == 0 || lanes > simt::MAX_LANES || (hd + lanes - 1) / lanes > 8) return -1;
  std::memset(&g_launch.L, 0, sizeof(g_launch.L));
  std::memset(&g_launch.P, 0, sizeof(g_launch.P));
  g_launch.q = q;
  g_launch.kv = kv;
  g_launch.out = out;
  g_launch.L.head_dim = hd;
  g_launch.L.n_kv_heads = n_kv_heads;
  g_launch.L.kv_ring_mask = ring_mask;
  g_launch.L.kv_region = 0;
  g_launch.P.kv_len = kv_len;
  g_launch.P.kv_write_end = 0xffffffffu;
  g_launch.dims.canvas = canvas;
  g_launch.dims.n_q_heads = n_q_heads;
  g_launch.dims.causal = causal;
  g_launch.dims.window = window;
  g_launch.tpg = {lanes, 1u, 1u};
  for (uint32_t tok = 0; tok < canvas; ++tok)
    for (uint32_t h = 0; h < n_q_heads; ++h) {
      g_launch.tgid = {tok, h, 0u};
      simt::run_threadgroup(int(lanes), lane_body);
    }
  return 0;
}
