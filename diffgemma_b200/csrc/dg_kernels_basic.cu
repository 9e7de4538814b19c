// Small kernels around the tensor-core attention kernel:
//   * qk_rope_kv / cache append  (per-head RMSNorm + RoPE + KV-cache write + RoPE table)
//   * general attention kernel   (any head_dim <= 512, any mask incl. a decoder bitmap)
//   * local merge of (O, m, l) partials, NCCL-merge helpers, visibility dump
// Reference behaviour restated (paths relative to the reference project):
//   src/shaders/attn/qk_rope_kv/qk_rope_kv.metal:29-149, src/shaders/attn/cpu.rs:67-145 (stage 1)
//   src/shaders/attn/attention/attention.metal:22-133, src/shaders/attn/cpu.rs:148-197 (stage 2)
#include "dg_common.cuh"
#include "dg_append_vec.cuh"
#include "dg_kernels.h"

namespace dg {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ------------------------------------------------------------------------------------------
// qk_rope_kv / append: one warp per (token, head-vector slot).
// slots: [Q heads (if q_in)] [K heads] [V heads] [1 RoPE-table slot (if rope_table)]
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32) dg_append_kernel(const AppendParams p, const RopeParams rp) {
  __shared__ float xs[kMaxHeadDim];
  // let a dependent kernel (the attention launch that follows on the stream) begin its set-up now;
  // it synchronises on this grid's completion before it reads the cache or the RoPE table
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // when this kernel was itself launched ahead of the end of its predecessor (programmatic dependent
  // launch), everything it reads or writes may still be in use by that kernel: wait for it here
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t tok = blockIdx.x, slot = blockIdx.y, lane = threadIdx.x;
  const uint32_t D = p.D;
  const uint32_t pos = p.pos0 + tok;
  const uint32_t nq = p.q_in ? p.Hq : 0u;
  const float fpos = float(pos);

  if (slot >= nq + 2u * p.Hkv) {  // RoPE table row: (cos, sin) of f32(pos) * inv_freq[i]
    if (p.rope_table == nullptr) return;
    for (uint32_t i = lane; i < rp.rot_half; i += 32) {
      const float a = fpos * rp.inv_freq[i];
      p.rope_table[size_t(tok) * rp.rot_half + i] = make_float2(cosf(a), sinf(a));
    }
    return;
  }
  const bool is_q = slot < nq;
  const bool is_k = !is_q && slot < nq + p.Hkv;
  const uint32_t H = is_q ? p.Hq : p.Hkv;
  const uint32_t h = is_q ? slot : (slot - nq) % p.Hkv;
  const __nv_bfloat16* src = (is_q ? p.q_in : (is_k ? p.k_in : p.v_in)) + (size_t(tok) * H + h) * D;
  __nv_bfloat16* wb = (is_q ? p.q_out : (is_k ? p.k_out : p.v_out));
  if (wb) wb += (size_t(tok) * H + h) * D;
  // ring caches keep position pos in slot pos & ring_mask; positions at or past write_end (the
  // zero-padded tail of a prefill chunk) must not reach the cache, where they would wrap onto live slots
  __nv_bfloat16* cache = (is_q || pos >= p.write_end || pos < p.pos_base)
                             ? nullptr
                             : (is_k ? p.cache_k : p.cache_v) + (size_t(h) * p.cap + ((pos - p.pos_base) & p.ring_mask)) * D;

  // sum of squares in the order of dg_append_table_kernel (a lane takes 8 consecutive elements, then a
  // butterfly), and the rotation through rope_rotate in both, so that the two kernels write the same bits
  float ss = 0.f;
  for (uint32_t c = lane; c < D / 8; c += 32) {
#pragma unroll
    for (uint32_t e = 0; e < 8; ++e) {
      const float x = __bfloat162float(src[c * 8 + e]);
      xs[c * 8 + e] = x;
      ss = __fmaf_rn(x, x, ss);
    }
  }
  ss = warp_sum(ss);
  const bool norm = is_q || is_k || p.v_norm;
  const float inv = norm ? 1.0f / sqrtf(ss / float(D) + p.eps) : 1.0f;
  const __nv_bfloat16* w = is_q ? p.qw : (is_k ? p.kw : nullptr);
  if (norm) {
    for (uint32_t d = lane; d < D; d += 32) {
      // the rotated elements of K get their norm inside the rotation (rope_norm_rotate)
      if (is_k && ((d < rp.rot_half) || (d >= rp.pair_off && d < rp.pair_off + rp.rot_half))) continue;
      const float wv = w ? __bfloat162float(w[d]) : 1.0f;
      xs[d] = xs[d] * (inv * wv);
    }
  }
  __syncwarp();
  if (is_q) {
    for (uint32_t i = lane; i < rp.rot_half; i += 32) {
      const float a = fpos * rp.inv_freq[i];
      const float c = cosf(a), s = sinf(a);
      const float x0 = xs[i], x1 = xs[rp.pair_off + i];
      xs[i] = rope_rotate_lo(x0, x1, c, s);
      xs[rp.pair_off + i] = rope_rotate_hi(x0, x1, c, s);
    }
    __syncwarp();
  } else if (is_k) {
    for (uint32_t i = lane; i < rp.rot_half; i += 32) {
      const float a = fpos * rp.inv_freq[i];
      const float c = cosf(a), s = sinf(a);
      const float x0 = xs[i], x1 = xs[rp.pair_off + i];
      const float w0 = w ? __bfloat162float(w[i]) : 1.0f, w1 = w ? __bfloat162float(w[rp.pair_off + i]) : 1.0f;
      xs[i] = rope_norm_rotate(x0, x1, rope_coef_a(w0, c), rope_coef_b(w1, s, true), inv);
      xs[rp.pair_off + i] = rope_norm_rotate(x1, x0, rope_coef_a(w1, c), rope_coef_b(w0, s, false), inv);
    }
    __syncwarp();
  }
  for (uint32_t d = lane; d < D; d += 32) {
    const __nv_bfloat16 y = __float2bfloat16_rn(xs[d]);
    if (wb) wb[d] = y;
    if (cache) cache[d] = y;
  }
}

// Canvas append when the RoPE table of these positions is already in memory (the denoise steps of a
// canvas revisit the same positions): head_dim 256, full split-half rotary, cache writes only.
// One warp per (token, K or V head vector), lane c owns the 16-byte chunk c, the RoPE partner of a
// chunk is chunk c ^ 16 (one shuffle away); eight warps per CTA.  No sincos, no shared memory, 512-byte
// coalesced loads and stores: the kernel is short enough to hide behind the attention kernel's Q
// prologue, which overlaps it through programmatic dependent launch.
__global__ void __launch_bounds__(256) dg_append_table_kernel(const AppendParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // see dg_append_kernel
  const uint32_t lane = threadIdx.x & 31u, w = blockIdx.x * 8u + (threadIdx.x >> 5);
  if (w >= p.n * 2u * p.Hkv) return;
  AppendVecArgs a;
  a.k_in = p.k_in;
  a.v_in = p.v_in;
  a.kw = p.kw;
  a.table = p.rope_table_in;
  a.cache_k = p.cache_k;
  a.cache_v = p.cache_v;
  a.cap = p.cap;
  a.pos0 = p.pos0;
  a.Hkv = p.Hkv;
  a.v_norm = p.v_norm;
  a.ring_mask = p.ring_mask;
  a.write_end = p.write_end;
  a.pos_base = p.pos_base;
  a.eps = p.eps;
  append_table_vector(a, w, lane);
}

void launch_append(const AppendParams& p, const RopeParams& rp, cudaStream_t st, bool early) {
  if (p.n == 0) return;
  // `early`: the kernel may be scheduled while its predecessor on the stream is still draining (it
  // waits for that kernel's completion before it touches memory), which hides its launch latency
  cudaLaunchConfig_t cfg = {};
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early ? 1 : 0;
  if (p.rope_table_in && !p.rope_table && !p.q_in && !p.k_out && !p.v_out && p.D == 256 && rp.rot_half == 128 &&
      rp.pair_off == 128) {
    const uint32_t warps = p.n * 2u * p.Hkv;
    cfg.gridDim = dim3((warps + 7u) / 8u);
    cfg.blockDim = dim3(256);
    cudaLaunchKernelEx(&cfg, dg_append_table_kernel, p);
    return;
  }
  const uint32_t slots = (p.q_in ? p.Hq : 0u) + 2u * p.Hkv + (p.rope_table ? 1u : 0u);
  cfg.gridDim = dim3(p.n, slots);
  cfg.blockDim = dim3(32);
  cudaLaunchKernelEx(&cfg, dg_append_kernel, p, rp);
}

// ------------------------------------------------------------------------------------------
// General attention: one CTA (4 warps) per (canvas row, q head); keys strided over warps;
// online softmax per warp, merged at the end.  Serves any head_dim <= 512 (multiple of 8),
// partial rotary / proportional pairing, and explicit decoder bitmaps.
// ------------------------------------------------------------------------------------------
constexpr int GEN_WARPS = 4;

__global__ void __launch_bounds__(GEN_WARPS * 32) dg_attn_general_kernel(const AttnParams p) {
  __shared__ float qs[kMaxHeadDim];
  __shared__ float red[GEN_WARPS];
  __shared__ float wm[GEN_WARPS], wl[GEN_WARPS];
  __shared__ float wo[GEN_WARPS][kMaxHeadDim];

  const uint32_t row = blockIdx.x, h = blockIdx.y;
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t D = p.D, kvh = h / p.G;

  // ---- Q prologue (norm + weight + RoPE from the table), then round to bf16
  const __nv_bfloat16* qsrc = p.q + (size_t(row) * p.Hq + h) * D;
  float ss = 0.f;
  for (uint32_t d = tid; d < D; d += GEN_WARPS * 32) {
    const float x = __bfloat162float(qsrc[d]);
    qs[d] = x;
    ss += x * x;
  }
  if (!p.q_prenormed) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < GEN_WARPS; ++w) tot += red[w];
    const float inv = 1.0f / sqrtf(tot / float(D) + p.eps);
    for (uint32_t d = tid; d < D; d += GEN_WARPS * 32) {
      const float wv = p.qw ? __bfloat162float(p.qw[d]) : 1.0f;
      qs[d] = qs[d] * (inv * wv);
    }
    __syncthreads();
    for (uint32_t i = tid; i < p.rot_half; i += GEN_WARPS * 32) {
      const float2 cs = p.rope_table[size_t(row) * p.rot_half + i];
      const float x0 = qs[i], x1 = qs[p.pair_off + i];
      qs[i] = x0 * cs.x - x1 * cs.y;
      qs[p.pair_off + i] = x0 * cs.y + x1 * cs.x;
    }
    __syncthreads();
    for (uint32_t d = tid; d < D; d += GEN_WARPS * 32) qs[d] = __bfloat162float(__float2bfloat16_rn(qs[d]));
  }
  __syncthreads();

  // ---- key sweep
  const uint32_t n_chunks = D / 8;  // 16-byte chunks per row
  float acc[2][8];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
  float m = -INFINITY, l = 0.f;

  const MaskParams mk = p.mask;
  const RowVis rv = mask_row(mk, row);
  const uint32_t T = mk.kv_len + p.C;
  const __nv_bfloat16* kbase = p.cache_k + size_t(kvh) * p.cap * D;
  const __nv_bfloat16* vbase = p.cache_v + size_t(kvh) * p.cap * D;

  for (int range = 0; range < 2; ++range) {
    uint32_t lo, hi;
    if (p.attend) {
      if (range == 1) break;
      lo = 0;
      hi = T;
    } else if (range == 0) {
      lo = rv.lo;
      hi = mk.pre_hi;
    } else {
      lo = rv.can_lo;
      hi = rv.can_hi;
    }
    for (uint32_t t = lo + warp; t < hi; t += GEN_WARPS) {
      if (p.attend) {
        if (!p.attend[size_t(row) * T + t]) continue;
      }
      const uint32_t ts = (t - p.pos_base) & p.ring_mask;   // cache slot of key position t
      const uint4* kr = reinterpret_cast<const uint4*>(kbase + size_t(ts) * D);
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t c = lane + 32u * j;
        if (c < n_chunks) {
          const uint4 kk = kr[c];
          const uint32_t w[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            dot += qs[c * 8 + 2 * e] * __uint_as_float(w[e] << 16);
            dot += qs[c * 8 + 2 * e + 1] * __uint_as_float(w[e] & 0xffff0000u);
          }
        }
      }
      dot = warp_sum(dot);
      const float s2 = dot * p.scale_log2;
      const float mn = fmaxf(m, s2);
      const float corr = exp2f(m - mn);  // exp2(-inf) = 0 on the first key
      const float pe = exp2f(s2 - mn);
      l = l * corr + pe;
      m = mn;
      const uint4* vr = reinterpret_cast<const uint4*>(vbase + size_t(ts) * D);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t c = lane + 32u * j;
        if (c < n_chunks) {
          const uint4 vv = vr[c];
          const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[j][2 * e] = acc[j][2 * e] * corr + pe * __uint_as_float(w[e] << 16);
            acc[j][2 * e + 1] = acc[j][2 * e + 1] * corr + pe * __uint_as_float(w[e] & 0xffff0000u);
          }
        }
      }
    }
  }

  // ---- merge the warps
  if (lane == 0) {
    wm[warp] = m;
    wl[warp] = l;
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const uint32_t c = lane + 32u * j;
    if (c < n_chunks)
#pragma unroll
      for (int e = 0; e < 8; ++e) wo[warp][c * 8 + e] = acc[j][e];
  }
  __syncthreads();
  float mg = -INFINITY;
  for (int w = 0; w < GEN_WARPS; ++w) mg = fmaxf(mg, wm[w]);
  float wgt[GEN_WARPS];
  float lg = 0.f;
  for (int w = 0; w < GEN_WARPS; ++w) {
    wgt[w] = (wm[w] == -INFINITY) ? 0.f : exp2f(wm[w] - mg);
    lg += wgt[w] * wl[w];
  }
  const size_t orow = size_t(row) * p.Hq + h;
  for (uint32_t d = tid; d < D; d += GEN_WARPS * 32) {
    float o = 0.f;
    for (int w = 0; w < GEN_WARPS; ++w) o += wgt[w] * wo[w][d];
    if (p.out) {
      p.out[orow * D + d] = __float2bfloat16_rn(lg > 0.f ? o / lg : 0.f);
    } else {
      p.out_o[orow * D + d] = o;
    }
  }
  if (!p.out && tid == 0) {
    p.out_m[orow] = mg * 0.6931471805599453f;  // log2 units -> natural units
    p.out_l[orow] = lg;
  }
}

void launch_attn_general(const AttnParams& p, cudaStream_t st) {
  dg_attn_general_kernel<<<dim3(p.C, p.Hq), GEN_WARPS * 32, 0, st>>>(p);
}

// ------------------------------------------------------------------------------------------
// Local merge of n_parts partials -> bf16.  One warp per row; m in natural-log units.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) dg_merge_local_kernel(uint32_t n_parts, uint32_t rows, uint32_t D,
                                                              const float* __restrict__ o,
                                                              const float* __restrict__ m,
                                                              const float* __restrict__ l,
                                                              __nv_bfloat16* __restrict__ out) {
  const uint32_t row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float mg = -INFINITY;
  for (uint32_t s = 0; s < n_parts; ++s) mg = fmaxf(mg, m[size_t(s) * rows + row]);
  float lg = 0.f;
  for (uint32_t s = 0; s < n_parts; ++s) {
    const float ms = m[size_t(s) * rows + row];
    lg += (ms == -INFINITY ? 0.f : expf(ms - mg)) * l[size_t(s) * rows + row];
  }
  for (uint32_t d = lane; d < D; d += 32) {
    float acc = 0.f;
    for (uint32_t s = 0; s < n_parts; ++s) {
      const float ms = m[size_t(s) * rows + row];
      const float w = ms == -INFINITY ? 0.f : expf(ms - mg);
      acc += w * o[(size_t(s) * rows + row) * D + d];
    }
    out[size_t(row) * D + d] = __float2bfloat16_rn(lg > 0.f ? acc / lg : 0.f);
  }
}

void launch_merge_local(uint32_t n_parts, uint32_t rows, uint32_t D, const float* o, const float* m,
                        const float* l, __nv_bfloat16* out, cudaStream_t st) {
  dg_merge_local_kernel<<<(rows + 3) / 4, 128, 0, st>>>(n_parts, rows, D, o, m, l, out);
}

// ------------------------------------------------------------------------------------------
// Cross-rank merge helpers.  Payload layout: pay[rows][D+1] = [O row | l]; m separate.
//   pack:     pay = [O | l] * exp(m_local - m_global)   (m_global already all-reduced into mg)
//   finalize: out = pay[:, :D] / pay[:, D]
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) dg_merge_pack_kernel(uint32_t rows, uint32_t D, const float* __restrict__ o,
                                                             const float* __restrict__ m_local,
                                                             const float* __restrict__ m_global,
                                                             const float* __restrict__ l, float* __restrict__ pay) {
  const uint32_t row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float ml = m_local[row], mg = m_global[row];
  const float w = (ml == -INFINITY) ? 0.f : expf(ml - mg);
  for (uint32_t d = lane; d < D; d += 32) pay[size_t(row) * (D + 1) + d] = w * o[size_t(row) * D + d];
  if (lane == 0) pay[size_t(row) * (D + 1) + D] = w * l[row];
}
__global__ void __launch_bounds__(128) dg_merge_finalize_kernel(uint32_t rows, uint32_t D, const float* __restrict__ pay,
                                                                 __nv_bfloat16* __restrict__ out) {
  const uint32_t row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float lg = pay[size_t(row) * (D + 1) + D];
  const float inv = lg > 0.f ? 1.0f / lg : 0.f;
  for (uint32_t d = lane; d < D; d += 32)
    out[size_t(row) * D + d] = __float2bfloat16_rn(pay[size_t(row) * (D + 1) + d] * inv);
}
void launch_merge_pack(uint32_t rows, uint32_t D, const float* o, const float* m_local, const float* m_global,
                       const float* l, float* pay, cudaStream_t st) {
  dg_merge_pack_kernel<<<(rows + 3) / 4, 128, 0, st>>>(rows, D, o, m_local, m_global, l, pay);
}
void launch_merge_finalize(uint32_t rows, uint32_t D, const float* pay, __nv_bfloat16* out, cudaStream_t st) {
  dg_merge_finalize_kernel<<<(rows + 3) / 4, 128, 0, st>>>(rows, D, pay, out);
}

// ------------------------------------------------------------------------------------------
// Visibility dump: the predicate of dg_common.cuh evaluated on the device.
// ------------------------------------------------------------------------------------------
__global__ void dg_visibility_kernel(MaskParams mk, uint32_t C, uint8_t* __restrict__ out) {
  const uint32_t T = mk.kv_len + C;
  const uint32_t row = blockIdx.y;
  const RowVis rv = mask_row(mk, row);
  for (uint32_t t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x)
    out[size_t(row) * T + t] = mask_visible_row(mk, rv, t) ? 1 : 0;
}
void launch_visibility(const MaskParams& mk, uint32_t C, uint8_t* out, cudaStream_t st) {
  const uint32_t T = mk.kv_len + C;
  uint32_t gx = (T + 255) / 256;
  if (gx > 1024) gx = 1024;
  dg_visibility_kernel<<<dim3(gx, C), 256, 0, st>>>(mk, C, out);
}

// ------------------------------------------------------------------------------------------
// Self-test of the bounded-wait / device-status path: one thread waits on a flag that nothing
// sets, gives up after `limit_cycles`, and reports DG_DEV_WAIT_TIMEOUT exactly like a kernel whose
// barrier wait ran out.  The context stays usable.
// ------------------------------------------------------------------------------------------
__global__ void dg_selftest_wait_kernel(volatile uint32_t* flag, long long limit_cycles, DevStatus* status) {
  const long long t0 = clock64();
  while (*flag == 0u) {
    if (clock64() - t0 > limit_cycles) {
      dev_status_set(status, DG_DEV_WAIT_TIMEOUT, KID_SELFTEST, blockIdx.x, 0u);
      return;
    }
  }
}
void launch_selftest_wait(uint32_t* flag, long long limit_cycles, DevStatus* status, cudaStream_t st) {
  dg_selftest_wait_kernel<<<1, 1, 0, st>>>(flag, limit_cycles, status);
}

// fill helpers for degenerate launches
__global__ void dg_fill_f32_kernel(float* p, float v, size_t n) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) p[i] = v;
}
void launch_fill_f32(float* p, float v, size_t n, cudaStream_t st) {
  if (n == 0) return;
  size_t g = (n + 255) / 256;
  if (g > 1024) g = 1024;
  dg_fill_f32_kernel<<<unsigned(g), 256, 0, st>>>(p, v, n);
}

}  // namespace dg
