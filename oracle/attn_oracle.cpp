// CPU oracle (C++/OpenMP twin) for the denoise-step canvas attention.
//
// TEST INFRASTRUCTURE ONLY: this file is the checker and the timed CPU baseline.
// Nothing in the shipped library links or calls it.
//
// It restates, in fp32 on bf16-rounded inputs, the arithmetic of the reference's own
// CPU code for this path (paths relative to the reference project):
//   rms_norm_head            src/shaders/attn/cpu.rs:67-75
//   apply_split_half_rope    src/shaders/attn/cpu.rs:31-44   (pairs (d, d+rot/2))
//   apply_proportional_rope  src/shaders/attn/cpu.rs:47-65   (pairs (d, hd/2+d))
//   qk_rope_kv               src/shaders/attn/cpu.rs:78-145
//   attention (online softmax, GQA kvh = qh / (Hq/Hkv))
//                            src/shaders/attn/cpu.rs:148-197
//   denoise window rule      src/shaders/attn/attention/attention.metal:52-63
//   causal (re-prefill) rule src/shaders/attn/attention/attention.metal:51,57-62
//   decoder bitmap mask      src/model/mask.rs:4-27, src/model/attention.rs:889-907
// The key loop is blocked (64-key tiles, online softmax carried as (m, l, O)) the way
// src/shaders/attn/attention_flash/mod.rs:20-95 blocks its CPU reference; the result is
// the same sum in a different association order.
//
// Parity pin: validated against the numpy oracle (<= 1e-5) and through it against the
// reference's known-answer values; the reference stores no golden attention outputs.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#include <limits>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

typedef struct {
  uint32_t n_q_heads, n_kv_heads, head_dim, canvas;
  uint32_t rotary_dim;
  float rope_theta, rms_eps, softmax_scale;
  uint32_t window, mask_mode, v_norm, rope_pairing;
} dgo_desc;

enum { DGO_MASK_NONE = 0, DGO_MASK_WINDOW_UNIFORM = 1, DGO_MASK_WINDOW_PER_ROW = 2, DGO_MASK_CAUSAL = 3 };

}  // extern "C"

namespace {

inline float bf16_to_f32(uint16_t b) {
  uint32_t u = uint32_t(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
  u += 0x7fffu + ((u >> 16) & 1u);
  return uint16_t(u >> 16);
}
inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

// norm (+weight) then RoPE of one head vector at one position, in place, fp32
void norm_rope_head(float* x, const float* w, const dgo_desc& d, const float* inv_freq, uint32_t pos,
                    bool rope) {
  const uint32_t D = d.head_dim;
  float ss = 0.f;
  for (uint32_t i = 0; i < D; ++i) ss += x[i] * x[i];
  const float inv = 1.0f / std::sqrt(ss / float(D) + d.rms_eps);
  for (uint32_t i = 0; i < D; ++i) x[i] = x[i] * inv * (w ? w[i] : 1.0f);
  if (!rope) return;
  const uint32_t half = d.rotary_dim / 2;
  const uint32_t off = d.rope_pairing == 0 ? half : D / 2;
  for (uint32_t i = 0; i < half; ++i) {
    const float a = float(pos) * inv_freq[i];
    const float c = std::cos(a), s = std::sin(a);
    const float x0 = x[i], x1 = x[off + i];
    x[i] = x0 * c - x1 * s;
    x[off + i] = x0 * s + x1 * c;
  }
}

constexpr int KT = 64;   // keys per tile
constexpr int RB = 16;   // stacked query rows per block

// S[r][k] = sum_d Q[r][d] * Kt[d][k]   (Kt is the key tile transposed: [D][KT])
__attribute__((target_clones("avx512f", "avx2,fma", "default")))
void score_tile(const float* __restrict__ Q, const float* __restrict__ Kt, float* __restrict__ S,
                int rows, int D) {
  for (int r0 = 0; r0 < rows; r0 += 4) {
    float acc[4][KT];
    for (int r = 0; r < 4; ++r)
      for (int k = 0; k < KT; ++k) acc[r][k] = 0.f;
    for (int d = 0; d < D; ++d) {
      const float* kr = Kt + size_t(d) * KT;
      for (int r = 0; r < 4; ++r) {
        const float qv = Q[size_t(r0 + r) * D + d];
#pragma omp simd
        for (int k = 0; k < KT; ++k) acc[r][k] += qv * kr[k];
      }
    }
    for (int r = 0; r < 4; ++r)
      for (int k = 0; k < KT; ++k) S[(r0 + r) * KT + k] = acc[r][k];
  }
}

// O[r][d] += sum_k P[r][k] * V[k][d]
__attribute__((target_clones("avx512f", "avx2,fma", "default")))
void pv_tile(const float* __restrict__ P, const float* __restrict__ V, float* __restrict__ O, int rows,
             int D) {
  for (int r = 0; r < rows; ++r) {
    float* o = O + size_t(r) * D;
    for (int k = 0; k < KT; k += 4) {
      const float p0 = P[r * KT + k], p1 = P[r * KT + k + 1], p2 = P[r * KT + k + 2],
                  p3 = P[r * KT + k + 3];
      if (p0 == 0.f && p1 == 0.f && p2 == 0.f && p3 == 0.f) continue;
      const float* v0 = V + size_t(k) * D;
      const float* v1 = v0 + D;
      const float* v2 = v1 + D;
      const float* v3 = v2 + D;
#pragma omp simd
      for (int dd = 0; dd < D; ++dd) o[dd] += p0 * v0[dd] + p1 * v1[dd] + p2 * v2[dd] + p3 * v3[dd];
    }
  }
}

}  // namespace

extern "C" {

// f32 inverse frequencies theta^(-2d/hd), d < rotary_dim/2 (src/shaders/attn/cpu.rs:35).
void dgo_rope_inv_freq(uint32_t rotary_dim, uint32_t head_dim, float theta, float* out) {
  for (uint32_t d = 0; d < rotary_dim / 2; ++d) out[d] = std::pow(theta, -2.0f * float(d) / float(head_dim));
}

// qk_rope_kv on canvas Q/K/V (bf16 bits in, bf16 bits out).  qw/kw may be NULL (unit).
void dgo_qk_rope_kv(const dgo_desc* dp, uint32_t kv_len, const uint16_t* q, const uint16_t* k,
                    const uint16_t* v, const uint16_t* qw, const uint16_t* kw, uint16_t* qn,
                    uint16_t* kn, uint16_t* vn) {
  const dgo_desc d = *dp;
  const uint32_t D = d.head_dim, C = d.canvas;
  std::vector<float> inv(std::max(1u, d.rotary_dim / 2));
  dgo_rope_inv_freq(d.rotary_dim, D, d.rope_theta, inv.data());
  std::vector<float> qwf, kwf;
  if (qw) { qwf.resize(D); for (uint32_t i = 0; i < D; ++i) qwf[i] = bf16_to_f32(qw[i]); }
  if (kw) { kwf.resize(D); for (uint32_t i = 0; i < D; ++i) kwf[i] = bf16_to_f32(kw[i]); }
#pragma omp parallel for schedule(static)
  for (int64_t tok = 0; tok < int64_t(C); ++tok) {
    std::vector<float> x(D);
    const uint32_t pos = kv_len + uint32_t(tok);
    for (uint32_t h = 0; h < d.n_q_heads; ++h) {
      const size_t off = (size_t(tok) * d.n_q_heads + h) * D;
      for (uint32_t i = 0; i < D; ++i) x[i] = bf16_to_f32(q[off + i]);
      norm_rope_head(x.data(), qw ? qwf.data() : nullptr, d, inv.data(), pos, true);
      for (uint32_t i = 0; i < D; ++i) qn[off + i] = f32_to_bf16(x[i]);
    }
    for (uint32_t h = 0; h < d.n_kv_heads; ++h) {
      const size_t off = (size_t(tok) * d.n_kv_heads + h) * D;
      for (uint32_t i = 0; i < D; ++i) x[i] = bf16_to_f32(k[off + i]);
      norm_rope_head(x.data(), kw ? kwf.data() : nullptr, d, inv.data(), pos, true);
      for (uint32_t i = 0; i < D; ++i) kn[off + i] = f32_to_bf16(x[i]);
      if (d.v_norm) {
        for (uint32_t i = 0; i < D; ++i) x[i] = bf16_to_f32(v[off + i]);
        norm_rope_head(x.data(), nullptr, d, inv.data(), pos, false);
        for (uint32_t i = 0; i < D; ++i) vn[off + i] = f32_to_bf16(x[i]);
      } else {
        for (uint32_t i = 0; i < D; ++i) vn[off + i] = v[off + i];
      }
    }
  }
}

// Visibility of key t for canvas row `row` (bit-exact mask rule).
int dgo_visible(const dgo_desc* d, uint32_t kv_len, uint32_t t0, uint32_t t1, int include_canvas,
                uint32_t row, uint32_t t) {
  uint32_t lo = 0;
  if (d->mask_mode != DGO_MASK_NONE && d->window != 0) {
    const uint32_t wm1 = d->window - 1;
    const uint32_t qpos = d->mask_mode == DGO_MASK_WINDOW_UNIFORM ? kv_len : kv_len + row;
    lo = qpos > wm1 ? qpos - wm1 : 0;
  }
  if (t >= kv_len) {
    if (!include_canvas || t >= kv_len + d->canvas) return 0;
    if (d->mask_mode == DGO_MASK_CAUSAL) return t <= kv_len + row && t >= lo;
    return 1;
  }
  return t >= lo && t >= t0 && t < t1;
}

void dgo_visibility(const dgo_desc* d, uint32_t kv_len, uint32_t t0, uint32_t t1, int include_canvas,
                    uint8_t* attend /*[C][kv_len+C]*/) {
  const uint32_t T = kv_len + d->canvas;
  if (t1 > kv_len) t1 = kv_len;
  for (uint32_t r = 0; r < d->canvas; ++r)
    for (uint32_t t = 0; t < T; ++t)
      attend[size_t(r) * T + t] = uint8_t(dgo_visible(d, kv_len, t0, t1, include_canvas, r, t));
}

// Attention of canvas rows [row_begin,row_end) over [prefix | canvas].
//   qn [C][Hq][D], kn/vn [C][Hkv][D]: outputs of dgo_qk_rope_kv (bf16 bits)
//   kp/vp [kv_len][Hkv][D]: the cache content (bf16 bits), token-major like the reference's
//   CPU KV view (K row stride = Hkv*D, src/model/attention.rs:861-887)
//   attend: optional bitmap [C][kv_len+C] overriding the window rule (may be NULL)
//   out [C][Hq][D] fp32; when m_out/l_out are non-NULL the output is left un-normalised.
// Returns 0.
int dgo_attention(const dgo_desc* dp, uint32_t kv_len, const uint16_t* qn, const uint16_t* kn,
                  const uint16_t* vn, const uint16_t* kp, const uint16_t* vp, const uint8_t* attend,
                  uint32_t t0, uint32_t t1, int include_canvas, uint32_t row_begin, uint32_t row_end,
                  float* out, float* m_out, float* l_out, int n_threads) {
  const dgo_desc d = *dp;
  const int D = int(d.head_dim);
  const uint32_t C = d.canvas, Hq = d.n_q_heads, Hkv = d.n_kv_heads, G = Hq / Hkv;
  const uint32_t T = kv_len + C;
  if (t1 > kv_len) t1 = kv_len;
  if (row_end > C) row_end = C;
  const bool partial = m_out != nullptr && l_out != nullptr;
  // key range that can be visible to any row
  uint32_t lo_any = t0;
  if (!attend && d.mask_mode != DGO_MASK_NONE && d.window != 0) {
    const uint32_t wm1 = d.window - 1;
    const uint32_t qpos = d.mask_mode == DGO_MASK_WINDOW_UNIFORM ? kv_len : kv_len + row_begin;
    lo_any = std::max(lo_any, qpos > wm1 ? qpos - wm1 : 0u);
  }
  if (attend) lo_any = 0;
  const uint32_t tile_lo = (lo_any / KT) * KT;
  const uint32_t n_rows = row_end > row_begin ? row_end - row_begin : 0;
  const uint32_t stacked = n_rows * G;                  // rows per kv head: (canvas row, group head)
  const uint32_t n_blocks = (stacked + RB - 1) / RB;
#ifdef _OPENMP
  if (n_threads > 0) omp_set_num_threads(n_threads);
#endif
#pragma omp parallel
  {
    std::vector<float> Qb(size_t(RB) * D), Kt(size_t(D) * KT), Vt(size_t(KT) * D), S(RB * KT),
        O(size_t(RB) * D);
    float mrun[RB], lrun[RB];
#pragma omp for collapse(2) schedule(dynamic, 1)
    for (int64_t kvh = 0; kvh < int64_t(Hkv); ++kvh) {
      for (int64_t blk = 0; blk < int64_t(n_blocks); ++blk) {
        const uint32_t s0 = uint32_t(blk) * RB;
        const int rows = int(std::min<uint32_t>(RB, stacked - s0));
        for (int r = 0; r < RB; ++r) {
          mrun[r] = -std::numeric_limits<float>::infinity();
          lrun[r] = 0.f;
          const uint32_t sidx = std::min<uint32_t>(s0 + r, stacked - 1);
          const uint32_t row = row_begin + sidx / G, h = uint32_t(kvh) * G + sidx % G;
          const uint16_t* src = qn + (size_t(row) * Hq + h) * D;
          for (int i = 0; i < D; ++i) Qb[size_t(r) * D + i] = bf16_to_f32(src[i]);
        }
        std::fill(O.begin(), O.end(), 0.f);
        for (uint32_t tb = tile_lo; tb < T; tb += KT) {
          // stage the key tile: K transposed, V as is (fp32)
          bool any_key = false;
          for (int k = 0; k < KT; ++k) {
            const uint32_t t = tb + k;
            const uint16_t *ks = nullptr, *vs = nullptr;
            if (t < kv_len) {
              ks = kp + (size_t(t) * Hkv + kvh) * D;
              vs = vp + (size_t(t) * Hkv + kvh) * D;
            } else if (t < T) {
              ks = kn + (size_t(t - kv_len) * Hkv + kvh) * D;
              vs = vn + (size_t(t - kv_len) * Hkv + kvh) * D;
            }
            if (ks) {
              any_key = true;
              for (int i = 0; i < D; ++i) {
                Kt[size_t(i) * KT + k] = bf16_to_f32(ks[i]);
                Vt[size_t(k) * D + i] = bf16_to_f32(vs[i]);
              }
            } else {
              for (int i = 0; i < D; ++i) {
                Kt[size_t(i) * KT + k] = 0.f;
                Vt[size_t(k) * D + i] = 0.f;
              }
            }
          }
          if (!any_key) continue;
          score_tile(Qb.data(), Kt.data(), S.data(), RB, D);
          for (int r = 0; r < rows; ++r) {
            const uint32_t sidx = s0 + r;
            const uint32_t row = row_begin + sidx / G;
            float* s = S.data() + r * KT;
            float mx = -std::numeric_limits<float>::infinity();
            for (int k = 0; k < KT; ++k) {
              const uint32_t t = tb + k;
              bool vis;
              if (t >= T) vis = false;
              else if (attend) vis = attend[size_t(row) * T + t] != 0;
              else vis = dgo_visible(&d, kv_len, t0, t1, include_canvas, row, t) != 0;
              s[k] = vis ? s[k] * d.softmax_scale : -std::numeric_limits<float>::infinity();
              mx = std::max(mx, s[k]);
            }
            if (mx == -std::numeric_limits<float>::infinity()) {
              for (int k = 0; k < KT; ++k) s[k] = 0.f;
              continue;
            }
            const float mn = std::max(mrun[r], mx);
            const float corr = std::exp(mrun[r] - mn);   // exp(-inf) = 0 on the first tile
            float sum = 0.f;
            for (int k = 0; k < KT; ++k) {
              const float p = std::exp(s[k] - mn);       // masked: exp(-inf) = 0
              s[k] = p;
              sum += p;
            }
            lrun[r] = lrun[r] * corr + sum;
            mrun[r] = mn;
            if (corr != 1.0f) {
              float* o = O.data() + size_t(r) * D;
              for (int i = 0; i < D; ++i) o[i] *= corr;
            }
          }
          for (int r = rows; r < RB; ++r)
            for (int k = 0; k < KT; ++k) S[r * KT + k] = 0.f;
          pv_tile(S.data(), Vt.data(), O.data(), rows, D);
        }
        for (int r = 0; r < rows; ++r) {
          const uint32_t sidx = s0 + r;
          const uint32_t row = row_begin + sidx / G, h = uint32_t(kvh) * G + sidx % G;
          float* dst = out + (size_t(row) * Hq + h) * D;
          const float* o = O.data() + size_t(r) * D;
          if (partial) {
            m_out[size_t(row) * Hq + h] = mrun[r];
            l_out[size_t(row) * Hq + h] = lrun[r];
            for (int i = 0; i < D; ++i) dst[i] = o[i];
          } else {
            const float invl = lrun[r] > 0.f ? 1.0f / lrun[r] : 0.f;
            for (int i = 0; i < D; ++i) dst[i] = o[i] * invl;
          }
        }
      }
    }
  }
  return 0;
}

int dgo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"
