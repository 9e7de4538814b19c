// Top-k sparse attention of the reference's full layers (DGQ_ATTN_TOPK_DECODE: src/shaders/attn/attention_topk/,
// oracle src/shaders/attn/attention_topk/cpu.rs:39-120), the selection and gathered-PV half.
//
// Per (canvas row, query head): only the k highest-scoring visible keys are kept (ties: lower index first), the
// softmax is renormalised over them and O = sum_j p_j V[idx_j].  The scores of all keys come from a tensor-core GEMM
// (dg_gemm_sm100_kernel: S[h][row][T] = Qn . K^T as bf16); this kernel
//   1. finds the k-th largest 16-bit score with two 256-bin radix histograms (the reference's two levels on its u16
//      key plane, attention_topk.metal:186-262), reading the row of the plane from L2;
//   2. keeps every key above that value and, of the keys that share it, the best by EXACT fp32 score (recomputed
//      from Q and K; ties by index) - or, when more than CAND_CAP keys share it (degenerate inputs: identical
//      scores), the lowest indices;
//   3. recomputes the exact fp32 scores of the k winners, softmax, and gathers V.
// One CTA of 256 threads per (row, head).
#include <cuda.h>

#include "dg_common.cuh"
#include "dg_kernels.h"
#include "sm100_ptx.cuh"

namespace dg {

namespace tk {
constexpr uint32_t THREADS = 256;
constexpr uint32_t K_CAP = 1024;      // most keys kept per row (the reference's largest slot capacity)
constexpr uint32_t CAND_CAP = 1024;   // keys sharing the threshold value that are still ranked by exact score
}  // namespace tk

// larger key = larger bf16 value; -0 and +0 differ, NaN sorts above +inf and is never produced by finite inputs
__device__ __forceinline__ uint32_t bf16_order_key(uint16_t b) {
  return (b & 0x8000u) ? (~uint32_t(b) & 0xffffu) : (uint32_t(b) | 0x8000u);
}

__device__ __forceinline__ float dot_row_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, uint32_t D, uint32_t lane) {
  // one warp, 16-byte loads; D is a multiple of 256 or the tail is handled by the stride loop
  float acc = 0.f;
  for (uint32_t c = lane; c < D / 8; c += 32) {
    const uint4 x = reinterpret_cast<const uint4*>(a)[c], y = reinterpret_cast<const uint4*>(b)[c];
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc = fmaf(__uint_as_float(xs[e] << 16), __uint_as_float(ys[e] << 16), acc);
      acc = fmaf(__uint_as_float(xs[e] & 0xffff0000u), __uint_as_float(ys[e] & 0xffff0000u), acc);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  return acc;
}

__global__ void __launch_bounds__(tk::THREADS) dg_topk_select_pv_kernel(const TopkParams p) {
  using namespace tk;
  __shared__ uint32_t hist[256];
  __shared__ uint32_t whist[THREADS / 32][256];   // one histogram per warp, added up into hist
  __shared__ float o_part[THREADS / 32][512];     // the warps' partial output rows
  __shared__ uint32_t s_idx[K_CAP];      // winners
  __shared__ float s_sc[K_CAP];          // their exact scores, then their probabilities
  __shared__ uint32_t c_idx[CAND_CAP];   // keys that share the threshold value
  __shared__ float c_sc[CAND_CAP];
  __shared__ uint32_t sh[8];             // 0 winners, 1 candidates, 2 bin, 3 need, 4 above, 5 n_valid
  __shared__ float red[8];
  __shared__ uint32_t scan[THREADS];
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t i = blockIdx.x, h = blockIdx.y;           // canvas row, query head
  const uint32_t kvh = h / p.G, g = h % p.G;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint16_t* srow = p.scores + (size_t(kvh) * p.head_rows + size_t(i) * p.G + g) * p.ld;
  const MaskParams mk = p.mask;
  const RowVis rv = mask_row(mk, i);
  const uint32_t T = mk.can_hi;
  const bool all_vis = mask_range_full(mk, rv, 0u, T);       // every key below T is visible to this row
  auto visible = [&](uint32_t t) { return all_vis || mask_visible_row(mk, rv, t); };
  // every visible key of the row, eight per 16-byte load (the row of the plane starts on a 16-byte boundary and is
  // padded to whole tiles), two loads in flight per thread: f(t, key)
  const uint4* row4 = reinterpret_cast<const uint4*>(srow);
  const uint32_t n8 = (T + 7u) / 8u;
  auto for_keys = [&](auto f) {
#pragma unroll 2
    for (uint32_t c = tid; c < n8; c += THREADS) {
      const uint4 x = row4[c];
      const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
      const uint32_t base = c * 8u;
      const bool whole = all_vis && base + 8u <= T;      // no key of the chunk needs a bounds or mask test
#pragma unroll
      for (uint32_t w = 0; w < 4; ++w) {
        // both order-preserving keys of the word at once: a negative value is complemented, a positive one gets
        // its sign bit set
        const uint32_t sg = (xs[w] >> 15) & 0x00010001u;
        const uint32_t k2 = xs[w] ^ ((sg * 0xffffu) | 0x80008000u);
        const uint32_t t = base + 2u * w;
        if (whole || (t < T && visible(t))) f(t, k2 & 0xffffu);
        if (whole || (t + 1u < T && visible(t + 1u))) f(t + 1u, k2 >> 16);
      }
    }
  };
  auto zero_whist = [&]() {
    for (uint32_t b = tid; b < (THREADS / 32) * 256; b += THREADS) (&whist[0][0])[b] = 0u;
  };
  auto fold_whist = [&]() {
    for (uint32_t b = tid; b < 256; b += THREADS) {
      uint32_t c = 0;
#pragma unroll
      for (uint32_t w = 0; w < THREADS / 32; ++w) c += whist[w][b];
      hist[b] = c;
    }
  };

  // ---- visible keys and k
  uint32_t nv = 0;
  if (!all_vis)
    for (uint32_t t = tid; t < T; t += THREADS) nv += visible(t) ? 1u : 0u;
  if (tid < 8) sh[tid] = 0u;
  zero_whist();
  __syncthreads();
  if (!all_vis) atomicAdd(&sh[5], nv);
  __syncthreads();
  const uint32_t n_valid = all_vis ? T : sh[5];
  uint32_t k_req = p.k_fixed;
  if (p.k_div != 0u) {
    k_req = n_valid / p.k_div;
    k_req = k_req < p.k_min ? p.k_min : k_req;
    k_req = k_req > p.k_max ? p.k_max : k_req;
  }
  uint32_t k = k_req < n_valid ? k_req : n_valid;
  if (k > K_CAP) k = K_CAP;
  __nv_bfloat16* orow = p.out + (size_t(i) * p.Hq + h) * p.D;
  if (k == 0u) {
    for (uint32_t d = tid; d < p.D; d += THREADS) orow[d] = __float2bfloat16(0.f);
    return;
  }

  // ---- level 1: top byte of the key
  // (one histogram per warp: scores cluster on a few exponent values, a single one would serialise on a few bins)
  for_keys([&](uint32_t, uint32_t key) { atomicAdd(&whist[warp][key >> 8], 1u); });
  __syncthreads();
  fold_whist();
  __syncthreads();
  if (tid == 0) {
    uint32_t cum = 0, b1 = 0;
    for (int b = 255; b >= 0; --b) {
      if (cum + hist[b] >= k) {
        b1 = uint32_t(b);
        break;
      }
      cum += hist[b];
    }
    sh[2] = b1;
    sh[4] = cum;          // keys whose top byte is larger
  }
  __syncthreads();
  const uint32_t bin1 = sh[2];
  uint32_t above = sh[4];
  __syncthreads();
  zero_whist();
  __syncthreads();
  // ---- level 2: low byte inside that bin
  for_keys([&](uint32_t, uint32_t key) {
    if ((key >> 8) == bin1) atomicAdd(&whist[warp][key & 0xffu], 1u);
  });
  __syncthreads();
  fold_whist();
  __syncthreads();
  if (tid == 0) {
    uint32_t cum = above, b2 = 0;
    for (int b = 255; b >= 0; --b) {
      if (cum + hist[b] >= k) {
        b2 = uint32_t(b);
        break;
      }
      cum += hist[b];
    }
    sh[2] = (bin1 << 8) | b2;     // the k-th largest 16-bit key
    sh[4] = cum;                  // keys strictly above it: all kept
    sh[3] = k - cum;              // still to take from the keys that share it
    sh[1] = hist[b2];             // how many share it
  }
  __syncthreads();
  const uint32_t thr = sh[2], need = sh[3], n_cand = sh[1];
  above = sh[4];
  const bool ranked = n_cand <= CAND_CAP;
  __syncthreads();
  if (tid == 0) sh[1] = 0u;
  __syncthreads();

  // ---- emit the keys above the threshold; collect (or count) the ones that share it
  uint32_t my_cand = 0;
  const uint32_t per = (T + THREADS - 1) / THREADS;          // contiguous index ranges, for the index-ordered path
  if (ranked) {
    for_keys([&](uint32_t t, uint32_t key) {
      if (key > thr) s_idx[atomicAdd(&sh[0], 1u)] = t;
      else if (key == thr) c_idx[atomicAdd(&sh[1], 1u)] = t;
    });
  } else {
    const uint32_t t_lo = tid * per, t_hi = (t_lo + per < T) ? t_lo + per : T;
    for (uint32_t t = t_lo; t < t_hi; ++t) {
      if (!visible(t)) continue;
      const uint32_t key = bf16_order_key(srow[t]);
      if (key > thr) s_idx[atomicAdd(&sh[0], 1u)] = t;
      else if (key == thr) ++my_cand;
    }
  }
  __syncthreads();
  const __nv_bfloat16* qrow = p.q + (size_t(i) * p.Hq + h) * p.D;
  const __nv_bfloat16* kbase = p.k + size_t(kvh) * p.cap * p.D;
  const __nv_bfloat16* vbase = p.v + size_t(kvh) * p.cap * p.D;
  if (ranked) {
    // exact scores of the candidates; a candidate is kept when fewer than `need` others beat it (score, then index)
    for (uint32_t c = warp; c < n_cand; c += THREADS / 32) {
      const float s = dot_row_bf16(qrow, kbase + size_t(c_idx[c]) * p.D, p.D, lane);
      if (lane == 0) c_sc[c] = s;
    }
    __syncthreads();
    for (uint32_t c = tid; c < n_cand; c += THREADS) {
      const float s = c_sc[c];
      const uint32_t t = c_idx[c];
      uint32_t better = 0;
      for (uint32_t o = 0; o < n_cand; ++o) {
        const float so = c_sc[o];
        better += (so > s || (so == s && c_idx[o] < t)) ? 1u : 0u;
      }
      if (better < need) s_idx[atomicAdd(&sh[0], 1u)] = t;
    }
  } else {
    // identical scores in bulk: the lowest indices, by an exclusive scan over the threads' index ranges
    scan[tid] = my_cand;
    __syncthreads();
    if (tid == 0) {
      uint32_t run = 0;
      for (uint32_t j = 0; j < THREADS; ++j) {
        const uint32_t c = scan[j];
        scan[j] = run;
        run += c;
      }
    }
    __syncthreads();
    uint32_t before = scan[tid];
    const uint32_t t_lo = tid * per, t_hi = (t_lo + per < T) ? t_lo + per : T;
    for (uint32_t t = t_lo; t < t_hi && before < need; ++t) {
      if (!visible(t)) continue;
      if (bf16_order_key(srow[t]) == thr) {
        s_idx[atomicAdd(&sh[0], 1u)] = t;
        ++before;
      }
    }
  }
  __syncthreads();
  // sh[0] == k now.  The winners were appended in the order the threads got to them: sort them by index, so that
  // every sum below is taken in the same order in every run.
  for (uint32_t j = tid; j < k; j += THREADS) {
    const uint32_t t = s_idx[j];
    uint32_t rank = 0;
    for (uint32_t o = 0; o < k; ++o) rank += s_idx[o] < t ? 1u : 0u;
    c_idx[rank] = t;
  }
  __syncthreads();
  for (uint32_t j = tid; j < k; j += THREADS) s_idx[j] = c_idx[j];
  __syncthreads();

  // ---- exact scores of the winners, softmax over them
#pragma unroll 2
  for (uint32_t j = warp; j < k; j += THREADS / 32) {
    const float s = dot_row_bf16(qrow, kbase + size_t(s_idx[j]) * p.D, p.D, lane);
    if (lane == 0) s_sc[j] = s * p.scale_log2;
  }
  __syncthreads();
  float mx = -INFINITY;
  for (uint32_t j = tid; j < k; j += THREADS) mx = fmaxf(mx, s_sc[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float l = 0.f;
  for (uint32_t j = tid; j < k; j += THREADS) {
    const float pj = fast_exp2(s_sc[j] - mx);
    s_sc[j] = pj;
    l += pj;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  if (lane == 0) red[warp] = l;
  __syncthreads();
  l = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) l += red[w];
  const float inv_l = l > 0.f ? 1.0f / l : 0.f;

  // ---- O = sum_j p_j V[idx_j]: a warp takes every eighth kept key, its lanes cover the value row with 16-byte
  // loads (several rows in flight), and the eight partial rows meet in shared memory
  __syncthreads();
  const uint32_t n_chunk = p.D / 256;            // 16-byte chunks per lane: 1 at head_dim 256, 2 at 512
  float acc[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) acc[e] = 0.f;
#pragma unroll 4
  for (uint32_t j = warp; j < k; j += THREADS / 32) {
    const uint4* vr = reinterpret_cast<const uint4*>(vbase + size_t(s_idx[j]) * p.D);
    const float pj = s_sc[j];
#pragma unroll
    for (uint32_t c = 0; c < 2; ++c) {
      if (c >= n_chunk) break;
      const uint4 x = vr[c * 32u + lane];
      const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[c * 8 + 2 * e] = fmaf(pj, __uint_as_float(xs[e] << 16), acc[c * 8 + 2 * e]);
        acc[c * 8 + 2 * e + 1] = fmaf(pj, __uint_as_float(xs[e] & 0xffff0000u), acc[c * 8 + 2 * e + 1]);
      }
    }
  }
#pragma unroll
  for (uint32_t c = 0; c < 2; ++c) {
    if (c >= n_chunk) break;
#pragma unroll
    for (int e = 0; e < 8; ++e) o_part[warp][(c * 32u + lane) * 8u + e] = acc[c * 8 + e];
  }
  __syncthreads();
  for (uint32_t d2 = tid; d2 < p.D / 2; d2 += THREADS) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (uint32_t w = 0; w < THREADS / 32; ++w) {      // fixed order: same bits every run
      a0 += o_part[w][2 * d2];
      a1 += o_part[w][2 * d2 + 1];
    }
    reinterpret_cast<uint32_t*>(orow)[d2] = pack_bf16x2(a0 * inv_l, a1 * inv_l);
  }
}

cudaError_t launch_topk_select_pv(const TopkParams& p, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.C, p.Hq);
  cfg.blockDim = dim3(tk::THREADS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, dg_topk_select_pv_kernel, p);
}

}  // namespace dg
