// The projections either side of the attention stage, for the canvas rows of one denoise step, on sm_100a:
//   D[M][N] = A[M][K] . W[N][K]^T      (bf16 in, fp32 accumulate in tensor memory, bf16 out)
// with M = canvas rows (<= 256), the stacked Q|K|V projection in front of the attention
// (src/metal/step_kernel/enc.rs:1560-1629 of the reference: 256 x 2816 -> 4096 + 2048 + 2048) and the output
// projection behind it (enc.rs:871-886), plus the row-wise kernels that frame them: the input RMS norm
// (enc.rs:1567-1573, src/shaders/elementwise/rms_norm_rows/rms_norm_rows_tiled.metal:16-78) and the
// post-attention norm + residual (enc.rs:888-911, src/shaders/elementwise/residual_half/residual_half.metal:9-22).
//
// GEMM: one CTA per 128 x BN tile of D.  Warp 0 streams A and W tiles of 64 contraction elements (TMA boxes
// {64, 128} and {64, BN}, 128-byte swizzle) through a ring of shared-memory stages, one lane of warp 1 issues
// tcgen05.mma M128 N(BN) K16 into BN columns of tensor memory, warps 2-5 (one per 32 TMEM lanes) convert and
// store.  The output columns are cut into up to three segments with their own destination and row stride (the
// reference's stacked segments: Q, K and V leave the one GEMM as three dense tensors, in the layout the
// attention stage reads), and the epilogue can write every row's sum of squares over the tile's columns, of
// the values as rounded to bf16, for the RMS norm that follows the output projection.
// With 256 rows the GEMM is bound by how fast the SMs pull the weight tiles through L2, not by the tensor pipe.
#include <cuda.h>

#include "dg_attn_sm100_common.cuh"
#include "dg_kernels.h"

namespace dg {

using namespace sm100;

namespace gm {
constexpr uint32_t GM = 128, BK = 64;   // rows of a tile, contraction elements per stage
constexpr uint32_t THREADS = 192;
constexpr uint32_t A_STAGE = GM * BK * 2;   // 16 KB
// stages of the ring: deep for the projections (44-128 contraction blocks per CTA); two for the score GEMM of the
// top-k path, whose contraction is four or eight blocks, so that three CTAs share an SM and one's epilogue overlaps
// another's loads
__host__ __device__ constexpr uint32_t stages(uint32_t bn, bool shallow) { return shallow ? 2u : bn >= 128 ? 6u : 8u; }
__host__ __device__ constexpr uint32_t smem_bytes(uint32_t bn, bool shallow) {
  return stages(bn, shallow) * (A_STAGE + bn * BK * 2) + 256 + 1024;
}
// pair form: every CTA stages its own 128 rows of A and HALF of the W tile
constexpr uint32_t PAIR_STAGES = 8;
__host__ __device__ constexpr uint32_t smem_bytes_pair(uint32_t bn) { return PAIR_STAGES * (A_STAGE + bn / 2 * BK * 2) + 256 + 1024; }
}  // namespace gm

// PAIR: the two row tiles of a 256-row problem form a cta_group::2 pair (cluster (2, 1, 1)): one lane of the leader's
// MMA warp issues M = 256 MMAs over both CTAs, each CTA supplies its own 128 rows of A and half of the N extent of W
// (tm_w then has boxes {64, BN / 2}), so a weight tile is staged once per pair instead of once per CTA: 24 KB instead
// of 32 KB cross L2 -> SM per CTA and contraction block.
template <uint32_t BN, bool SHALLOW, bool PAIR>
__global__ void __launch_bounds__(gm::THREADS, 1)
dg_gemm_sm100_kernel(const GemmParams g, const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w) {
  using namespace gm;
  constexpr uint32_t ST = PAIR ? PAIR_STAGES : stages(BN, SHALLOW), B_STAGE = (PAIR ? BN / 2 : BN) * BK * 2,
                     STAGE = A_STAGE + B_STAGE;
  enum : uint32_t { B_FULL = 0, B_EMPTY = ST, B_ACC = 2 * ST, B_COUNT = 2 * ST + 1 };
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_base = smem_base + ST * STAGE;
  volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + ST * STAGE + B_COUNT * 8);
  // pair form: blockIdx.x is the row tile (= the rank inside the cluster of (2, 1, 1)), blockIdx.y the column tile
  const uint32_t n_tile = PAIR ? blockIdx.y : blockIdx.x, n_tiles = PAIR ? gridDim.y : gridDim.x;
  const uint32_t n0 = n_tile * BN, m0 = (PAIR ? blockIdx.x : blockIdx.y) * GM;
  const uint32_t xi = PAIR ? cluster_ctarank() : 0u;       // position inside the pair = the row tile
  const bool is_leader = xi == 0u;
  auto lead_bar = [&](uint32_t idx) { return dsmem_addr(bar_addr(bar_base, idx), 0u); };
  auto pair_bar = [&](uint32_t idx) { return dsmem_addr(bar_addr(bar_base, idx), 1u); };
  // split-K: slice blockIdx.z of the contraction; its fp32 partial tile goes to plane blockIdx.z of g.part
  const uint32_t kb_all = g.K / BK;
  const uint32_t kb0 = uint32_t((uint64_t(blockIdx.z) * kb_all) / gridDim.z);
  const uint32_t n_kb = uint32_t((uint64_t(blockIdx.z + 1) * kb_all) / gridDim.z) - kb0;

  if (tid == 0) {
    for (uint32_t s = 0; s < ST; ++s) {
      mbar_init(bar_addr(bar_base, B_FULL + s), 1);
      mbar_init(bar_addr(bar_base, B_EMPTY + s), 1);
    }
    mbar_init(bar_addr(bar_base, B_ACC), 1);
    ctl[1] = 0u;
    fence_mbar_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(&ctl[0])), BN);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(const_cast<uint32_t*>(&ctl[0])), BN < 32 ? 32 : BN);
      tmem_relinquish();
    }
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();      // the other CTA's barriers exist before anything of ours can signal them
  tc_fence_after();
  const uint32_t tmem = ctl[0];
  volatile uint32_t* abort_flag = &ctl[1];
  // the kernel behind this one may start its set-up; A was written by the kernel in front
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      for (uint32_t kb = 0; kb < n_kb; ++kb) {
        const uint32_t s = kb % ST, use = kb / ST;
        if (use > 0 && !mbar_wait(bar_addr(bar_base, B_EMPTY + s), (use - 1u) & 1u, abort_flag)) break;
        if (PAIR) {
          // both CTAs' bytes are counted on the leader's barrier
          if (is_leader) mbar_expect_tx(bar_addr(bar_base, B_FULL + s), 2 * STAGE);
          const uint32_t full = lead_bar(B_FULL + s);
          tma_load_3d_pair(smem_base + s * STAGE, &tm_a, full, int32_t((kb0 + kb) * BK), int32_t(m0), 0);
          tma_load_3d_pair(smem_base + s * STAGE + A_STAGE, &tm_w, full, int32_t((kb0 + kb) * BK), int32_t(n0 + xi * (BN / 2)),
                           int32_t(g.w_z));
          continue;
        }
        const uint32_t full = bar_addr(bar_base, B_FULL + s);
        mbar_expect_tx(full, STAGE);
        if (g.a_inner == 0u) tma_load_3d(smem_base + s * STAGE, &tm_a, full, int32_t((kb0 + kb) * BK), int32_t(m0), 0);
        else tma_load_3d(smem_base + s * STAGE, &tm_a, full, int32_t((kb0 + kb) * BK), 0, int32_t(m0 / g.a_inner));
        tma_load_3d(smem_base + s * STAGE + A_STAGE, &tm_w, full, int32_t((kb0 + kb) * BK), int32_t(n0), int32_t(g.w_z));
      }
    }
  } else if (warp == 1) {
    // the whole warp waits, one elected lane issues
    constexpr uint32_t IDESC = umma_idesc_bf16(PAIR ? 2 * GM : GM, BN, 0, 0);
    constexpr uint32_t HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version 1, 128-byte swizzle
    auto mkdesc = [](uint32_t lo, uint32_t hi) { return (uint64_t(hi) << 32) | uint64_t(lo); };
    for (uint32_t kb = 0; kb < n_kb && (!PAIR || is_leader); ++kb) {
      const uint32_t s = kb % ST, use = kb / ST;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, B_FULL + s), use & 1u, abort_flag))) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t a_lo = (((smem_base + s * STAGE) >> 4) & 0x3FFFu) | ((16u >> 4) << 16);
        const uint32_t b_lo = (((smem_base + s * STAGE + A_STAGE) >> 4) & 0x3FFFu) | ((16u >> 4) << 16);
#pragma unroll
        for (uint32_t kk = 0; kk < BK / 16; ++kk) {
          if (PAIR) umma_ss_pair(tmem, mkdesc(a_lo + kk * 2u, HI), mkdesc(b_lo + kk * 2u, HI), IDESC, (kb | kk) != 0u);
          else umma_ss(tmem, mkdesc(a_lo + kk * 2u, HI), mkdesc(b_lo + kk * 2u, HI), IDESC, (kb | kk) != 0u);
        }
        if (PAIR) {
          // the stage is free, and at the end the accumulator complete, in both CTAs
          umma_commit_pair(lead_bar(B_EMPTY + s));
          umma_commit_pair(pair_bar(B_EMPTY + s));
          if (kb + 1 == n_kb) {
            umma_commit_pair(lead_bar(B_ACC));
            umma_commit_pair(pair_bar(B_ACC));
          }
        } else {
          umma_commit(bar_addr(bar_base, B_EMPTY + s));
          if (kb + 1 == n_kb) umma_commit(bar_addr(bar_base, B_ACC));
        }
      }
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------------------- epilogue: thread = one row of the tile
    const uint32_t q4 = warp & 3u;                       // the 32 TMEM lanes this warp may read
    const uint32_t row = m0 + q4 * 32u + lane;
    const bool ok = __all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, B_ACC), 0u, abort_flag));
    tc_fence_after();
    // the tile lies inside one segment (segment starts are multiples of the tile width)
    uint32_t sg = 0;
    if (g.n_seg > 1 && n0 >= g.seg[1].col_begin) sg = 1;
    if (g.n_seg > 2 && n0 >= g.seg[2].col_begin) sg = 2;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(g.seg[sg].dst) + size_t(row) * g.seg[sg].ld + (n0 - g.seg[sg].col_begin);
    if (g.part != nullptr) {
      // fp32 partial sums of this slice of the contraction, row-major [slice][M][N]
      float* dp = g.part + (size_t(blockIdx.z) * g.M + row) * g.N + n0;
#pragma unroll 1
      for (uint32_t c = 0; ok && c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem + ((q4 * 32u) << 16) + c * 32u, v);
        tmem_wait_ld();
        if (row < g.M) {
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(dp + c * 32u + j * 4u) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
      }
    } else {
    float ss = 0.f;
    if (ok) {
#pragma unroll 1
      for (uint32_t c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem + ((q4 * 32u) << 16) + c * 32u, v);
        tmem_wait_ld();
        if (row < g.M) {
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            uint4 w4;
            w4.x = pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
            w4.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
            w4.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
            w4.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32u + j * 8u) = w4;
            if (g.rowsq != nullptr) {
              const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
              for (uint32_t e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(ws[e] << 16), hi = __uint_as_float(ws[e] & 0xffff0000u);
                ss = fmaf(lo, lo, ss);
                ss = fmaf(hi, hi, ss);
              }
            }
          }
        }
      }
    }
    if (g.rowsq != nullptr && row < g.M) g.rowsq[size_t(row) * n_tiles + n_tile] = ok ? ss : 0.f;
    }
  }

  if (*abort_flag) {
    if (tid == 0) dev_status_set(g.status, DG_DEV_WAIT_TIMEOUT, KID_GEMM, blockIdx.x + gridDim.x * blockIdx.y, n_kb);
    if (warp == 0 && lane == 0) {
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000ll) {}   // ~1 ms: far longer than any tile load in flight
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) {
    // neither CTA frees tensor memory or leaves while the other can still be the target of a pair-wide MMA or commit
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem, BN);
  } else if (warp == 1) {
    tmem_dealloc(tmem, BN < 32 ? 32 : BN);
  }
}

// Row-wise kernels: one block of 256 threads per row, a thread holds up to ROW_VEC 8-element vectors of the row in
// registers, so the row crosses memory once.
constexpr uint32_t ROW_VEC = 4;        // rows of up to 256 * 4 * 8 = 8192 elements

__device__ __forceinline__ float block_sum_256(float acc, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t += red[i];
  return t;
}

// y[row] = bf16(x[row] * rsqrt(mean(x[row]^2) + 1e-6) * w)
// (rms_norm_rows_tiled.metal:16-78: f32 sum of squares, v * inv, then * weight).
__global__ void __launch_bounds__(256) dg_rmsnorm_rows_kernel(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* y,
                                                              uint32_t dim) {
  __shared__ float red[8];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t n_vec = dim / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(blockIdx.x) * dim);
  uint4 v[ROW_VEC];
  float acc = 0.f;
#pragma unroll
  for (uint32_t j = 0; j < ROW_VEC; ++j) {
    const uint32_t i = threadIdx.x + j * 256u;
    v[j] = i < n_vec ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t ws[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
    for (uint32_t e = 0; e < 4; ++e) {
      const float lo = __uint_as_float(ws[e] << 16), hi = __uint_as_float(ws[e] & 0xffff0000u);
      acc = fmaf(lo, lo, acc);
      acc = fmaf(hi, hi, acc);
    }
  }
  const float inv = rsqrtf(block_sum_256(acc, red) / float(dim) + 1e-6f);
  uint4* yr = reinterpret_cast<uint4*>(y + size_t(blockIdx.x) * dim);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (uint32_t j = 0; j < ROW_VEC; ++j) {
    const uint32_t i = threadIdx.x + j * 256u;
    if (i >= n_vec) continue;
    const uint4 w4 = w != nullptr ? wr[i] : make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
    const uint32_t xs[4] = {v[j].x, v[j].y, v[j].z, v[j].w}, ws[4] = {w4.x, w4.y, w4.z, w4.w};
    uint32_t o[4];
#pragma unroll
    for (uint32_t e = 0; e < 4; ++e) {
      float lo = __uint_as_float(xs[e] << 16) * inv, hi = __uint_as_float(xs[e] & 0xffff0000u) * inv;
      if (w != nullptr) {
        lo *= __uint_as_float(ws[e] << 16);
        hi *= __uint_as_float(ws[e] & 0xffff0000u);
      }
      o[e] = pack_bf16x2(lo, hi);
    }
    yr[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// out[row] = bf16(hidden[row] + bf16(t[row] * inv * w)) with t[row] = bf16(sum over the n_part fp32 partial planes of
// the output projection), inv = rsqrt(mean(t[row]^2) + 1e-6)
// (enc.rs:888-911: the projection stored to the bf16 arena, its RMS norm in place, then the residual add).
// The planes are added in a fixed order: same bits every run.
__global__ void __launch_bounds__(256) dg_norm_residual_kernel(const float* part, uint32_t n_part, size_t plane,
                                                               const __nv_bfloat16* w, const __nv_bfloat16* hidden,
                                                               __nv_bfloat16* out, uint32_t dim) {
  __shared__ float red[8];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t n_vec = dim / 8;
  float t[ROW_VEC][8];
  float acc = 0.f;
#pragma unroll
  for (uint32_t j = 0; j < ROW_VEC; ++j) {
    const uint32_t i = threadIdx.x + j * 256u;
#pragma unroll
    for (uint32_t e = 0; e < 8; ++e) t[j][e] = 0.f;
    if (i >= n_vec) continue;
    for (uint32_t s = 0; s < n_part; ++s) {
      const float4* pr = reinterpret_cast<const float4*>(part + s * plane + size_t(blockIdx.x) * dim) + 2 * i;
      const float4 a = pr[0], b = pr[1];
      t[j][0] += a.x; t[j][1] += a.y; t[j][2] += a.z; t[j][3] += a.w;
      t[j][4] += b.x; t[j][5] += b.y; t[j][6] += b.z; t[j][7] += b.w;
    }
#pragma unroll
    for (uint32_t e = 0; e < 8; ++e) {
      t[j][e] = __bfloat162float(__float2bfloat16(t[j][e]));      // the projection as stored
      acc = fmaf(t[j][e], t[j][e], acc);
    }
  }
  const float inv = rsqrtf(block_sum_256(acc, red) / float(dim) + 1e-6f);
  const uint4* hr = reinterpret_cast<const uint4*>(hidden + size_t(blockIdx.x) * dim);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* orow = reinterpret_cast<uint4*>(out + size_t(blockIdx.x) * dim);
#pragma unroll
  for (uint32_t j = 0; j < ROW_VEC; ++j) {
    const uint32_t i = threadIdx.x + j * 256u;
    if (i >= n_vec) continue;
    const uint4 h4 = hr[i];
    const uint4 w4 = w != nullptr ? wr[i] : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t hs[4] = {h4.x, h4.y, h4.z, h4.w}, ws[4] = {w4.x, w4.y, w4.z, w4.w};
    uint32_t o[4];
#pragma unroll
    for (uint32_t e = 0; e < 4; ++e) {
      float lo = t[j][2 * e] * inv, hi = t[j][2 * e + 1] * inv;
      if (w != nullptr) {
        lo *= __uint_as_float(ws[e] << 16);
        hi *= __uint_as_float(ws[e] & 0xffff0000u);
      }
      lo = __bfloat162float(__float2bfloat16(lo));               // the normed projection as stored
      hi = __bfloat162float(__float2bfloat16(hi));
      o[e] = pack_bf16x2(__uint_as_float(hs[e] << 16) + lo, __uint_as_float(hs[e] & 0xffff0000u) + hi);
    }
    orow[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

cudaError_t sm100_gemm_configure() {
  cudaError_t e = cudaFuncSetAttribute(dg_gemm_sm100_kernel<128, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       int(gm::smem_bytes(128, false)));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(dg_gemm_sm100_kernel<64, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(gm::smem_bytes(64, false)));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(dg_gemm_sm100_kernel<128, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(gm::smem_bytes(128, true)));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(dg_gemm_sm100_kernel<64, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(gm::smem_bytes(64, true)));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(dg_gemm_sm100_kernel<128, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(gm::smem_bytes_pair(128)));
  return e;
}

static void pdl_cfg(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
  cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
}

// tm_a: {K, M, 1} map with boxes {64, 128, 1}; tm_w: {K, N, 1} map with boxes {64, bn, 1}
cudaError_t launch_gemm_sm100(const GemmParams& g, const CUtensorMap& tm_a, const CUtensorMap& tm_w, uint32_t bn,
                              cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  const dim3 grid(g.N / bn, (g.M + gm::GM - 1) / gm::GM, g.part != nullptr ? g.k_slices : 1u);
  const bool shallow = g.K / gm::BK <= 8;
  pdl_cfg(cfg, attr, grid, dim3(gm::THREADS), gm::smem_bytes(bn, shallow), st);
  if (shallow) {
    if (bn == 128) return cudaLaunchKernelEx(&cfg, dg_gemm_sm100_kernel<128, true, false>, g, tm_a, tm_w);
    return cudaLaunchKernelEx(&cfg, dg_gemm_sm100_kernel<64, true, false>, g, tm_a, tm_w);
  }
  if (bn == 128) return cudaLaunchKernelEx(&cfg, dg_gemm_sm100_kernel<128, false, false>, g, tm_a, tm_w);
  return cudaLaunchKernelEx(&cfg, dg_gemm_sm100_kernel<64, false, false>, g, tm_a, tm_w);
}

// Pair form: exactly two row tiles (128 < M <= 256), 128 output columns per tile; tm_w has boxes {64, 64, 1}.
cudaError_t launch_gemm_sm100_pair(const GemmParams& g, const CUtensorMap& tm_a, const CUtensorMap& tm_w, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, g.N / 128, g.part != nullptr ? g.k_slices : 1u);
  cfg.blockDim = dim3(gm::THREADS);
  cfg.dynamicSmemBytes = gm::smem_bytes_pair(128);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, dg_gemm_sm100_kernel<128, false, true>, g, tm_a, tm_w);
}

cudaError_t launch_rmsnorm_rows(const void* x, const void* w, void* y, uint32_t rows, uint32_t dim, cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  pdl_cfg(cfg, attr, dim3(rows), dim3(256), 0, st);
  return cudaLaunchKernelEx(&cfg, dg_rmsnorm_rows_kernel, static_cast<const __nv_bfloat16*>(x),
                            static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), dim);
}

cudaError_t launch_norm_residual(const float* part, uint32_t n_part, const void* w, const void* hidden, void* out,
                                 uint32_t rows, uint32_t dim, cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  pdl_cfg(cfg, attr, dim3(rows), dim3(256), 0, st);
  return cudaLaunchKernelEx(&cfg, dg_norm_residual_kernel, part, n_part, size_t(rows) * dim,
                            static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(hidden),
                            static_cast<__nv_bfloat16*>(out), dim);
}

}  // namespace dg
