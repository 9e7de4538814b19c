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
__host__ __device__ constexpr uint32_t stages(uint32_t bn) { return bn >= 128 ? 6u : 8u; }
__host__ __device__ constexpr uint32_t smem_bytes(uint32_t bn) { return stages(bn) * (A_STAGE + bn * BK * 2) + 256 + 1024; }
}  // namespace gm

template <uint32_t BN>
__global__ void __launch_bounds__(gm::THREADS, 1)
dg_gemm_sm100_kernel(const GemmParams g, const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w) {
  using namespace gm;
  constexpr uint32_t ST = stages(BN), B_STAGE = BN * BK * 2, STAGE = A_STAGE + B_STAGE;
  enum : uint32_t { B_FULL = 0, B_EMPTY = ST, B_ACC = 2 * ST, B_COUNT = 2 * ST + 1 };
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_base = smem_base + ST * STAGE;
  volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + ST * STAGE + B_COUNT * 8);
  const uint32_t n0 = blockIdx.x * BN, m0 = blockIdx.y * GM;
  const uint32_t n_kb = g.K / BK;

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
    tmem_alloc(smem_u32(const_cast<uint32_t*>(&ctl[0])), BN < 32 ? 32 : BN);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
  }
  tc_fence_before();
  __syncthreads();
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
        const uint32_t full = bar_addr(bar_base, B_FULL + s);
        mbar_expect_tx(full, STAGE);
        tma_load_3d(smem_base + s * STAGE, &tm_a, full, int32_t(kb * BK), int32_t(m0), 0);
        tma_load_3d(smem_base + s * STAGE + A_STAGE, &tm_w, full, int32_t(kb * BK), int32_t(n0), 0);
      }
    }
  } else if (warp == 1) {
    // the whole warp waits, one elected lane issues
    constexpr uint32_t IDESC = umma_idesc_bf16(GM, BN, 0, 0);
    constexpr uint32_t HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version 1, 128-byte swizzle
    auto mkdesc = [](uint32_t lo, uint32_t hi) { return (uint64_t(hi) << 32) | uint64_t(lo); };
    for (uint32_t kb = 0; kb < n_kb; ++kb) {
      const uint32_t s = kb % ST, use = kb / ST;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_addr(bar_base, B_FULL + s), use & 1u, abort_flag))) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t a_lo = (((smem_base + s * STAGE) >> 4) & 0x3FFFu) | ((16u >> 4) << 16);
        const uint32_t b_lo = (((smem_base + s * STAGE + A_STAGE) >> 4) & 0x3FFFu) | ((16u >> 4) << 16);
#pragma unroll
        for (uint32_t kk = 0; kk < BK / 16; ++kk)
          umma_ss(tmem, mkdesc(a_lo + kk * 2u, HI), mkdesc(b_lo + kk * 2u, HI), IDESC, (kb | kk) != 0u);
        umma_commit(bar_addr(bar_base, B_EMPTY + s));
        if (kb + 1 == n_kb) umma_commit(bar_addr(bar_base, B_ACC));
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
    if (g.rowsq != nullptr && row < g.M) g.rowsq[size_t(row) * gridDim.x + blockIdx.x] = ok ? ss : 0.f;
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
  if (warp == 1) tmem_dealloc(tmem, BN < 32 ? 32 : BN);
}

// y[row] = bf16(x[row] * rsqrt(mean(x[row]^2) + 1e-6) * w), one block per row
// (rms_norm_rows_tiled.metal:16-78: f32 sum of squares, v * inv, then * weight).
__global__ void __launch_bounds__(256) dg_rmsnorm_rows_kernel(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* y,
                                                              uint32_t dim) {
  __shared__ float red[8];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const size_t base = size_t(blockIdx.x) * dim;
  float acc = 0.f;
  for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = __bfloat162float(x[base + i]);
    acc = fmaf(v, v, acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t += red[i];
  const float inv = rsqrtf(t / float(dim) + 1e-6f);
  for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = __bfloat162float(x[base + i]) * inv;
    if (w != nullptr) v *= __bfloat162float(w[i]);
    y[base + i] = __float2bfloat16(v);
  }
}

// out[row] = bf16(hidden[row] + bf16(t[row] * inv * w)), inv from the per-tile sums of squares the output
// projection left (enc.rs:888-911: RMS norm of the projection in place, then the residual add).
__global__ void __launch_bounds__(256) dg_norm_residual_kernel(const __nv_bfloat16* t, const float* rowsq, uint32_t n_part,
                                                               const __nv_bfloat16* w, const __nv_bfloat16* hidden,
                                                               __nv_bfloat16* out, uint32_t dim) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const size_t base = size_t(blockIdx.x) * dim;
  float s = 0.f;
  for (uint32_t i = 0; i < n_part; ++i) s += rowsq[size_t(blockIdx.x) * n_part + i];   // fixed order: same bits every run
  const float inv = rsqrtf(s / float(dim) + 1e-6f);
  for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = __bfloat162float(t[base + i]) * inv;
    if (w != nullptr) v *= __bfloat162float(w[i]);
    const float nv = __bfloat162float(__float2bfloat16(v));
    out[base + i] = __float2bfloat16(__bfloat162float(hidden[base + i]) + nv);
  }
}

cudaError_t sm100_gemm_configure() {
  cudaError_t e = cudaFuncSetAttribute(dg_gemm_sm100_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gm::smem_bytes(128)));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(dg_gemm_sm100_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gm::smem_bytes(64)));
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
  const dim3 grid(g.N / bn, (g.M + gm::GM - 1) / gm::GM);
  pdl_cfg(cfg, attr, grid, dim3(gm::THREADS), gm::smem_bytes(bn), st);
  if (bn == 128) return cudaLaunchKernelEx(&cfg, dg_gemm_sm100_kernel<128>, g, tm_a, tm_w);
  return cudaLaunchKernelEx(&cfg, dg_gemm_sm100_kernel<64>, g, tm_a, tm_w);
}

cudaError_t launch_rmsnorm_rows(const void* x, const void* w, void* y, uint32_t rows, uint32_t dim, cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  pdl_cfg(cfg, attr, dim3(rows), dim3(256), 0, st);
  return cudaLaunchKernelEx(&cfg, dg_rmsnorm_rows_kernel, static_cast<const __nv_bfloat16*>(x),
                            static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), dim);
}

cudaError_t launch_norm_residual(const void* t, const float* rowsq, uint32_t n_part, const void* w, const void* hidden,
                                 void* out, uint32_t rows, uint32_t dim, cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  pdl_cfg(cfg, attr, dim3(rows), dim3(256), 0, st);
  return cudaLaunchKernelEx(&cfg, dg_norm_residual_kernel, static_cast<const __nv_bfloat16*>(t), rowsq, n_part,
                            static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(hidden),
                            static_cast<__nv_bfloat16*>(out), dim);
}

}  // namespace dg
