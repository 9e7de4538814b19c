// Host-callable launchers of the kernels in this directory.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "dg_common.cuh"

namespace dg {

void launch_append(const AppendParams& p, const RopeParams& rp, cudaStream_t st, bool early = false);
void launch_attn_general(const AttnParams& p, cudaStream_t st);
void launch_merge_local(uint32_t n_parts, uint32_t rows, uint32_t D, const float* o, const float* m,
                        const float* l, __nv_bfloat16* out, cudaStream_t st);
void launch_merge_pack(uint32_t rows, uint32_t D, const float* o, const float* m_local, const float* m_global,
                       const float* l, float* pay, cudaStream_t st);
void launch_merge_finalize(uint32_t rows, uint32_t D, const float* pay, __nv_bfloat16* out, cudaStream_t st);
void launch_visibility(const MaskParams& mk, uint32_t C, uint8_t* out, cudaStream_t st);
void launch_fill_f32(float* p, float v, size_t n, cudaStream_t st);
void launch_p2p_merge(const P2pParams& q, void* out, int num_sms, cudaStream_t st);
// push form: every rank sends each row of its partial to the rank that owns the row, the owner merges;
// `out` receives this rank's row slice only (rows [rank * rows / world, (rank + 1) * rows / world))
cudaError_t launch_p2p_push_merge(const P2pParams& q, void* out, int num_sms, cudaStream_t st);
// host pipeline: push this rank's row slice of the staged queries (slot) to every peer and wait for theirs
cudaError_t launch_p2p_qgather(const P2pParams& q, uint32_t slot, uint32_t uses, cudaStream_t st);
void launch_selftest_wait(uint32_t* flag, long long limit_cycles, DevStatus* status, cudaStream_t st);

// Tensor-core kernel (head_dim 256).  tm_k / tm_v: 3-D tensor maps {D, cap, Hkv}, box {64, 128, 1},
// 128-byte swizzle.  Returns the CUDA error of the launch.
constexpr uint32_t kSm100MaxSplits = 32;
cudaError_t sm100_attn_configure();   // one-time cudaFuncSetAttribute
cudaError_t launch_attn_sm100(const AttnParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                              cudaStream_t st);
uint32_t sm100_query_tiles(uint32_t C, uint32_t G, uint32_t Hkv);   // CTAs in grid.x
// CTA-pair variant (cta_group::2): tm_k64 is the K tensor map with box {64, 64, 1}
cudaError_t sm100_pair_configure();
cudaError_t launch_attn_sm100_pair(const AttnParams& p, const CUtensorMap& tm_k64, const CUtensorMap& tm_v,
                                   cudaStream_t st);
uint32_t sm100_pair_query_tiles(uint32_t C, uint32_t G, uint32_t Hkv);
// up to kMaxBatchLaunch independent canvases of one geometry, split count and kernel form in ONE launch
cudaError_t launch_attn_sm100_batch(const AttnParams* p, const CUtensorMap* const* tm_k, const CUtensorMap* const* tm_v,
                                    uint32_t n, bool pair, cudaStream_t st);
int sm100_max_active_clusters(uint32_t cluster_y);        // single-CTA kernel, clusters (1, y, 1)
int sm100_pair_max_active_clusters(uint32_t cluster_y);   // pair kernel, clusters (2, y, 1)
// head_dim 512 (csrc/dg_attn_sm100_hd512.cu): tm_k / tm_v are {512, cap, Hkv} maps with boxes {64, 64, 1}
cudaError_t sm100_hd512_configure();
cudaError_t launch_attn_sm100_hd512(const AttnParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                                    cudaStream_t st);
uint32_t sm100_hd512_key_tiles(const MaskParams& mk);             // key tiles of 64 keys per CTA
// head_dim 512, CTA-pair form (csrc/dg_attn_sm100_hd512x.cu): same maps; clusters of two CTAs that exchange P
cudaError_t sm100_hd512x_configure();
cudaError_t launch_attn_sm100_hd512x(const AttnParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                                     cudaStream_t st);
uint32_t sm100_hd512x_key_steps(const MaskParams& mk);            // pairs of 64-key tiles per cluster
// head_dim 512, four CTAs per cluster (csrc/dg_attn_sm100_hd512q.cu): the exchange above plus cta_group::2 MMAs over
// two query tiles; tm_k has boxes {64, 32, 1} (each CTA stages half of a key tile), tm_v as above
cudaError_t sm100_hd512q_configure();
cudaError_t launch_attn_sm100_hd512q(const AttnParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                                     cudaStream_t st);
uint32_t sm100_key_tiles(const MaskParams& mk);                     // upper bound of key tiles per CTA
// projections and row-wise kernels either side of the attention stage (csrc/dg_gemm_sm100.cu)
cudaError_t sm100_gemm_configure();
cudaError_t launch_gemm_sm100(const GemmParams& g, const CUtensorMap& tm_a, const CUtensorMap& tm_w, uint32_t bn,
                              cudaStream_t st);
// top-k selection + gathered PV (csrc/dg_topk.cu)
cudaError_t launch_topk_select_pv(const TopkParams& p, cudaStream_t st);
cudaError_t launch_gemm_sm100_pair(const GemmParams& g, const CUtensorMap& tm_a, const CUtensorMap& tm_w, cudaStream_t st);
cudaError_t launch_rmsnorm_rows(const void* x, const void* w, void* y, uint32_t rows, uint32_t dim, cudaStream_t st);
cudaError_t launch_norm_residual(const float* part, uint32_t n_part, const void* w, const void* hidden, void* out,
                                 uint32_t rows, uint32_t dim, cudaStream_t st);

}  // namespace dg
