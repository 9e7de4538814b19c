// Definitions shared by the single-CTA and the CTA-pair variants of the head_dim-256 attention
// kernel: tile geometry, key-tile schedule, barrier slots, phase stamps.
#pragma once
#include <cuda.h>

#include "dg_common.cuh"
#include "sm100_ptx.cuh"

namespace dg {
namespace sm100 {


constexpr uint32_t BM = 128;            // query rows per CTA
constexpr uint32_t BN = 128;            // keys per tile
constexpr uint32_t HD = 256;            // head_dim
constexpr uint32_t ATOM_BYTES = 128 * 128;        // 128 rows x 128 B (64 bf16): one swizzle-atom column
constexpr uint32_t TILE_BYTES = 4 * ATOM_BYTES;   // 128 rows x 256 bf16
constexpr uint32_t OFF_Q = 0;
constexpr uint32_t OFF_K = TILE_BYTES;
constexpr uint32_t OFF_V = 2 * TILE_BYTES;
constexpr uint32_t OFF_BAR = 3 * TILE_BYTES;
constexpr uint32_t OFF_XCH = OFF_BAR + 256;             // row-group exchange scratch (8 KB)
constexpr uint32_t OFF_ML = OFF_XCH + 8192;             // (m, l) of the on-chip partial, [BM] float2
constexpr uint32_t OBUF_LD = 260;                       // floats per row of the on-chip partial (padded 256)
constexpr uint32_t SMEM_BYTES = OFF_ML + 1024 + 1024;   // + alignment slack
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_S = 0;            // two S buffers of 128 columns
constexpr uint32_t TM_O = 256;          // O accumulator, 256 columns
// CTA-pair variant: warps 0-7 = two softmax warpgroups (warp w and w+4 share the 32 query rows of
// TMEM quadrant w & 3; the first handles key columns 0-63 of every tile, the second 64-127),
// 8: K loader, 9: V loader, 10: TMEM allocation + the MMA-issuing thread
constexpr uint32_t N_SM_WARPS = 8;
constexpr uint32_t WARP_K = 8, WARP_V = 9, WARP_MMA = 10;
constexpr uint32_t N_THREADS = 352;
constexpr float RESCALE_THRESHOLD = 8.0f;   // log2 units

// barrier slots (8 bytes each) inside the barrier block
enum : uint32_t {
  BAR_Q = 0,
  BAR_K_FULL = 1,
  BAR_K_EMPTY = 2,
  BAR_V_FULL = 3,
  BAR_V_EMPTY = 4,
  BAR_S_FULL0 = 5,   // +1 for buffer 1
  BAR_P_FULL0 = 7,   // +1 for buffer 1
  BAR_PV_DONE = 9,   // one phase per key tile; only waited on when O must be rescaled
  BAR_O_FINAL = 10,  // single phase: every PV of this CTA has completed
  N_BARS = 11
};

struct TileSched {
  uint32_t a0, nA, b0, nB;
};
// Key tiles (absolute index = key / 128) a CTA whose first canvas row is `row_first` must visit:
// the prefix interval [lo, pre_hi) and the canvas interval [kv_len, can_hi), merged when they touch.
__host__ __device__ inline TileSched tile_sched(const MaskParams& mk, uint32_t row_first) {
  TileSched t{0, 0, 0, 0};
  const uint32_t lo = mask_row_lo(mk, row_first);
  if (mk.pre_hi > lo) {
    t.a0 = lo / BN;
    t.nA = (mk.pre_hi + BN - 1) / BN - t.a0;
  }
  if (mk.can_hi > mk.kv_len) {
    const uint32_t b0 = mk.kv_len / BN, b1 = (mk.can_hi + BN - 1) / BN;
    if (t.nA > 0 && b0 < t.a0 + t.nA) {
      const uint32_t a1 = (t.a0 + t.nA) > b1 ? (t.a0 + t.nA) : b1;
      t.nA = a1 - t.a0;
    } else {
      t.b0 = b0;
      t.nB = b1 - b0;
    }
  }
  return t;
}

__device__ __forceinline__ uint32_t bar_addr(uint32_t bar_base, uint32_t idx) { return bar_base + idx * 8u; }

// Phase time stamps (globaltimer, ns) of one CTA, written by thread 0 when a stamp buffer is given:
// 0 start, 1 set-up done, 2 Q prologue done, 3 main loop done, 4 epilogue done, 5 merge done.
__device__ __forceinline__ void stamp(const AttnParams& p, uint32_t slot) {
  if (p.stamps != nullptr && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.stamps[(size_t(blockIdx.y) * gridDim.x + blockIdx.x) * 8 + slot] = t;
  }
}


// named barrier shared by the two warps that own the same 32 query rows
__device__ __forceinline__ void pair_sync(uint32_t smw) {
  asm volatile("bar.sync %0, 64;" ::"r"(smw + 1u) : "memory");
}


}  // namespace sm100
}  // namespace dg
