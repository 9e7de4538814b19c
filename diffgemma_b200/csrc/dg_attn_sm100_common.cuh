// Definitions of the head_dim-256 attention kernel that the host side shares: tile geometry,
// shared-memory map, key-tile schedule, phase stamps.
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
constexpr uint32_t OFF_ML = OFF_XCH + 8192;             // (m, l, 1 / scale, -) of the on-chip partial rows, [BM] float4
constexpr uint32_t HBUF_LD = 264;                       // halves per row of the on-chip partial (padded 256)
constexpr uint32_t SMEM_BYTES = OFF_ML + 2048 + 1024;   // + alignment slack
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_S = 0;            // two S buffers of 128 columns
constexpr uint32_t TM_O = 256;          // O accumulator, 256 columns
constexpr float RESCALE_THRESHOLD = 8.0f;   // log2 units

struct TileSched {
  uint32_t a0, nA, b0, nB;
};
// Key tiles (absolute index = key / 128) a CTA whose canvas rows are [row_first, row_last] must visit:
// the prefix interval [lo(row_first), pre_hi) and the canvas interval [kv_len, can_hi) - in the causal
// mode only up to row_last's own position -, merged when they touch.  (The lower bounds grow with the
// row, the causal upper bound too, so the first row gives the lowest key and the last row the highest.)
__host__ __device__ inline TileSched tile_sched(const MaskParams& mk, uint32_t row_first, uint32_t row_last) {
  TileSched t{0, 0, 0, 0};
  const uint32_t lo = mask_row_lo(mk, row_first);
  if (mk.pre_hi > lo) {
    t.a0 = lo / BN;
    t.nA = (mk.pre_hi + BN - 1) / BN - t.a0;
  }
  const uint32_t can_hi = mask_can_hi_rows(mk, row_last);
  if (can_hi > mk.kv_len) {
    const uint32_t b0 = mk.kv_len / BN, b1 = (can_hi + BN - 1) / BN;
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
// Slots 6-11 hold SM-clock cycles that single threads spent waiting inside the key loop:
// 6 MMA issuer on K tiles, 7 on V tiles, 8 on P (softmax output), 9 its whole loop,
// 10 softmax thread 0 on S (scores), 11 softmax thread 0 on the rescale barrier.
// Slots 12-14 are time stamps inside the tail: 12 the last PV has completed, 13 the cluster's CTAs have all
// finished their MMAs (cluster merge only), 14 the partial rows of the cluster have all arrived.
constexpr uint32_t STAMP_SLOTS = 16;
__device__ __forceinline__ void stamp(const AttnParams& p, uint32_t slot) {
  if (p.stamps != nullptr && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.stamps[((size_t(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * STAMP_SLOTS + slot] = t;
  }
}
__device__ __forceinline__ void stamp_cycles(const AttnParams& p, uint32_t slot, long long cycles) {
  if (p.stamps != nullptr)
    p.stamps[((size_t(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * STAMP_SLOTS + slot] = (unsigned long long)cycles;
}
// runs a wait and, when profiling, adds the cycles it took to acc
template <class F>
__device__ __forceinline__ bool timed_wait(bool prof, long long& acc, F f) {
  if (!prof) return f();
  const long long t = clock64();
  const bool r = f();
  acc += clock64() - t;
  return r;
}


}  // namespace sm100
}  // namespace dg
