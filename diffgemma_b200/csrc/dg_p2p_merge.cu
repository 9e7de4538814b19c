// Split-KV merge over peer memory (NVLink / NVSwitch), one process per GPU.
//
// Every rank owns an exchange buffer that the other ranks have mapped (CUDA IPC).  After its
// partial attention kernel a rank publishes "partial ready"; the merge kernel of rank r then reads
// the W partial rows of ITS slice of the query rows straight from the peers' buffers (plain
// loads over NVLink, no TMA, no multicast), merges them by log-sum-exp and stores the bf16 result
// rows into every rank's result area, publishes "slice r done" to every rank, and - once all W
// slices have landed locally - copies the result to the caller's output.  Two parities
// of every buffer and flag alternate between steps; flags carry a monotonically increasing step id.
//
// With two ranks the slices are not worth their second exchange: each rank reads the peer's whole
// partial (4.2 MB, a few microseconds of NVLink) and merges every row itself, so there is one flag
// round trip instead of two and no result scatter.
//
// All waits are bounded: a flag that does not arrive within the limit records DG_DEV_WAIT_TIMEOUT
// and the kernel carries on without it.
#include <cuda_fp16.h>

#include "dg_common.cuh"
#include "dg_kernels.h"

namespace dg {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_sys_f4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ float ld_sys_f(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// wait until *flag >= want (step ids only grow); false on timeout
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, long long limit_cycles) {
  const long long t0 = clock64();
  while (int32_t(ld_acquire_sys(flag) - want) < 0) {
    if (clock64() - t0 > limit_cycles) return false;
  }
  return true;
}

__global__ void __launch_bounds__(256) dg_p2p_merge_kernel(const P2pParams q, uint4* __restrict__ out) {
  __shared__ uint32_t s_ok;
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t par = q.parity;
  uint8_t* mine = q.peer[q.rank];
  if (tid == 0) s_ok = 1u;
  // 1. publish this rank's partial (written by the preceding kernel on the stream)
  //    by WRITING the step id into every rank's flag array, so that waiting is a poll of local memory
  if (blockIdx.x == 0 && tid < q.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(q.peer[tid] + q.off_pflag) + par * 8 + q.rank, q.step);
  }
  __syncthreads();
  // 2. every CTA waits for every peer's partial
  if (tid < q.world) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(mine + q.off_pflag) + par * 8 + tid;
    if (!wait_flag(f, q.step, q.wait_limit)) {
      s_ok = 0u;
      dev_status_set(q.status, DG_DEV_WAIT_TIMEOUT, KID_MERGE, blockIdx.x, tid);
    }
  }
  __syncthreads();
  // 3. merge this rank's slice of the rows (two ranks: every row, written straight to the output)
  const bool all_rows = q.all_rows != 0u;
  const uint32_t r0 = all_rows ? 0u : uint32_t((uint64_t(q.rank) * q.rows) / q.world);
  const uint32_t r1 = all_rows ? q.rows : uint32_t((uint64_t(q.rank + 1) * q.rows) / q.world);
  const uint32_t D = q.D, W = q.world;
  if (s_ok) {
    for (uint32_t row = r0 + blockIdx.x * 8 + warp; row < r1; row += gridDim.x * 8) {
      // the row's first 256 columns of every partial are requested together with its (m, l) pairs, so
      // that one NVLink round trip covers both
      float4 a0[8], b0[8];
#pragma unroll
      for (uint32_t w = 0; w < 8; ++w) {
        a0[w] = b0[w] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (w < W) {
          const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(q.peer[w] + q.off_o[par]) + size_t(row) * D + lane * 8);
          a0[w] = ld_sys_f4(src);
          b0[w] = ld_sys_f4(src + 1);
        }
      }
      float mw = -INFINITY, lw = 0.f;
      if (lane < W) {
        mw = ld_sys_f(reinterpret_cast<const float*>(q.peer[lane] + q.off_m[par]) + row);
        lw = ld_sys_f(reinterpret_cast<const float*>(q.peer[lane] + q.off_l[par]) + row);
      }
      float mg = mw;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, o));
      const float w_mine = (mw == -INFINITY) ? 0.f : expf(mw - mg);
      float lg = w_mine * lw;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) lg += __shfl_xor_sync(0xffffffffu, lg, o);
      const float inv = lg > 0.f ? 1.0f / lg : 0.f;
      for (uint32_t c0 = lane * 8; c0 < D; c0 += 256) {
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        float4 a[8], b[8];
#pragma unroll
        for (uint32_t w = 0; w < 8; ++w) {
          a[w] = a0[w];
          b[w] = b0[w];
          if (c0 >= 256u) {
            a[w] = b[w] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (w < W) {   // uniform: only the W real partials cross the link, all issued before first use
              const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(q.peer[w] + q.off_o[par]) + size_t(row) * D + c0);
              a[w] = ld_sys_f4(src);
              b[w] = ld_sys_f4(src + 1);
            }
          }
        }
#pragma unroll
        for (uint32_t w = 0; w < 8; ++w) {
          float wt = __shfl_sync(0xffffffffu, w_mine, int(w));
          if (w >= W) wt = 0.f;
          acc[0] += wt * a[w].x; acc[1] += wt * a[w].y; acc[2] += wt * a[w].z; acc[3] += wt * a[w].w;
          acc[4] += wt * b[w].x; acc[5] += wt * b[w].y; acc[6] += wt * b[w].z; acc[7] += wt * b[w].w;
        }
        __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv), h1 = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[4] * inv, acc[5] * inv), h3 = __floats2bfloat162_rn(acc[6] * inv, acc[7] * inv);
        uint4 o4;
        o4.x = *reinterpret_cast<uint32_t*>(&h0);
        o4.y = *reinterpret_cast<uint32_t*>(&h1);
        o4.z = *reinterpret_cast<uint32_t*>(&h2);
        o4.w = *reinterpret_cast<uint32_t*>(&h3);
        if (all_rows) {
          out[(size_t(row) * D + c0) / 8] = o4;
        } else {
          for (uint32_t w = 0; w < W; ++w)
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(q.peer[w] + q.off_res[par]) + size_t(row) * D + c0) = o4;
        }
      }
    }
  }
  if (all_rows) return;   // nothing was sent: no second exchange
  // 4. the last CTA to finish tells every rank that this rank's slice has landed.  One
  //    system-scope fence per CTA, issued after the CTA barrier, covers the stores of all its threads.
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    uint32_t* done = reinterpret_cast<uint32_t*>(mine + q.off_done) + par;
    const uint32_t old = atomicAdd(done, 1u);
    if (old == gridDim.x - 1) {
      *done = 0u;
      __threadfence_system();
      for (uint32_t w = 0; w < W; ++w)
        st_release_sys(reinterpret_cast<uint32_t*>(q.peer[w] + q.off_rflag) + par * 8 + q.rank, q.step);
    }
  }
  // 5. once every rank's slice has landed here, copy the result to the caller's output.  Every CTA
  //    of this grid is resident (at most one per SM), so waiting here cannot starve the CTA that
  //    publishes this rank's own flag.
  if (tid < W) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(mine + q.off_rflag) + par * 8 + tid;
    if (!wait_flag(f, q.step, q.wait_limit)) {
      s_ok = 0u;
      dev_status_set(q.status, DG_DEV_WAIT_TIMEOUT, KID_MERGE, blockIdx.x, 100u + tid);
    }
  }
  __syncthreads();
  if (!s_ok) return;   // a slice never arrived: the status word says so, the output is left alone
  const uint4* src = reinterpret_cast<const uint4*>(mine + q.off_res[par]);
  const size_t n = size_t(q.rows) * q.D / 8;   // 16-byte units
  for (size_t i = size_t(blockIdx.x) * 256 + tid; i < n; i += size_t(gridDim.x) * 256) out[i] = src[i];
}

// ------------------------------------------------------------------------------------------
// Push form (reduce-scatter): rank r owns the row slice [r * rows / W, (r + 1) * rows / W) of the
// output.  Phase A: every rank converts each row of its local fp32 partial to fp16 with one
// power-of-two scale per row (the row's largest magnitude lands in [2^14, 2^15): 11 significant bits
// relative to it, half the bytes) and STORES it, with its (m, l, 1 / scale) record, into the receive
// area of the rank that owns the row - posted writes over NVLink, nobody waits for a load to come
// back - then adds the number of rows it delivered to that owner's arrival counter (system-scope
// release after a system fence).  Phase B: the owner polls its own counter in LOCAL memory until all
// W x slice rows of this step have arrived, merges the W partial rows from local memory and writes
// the finished bf16 rows of its slice to `out`.  Nothing is scattered back and there is no second
// flag round: a host that needs every row on every rank gathers the slices afterwards.
// The counters only grow (the host passes how many steps have used this parity), so no kernel ever
// resets a word that a peer may still be adding to.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void p2p_stamp(const P2pParams& q, uint32_t slot) {
  if (q.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    q.stamps[slot] = t;
  }
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Phase A: convert the rows of this rank's fp32 partial (written by the attention kernel of the same step, buffer
// parity q.parity) and store them into the owners' receive slot q.send_slot; publish the delivered row counts.
__device__ __forceinline__ void p2p_phase_send(const P2pParams& q, uint32_t* s_rows) {
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t par = q.parity, slot = q.send_slot, W = q.world, D = q.D;
  uint8_t* mine = q.peer[q.rank];
  // ---- phase A: this CTA serves ONE owner, so that it signals exactly one counter, once
  {
    const uint32_t o = blockIdx.x % W, j = blockIdx.x / W;
    const uint32_t n_o = (gridDim.x - o + W - 1u) / W;   // CTAs that serve owner o
    const uint32_t r0 = uint32_t((uint64_t(o) * q.rows) / W), r1 = uint32_t((uint64_t(o + 1) * q.rows) / W);
    const float* src_o = reinterpret_cast<const float*>(mine + q.off_o[par]);
    const float* src_m = reinterpret_cast<const float*>(mine + q.off_m[par]);
    const float* src_l = reinterpret_cast<const float*>(mine + q.off_l[par]);
    __half* dst_rows = reinterpret_cast<__half*>(q.peer[o] + q.off_recv[slot]) + size_t(q.rank) * q.slice_cap * D;
    float4* dst_ml = reinterpret_cast<float4*>(q.peer[o] + q.off_rml[slot]) + size_t(q.rank) * q.slice_cap;
    uint32_t done = 0;
    // two rows per warp and iteration, all their loads issued before the first use: the pass is bound by the
    // latency of the loads, not by their bytes
    constexpr uint32_t RA = 2;
    for (uint32_t row0 = r0 + (j * 8u + warp) * RA; row0 < r1; row0 += n_o * 8u * RA) {
      float4 a[RA][2][2];
      float rm[RA], rl[RA];
#pragma unroll
      for (uint32_t k = 0; k < RA; ++k) {
        const uint32_t row = row0 + k < r1 ? row0 + k : r1 - 1u;
#pragma unroll
        for (uint32_t c = 0; c < 2; ++c) {
          a[k][c][0] = a[k][c][1] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (c * 256u < D) {
            const float4* s4 = reinterpret_cast<const float4*>(src_o + size_t(row) * D + c * 256u + lane * 8u);
            a[k][c][0] = s4[0];
            a[k][c][1] = s4[1];
          }
        }
        rm[k] = src_m[row];
        rl[k] = src_l[row];
      }
#pragma unroll
      for (uint32_t k = 0; k < RA; ++k) {
        const uint32_t row = row0 + k;
        if (row >= r1) break;   // warp-uniform
        float amax = 0.f;
#pragma unroll
        for (uint32_t c = 0; c < 2; ++c)
#pragma unroll
          for (uint32_t h = 0; h < 2; ++h)
            amax = fmaxf(fmaxf(amax, fmaxf(fabsf(a[k][c][h].x), fabsf(a[k][c][h].y))), fmaxf(fabsf(a[k][c][h].z), fabsf(a[k][c][h].w)));
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sft));
        // biased exponent of the row maximum; tiny, zero, infinite or NaN maxima travel unscaled
        const uint32_t eb = (__float_as_uint(amax) >> 23) & 0xffu;
        const bool scaled = eb >= 15u && eb < 255u;
        const float sc = scaled ? __uint_as_float((268u - eb) << 23) : 1.0f;       // 2^(14 - exponent)
        const float inv_sc = scaled ? __uint_as_float((eb - 14u) << 23) : 1.0f;
#pragma unroll
        for (uint32_t c = 0; c < 2; ++c) {
          if (c * 256u >= D) break;
          __half2 h0 = __floats2half2_rn(a[k][c][0].x * sc, a[k][c][0].y * sc), h1 = __floats2half2_rn(a[k][c][0].z * sc, a[k][c][0].w * sc);
          __half2 h2 = __floats2half2_rn(a[k][c][1].x * sc, a[k][c][1].y * sc), h3 = __floats2half2_rn(a[k][c][1].z * sc, a[k][c][1].w * sc);
          uint4 pk;
          pk.x = *reinterpret_cast<uint32_t*>(&h0);
          pk.y = *reinterpret_cast<uint32_t*>(&h1);
          pk.z = *reinterpret_cast<uint32_t*>(&h2);
          pk.w = *reinterpret_cast<uint32_t*>(&h3);
          *reinterpret_cast<uint4*>(dst_rows + size_t(row - r0) * D + c * 256u + lane * 8u) = pk;
        }
        if (lane == 0) dst_ml[row - r0] = make_float4(rm[k], rl[k], inv_sc, 0.f);
        ++done;
      }
    }
    if (lane == 0 && done) atomicAdd(s_rows, done);
    __syncthreads();
    p2p_stamp(q, 2);
    if (tid == 0 && *s_rows) {
      // A release at system scope by one thread, after the CTA barrier, publishes the stores of every thread
      // of the CTA (release is cumulative over what the barrier ordered before it).  No sequentially
      // consistent fence: those are totally ordered among all CTAs and cost 10 us here with 148 of them.
      red_release_sys_add(reinterpret_cast<uint32_t*>(q.peer[o] + q.off_cnt) + slot, *s_rows);
    }
  }

}

// Phase B: wait (bounded, on this rank's own memory) until every rank's rows of this rank's slice have landed in
// receive slot q.merge_slot, merge them and write the finished bf16 rows of the slice to `out`.
__device__ __forceinline__ void p2p_phase_merge(const P2pParams& q, __nv_bfloat16* __restrict__ out, uint32_t* s_ok) {
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t slot = q.merge_slot, W = q.world, D = q.D;
  uint8_t* mine = q.peer[q.rank];
  // ---- phase B: wait until every rank's rows of this rank's slice have landed here
  const uint32_t r0 = uint32_t((uint64_t(q.rank) * q.rows) / W), r1 = uint32_t((uint64_t(q.rank + 1) * q.rows) / W);
  if (tid == 0) {
    const uint32_t want = q.merge_uses * (r1 - r0) * W;
    if (!wait_flag(reinterpret_cast<const uint32_t*>(mine + q.off_cnt) + slot, want, q.wait_limit)) {
      *s_ok = 0u;
      dev_status_set(q.status, DG_DEV_WAIT_TIMEOUT, KID_MERGE, blockIdx.x, 200u);
    }
  }
  __syncthreads();
  p2p_stamp(q, 4);
  if (!*s_ok) return;   // some rank's rows never arrived: the status word says so, the output is left alone
  const __half* rows_in = reinterpret_cast<const __half*>(mine + q.off_recv[slot]);
  const float4* ml_in = reinterpret_cast<const float4*>(mine + q.off_rml[slot]);
  // D = 256: two rows per warp and iteration with every load in flight before the first use (the pass is bound
  // by load latency); wider rows go one at a time
  const uint32_t RB = (D <= 256u) ? 2u : 1u;
  for (uint32_t row0 = r0 + (blockIdx.x * 8u + warp) * RB; row0 < r1; row0 += gridDim.x * 8u * RB) {
    float4 rec[2];
    uint4 x[2][8];
#pragma unroll
    for (uint32_t k = 0; k < 2; ++k) {
      const uint32_t row = (k < RB && row0 + k < r1) ? row0 + k : row0;
      const uint32_t rl = row - r0;
      rec[k] = make_float4(-INFINITY, 0.f, 1.f, 0.f);
      if (lane < W) rec[k] = ml_in[size_t(lane) * q.slice_cap + rl];
#pragma unroll
      for (uint32_t w = 0; w < 8; ++w) {
        x[k][w] = make_uint4(0u, 0u, 0u, 0u);
        if (w < W) x[k][w] = *reinterpret_cast<const uint4*>(rows_in + (size_t(w) * q.slice_cap + rl) * D + lane * 8u);
      }
    }
#pragma unroll
    for (uint32_t k = 0; k < 2; ++k) {
      const uint32_t row = row0 + k;
      if (k >= RB || row >= r1) break;   // warp-uniform
      const uint32_t rl = row - r0;
      float mg = rec[k].x;
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, sft));
      const float w_mine = (rec[k].x == -INFINITY) ? 0.f : expf(rec[k].x - mg);
      float lg = w_mine * rec[k].y;
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) lg += __shfl_xor_sync(0xffffffffu, lg, sft);
      const float inv = lg > 0.f ? 1.0f / lg : 0.f;
      const float ws_mine = w_mine * rec[k].z;   // the row's scale folded into its weight
      for (uint32_t c0 = lane * 8u; c0 < D; c0 += 256u) {
        if (c0 >= 256u) {
#pragma unroll
          for (uint32_t w = 0; w < 8; ++w)
            if (w < W) x[k][w] = *reinterpret_cast<const uint4*>(rows_in + (size_t(w) * q.slice_cap + rl) * D + c0);
        }
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
        for (uint32_t w = 0; w < 8; ++w) {
          float wt = __shfl_sync(0xffffffffu, ws_mine, int(w));
          if (w >= W) wt = 0.f;
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&x[k][w].x));
          const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&x[k][w].y));
          const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&x[k][w].z));
          const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&x[k][w].w));
          acc[0] += wt * f0.x; acc[1] += wt * f0.y; acc[2] += wt * f1.x; acc[3] += wt * f1.y;
          acc[4] += wt * f2.x; acc[5] += wt * f2.y; acc[6] += wt * f3.x; acc[7] += wt * f3.y;
        }
        __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv), h1 = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[4] * inv, acc[5] * inv), h3 = __floats2bfloat162_rn(acc[6] * inv, acc[7] * inv);
        uint4 o4;
        o4.x = *reinterpret_cast<uint32_t*>(&h0);
        o4.y = *reinterpret_cast<uint32_t*>(&h1);
        o4.z = *reinterpret_cast<uint32_t*>(&h2);
        o4.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(out + size_t(row) * D + c0) = o4;
      }
    }
  }
}

__global__ void __launch_bounds__(256) dg_p2p_push_merge_kernel(const P2pParams q, __nv_bfloat16* __restrict__ out) {
  __shared__ uint32_t s_ok, s_rows;
  if (threadIdx.x == 0) {
    s_ok = 1u;
    s_rows = 0u;
  }
  // the partial was written by the attention kernel that precedes this one on the stream
  p2p_stamp(q, 0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();
  p2p_stamp(q, 1);
  if (q.merge_on && q.merge_first) {
    // pipelined form: the slice of the PREVIOUS step first (its rows arrived a step ago), then this step's rows.
    // A CTA signals this step's rows only after it has finished reading the previous step's slot, so a peer that
    // has seen this rank's rows of step i+1 knows that this rank is done with the slot of step i.
    p2p_phase_merge(q, out, &s_ok);
    __syncthreads();
  }
  if (q.send_on) p2p_phase_send(q, &s_rows);
  p2p_stamp(q, 3);
  if (q.merge_on && !q.merge_first) p2p_phase_merge(q, out, &s_ok);
  p2p_stamp(q, 5);
}

cudaError_t launch_p2p_push_merge(const P2pParams& q, void* out, int num_sms, cudaStream_t st) {
  // every CTA must be resident while it waits (at most one per SM), and every owner needs a CTA
  uint32_t grid = (q.rows + 7u) / 8u;
  if (grid > uint32_t(num_sms)) grid = uint32_t(num_sms);
  if (grid < q.world) grid = q.world;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  // start while the attention kernel drains; the kernel waits (griddepcontrol.wait) before it reads
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, dg_p2p_push_merge_kernel, q, static_cast<__nv_bfloat16*>(out));
}

// ------------------------------------------------------------------------------------------
// Query all-gather of the host pipeline: split-KV replicates Q on every rank, but N copies of it from host memory
// share the host's PCIe links.  Every rank copies in only its own row slice; this kernel stores that slice into the
// same slot of every peer's query staging (posted stores over NVLink), publishes the row count with a system-scope
// release per peer, and waits (bounded, on this rank's own memory) until the other ranks' slices have landed here.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) dg_p2p_qgather_kernel(const P2pParams q, uint32_t slot, uint32_t uses) {
  const uint32_t tid = threadIdx.x, W = q.world;
  const uint32_t r0 = uint32_t((uint64_t(q.rank) * q.rows) / W), r1 = uint32_t((uint64_t(q.rank + 1) * q.rows) / W);
  const size_t row_units = size_t(q.D) * 2 / 16;                       // 16-byte units per row
  const uint4* src = reinterpret_cast<const uint4*>(q.peer[q.rank] + q.off_qstage[slot]) + size_t(r0) * row_units;
  // this CTA's share of the slice, whole rows
  const uint32_t n_rows = r1 - r0;
  const uint32_t per = (n_rows + gridDim.x - 1) / gridDim.x;
  const uint32_t a = blockIdx.x * per < n_rows ? blockIdx.x * per : n_rows;
  const uint32_t b = a + per < n_rows ? a + per : n_rows;
  for (uint32_t w = 1; w < W; ++w) {
    const uint32_t peer = (q.rank + w) % W;
    uint4* dst = reinterpret_cast<uint4*>(q.peer[peer] + q.off_qstage[slot]) + size_t(r0) * row_units;
    for (size_t i = size_t(a) * row_units + tid; i < size_t(b) * row_units; i += 256) dst[i] = src[i];
  }
  __syncthreads();
  if (tid < W && tid != q.rank && b > a)
    red_release_sys_add(reinterpret_cast<uint32_t*>(q.peer[tid] + q.off_qcnt) + slot, b - a);
  if (blockIdx.x == 0 && tid == 0) {
    const uint32_t want = uses * (q.rows - n_rows);
    if (!wait_flag(reinterpret_cast<const uint32_t*>(q.peer[q.rank] + q.off_qcnt) + slot, want, q.wait_limit))
      dev_status_set(q.status, DG_DEV_WAIT_TIMEOUT, KID_MERGE, blockIdx.x, 300u + slot);
  }
}

cudaError_t launch_p2p_qgather(const P2pParams& q, uint32_t slot, uint32_t uses, cudaStream_t st) {
  dg_p2p_qgather_kernel<<<16, 256, 0, st>>>(q, slot, uses);
  return cudaGetLastError();
}

void launch_p2p_merge(const P2pParams& q, void* out, int num_sms, cudaStream_t st) {
  const uint32_t slice = q.all_rows ? q.rows : (q.rows + q.world - 1) / q.world;
  uint32_t grid = (slice + 7) / 8;
  if (grid > uint32_t(num_sms)) grid = uint32_t(num_sms);
  if (grid == 0) grid = 1;
  dg_p2p_merge_kernel<<<grid, 256, 0, st>>>(q, static_cast<uint4*>(out));
}

}  // namespace dg
