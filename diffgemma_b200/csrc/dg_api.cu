// Host side of the C ABI declared in include/dg_attn.h: context, KV cache objects, argument
// validation, kernel selection and launch, split planning, NCCL merge.  The host mirrors what the
// reference's step encoder does for its two attention stages (paths relative to the reference
// project): encode_layer_qk_rope_kv_dispatch src/metal/step_kernel/enc.rs:1733-1806 and
// encode_layer_attention_dispatch src/metal/step_kernel/enc.rs:2102-2296 (kernel choice by layer
// geometry, buffer binding, grids).  There is no CPU fallback: without a usable GPU every call
// returns an error.
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <deque>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "dg_common.cuh"
#include "dg_kernels.h"

using namespace dg;

// ------------------------------------------------------------------------------------------
// error plumbing
// ------------------------------------------------------------------------------------------
static thread_local std::string g_last_error;

static int32_t fail_cuda(cudaError_t e, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return DG_ERR_CUDA;
}
#define DG_CUDA(call)                                \
  do {                                               \
    cudaError_t e__ = (call);                        \
    if (e__ != cudaSuccess) return fail_cuda(e__, #call); \
  } while (0)

static int32_t fail(int32_t code, const char* msg) {
  g_last_error = msg;
  return code;
}

// ------------------------------------------------------------------------------------------
// objects
// ------------------------------------------------------------------------------------------
struct dg_ctx {
  int device = 0;
  int num_sms = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  DevStatus* d_status = nullptr;
  uint32_t concurrent = 1;             // canvases in flight together: the split heuristic counts their CTAs
  uint32_t* counters = nullptr;        // [kCounterSlots], zero between launches
  float* ws_o = nullptr;               // split partials
  float* ws_ml = nullptr;
  size_t ws_splits = 0, ws_rows = 0;   // capacity of ws_o / ws_ml: splits x rows (x 256 / x 2)
  __nv_bfloat16* stage_q = nullptr;    // device staging for host-buffer calls / pre-normed Q
  __nv_bfloat16* stage_k = nullptr;
  __nv_bfloat16* stage_v = nullptr;
  __nv_bfloat16* stage_o = nullptr;
  size_t stage_q_elems = 0, stage_kv_elems = 0;
  float* nccl_pay = nullptr;           // [rows][D+1] payload of the cross-rank merge
  float* nccl_mg = nullptr;            // [rows]
  size_t nccl_rows = 0, nccl_d = 0;
  // dg_attn_block: activations between its kernels (normed input, Q, K, V, O, projected O, row sums of squares)
  __nv_bfloat16* blk_xn = nullptr;
  __nv_bfloat16* blk_q = nullptr;
  __nv_bfloat16* blk_k = nullptr;
  __nv_bfloat16* blk_v = nullptr;
  __nv_bfloat16* blk_o = nullptr;
  float* blk_part = nullptr;           // fp32 partial planes of the output projection, [4][rows][hidden]
  uint16_t* topk_scores = nullptr;     // dg_attn_denoise_topk: bf16 score plane [Hkv][canvas * G][ld]
  size_t topk_elems = 0;
  size_t blk_rows = 0, blk_hidden = 0, blk_qe = 0, blk_ke = 0;
  CUtensorMap blk_tm_xn, blk_tm_o;
  struct WMap {
    const void* w;
    uint32_t n, k, bn;
    CUtensorMap tm;
  };
  std::deque<WMap> blk_wmaps;          // tensor maps of the weight matrices seen so far (a deque: growing it leaves
                                       // the addresses of its elements, which a call holds across two look-ups, alone)
  int q_from_prev_kernel = 0;          // 1 while dg_attn_block runs: Q is written by the kernel queued just ahead
  int force_general = 0;
  int fused_append = 1;                // 1: the canvas append runs inside the attention launch where it can
  int inputs_stable = 0;               // 1: the caller's q/k/v are not written by work queued ahead of a call
  int pair_mode = 2;                   // tensor path: 0 single-CTA kernel, 1 CTA-pair (cta_group::2) kernel, 2 automatic
  uint32_t forced_splits = 0;
  uint32_t last_launches = 0;
  // optional per-launch timing of the attention kernel (event pairs on the launching stream)
  unsigned long long* stamps = nullptr;   // caller-owned device buffer for per-CTA phase stamps
  bool timing = false;
  std::vector<cudaEvent_t> ev;
  size_t ev_used = 0;
};

// What a cache's RoPE table currently holds.  Denoise steps repeat at the same positions, so the
// table is rewritten only when this key changes.
struct RopeKey {
  bool valid = false;
  uint32_t kv_len = 0, canvas = 0, rotary_dim = 0, pairing = 0, head_dim = 0;
  float theta = 0.f;
};

struct dg_kv {
  dg_ctx* ctx = nullptr;
  // (cos, sin) of the canvas positions [kv_len, kv_len + canvas) of the fused path, two regions of
  // [kMaxCanvas][head_dim / 2] entries.  The table belongs to the CACHE, so that a step replayed from a CUDA
  // graph reads the table of its own cache and positions whatever other caches were used since.
  // Region 0 is maintained by eager calls and described by rope_key.  Launches recorded under stream
  // capture may read region 0 (when it already holds their positions) but never write it: a replay is
  // invisible to the host, so a table a graph writes lives in region 1, which only that graph reads.
  float2* rope_table = nullptr;
  RopeKey rope_key;
  uint32_t* ap_ctl = nullptr;   // {ticket, vectors done, CTAs finished} of the in-launch canvas append; zero between launches
  __nv_bfloat16* k = nullptr;   // [Hkv][cap][D]
  __nv_bfloat16* v = nullptr;
  uint64_t cap = 0;
  uint32_t ring_mask = 0;       // 0: linear cache; else slots - 1 of a ring (slot = pos & ring_mask)
  uint32_t pos_base = 0;        // shard caches: the first position held, multiple of 128
  bool shard = false;           // holds [pos_base, pos_base + cap) of a longer prefix (dg_kv_create_shard)
  uint32_t Hkv = 0, D = 0;
  bool has_tmap = false;
  CUtensorMap tm_k, tm_v;
  CUtensorMap tm_k64;   // K with half-tile boxes (64 keys at head_dim 256, 32 at 512): each CTA of a cta_group::2 pair stages half of a key tile
};

constexpr uint32_t kMaxQueryTiles = 4096;
constexpr uint32_t kCounterSlots = kMaxQueryTiles * 32 + 1;   // (query tile, four-row slice) arrival counters + the self-test flag

// ------------------------------------------------------------------------------------------
// driver entry point for tensor-map encoding (no link-time dependency on libcuda)
// ------------------------------------------------------------------------------------------
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PFN_encodeTiled get_encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<PFN_encodeTiled>(p);
  return fn;
}

static int32_t make_kv_tmap(CUtensorMap* tm, void* base, uint64_t cap, uint32_t Hkv, uint32_t box_keys = 128,
                            uint32_t D = 256) {
  PFN_encodeTiled enc = get_encode_fn();
  if (!enc) return fail(DG_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  const cuuint64_t dims[3] = {D, cap, Hkv};
  const cuuint64_t strides[2] = {cuuint64_t(D) * 2, cap * D * 2};   // bytes, dims 1 and 2
  const cuuint32_t box[3] = {64, box_keys, 1};               // 128 B x box_keys keys
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_error = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r));
    return DG_ERR_CUDA;
  }
  return DG_OK;
}

// ------------------------------------------------------------------------------------------
// validation helpers
// ------------------------------------------------------------------------------------------
static int32_t check_desc(const dg_layer_desc* d) {
  if (!d) return fail(DG_ERR_INVALID_ARG, "desc is NULL");
  if (d->n_q_heads == 0 || d->n_kv_heads == 0 || d->n_q_heads % d->n_kv_heads != 0)
    return fail(DG_ERR_INVALID_ARG, "n_q_heads must be a positive multiple of n_kv_heads");
  if (d->head_dim == 0 || d->head_dim % 8 != 0 || d->head_dim > kMaxHeadDim)
    return fail(DG_ERR_UNSUPPORTED, "head_dim must be a multiple of 8, at most 512");
  if (d->canvas == 0 || d->canvas > kMaxCanvas) return fail(DG_ERR_UNSUPPORTED, "canvas must be in 1..256");
  if (d->rotary_dim > d->head_dim || d->rotary_dim % 2 != 0)
    return fail(DG_ERR_INVALID_ARG, "rotary_dim must be even and <= head_dim");
  if (d->mask_mode > DG_MASK_CAUSAL) return fail(DG_ERR_INVALID_ARG, "unknown mask_mode");
  if (d->rope_pairing > DG_ROPE_PROPORTIONAL) return fail(DG_ERR_INVALID_ARG, "unknown rope_pairing");
  if (d->rope_pairing == DG_ROPE_SPLIT_HALF && d->rotary_dim / 2 + d->rotary_dim / 2 > d->head_dim)
    return fail(DG_ERR_INVALID_ARG, "rotary_dim too large");
  if (d->rope_pairing == DG_ROPE_PROPORTIONAL && d->rotary_dim / 2 > d->head_dim / 2)
    return fail(DG_ERR_INVALID_ARG, "rotary_dim too large for proportional pairing");
  if (!(d->softmax_scale > 0.f) || !std::isfinite(d->softmax_scale))
    return fail(DG_ERR_INVALID_ARG, "softmax_scale must be positive and finite");
  if (!(d->rope_theta > 0.f)) return fail(DG_ERR_INVALID_ARG, "rope_theta must be positive");
  return DG_OK;
}
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static RopeParams make_rope(const dg_layer_desc& d) {
  RopeParams rp;
  rp.rot_half = d.rotary_dim / 2;
  rp.pair_off = d.rope_pairing == DG_ROPE_SPLIT_HALF ? d.rotary_dim / 2 : d.head_dim / 2;
  // theta^(-2i/head_dim) evaluated in f32 on the host (src/shaders/attn/cpu.rs:35); the device only
  // multiplies by the position and takes cosf/sinf of the f32 angle.
  for (uint32_t i = 0; i < kMaxRotHalf; ++i)
    rp.inv_freq[i] = i < rp.rot_half ? std::pow(d.rope_theta, -2.0f * float(i) / float(d.head_dim)) : 0.f;
  return rp;
}

// tensor-core kernels exist for head_dim 256 (all benchmark layers) and 512 (the reference's full layers)
static bool tensor_path_ok(const dg_layer_desc& d) {
  return (d.head_dim == 256 || d.head_dim == 512) && d.canvas <= kMaxCanvas;
}
// the in-kernel Q prologue covers full split-half rotary only
static bool fused_q_prologue_ok(const dg_layer_desc& d) {
  return d.head_dim == 256 && d.rotary_dim == 256 && d.rope_pairing == DG_ROPE_SPLIT_HALF;
}

static uint32_t choose_splits(const dg_ctx* ctx, uint32_t q_tiles, uint32_t k_tiles) {
  uint32_t smax = k_tiles < kSm100MaxSplits ? k_tiles : kSm100MaxSplits;
  if (smax < 1) smax = 1;
  if (ctx->forced_splits) return ctx->forced_splits < smax ? ctx->forced_splits : smax;
  const uint32_t sms = ctx->num_sms > 0 ? uint32_t(ctx->num_sms) : 148u;
  uint32_t best = 1;
  uint64_t best_cost = ~0ull;
  // automatic choice: powers of two up to 8, the split counts that merge inside a cluster
  for (uint32_t s = 1; s <= smax && s <= 8u; s *= 2) {
    const uint64_t waves = (uint64_t(q_tiles) * s + sms - 1) / sms;
    // in tenths of a key tile's time (about 1.75 us): the fixed cost of a step (launches, set-up, Q
    // prologue, epilogue: about 12 us) and the measured cost of exchanging and merging the partial rows
    // of s splits (about 6.3 us for two, 7.7 us for four), so that a short key range is not split at all
    const uint64_t merge = s == 1 ? 0 : s == 2 ? 36 : s == 4 ? 44 : 55;
    const uint64_t per = 10 * ((k_tiles + s - 1) / s) + 70 + merge;
    const uint64_t cost = waves * per;
    if (cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

static int32_t ensure_split_ws(dg_ctx* ctx, uint32_t splits, uint32_t rows) {
  if (splits <= ctx->ws_splits && rows <= ctx->ws_rows) return DG_OK;
  const size_t s = splits > ctx->ws_splits ? splits : ctx->ws_splits;
  const size_t r = rows > ctx->ws_rows ? rows : ctx->ws_rows;
  DG_CUDA(cudaStreamSynchronize(ctx->stream));
  if (ctx->ws_o) cudaFree(ctx->ws_o);
  if (ctx->ws_ml) cudaFree(ctx->ws_ml);
  ctx->ws_o = ctx->ws_ml = nullptr;
  ctx->ws_splits = ctx->ws_rows = 0;
  DG_CUDA(cudaMalloc(&ctx->ws_o, s * r * 256 * sizeof(float)));
  DG_CUDA(cudaMalloc(&ctx->ws_ml, s * r * 2 * sizeof(float)));
  ctx->ws_splits = s;
  ctx->ws_rows = r;
  return DG_OK;
}

static int32_t ensure_stage(dg_ctx* ctx, size_t q_elems, size_t kv_elems) {
  if (q_elems > ctx->stage_q_elems) {
    DG_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->stage_q) cudaFree(ctx->stage_q);
    if (ctx->stage_o) cudaFree(ctx->stage_o);
    ctx->stage_q = ctx->stage_o = nullptr;
    ctx->stage_q_elems = 0;
    DG_CUDA(cudaMalloc(&ctx->stage_q, q_elems * 2));
    DG_CUDA(cudaMalloc(&ctx->stage_o, q_elems * 2));
    ctx->stage_q_elems = q_elems;
  }
  if (kv_elems > ctx->stage_kv_elems) {
    DG_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->stage_k) cudaFree(ctx->stage_k);
    if (ctx->stage_v) cudaFree(ctx->stage_v);
    ctx->stage_k = ctx->stage_v = nullptr;
    ctx->stage_kv_elems = 0;
    DG_CUDA(cudaMalloc(&ctx->stage_k, kv_elems * 2));
    DG_CUDA(cudaMalloc(&ctx->stage_v, kv_elems * 2));
    ctx->stage_kv_elems = kv_elems;
  }
  return DG_OK;
}

// ------------------------------------------------------------------------------------------
// context
// ------------------------------------------------------------------------------------------
extern "C" const char* dg_last_error_message(void) { return g_last_error.c_str(); }

extern "C" const char* dg_status_str(int32_t s) {
  switch (s) {
    case DG_OK: return "ok";
    case DG_ERR_INVALID_ARG: return "invalid argument";
    case DG_ERR_UNSUPPORTED: return "unsupported geometry";
    case DG_ERR_CAPACITY: return "kv_len + canvas exceeds the cache capacity";
    case DG_ERR_CUDA: return "CUDA error";
    case DG_ERR_NO_DEVICE: return "no sm_100 device";
    case DG_ERR_NCCL: return "NCCL error";
    case DG_ERR_ALIGNMENT: return "pointer not 16-byte aligned";
    case DG_DEV_WAIT_TIMEOUT: return "device-side wait timed out";
    case DG_DEV_SMEM_LAYOUT: return "shared-memory map did not fit the block's window";
    case DG_DEV_BAD_SHAPE: return "device-side shape check failed";
    default: return "unknown status";
  }
}

extern "C" int32_t dg_ctx_create(int32_t device, dg_ctx** out) {
  if (!out) return fail(DG_ERR_INVALID_ARG, "out is NULL");
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    cudaGetLastError();
    return fail(DG_ERR_NO_DEVICE, "no CUDA device visible; this library has no CPU path");
  }
  if (device < 0 || device >= n) return fail(DG_ERR_INVALID_ARG, "device index out of range");
  cudaDeviceProp prop;
  DG_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return fail(DG_ERR_NO_DEVICE, "device is not sm_100 (B200); kernels are built for sm_100a only");
  DG_CUDA(cudaSetDevice(device));
  dg_ctx* c = new (std::nothrow) dg_ctx();
  if (!c) return fail(DG_ERR_INVALID_ARG, "out of host memory");
  c->device = device;
  c->num_sms = prop.multiProcessorCount;
  cudaError_t e = cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_status, sizeof(DevStatus));
  if (e == cudaSuccess) e = cudaMemset(c->d_status, 0, sizeof(DevStatus));
  if (e == cudaSuccess) e = cudaMalloc(&c->counters, kCounterSlots * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(c->counters, 0, kCounterSlots * sizeof(uint32_t));
  if (e == cudaSuccess) e = sm100_attn_configure();
  if (e == cudaSuccess) e = sm100_pair_configure();
  if (e == cudaSuccess) e = sm100_hd512_configure();
  if (e == cudaSuccess) e = sm100_hd512x_configure();
  if (e == cudaSuccess) e = sm100_hd512q_configure();
  if (e == cudaSuccess) e = sm100_gemm_configure();
  if (e != cudaSuccess) {
    dg_ctx_destroy(c);
    return fail_cuda(e, "dg_ctx_create");
  }
  c->stream = c->own_stream;
  *out = c;
  return DG_OK;
}

extern "C" int32_t dg_ctx_destroy(dg_ctx* c) {
  if (!c) return DG_OK;
  cudaSetDevice(c->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  cudaFree(c->d_status);
  cudaFree(c->counters);
  cudaFree(c->ws_o);
  cudaFree(c->ws_ml);
  cudaFree(c->stage_q);
  cudaFree(c->stage_k);
  cudaFree(c->stage_v);
  cudaFree(c->stage_o);
  cudaFree(c->nccl_pay);
  cudaFree(c->nccl_mg);
  cudaFree(c->blk_xn);
  cudaFree(c->blk_q);
  cudaFree(c->blk_k);
  cudaFree(c->blk_v);
  cudaFree(c->blk_o);
  cudaFree(c->blk_part);
  cudaFree(c->topk_scores);
  for (cudaEvent_t e : c->ev) cudaEventDestroy(e);
  if (c->own_stream) cudaStreamDestroy(c->own_stream);
  delete c;
  return DG_OK;
}

extern "C" int32_t dg_ctx_set_stream(dg_ctx* c, void* s) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  c->stream = s ? static_cast<cudaStream_t>(s) : c->own_stream;
  return DG_OK;
}
extern "C" void* dg_ctx_stream(dg_ctx* c) { return c ? static_cast<void*>(c->stream) : nullptr; }

static int32_t read_status(dg_ctx* c, DevStatus* h) {
  DG_CUDA(cudaMemcpyAsync(h, c->d_status, sizeof(DevStatus), cudaMemcpyDeviceToHost, c->stream));
  DG_CUDA(cudaStreamSynchronize(c->stream));
  return DG_OK;
}

extern "C" int32_t dg_ctx_synchronize(dg_ctx* c) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  DG_CUDA(cudaSetDevice(c->device));
  DevStatus h;
  const int32_t r = read_status(c, &h);
  if (r != DG_OK) return r;
  return int32_t(h.code);
}

extern "C" int32_t dg_ctx_last_device_status(dg_ctx* c, uint32_t out[4]) {
  if (!c || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  DG_CUDA(cudaSetDevice(c->device));
  DevStatus h;
  const int32_t r = read_status(c, &h);
  if (r != DG_OK) return r;
  out[0] = h.code; out[1] = h.kernel_id; out[2] = h.cta; out[3] = h.value;
  return DG_OK;
}

extern "C" int32_t dg_ctx_clear_device_status(dg_ctx* c) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  DG_CUDA(cudaSetDevice(c->device));
  DG_CUDA(cudaMemsetAsync(c->d_status, 0, sizeof(DevStatus), c->stream));
  return DG_OK;
}

extern "C" int32_t dg_ctx_selftest_wait_timeout(dg_ctx* c, uint64_t limit_cycles) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  if (limit_cycles == 0 || limit_cycles > 2000000000ull) return fail(DG_ERR_INVALID_ARG, "limit must be in 1..2e9 cycles");
  DG_CUDA(cudaSetDevice(c->device));
  // the flag is one of the (always zero between launches) query-tile counters: nothing sets it
  launch_selftest_wait(c->counters + (kCounterSlots - 1), (long long)limit_cycles, c->d_status, c->stream);
  DG_CUDA(cudaGetLastError());
  return DG_OK;
}

extern "C" int32_t dg_uses_tensor_path(const dg_layer_desc* d) {
  if (check_desc(d) != DG_OK) return 0;
  return tensor_path_ok(*d) ? 1 : 0;
}
extern "C" int32_t dg_ctx_force_general(dg_ctx* c, int32_t on) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  c->force_general = on ? 1 : 0;
  return DG_OK;
}
extern "C" int32_t dg_ctx_max_active_clusters(dg_ctx* c, int32_t pair, uint32_t cluster_y) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  cudaSetDevice(c->device);
  return pair ? sm100_pair_max_active_clusters(cluster_y) : sm100_max_active_clusters(cluster_y);
}
extern "C" int32_t dg_ctx_set_pair_mode(dg_ctx* c, int32_t mode) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  if (mode < 0 || mode > 2) return fail(DG_ERR_INVALID_ARG, "pair mode must be 0 (single), 1 (pair) or 2 (automatic)");
  c->pair_mode = mode;
  return DG_OK;
}
extern "C" int32_t dg_ctx_set_fused_append(dg_ctx* c, int32_t on) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  c->fused_append = on ? 1 : 0;
  return DG_OK;
}
extern "C" int32_t dg_ctx_set_inputs_stable(dg_ctx* c, int32_t on) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  c->inputs_stable = on ? 1 : 0;
  return DG_OK;
}
extern "C" int32_t dg_ctx_set_splits(dg_ctx* c, uint32_t n) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  if (n > kSm100MaxSplits) return fail(DG_ERR_INVALID_ARG, "at most 32 splits");
  c->forced_splits = n;
  return DG_OK;
}
extern "C" uint32_t dg_ctx_last_launch_count(const dg_ctx* c) { return c ? c->last_launches : 0; }

extern "C" int32_t dg_ctx_phase_stamps(dg_ctx* c, void* device_buffer) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  c->stamps = static_cast<unsigned long long*>(device_buffer);
  return DG_OK;
}

extern "C" int32_t dg_ctx_kernel_timing(dg_ctx* c, int32_t on, uint32_t max_launches) {
  if (!c) return fail(DG_ERR_INVALID_ARG, "ctx is NULL");
  DG_CUDA(cudaSetDevice(c->device));
  c->timing = on != 0;
  c->ev_used = 0;
  while (on && c->ev.size() < size_t(max_launches) * 2) {
    cudaEvent_t e;
    DG_CUDA(cudaEventCreate(&e));
    c->ev.push_back(e);
  }
  return DG_OK;
}

extern "C" int32_t dg_ctx_kernel_time(dg_ctx* c, double* total_ms, uint32_t* launches) {
  if (!c || !total_ms || !launches) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  DG_CUDA(cudaSetDevice(c->device));
  DG_CUDA(cudaStreamSynchronize(c->stream));
  double sum = 0.0;
  for (size_t i = 0; i + 1 < c->ev_used; i += 2) {
    float ms = 0.f;
    DG_CUDA(cudaEventElapsedTime(&ms, c->ev[i], c->ev[i + 1]));
    sum += ms;
  }
  *total_ms = sum;
  *launches = uint32_t(c->ev_used / 2);
  return DG_OK;
}

// ------------------------------------------------------------------------------------------
// KV cache
// ------------------------------------------------------------------------------------------
static int32_t kv_create(dg_ctx* c, const dg_layer_desc* d, uint64_t capacity_tokens, uint32_t ring_mask, dg_kv** out,
                         uint32_t pos_base = 0, bool shard = false) {
  if (!c || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  *out = nullptr;
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  if (capacity_tokens == 0 || capacity_tokens > (1ull << 31)) return fail(DG_ERR_INVALID_ARG, "bad capacity");
  DG_CUDA(cudaSetDevice(c->device));
  dg_kv* kv = new (std::nothrow) dg_kv();
  if (!kv) return fail(DG_ERR_INVALID_ARG, "out of host memory");
  kv->ctx = c;
  kv->cap = (capacity_tokens + 127) / 128 * 128;
  kv->ring_mask = ring_mask;
  kv->pos_base = pos_base;
  kv->shard = shard;
  kv->Hkv = d->n_kv_heads;
  kv->D = d->head_dim;
  const size_t bytes = size_t(kv->Hkv) * kv->cap * kv->D * 2;
  cudaError_t e = cudaMalloc(&kv->k, bytes);
  if (e == cudaSuccess) e = cudaMalloc(&kv->v, bytes);
  // rows in [T, cap) are read by whole-tile loads and masked afterwards: they must be finite
  if (e == cudaSuccess) e = cudaMemsetAsync(kv->k, 0, bytes, c->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(kv->v, 0, bytes, c->stream);
  if (e == cudaSuccess) e = cudaMalloc(&kv->rope_table, 2 * size_t(kMaxCanvas) * (kv->D / 2) * sizeof(float2));
  if (e == cudaSuccess) e = cudaMalloc(&kv->ap_ctl, 4 * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemsetAsync(kv->ap_ctl, 0, 4 * sizeof(uint32_t), c->stream);
  if (e != cudaSuccess) {
    dg_kv_destroy(kv);
    return fail_cuda(e, "dg_kv_create");
  }
  if (kv->D == 256) {
    r = make_kv_tmap(&kv->tm_k, kv->k, kv->cap, kv->Hkv);
    if (r == DG_OK) r = make_kv_tmap(&kv->tm_v, kv->v, kv->cap, kv->Hkv);
    if (r == DG_OK) r = make_kv_tmap(&kv->tm_k64, kv->k, kv->cap, kv->Hkv, 64);
    if (r != DG_OK) {
      dg_kv_destroy(kv);
      return r;
    }
    kv->has_tmap = true;
  } else if (kv->D == 512) {
    // head_dim-512 kernel: key tiles of 64 keys for both K and V
    r = make_kv_tmap(&kv->tm_k, kv->k, kv->cap, kv->Hkv, 64, 512);
    if (r == DG_OK) r = make_kv_tmap(&kv->tm_v, kv->v, kv->cap, kv->Hkv, 64, 512);
    if (r == DG_OK) r = make_kv_tmap(&kv->tm_k64, kv->k, kv->cap, kv->Hkv, 32, 512);   // half of a key tile per CTA of a pair
    if (r != DG_OK) {
      dg_kv_destroy(kv);
      return r;
    }
    kv->has_tmap = true;
  }
  *out = kv;
  return DG_OK;
}
extern "C" int32_t dg_kv_create(dg_ctx* c, const dg_layer_desc* d, uint64_t capacity_tokens, dg_kv** out) {
  return kv_create(c, d, capacity_tokens, 0u, out);
}
extern "C" int32_t dg_kv_create_ring(dg_ctx* c, const dg_layer_desc* d, uint32_t ring_slots, dg_kv** out) {
  if (ring_slots < 256 || (ring_slots & (ring_slots - 1)) != 0)
    return fail(DG_ERR_INVALID_ARG, "ring_slots must be a power of two, at least 256");
  return kv_create(c, d, ring_slots, ring_slots - 1u, out);
}
extern "C" int32_t dg_kv_create_shard(dg_ctx* c, const dg_layer_desc* d, uint64_t pos_base, uint64_t capacity_tokens,
                                      dg_kv** out) {
  if (pos_base % 128 != 0 || pos_base >= (1ull << 31))
    return fail(DG_ERR_INVALID_ARG, "pos_base must be a multiple of 128 below 2^31");
  return kv_create(c, d, capacity_tokens, 0u, out, uint32_t(pos_base), true);
}
extern "C" uint32_t dg_kv_ring_mask(const dg_kv* kv) { return kv ? kv->ring_mask : 0u; }
extern "C" uint64_t dg_kv_pos_base(const dg_kv* kv) { return kv ? kv->pos_base : 0u; }

extern "C" int32_t dg_kv_destroy(dg_kv* kv) {
  if (!kv) return DG_OK;
  if (kv->ctx) {
    cudaSetDevice(kv->ctx->device);
    cudaStreamSynchronize(kv->ctx->stream);
  }
  cudaFree(kv->k);
  cudaFree(kv->v);
  cudaFree(kv->rope_table);
  cudaFree(kv->ap_ctl);
  delete kv;
  return DG_OK;
}
extern "C" uint64_t dg_kv_capacity(const dg_kv* kv) { return kv ? kv->cap : 0; }

// A run of positions [pos0, pos0 + n) as at most two runs of contiguous cache slots.  In a ring only the
// last `cap` positions of the run still have a slot (older ones were overwritten by them).
struct SlotRuns {
  uint64_t skip = 0;                 // leading positions of the run that no longer have a slot
  uint64_t slot[2] = {0, 0}, len[2] = {0, 0};
};
static SlotRuns slot_runs(const dg_kv* kv, uint64_t pos0, uint64_t n) {
  SlotRuns r;
  if (kv->ring_mask == 0) {
    r.slot[0] = pos0 - kv->pos_base;
    r.len[0] = n;
    return r;
  }
  if (n > kv->cap) {
    r.skip = n - kv->cap;
    pos0 += r.skip;
    n = kv->cap;
  }
  const uint64_t s0 = pos0 & kv->ring_mask;
  r.slot[0] = s0;
  r.len[0] = (s0 + n <= kv->cap) ? n : kv->cap - s0;
  r.slot[1] = 0;
  r.len[1] = n - r.len[0];
  return r;
}

extern "C" int32_t dg_kv_load_prefix(dg_kv* kv, const void* k, const void* v, uint64_t pos0, uint64_t n) {
  if (!kv || !k || !v) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (kv->ring_mask == 0 && (pos0 < kv->pos_base || pos0 + n > kv->pos_base + kv->cap))
    return fail(DG_ERR_CAPACITY, "prefix does not fit the cache");
  if (n == 0) return DG_OK;
  DG_CUDA(cudaSetDevice(kv->ctx->device));
  const size_t row = size_t(kv->D) * 2, spitch = size_t(kv->Hkv) * row;
  const SlotRuns runs = slot_runs(kv, pos0, n);
  uint64_t done = runs.skip;
  for (int s = 0; s < 2; ++s) {
    if (runs.len[s] == 0) continue;
    for (uint32_t h = 0; h < kv->Hkv; ++h) {
      DG_CUDA(cudaMemcpy2DAsync(kv->k + (size_t(h) * kv->cap + runs.slot[s]) * kv->D, row,
                                static_cast<const uint8_t*>(k) + done * spitch + h * row, spitch, row, runs.len[s],
                                cudaMemcpyDefault, kv->ctx->stream));
      DG_CUDA(cudaMemcpy2DAsync(kv->v + (size_t(h) * kv->cap + runs.slot[s]) * kv->D, row,
                                static_cast<const uint8_t*>(v) + done * spitch + h * row, spitch, row, runs.len[s],
                                cudaMemcpyDefault, kv->ctx->stream));
    }
    done += runs.len[s];
  }
  return DG_OK;
}

extern "C" int32_t dg_kv_read(dg_kv* kv, void* k_out, void* v_out, uint64_t pos0, uint64_t n) {
  if (!kv || !k_out || !v_out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (kv->ring_mask == 0 ? (pos0 < kv->pos_base || pos0 + n > kv->pos_base + kv->cap) : (n > kv->cap))
    return fail(DG_ERR_CAPACITY, "range outside the cache");
  DG_CUDA(cudaSetDevice(kv->ctx->device));
  const size_t row = size_t(kv->D) * 2, dpitch = size_t(kv->Hkv) * row;
  const SlotRuns runs = slot_runs(kv, pos0, n);
  uint64_t done = 0;
  for (int s = 0; s < 2; ++s) {
    if (runs.len[s] == 0) continue;
    for (uint32_t h = 0; h < kv->Hkv; ++h) {
      DG_CUDA(cudaMemcpy2DAsync(static_cast<uint8_t*>(k_out) + done * dpitch + h * row, dpitch,
                                kv->k + (size_t(h) * kv->cap + runs.slot[s]) * kv->D, row, row, runs.len[s],
                                cudaMemcpyDefault, kv->ctx->stream));
      DG_CUDA(cudaMemcpy2DAsync(static_cast<uint8_t*>(v_out) + done * dpitch + h * row, dpitch,
                                kv->v + (size_t(h) * kv->cap + runs.slot[s]) * kv->D, row, row, runs.len[s],
                                cudaMemcpyDefault, kv->ctx->stream));
    }
    done += runs.len[s];
  }
  DG_CUDA(cudaStreamSynchronize(kv->ctx->stream));
  return DG_OK;
}

static int32_t check_kv(const dg_layer_desc& d, const dg_kv* kv, uint64_t end_pos) {
  if (!kv) return fail(DG_ERR_INVALID_ARG, "kv is NULL");
  if (kv->Hkv != d.n_kv_heads || kv->D != d.head_dim) return fail(DG_ERR_INVALID_ARG, "kv geometry differs from desc");
  // a shard holds part of the positions only: what a call may touch is checked against
  // its visible key range (check_ring_span), and appends outside the shard are dropped
  if (kv->ring_mask == 0 && !kv->shard && end_pos > kv->cap)
    return fail(DG_ERR_CAPACITY, "kv_len + canvas exceeds the cache capacity");
  if (end_pos > (1ull << 31)) return fail(DG_ERR_CAPACITY, "position beyond 2^31");
  return DG_OK;
}
// A ring holds the last `cap` positions, a shard the positions [pos_base, pos_base + cap): every key an
// attention call can load (whole 128-key tiles from the first visible position of canvas row 0 to the
// end of what it sees) must be in the cache.
static int32_t check_ring_span(const dg_kv* kv, const MaskParams& mk, uint32_t canvas) {
  if (kv->ring_mask == 0 && !kv->shard) return DG_OK;
  const uint32_t lo0 = mask_row_lo(mk, 0);
  const uint32_t lo = lo0 / 128u * 128u;
  if (kv->ring_mask != 0) {
    const uint64_t end = uint64_t(mk.kv_len) + canvas;
    if (end - lo > kv->cap)
      return fail(DG_ERR_CAPACITY, "the visible key range (window + canvas, tile aligned) exceeds the ring");
    return DG_OK;
  }
  const bool sees_prefix = mk.pre_hi > lo0, sees_canvas = mk.can_hi > mk.kv_len;
  if (!sees_prefix && !sees_canvas) return DG_OK;
  const uint64_t first = sees_prefix ? lo : mk.kv_len / 128u * 128u;
  const uint64_t last = sees_canvas ? mk.can_hi : mk.pre_hi;   // one past the last visible key
  if (first < kv->pos_base || (last + 127u) / 128u * 128u > uint64_t(kv->pos_base) + kv->cap)
    return fail(DG_ERR_CAPACITY, "the visible key range (tile aligned) lies outside this shard of the cache");
  return DG_OK;
}

// stream the kernels of the current call go to
static cudaStream_t launch_stream(const dg_ctx* c) { return c->stream; }

// append n tokens (norm + RoPE + cache write); optionally also Q (stage 1) and the RoPE table
static int32_t do_append(dg_ctx* c, const dg_layer_desc& d, dg_kv* kv, uint64_t pos0, uint32_t n, const void* q_in,
                         void* q_out, const void* k_in, void* k_out, const void* v_in, void* v_out, const void* qw,
                         const void* kw, float2* table, uint32_t write_end = 0xffffffffu,
                         const float2* table_in = nullptr) {
  AppendParams ap;
  ap.q_in = static_cast<const __nv_bfloat16*>(q_in);
  ap.q_out = static_cast<__nv_bfloat16*>(q_out);
  ap.k_in = static_cast<const __nv_bfloat16*>(k_in);
  ap.k_out = static_cast<__nv_bfloat16*>(k_out);
  ap.v_in = static_cast<const __nv_bfloat16*>(v_in);
  ap.v_out = static_cast<__nv_bfloat16*>(v_out);
  ap.qw = static_cast<const __nv_bfloat16*>(qw);
  ap.kw = static_cast<const __nv_bfloat16*>(kw);
  ap.cache_k = kv->k;
  ap.cache_v = kv->v;
  ap.rope_table = table;
  ap.rope_table_in = table_in;
  ap.cap = kv->cap;
  ap.pos0 = uint32_t(pos0);
  ap.n = n;
  ap.Hq = d.n_q_heads;
  ap.Hkv = d.n_kv_heads;
  ap.D = d.head_dim;
  ap.v_norm = d.v_norm;
  ap.eps = d.rms_eps;
  ap.ring_mask = kv->ring_mask ? kv->ring_mask : 0xffffffffu;
  ap.write_end = write_end;
  ap.pos_base = kv->pos_base;
  if (kv->shard) {
    // positions outside the shard are not stored (a rank that does not own the canvas keys still
    // runs the step with the replicated canvas K/V)
    const uint64_t end = uint64_t(kv->pos_base) + kv->cap;
    if (end < ap.write_end) ap.write_end = uint32_t(end);
  }
  const RopeParams rp = make_rope(d);
  // scheduled while the kernel ahead of it on the stream drains (it waits for that kernel's completion
  // before it touches memory): 1-3 us per step of launch latency hidden
  launch_append(ap, rp, launch_stream(c), true);
  DG_CUDA(cudaGetLastError());
  c->last_launches += 1;
  return DG_OK;
}

extern "C" int32_t dg_kv_append_guarded(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint64_t pos0, uint32_t n,
                                        const void* k, const void* v, const void* kw, uint32_t write_end);
extern "C" int32_t dg_kv_append(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint64_t pos0, uint32_t n, const void* k,
                                const void* v, const void* kw) {
  return dg_kv_append_guarded(c, d, kv, pos0, n, k, v, kw, 0xffffffffu);
}
extern "C" int32_t dg_kv_append_guarded(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint64_t pos0, uint32_t n,
                                        const void* k, const void* v, const void* kw, uint32_t write_end) {
  if (!c || !k || !v) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  r = check_kv(*d, kv, (pos0 + n < write_end) ? pos0 + n : (write_end > pos0 ? uint64_t(write_end) : pos0));
  if (r != DG_OK) return r;
  if (n > 65535) return fail(DG_ERR_INVALID_ARG, "append at most 65535 tokens per call");
  DG_CUDA(cudaSetDevice(c->device));
  c->last_launches = 0;
  return do_append(c, *d, kv, pos0, n, nullptr, nullptr, k, nullptr, v, nullptr, nullptr, kw, nullptr, write_end);
}

// ------------------------------------------------------------------------------------------
// attention launch (stage 2), shared by every entry point
// ------------------------------------------------------------------------------------------
// A head_dim-256 tensor-kernel launch that has been prepared but not issued: the canvases of a batch are
// collected and go out as one launch.
struct Prepared {
  bool filled = false;
  bool pair = false;
  AttnParams p;
  const CUtensorMap* tm_k = nullptr;
  const CUtensorMap* tm_v = nullptr;
};

struct AttnCall {
  Prepared* defer = nullptr;     // non-null: do not launch the head_dim-256 tensor kernel, describe it here
  const void* q = nullptr;       // [C][Hq][D]
  const void* qw = nullptr;
  const float2* table = nullptr;
  bool q_prenormed = false;
  bool early_q = false;          // the table was not written by the append launched just before
  const uint8_t* attend = nullptr;
  void* out = nullptr;           // bf16, or NULL for partial
  float* out_o = nullptr;
  float* out_m = nullptr;
  float* out_l = nullptr;
  uint32_t kv_len = 0, t0 = 0, t1 = 0xffffffffu;
  int include_canvas = 1;
  // canvas append inside the attention launch (raw canvas K / V, K norm weight); null: already appended
  const void* ap_k = nullptr;
  const void* ap_v = nullptr;
  const void* ap_kw = nullptr;
  uint32_t ap_write_end = 0xffffffffu;
};

// A split workspace that the caller provides instead of the context's grown cudaMalloc buffers
// (dg_attention_static_scratch): partial O, partial (m, l), arrival counters, with their capacities.
struct FixedWs {
  float* o = nullptr;
  float* ml = nullptr;
  uint32_t* counters = nullptr;
  size_t o_floats = 0, ml_floats = 0;
  uint32_t n_counters = 0;
};

static int32_t do_attention(dg_ctx* c, const dg_layer_desc& d, dg_kv* kv, const AttnCall& a,
                            const FixedWs* fixed = nullptr) {
  AttnParams p;
  std::memset(&p, 0, sizeof(p));
  p.q = static_cast<const __nv_bfloat16*>(a.q);
  p.qw = static_cast<const __nv_bfloat16*>(a.qw);
  p.rope_table = a.table;
  p.early_q = a.early_q ? 1u : 0u;
  p.cache_k = kv->k;
  p.cache_v = kv->v;
  p.attend = a.attend;
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.out_o = a.out_o;
  p.out_m = a.out_m;
  p.out_l = a.out_l;
  p.status = c->d_status;
  p.stamps = c->stamps;
  p.cap = kv->cap;
  p.mask = make_mask(d, a.kv_len, a.t0, a.t1, a.include_canvas);
  p.ring_mask = kv->ring_mask ? kv->ring_mask : 0xffffffffu;
  p.pos_base = kv->pos_base;
  {
    const int32_t rr = check_ring_span(kv, p.mask, d.canvas);
    if (rr != DG_OK) return rr;
  }
  p.C = d.canvas;
  p.Hq = d.n_q_heads;
  p.Hkv = d.n_kv_heads;
  p.G = d.n_q_heads / d.n_kv_heads;
  p.D = d.head_dim;
  p.q_prenormed = a.q_prenormed ? 1u : 0u;
  p.n_splits = 1;
  p.rot_half = d.rotary_dim / 2;
  p.pair_off = d.rope_pairing == DG_ROPE_SPLIT_HALF ? d.rotary_dim / 2 : d.head_dim / 2;
  p.scale_log2 = d.softmax_scale * 1.4426950408889634f;
  p.eps = d.rms_eps;
  if (a.ap_k != nullptr) {
    p.ap_k = static_cast<const __nv_bfloat16*>(a.ap_k);
    p.ap_v = static_cast<const __nv_bfloat16*>(a.ap_v);
    p.ap_kw = static_cast<const __nv_bfloat16*>(a.ap_kw);
    p.ap_cache_k = kv->k;
    p.ap_cache_v = kv->v;
    p.ap_ctl = kv->ap_ctl;
    p.ap_vectors = d.canvas * 2u * d.n_kv_heads;
    p.ap_v_norm = d.v_norm;
    p.ap_write_end = a.ap_write_end;
  }

  const bool tensor = tensor_path_ok(d) && kv->has_tmap && !c->force_general && a.attend == nullptr &&
                      (a.q_prenormed || fused_q_prologue_ok(d));
  if (a.ap_k != nullptr && !(tensor && d.head_dim == 256))
    return fail(DG_ERR_INVALID_ARG, "internal: in-launch append needs the head_dim-256 tensor kernel");
  if (!tensor) {
    launch_attn_general(p, launch_stream(c));
    DG_CUDA(cudaGetLastError());
    c->last_launches += 1;
    return DG_OK;
  }
  if (d.head_dim == 512) {
    // value columns split over two CTAs per (query tile, key split); splits meet in the workspace
    if (!a.q_prenormed) return fail(DG_ERR_UNSUPPORTED, "head_dim 512 tensor path needs a prenormed Q");
    const uint32_t q_tiles5 = sm100_query_tiles(p.C, p.G, p.Hkv);
    if (q_tiles5 * 2 > (fixed ? fixed->n_counters : kMaxQueryTiles)) return fail(DG_ERR_UNSUPPORTED, "too many query tiles");
    // The two value halves split the score work and exchange P unless the single form is asked for; on top of
    // that, pairs of query tiles of one KV head share their K and V stages (cta_group::2) when the head has an
    // even number of tiles (pair mode 1 = the exchange alone, 2 = automatic)
    const bool pair5 = !fixed && c->pair_mode != 0;
    const bool quad5 = pair5 && c->pair_mode == 2 && sm100_query_tiles(p.C, p.G, 1) % 2 == 0;
    p.n_splits = choose_splits(c, q_tiles5 * 2, pair5 ? sm100_hd512x_key_steps(p.mask) : sm100_hd512_key_tiles(p.mask));
    p.cluster_splits = 1;
    if (fixed) {
      // as many splits as the fixed arrays hold: [splits][rows][512] partial O, [2 splits][rows] (m, l) pairs
      const size_t rows5 = size_t(p.C) * p.Hq;
      const size_t cap_o = fixed->o_floats / (rows5 * 512), cap_ml = fixed->ml_floats / (rows5 * 4);
      const size_t cap = cap_o < cap_ml ? cap_o : cap_ml;
      if (cap == 0) return fail(DG_ERR_UNSUPPORTED, "rows exceed the fixed workspace");
      if (p.n_splits > cap) p.n_splits = uint32_t(cap);
      p.ws_o = fixed->o;
      p.ws_ml = fixed->ml;
      p.ws_counters = fixed->counters;
    } else if (p.n_splits > 1) {
      const int32_t r5 = ensure_split_ws(c, 2 * p.n_splits, p.C * p.Hq);
      if (r5 != DG_OK) return r5;
      p.ws_o = c->ws_o;
      p.ws_ml = c->ws_ml;
      p.ws_counters = c->counters;
    }
    const bool timed5 = c->timing && c->ev_used + 2 <= c->ev.size();
    if (timed5) DG_CUDA(cudaEventRecord(c->ev[c->ev_used], c->stream));
    const cudaError_t e5 = quad5   ? launch_attn_sm100_hd512q(p, kv->tm_k64, kv->tm_v, launch_stream(c))
                           : pair5 ? launch_attn_sm100_hd512x(p, kv->tm_k, kv->tm_v, launch_stream(c))
                                   : launch_attn_sm100_hd512(p, kv->tm_k, kv->tm_v, launch_stream(c));
    if (e5 != cudaSuccess) return fail_cuda(e5, "launch_attn_sm100_hd512");
    if (timed5) {
      DG_CUDA(cudaEventRecord(c->ev[c->ev_used + 1], c->stream));
      c->ev_used += 2;
    }
    c->last_launches += 1;
    return DG_OK;
  }
  // CTA pairs halve the shared-memory traffic per query tile (the kernel's limiter); they need two
  // query tiles of one KV head to share a key schedule, so a head with a single tile runs unpaired
  // Short key ranges stay unpaired too: the pair form's longer set-up and its workspace merge cost
  // more than the per-tile saving returns below about a hundred key tiles.
  const uint32_t tiles_per_head = sm100_query_tiles(p.C, p.G, 1);
  const uint32_t k_tiles = sm100_key_tiles(p.mask);
  const bool pair = !fixed && (c->pair_mode == 1 || (c->pair_mode == 2 && tiles_per_head >= 2 && k_tiles >= 96));
  const uint32_t q_tiles = pair ? sm100_pair_query_tiles(p.C, p.G, p.Hkv) : sm100_query_tiles(p.C, p.G, p.Hkv);
  if (q_tiles > (fixed ? fixed->n_counters : kMaxQueryTiles)) return fail(DG_ERR_UNSUPPORTED, "too many query tiles");
  p.n_splits = choose_splits(c, q_tiles * c->concurrent, k_tiles);
  // Split merge: consecutive splits of a query tile form a thread-block cluster and merge through
  // shared memory; what is left meets in the workspace.  Clusters stay at 4 CTAs in the pair form
  // (2 x 2): too few clusters of 8 are co-resident on the device.
  p.cluster_splits = 1;
  if (fixed) {
    // every split meets in the caller's arrays (single-CTA form, no cluster merge): as many splits
    // as they hold, [splits][rows][256] partial O and [splits][rows] (m, l) pairs
    const size_t rows = size_t(p.C) * p.Hq;
    const size_t cap_o = fixed->o_floats / (rows * 256), cap_ml = fixed->ml_floats / (rows * 2);
    const size_t cap = cap_o < cap_ml ? cap_o : cap_ml;
    if (cap == 0) return fail(DG_ERR_UNSUPPORTED, "rows exceed the fixed workspace");
    if (p.n_splits > cap) p.n_splits = uint32_t(cap);
    p.ws_o = fixed->o;
    p.ws_ml = fixed->ml;
    p.ws_counters = fixed->counters;
  } else if (p.n_splits % 2 == 0) {
    if (pair) p.cluster_splits = 2;
    else if (p.n_splits == 2 || p.n_splits == 4 || p.n_splits == 8) p.cluster_splits = p.n_splits;
  }
  if (!fixed && p.n_splits / p.cluster_splits > 1) {
    const int32_t r = ensure_split_ws(c, p.n_splits, p.C * p.Hq);
    if (r != DG_OK) return r;
    p.ws_o = c->ws_o;
    p.ws_ml = c->ws_ml;
    p.ws_counters = c->counters;
  }
  if (a.defer != nullptr) {
    a.defer->filled = true;
    a.defer->pair = pair;
    a.defer->p = p;
    a.defer->tm_k = pair ? &kv->tm_k64 : &kv->tm_k;
    a.defer->tm_v = &kv->tm_v;
    return DG_OK;
  }
  const bool timed = c->timing && c->ev_used + 2 <= c->ev.size();
  if (timed) DG_CUDA(cudaEventRecord(c->ev[c->ev_used], c->stream));
  const cudaError_t e = pair ? launch_attn_sm100_pair(p, kv->tm_k64, kv->tm_v, launch_stream(c))
                             : launch_attn_sm100(p, kv->tm_k, kv->tm_v, launch_stream(c));
  if (e != cudaSuccess) return fail_cuda(e, "launch_attn_sm100");
  if (timed) {
    DG_CUDA(cudaEventRecord(c->ev[c->ev_used + 1], c->stream));
    c->ev_used += 2;
  }
  c->last_launches += 1;
  return DG_OK;
}

static int32_t check_ptrs16(std::initializer_list<const void*> ps) {
  for (const void* p : ps)
    if (p && !aligned16(p)) return fail(DG_ERR_ALIGNMENT, "device pointers must be 16-byte aligned");
  return DG_OK;
}

// one canvas: stage 1 on K/V (+ table), then stage 2 with the fused Q prologue
static int32_t denoise_one(dg_ctx* c, const dg_layer_desc& d, dg_kv* kv, uint32_t kv_len, const void* q,
                           const void* k, const void* v, const void* qw, const void* kw, const uint8_t* attend,
                           AttnCall a) {
  int32_t r = check_kv(d, kv, uint64_t(kv_len) + d.canvas);
  if (r != DG_OK) return r;
  // everything that can refuse the call is checked before the first launch, so that a refused call
  // leaves nothing queued (a split-KV group then stays in step with its peers)
  r = check_ring_span(kv, make_mask(d, kv_len, a.t0, a.t1, a.include_canvas), d.canvas);
  if (r != DG_OK) return r;
  const bool tensor = tensor_path_ok(d) && kv->has_tmap && !c->force_general && attend == nullptr;
  if (tensor && !fused_q_prologue_ok(d)) {
    // partial / proportional rotary: run the stand-alone Q prologue into the staging buffer
    r = ensure_stage(c, size_t(d.canvas) * d.n_q_heads * d.head_dim, 0);
    if (r != DG_OK) return r;
    r = do_append(c, d, kv, kv_len, d.canvas, q, c->stage_q, k, nullptr, v, nullptr, qw, kw, nullptr);
    if (r != DG_OK) return r;
    a.q = c->stage_q;
    a.q_prenormed = true;
  } else {
    RopeKey& key = kv->rope_key;
    const bool cached = key.valid && key.kv_len == kv_len && key.canvas == d.canvas && key.rotary_dim == d.rotary_dim &&
                        key.pairing == d.rope_pairing && key.head_dim == d.head_dim && key.theta == d.rope_theta;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    DG_CUDA(cudaStreamIsCapturing(launch_stream(c), &cap));
    const bool capturing = cap != cudaStreamCaptureStatusNone;
    // eager: region 0, rewritten when the key changes.  captured: region 0 read-only when it already
    // holds these positions, else region 1, written and read by the recorded launches themselves.
    float2* table = kv->rope_table + ((capturing && !cached) ? size_t(kMaxCanvas) * (kv->D / 2) : 0);
    // what of the canvas positions this cache stores at all (a shard may hold none of them)
    uint32_t write_end = 0xffffffffu;
    if (kv->shard) {
      const uint64_t end = uint64_t(kv->pos_base) + kv->cap;
      if (end < write_end) write_end = uint32_t(end);
    }
    const bool stores_canvas = write_end > kv_len;
    // With the table in memory the append can run inside the attention launch (one kernel per step);
    // the first step at new positions still goes through the stand-alone kernel, which writes the table.
    const bool in_launch = cached && tensor && c->fused_append && d.head_dim == 256;
    if (in_launch) {
      if (stores_canvas) {
        a.ap_k = k;
        a.ap_v = v;
        a.ap_kw = kw;
        a.ap_write_end = write_end;
      }
    } else if (stores_canvas || !cached) {
      r = do_append(c, d, kv, kv_len, d.canvas, nullptr, nullptr, k, nullptr, v, nullptr, nullptr, kw, cached ? nullptr : table,
                    0xffffffffu, cached ? table : nullptr);
      if (r != DG_OK) return r;
    }
    if (!cached && !capturing) {
      key.valid = true;
      key.kv_len = kv_len;
      key.canvas = d.canvas;
      key.rotary_dim = d.rotary_dim;
      key.pairing = d.rope_pairing;
      key.head_dim = d.head_dim;
      key.theta = d.rope_theta;
    }
    a.q = q;
    a.qw = qw;
    a.table = table;
    a.q_prenormed = false;
    // the Q prologue may start before the kernel ahead of this launch has drained when nothing it reads
    // (Q, its weight, the table) comes from that kernel: the stand-alone append kernel is known not to
    // write them; with the append inside the launch the kernel ahead is the caller's, so the caller must
    // have said that its inputs are stable
    a.early_q = !c->q_from_prev_kernel && (in_launch ? (c->inputs_stable != 0) : cached);
  }
  a.kv_len = kv_len;
  a.attend = attend;
  return do_attention(c, d, kv, a);
}

extern "C" int32_t dg_qk_rope_kv(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint32_t kv_len, void* q, void* k, void* v,
                                 const void* qw, const void* kw) {
  if (!c || !q || !k || !v) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  r = check_kv(*d, kv, uint64_t(kv_len) + d->canvas);
  if (r != DG_OK) return r;
  DG_CUDA(cudaSetDevice(c->device));
  c->last_launches = 0;
  return do_append(c, *d, kv, kv_len, d->canvas, q, q, k, k, v, d->v_norm ? v : nullptr, qw, kw, nullptr);
}

extern "C" int32_t dg_attention(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint32_t kv_len, const void* q, void* out) {
  if (!c || !q || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  r = check_kv(*d, kv, uint64_t(kv_len) + d->canvas);
  if (r != DG_OK) return r;
  r = check_ptrs16({q, out});
  if (r != DG_OK) return r;
  DG_CUDA(cudaSetDevice(c->device));
  c->last_launches = 0;
  AttnCall a;
  a.q = q;
  a.q_prenormed = true;
  a.out = out;
  a.kv_len = kv_len;
  return do_attention(c, *d, kv, a);
}

extern "C" int32_t dg_attn_denoise(dg_ctx* c, const dg_layer_desc* d, dg_kv* const* kv, const uint32_t* kv_len,
                                   uint32_t batch, const void* q, const void* k, const void* v, const void* qw,
                                   const void* kw, void* out) {
  if (!c || !kv || !kv_len || !q || !k || !v || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  r = check_ptrs16({q, k, v, qw, kw, out});
  if (r != DG_OK) return r;
  DG_CUDA(cudaSetDevice(c->device));
  c->last_launches = 0;
  const size_t qe = size_t(d->canvas) * d->n_q_heads * d->head_dim, ke = size_t(d->canvas) * d->n_kv_heads * d->head_dim;
  // Independent canvases go out as ONE launch (grid z = canvas) when nothing they use is shared, with a
  // split count chosen for all their CTAs together (short key ranges then need no key split at all and so
  // no merge).  That holds on the fused tensor path with splits merged inside clusters; anything that
  // needs the shared staging buffer or the split workspace runs one canvas after the other.
  bool concurrent = batch > 1 && batch <= 8 && d->head_dim == 256 && tensor_path_ok(*d) && fused_q_prologue_ok(*d) &&
                    !c->force_general && !c->timing;
  for (uint32_t b = 0; concurrent && b < batch; ++b) concurrent = kv[b] != nullptr && kv[b]->has_tmap;
  uint32_t conc_splits = 0;
  bool conc_pair = false;
  if (concurrent) {
    // one kernel form and one split count for every canvas, and only if that needs no workspace
    const uint32_t G = d->n_q_heads / d->n_kv_heads;
    const uint32_t tph = sm100_query_tiles(d->canvas, G, 1);
    uint32_t k_min = 0xffffffffu, k_max = 0;
    for (uint32_t b = 0; b < batch; ++b) {
      const uint32_t kt = sm100_key_tiles(make_mask(*d, kv_len[b], 0, 0xffffffffu, 1));
      k_min = kt < k_min ? kt : k_min;
      k_max = kt > k_max ? kt : k_max;
    }
    const bool pair_lo = c->pair_mode == 1 || (c->pair_mode == 2 && tph >= 2 && k_min >= 96);
    const bool pair_hi = c->pair_mode == 1 || (c->pair_mode == 2 && tph >= 2 && k_max >= 96);
    conc_pair = pair_lo;
    const uint32_t q_tiles = conc_pair ? sm100_pair_query_tiles(d->canvas, G, d->n_kv_heads)
                                       : sm100_query_tiles(d->canvas, G, d->n_kv_heads);
    conc_splits = choose_splits(c, q_tiles * batch, k_max);
    const bool no_ws = conc_splits == 1 || (conc_pair ? conc_splits == 2 : (conc_splits == 2 || conc_splits == 4 || conc_splits == 8));
    concurrent = pair_lo == pair_hi && no_ws && conc_splits <= k_min;
  }
  const uint32_t saved_splits = c->forced_splits;
  const int saved_pair = c->pair_mode;
  int32_t rc = DG_OK;
  if (concurrent) {
    // one launch per group of up to kMaxBatchLaunch canvases (blockIdx.z = canvas): the appends that are
    // still needed (first step at new positions) are queued first, the attention launches are described
    // by denoise_one and issued together
    c->concurrent = batch;
    c->forced_splits = conc_splits;
    c->pair_mode = conc_pair ? 1 : 0;
    Prepared prep[8];
    for (uint32_t b = 0; b < batch && rc == DG_OK; ++b) {
      AttnCall a;
      a.out = static_cast<__nv_bfloat16*>(out) + b * qe;
      a.defer = &prep[b];
      rc = denoise_one(c, *d, kv[b], kv_len[b], static_cast<const __nv_bfloat16*>(q) + b * qe,
                       static_cast<const __nv_bfloat16*>(k) + b * ke, static_cast<const __nv_bfloat16*>(v) + b * ke, qw, kw,
                       nullptr, a);
      if (rc == DG_OK && !prep[b].filled) rc = fail(DG_ERR_INVALID_ARG, "internal: batched canvas did not take the tensor path");
    }
    c->concurrent = 1;
    c->forced_splits = saved_splits;
    c->pair_mode = saved_pair;
    for (uint32_t b0 = 0; b0 < batch && rc == DG_OK; b0 += kMaxBatchLaunch) {
      const uint32_t n = batch - b0 < kMaxBatchLaunch ? batch - b0 : kMaxBatchLaunch;
      AttnParams ps[kMaxBatchLaunch];
      const CUtensorMap* tk[kMaxBatchLaunch];
      const CUtensorMap* tv[kMaxBatchLaunch];
      for (uint32_t i = 0; i < n; ++i) {
        ps[i] = prep[b0 + i].p;
        tk[i] = prep[b0 + i].tm_k;
        tv[i] = prep[b0 + i].tm_v;
      }
      const cudaError_t e = launch_attn_sm100_batch(ps, tk, tv, n, prep[b0].pair, c->stream);
      if (e != cudaSuccess) rc = fail_cuda(e, "launch_attn_sm100_batch");
      c->last_launches += 1;
    }
    return rc;
  }
  for (uint32_t b = 0; b < batch && rc == DG_OK; ++b) {
    AttnCall a;
    a.out = static_cast<__nv_bfloat16*>(out) + b * qe;
    rc = denoise_one(c, *d, kv[b], kv_len[b], static_cast<const __nv_bfloat16*>(q) + b * qe,
                     static_cast<const __nv_bfloat16*>(k) + b * ke, static_cast<const __nv_bfloat16*>(v) + b * ke, qw, kw,
                     nullptr, a);
  }
  return rc;
}

extern "C" int32_t dg_attn_denoise_host(dg_ctx* c, const dg_layer_desc* d, dg_kv* const* kv, const uint32_t* kv_len,
                                        uint32_t batch, const void* q, const void* k, const void* v, const void* qw,
                                        const void* kw, void* out) {
  if (!c || !kv || !kv_len || !q || !k || !v || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  DG_CUDA(cudaSetDevice(c->device));
  const size_t qe = size_t(batch) * d->canvas * d->n_q_heads * d->head_dim;
  const size_t ke = size_t(batch) * d->canvas * d->n_kv_heads * d->head_dim;
  r = ensure_stage(c, qe, ke);
  if (r != DG_OK) return r;
  DG_CUDA(cudaMemcpyAsync(c->stage_q, q, qe * 2, cudaMemcpyHostToDevice, c->stream));
  DG_CUDA(cudaMemcpyAsync(c->stage_k, k, ke * 2, cudaMemcpyHostToDevice, c->stream));
  DG_CUDA(cudaMemcpyAsync(c->stage_v, v, ke * 2, cudaMemcpyHostToDevice, c->stream));
  // qw / kw are tiny and constant per layer: they stay device pointers.  When the stand-alone Q
  // prologue runs it normalises stage_q in place, which is safe (one warp owns one head vector).
  r = dg_attn_denoise(c, d, kv, kv_len, batch, c->stage_q, c->stage_k, c->stage_v, qw, kw, c->stage_o);
  if (r != DG_OK) return r;
  const uint32_t launches = c->last_launches;
  DG_CUDA(cudaMemcpyAsync(out, c->stage_o, qe * 2, cudaMemcpyDeviceToHost, c->stream));
  const int32_t s = dg_ctx_synchronize(c);
  c->last_launches = launches;
  return s;
}

// ------------------------------------------------------------------------------------------
// Host-buffer pipeline: the copies of step i+1 and i-1 overlap the kernels of step i
// ------------------------------------------------------------------------------------------
struct dg_p2p;
static bool p2p_is_push(const dg_p2p* x);
static void p2p_slice_bytes(const dg_p2p* x, size_t* off, size_t* bytes);
extern "C" int32_t dg_attn_denoise_split_p2p(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint32_t kv_len, uint32_t t0,
                                             uint32_t t1, int32_t include_canvas, dg_p2p* x, const void* q, const void* k,
                                             const void* v, const void* qw, const void* kw, void* out);

struct dg_host_pipe {
  dg_ctx* ctx = nullptr;
  uint32_t depth = 0;
  size_t q_elems = 0, kv_elems = 0;
  cudaStream_t h2d = nullptr, d2h = nullptr;
  struct Slot {
    __nv_bfloat16 *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr;
    cudaEvent_t in = nullptr, cmp = nullptr, out = nullptr;
    bool used = false;      // the events have been recorded at least once
    bool pending = false;   // submitted and not yet waited for
    // dg_host_pipe_submit: the step's copies in are queued at once, its kernels one submit later (pipe_launch)
    bool launched = true;
    dg_layer_desc d;
    std::vector<dg_kv*> kv;
    std::vector<uint32_t> len;
    uint32_t batch = 0;
    const void *qw = nullptr, *kw = nullptr;
    void* out_host = nullptr;
    size_t qe = 0;
    // dg_host_pipe_submit_split: the step of one rank of a split-KV group
    bool split = false;
    uint32_t t0 = 0, t1 = 0;
    int32_t include_canvas = 0;
    struct dg_p2p* x = nullptr;
    const void* q_dev = nullptr;
  } slot[8];
  uint64_t next = 0;        // ticket of the next submit
  bool deferred = false;    // dg_host_pipe_set_deferred_launch
};

// Kernels and copy out of a submitted step whose copies in have been queued.  Deferred form: the HOST waits for those
// copies here (they were queued a whole submit ago, so this normally returns at once) instead of making the compute
// stream wait for their event: with nothing between this step's kernel and the previous step's on the stream the
// launch stays programmatic, and the kernel's set-up and Q prologue overlap the tail of the kernel before it.
static int32_t pipe_launch(dg_host_pipe* hp, dg_host_pipe::Slot& sl) {
  if (sl.launched) return DG_OK;
  sl.launched = true;
  dg_ctx* c = hp->ctx;
  if (hp->deferred) DG_CUDA(cudaEventSynchronize(sl.in));
  else DG_CUDA(cudaStreamWaitEvent(c->stream, sl.in, 0));
  // the slot's staging buffers are complete and are not rewritten before sl.cmp: the Q prologue may read them as
  // early as it likes.  (The slot's previous output left long ago: its submitter or a wait synchronised on sl.out.)
  const int saved = c->inputs_stable;
  c->inputs_stable = 1;
  const int32_t r = sl.split ? dg_attn_denoise_split_p2p(c, &sl.d, sl.kv[0], sl.len[0], sl.t0, sl.t1, sl.include_canvas, sl.x,
                                                         sl.q_dev, sl.k, sl.v, sl.qw, sl.kw, sl.o)
                             : dg_attn_denoise(c, &sl.d, sl.kv.data(), sl.len.data(), sl.batch, sl.q, sl.k, sl.v, sl.qw, sl.kw, sl.o);
  c->inputs_stable = saved;
  if (r != DG_OK) return r;
  DG_CUDA(cudaEventRecord(sl.cmp, c->stream));
  DG_CUDA(cudaStreamWaitEvent(hp->d2h, sl.cmp, 0));
  // a split-KV step in the push form of the exchange leaves only this rank's row slice
  size_t off = 0, bytes = sl.qe * 2;
  if (sl.split && p2p_is_push(sl.x)) p2p_slice_bytes(sl.x, &off, &bytes);
  DG_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(sl.out_host) + off, reinterpret_cast<uint8_t*>(sl.o) + off, bytes,
                          cudaMemcpyDeviceToHost, hp->d2h));
  DG_CUDA(cudaEventRecord(sl.out, hp->d2h));
  sl.used = true;
  return DG_OK;
}
// every submitted step up to and including `upto`, in submission order
static int32_t pipe_launch_upto(dg_host_pipe* hp, uint64_t upto) {
  const uint64_t first = hp->next > hp->depth ? hp->next - hp->depth : 0;
  for (uint64_t t = first; t <= upto && t < hp->next; ++t) {
    const int32_t r = pipe_launch(hp, hp->slot[t % hp->depth]);
    if (r != DG_OK) return r;
  }
  return DG_OK;
}

extern "C" int32_t dg_host_pipe_destroy(dg_host_pipe* hp) {
  if (!hp) return DG_OK;
  cudaSetDevice(hp->ctx->device);
  if (hp->next > 0) pipe_launch_upto(hp, hp->next - 1);
  cudaStreamSynchronize(hp->ctx->stream);
  if (hp->h2d) cudaStreamSynchronize(hp->h2d);
  if (hp->d2h) cudaStreamSynchronize(hp->d2h);
  for (uint32_t i = 0; i < hp->depth; ++i) {
    dg_host_pipe::Slot& sl = hp->slot[i];
    cudaFree(sl.q);
    cudaFree(sl.k);
    cudaFree(sl.v);
    cudaFree(sl.o);
    if (sl.in) cudaEventDestroy(sl.in);
    if (sl.cmp) cudaEventDestroy(sl.cmp);
    if (sl.out) cudaEventDestroy(sl.out);
  }
  if (hp->h2d) cudaStreamDestroy(hp->h2d);
  if (hp->d2h) cudaStreamDestroy(hp->d2h);
  delete hp;
  return DG_OK;
}

extern "C" int32_t dg_host_pipe_create(dg_ctx* c, const dg_layer_desc* d, uint32_t max_batch, uint32_t depth,
                                       dg_host_pipe** out) {
  if (!c || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  *out = nullptr;
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  if (depth < 1 || depth > 8 || max_batch < 1) return fail(DG_ERR_INVALID_ARG, "depth must be 1..8, max_batch >= 1");
  DG_CUDA(cudaSetDevice(c->device));
  dg_host_pipe* hp = new (std::nothrow) dg_host_pipe();
  if (!hp) return fail(DG_ERR_INVALID_ARG, "out of host memory");
  hp->ctx = c;
  hp->depth = depth;
  hp->q_elems = size_t(max_batch) * d->canvas * d->n_q_heads * d->head_dim;
  hp->kv_elems = size_t(max_batch) * d->canvas * d->n_kv_heads * d->head_dim;
  cudaError_t e = cudaStreamCreateWithFlags(&hp->h2d, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&hp->d2h, cudaStreamNonBlocking);
  for (uint32_t i = 0; i < depth && e == cudaSuccess; ++i) {
    dg_host_pipe::Slot& sl = hp->slot[i];
    e = cudaMalloc(&sl.q, hp->q_elems * 2);
    if (e == cudaSuccess) e = cudaMalloc(&sl.k, hp->kv_elems * 2);
    if (e == cudaSuccess) e = cudaMalloc(&sl.v, hp->kv_elems * 2);
    if (e == cudaSuccess) e = cudaMalloc(&sl.o, hp->q_elems * 2);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&sl.in, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&sl.cmp, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&sl.out, cudaEventDisableTiming);
  }
  if (e != cudaSuccess) {
    dg_host_pipe_destroy(hp);
    return fail_cuda(e, "dg_host_pipe_create");
  }
  *out = hp;
  return DG_OK;
}

extern "C" int32_t dg_host_pipe_wait(dg_host_pipe* hp, uint64_t ticket) {
  if (!hp) return fail(DG_ERR_INVALID_ARG, "pipe is NULL");
  if (ticket >= hp->next) return fail(DG_ERR_INVALID_ARG, "ticket was never issued");
  if (ticket + hp->depth < hp->next) return DG_OK;   // its slot has been reused: that submit waited for it
  dg_host_pipe::Slot& sl = hp->slot[ticket % hp->depth];
  if (!sl.pending) return DG_OK;
  DG_CUDA(cudaSetDevice(hp->ctx->device));
  const int32_t r = pipe_launch_upto(hp, ticket);
  if (r != DG_OK) return r;
  DG_CUDA(cudaEventSynchronize(sl.out));
  sl.pending = false;
  return DG_OK;
}

extern "C" int32_t dg_host_pipe_submit(dg_host_pipe* hp, const dg_layer_desc* d, dg_kv* const* kv, const uint32_t* kv_len,
                                       uint32_t batch, const void* q, const void* k, const void* v, const void* qw,
                                       const void* kw, void* out, uint64_t* ticket) {
  if (!hp || !kv || !kv_len || !q || !k || !v || !out || !ticket) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  dg_ctx* c = hp->ctx;
  const size_t qe = size_t(batch) * d->canvas * d->n_q_heads * d->head_dim;
  const size_t ke = size_t(batch) * d->canvas * d->n_kv_heads * d->head_dim;
  if (qe > hp->q_elems || ke > hp->kv_elems) return fail(DG_ERR_CAPACITY, "batch / geometry larger than the pipe was created for");
  DG_CUDA(cudaSetDevice(c->device));
  // the steps submitted before this one: their copies in were queued a submit ago
  if (hp->next > 0) {
    r = pipe_launch_upto(hp, hp->next - 1);
    if (r != DG_OK) return r;
  }
  dg_host_pipe::Slot& sl = hp->slot[hp->next % hp->depth];
  if (sl.pending) {   // the caller has not collected this slot's previous result: finish it first
    DG_CUDA(cudaEventSynchronize(sl.out));
    sl.pending = false;
  }
  // copies in: after the previous kernels that read this slot's staging buffers
  if (sl.used) DG_CUDA(cudaStreamWaitEvent(hp->h2d, sl.cmp, 0));
  DG_CUDA(cudaMemcpyAsync(sl.q, q, qe * 2, cudaMemcpyHostToDevice, hp->h2d));
  DG_CUDA(cudaMemcpyAsync(sl.k, k, ke * 2, cudaMemcpyHostToDevice, hp->h2d));
  DG_CUDA(cudaMemcpyAsync(sl.v, v, ke * 2, cudaMemcpyHostToDevice, hp->h2d));
  DG_CUDA(cudaEventRecord(sl.in, hp->h2d));
  sl.d = *d;
  sl.kv.assign(kv, kv + batch);
  sl.len.assign(kv_len, kv_len + batch);
  sl.batch = batch;
  sl.qw = qw;
  sl.kw = kw;
  sl.out_host = out;
  sl.qe = qe;
  sl.split = false;
  sl.launched = false;
  sl.pending = true;
  *ticket = hp->next++;
  // deferred form: the kernels follow at the next submit, or at the wait for this step, whichever comes first
  return hp->deferred ? DG_OK : pipe_launch(hp, sl);
}

extern "C" int32_t dg_host_pipe_set_deferred_launch(dg_host_pipe* hp, int32_t on) {
  if (!hp) return fail(DG_ERR_INVALID_ARG, "pipe is NULL");
  if (hp->next > 0) {
    DG_CUDA(cudaSetDevice(hp->ctx->device));
    const int32_t r = pipe_launch_upto(hp, hp->next - 1);
    if (r != DG_OK) return r;
  }
  hp->deferred = on != 0;
  return DG_OK;
}

// One split-KV step through the pipe: like dg_host_pipe_submit for one canvas, with the kernels of
// dg_attn_denoise_split_p2p.  A rank that does not count the canvas keys and whose cache is a shard
// never stores the canvas K/V, so their host-to-device copies are left out; in the push form of the
// exchange only this rank's row slice of the output is copied back.
// shared query staging: null when the group does not share Q; else the slot's device buffer, after the slice
// exchange has been queued on `st`
static int32_t p2p_share_q(dg_p2p* x, uint32_t slot, const void* q_host, cudaStream_t st, __nv_bfloat16** q_dev);
extern "C" int32_t dg_host_pipe_submit_split(dg_host_pipe* hp, const dg_layer_desc* d, dg_kv* kv, uint32_t kv_len,
                                             uint32_t t0, uint32_t t1, int32_t include_canvas, dg_p2p* x, const void* q,
                                             const void* k, const void* v, const void* qw, const void* kw, void* out,
                                             uint64_t* ticket) {
  if (!hp || !kv || !x || !q || !k || !v || !out || !ticket) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  dg_ctx* c = hp->ctx;
  const size_t qe = size_t(d->canvas) * d->n_q_heads * d->head_dim;
  const size_t ke = size_t(d->canvas) * d->n_kv_heads * d->head_dim;
  if (qe > hp->q_elems || ke > hp->kv_elems) return fail(DG_ERR_CAPACITY, "geometry larger than the pipe was created for");
  DG_CUDA(cudaSetDevice(c->device));
  if (hp->next > 0) {
    r = pipe_launch_upto(hp, hp->next - 1);
    if (r != DG_OK) return r;
  }
  dg_host_pipe::Slot& sl = hp->slot[hp->next % hp->depth];
  if (sl.pending) {
    DG_CUDA(cudaEventSynchronize(sl.out));
    sl.pending = false;
  }
  if (sl.used) DG_CUDA(cudaStreamWaitEvent(hp->h2d, sl.cmp, 0));
  // Q: the whole block from this rank's host memory, or (dg_p2p_set_share_q) only this rank's row slice, the
  // other slices arriving from the peers over NVLink
  __nv_bfloat16* q_dev = nullptr;
  r = p2p_share_q(x, uint32_t(hp->next % hp->depth), q, hp->h2d, &q_dev);
  if (r != DG_OK) return r;
  if (q_dev == nullptr) {
    DG_CUDA(cudaMemcpyAsync(sl.q, q, qe * 2, cudaMemcpyHostToDevice, hp->h2d));
    q_dev = sl.q;
  }
  const bool stores_canvas = include_canvas != 0 || !kv->shard;
  if (stores_canvas) {
    DG_CUDA(cudaMemcpyAsync(sl.k, k, ke * 2, cudaMemcpyHostToDevice, hp->h2d));
    DG_CUDA(cudaMemcpyAsync(sl.v, v, ke * 2, cudaMemcpyHostToDevice, hp->h2d));
  }
  DG_CUDA(cudaEventRecord(sl.in, hp->h2d));
  sl.d = *d;
  sl.kv.assign(1, kv);
  sl.len.assign(1, kv_len);
  sl.batch = 1;
  sl.qw = qw;
  sl.kw = kw;
  sl.out_host = out;
  sl.qe = qe;
  sl.split = true;
  sl.t0 = t0;
  sl.t1 = t1;
  sl.include_canvas = include_canvas;
  sl.x = x;
  sl.q_dev = q_dev;
  sl.launched = false;
  sl.pending = true;
  *ticket = hp->next++;
  return hp->deferred ? DG_OK : pipe_launch(hp, sl);
}

extern "C" int32_t dg_attn_denoise_bitmap(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint32_t kv_len, const void* q,
                                          const void* k, const void* v, const void* qw, const void* kw,
                                          const uint8_t* attend, void* out) {
  if (!c || !q || !k || !v || !attend || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  DG_CUDA(cudaSetDevice(c->device));
  c->last_launches = 0;
  AttnCall a;
  a.out = out;
  return denoise_one(c, *d, kv, kv_len, q, k, v, qw, kw, attend, a);
}

extern "C" int32_t dg_attn_partial(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint32_t kv_len, uint32_t t0, uint32_t t1,
                                   int32_t include_canvas, const void* q, const void* k, const void* v, const void* qw,
                                   const void* kw, float* o_unnorm, float* m, float* l) {
  if (!c || !q || !k || !v || !o_unnorm || !m || !l) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  r = check_ptrs16({q, k, v, qw, kw, o_unnorm});
  if (r != DG_OK) return r;
  DG_CUDA(cudaSetDevice(c->device));
  c->last_launches = 0;
  AttnCall a;
  a.out = nullptr;
  a.out_o = o_unnorm;
  a.out_m = m;
  a.out_l = l;
  a.t0 = t0;
  a.t1 = t1;
  a.include_canvas = include_canvas ? 1 : 0;
  return denoise_one(c, *d, kv, kv_len, q, k, v, qw, kw, nullptr, a);
}

extern "C" int32_t dg_attn_merge_local(dg_ctx* c, uint32_t n_parts, uint32_t rows, uint32_t head_dim, const float* o,
                                       const float* m, const float* l, void* out) {
  if (!c || !o || !m || !l || !out || n_parts == 0) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  DG_CUDA(cudaSetDevice(c->device));
  launch_merge_local(n_parts, rows, head_dim, o, m, l, static_cast<__nv_bfloat16*>(out), c->stream);
  DG_CUDA(cudaGetLastError());
  c->last_launches = 1;
  return DG_OK;
}

extern "C" int32_t dg_attn_visibility(dg_ctx* c, const dg_layer_desc* d, uint32_t kv_len, uint32_t t0, uint32_t t1,
                                      int32_t include_canvas, uint8_t* attend_out) {
  if (!c || !attend_out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  const int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  DG_CUDA(cudaSetDevice(c->device));
  launch_visibility(make_mask(*d, kv_len, t0, t1, include_canvas), d->canvas, attend_out, c->stream);
  DG_CUDA(cudaGetLastError());
  return DG_OK;
}

extern "C" double dg_attn_flops(const dg_layer_desc* d, uint32_t kv_len) {
  if (check_desc(d) != DG_OK) return 0.0;
  const MaskParams mk = make_mask(*d, kv_len, 0, 0xffffffffu, 1);
  double vis = 0.0;
  for (uint32_t r = 0; r < d->canvas; ++r) {
    const RowVis rv = mask_row(mk, r);
    vis += double(mk.pre_hi > rv.lo ? mk.pre_hi - rv.lo : 0u) + double(rv.can_hi - rv.can_lo);
  }
  return 4.0 * d->head_dim * d->n_q_heads * vis;
}

// ------------------------------------------------------------------------------------------
// NCCL (loaded at run time so that the library itself has no hard dependency on it)
// ------------------------------------------------------------------------------------------
namespace {
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;   // optional: the host-side watchdog
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  bool ok = false;
};
NcclApi& nccl() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api;
  tried = true;
  const char* env = getenv("DG_NCCL_LIB");
  const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    if (!n) continue;
    api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (api.handle) break;
  }
  if (!api.handle) return api;
  api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(api.handle, "ncclGetUniqueId"));
  api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(api.handle, "ncclCommInitRank"));
  api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(api.handle, "ncclCommDestroy"));
  api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(api.handle, "ncclAllReduce"));
  api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(api.handle, "ncclAllGather"));
  api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(api.handle, "ncclGetErrorString"));
  api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(dlsym(api.handle, "ncclCommGetAsyncError"));
  api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(dlsym(api.handle, "ncclCommAbort"));
  api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather && api.GetErrorString;
  return api;
}
int32_t fail_nccl(ncclResult_t r, const char* what) {
  g_last_error = std::string(what) + ": " + (nccl().GetErrorString ? nccl().GetErrorString(r) : "nccl error");
  return DG_ERR_NCCL;
}
}  // namespace
#define DG_NCCL(call)                                  \
  do {                                                 \
    ncclResult_t r__ = (call);                         \
    if (r__ != ncclSuccess) return fail_nccl(r__, #call); \
  } while (0)

extern "C" int32_t dg_nccl_unique_id(uint8_t id_out[128]) {
  if (!id_out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (!nccl().ok) return fail(DG_ERR_NCCL, "libnccl.so.2 could not be loaded (set DG_NCCL_LIB)");
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  DG_NCCL(nccl().GetUniqueId(&id));
  std::memcpy(id_out, &id, 128);
  return DG_OK;
}
extern "C" int32_t dg_nccl_comm_create(dg_ctx* c, const uint8_t id[128], int32_t world, int32_t rank, void** comm_out) {
  if (!c || !id || !comm_out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (!nccl().ok) return fail(DG_ERR_NCCL, "libnccl.so.2 could not be loaded (set DG_NCCL_LIB)");
  DG_CUDA(cudaSetDevice(c->device));
  ncclUniqueId uid;
  std::memcpy(&uid, id, 128);
  ncclComm_t comm;
  DG_NCCL(nccl().CommInitRank(&comm, world, uid, rank));
  *comm_out = comm;
  return DG_OK;
}
extern "C" int32_t dg_nccl_comm_destroy(void* comm) {
  if (!comm) return DG_OK;
  if (!nccl().ok) return fail(DG_ERR_NCCL, "NCCL not loaded");
  DG_NCCL(nccl().CommDestroy(static_cast<ncclComm_t>(comm)));
  return DG_OK;
}

// Host-side watchdog of a communicator: NCCL reports failures of collectives that are already queued (a
// peer that died, a network error) asynchronously; a host loop polls this between steps and, on an error,
// aborts the communicator so that the kernels still waiting on it return instead of spinning.
extern "C" int32_t dg_nccl_comm_check(void* comm) {
  if (!comm) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (!nccl().ok || !nccl().CommGetAsyncError) return fail(DG_ERR_NCCL, "ncclCommGetAsyncError not available");
  ncclResult_t async = ncclSuccess;
  DG_NCCL(nccl().CommGetAsyncError(static_cast<ncclComm_t>(comm), &async));
  if (async != ncclSuccess && async != ncclInProgress) return fail_nccl(async, "asynchronous NCCL error");
  return DG_OK;
}
extern "C" int32_t dg_nccl_comm_abort(void* comm) {
  if (!comm) return DG_OK;
  if (!nccl().ok || !nccl().CommAbort) return fail(DG_ERR_NCCL, "ncclCommAbort not available");
  DG_NCCL(nccl().CommAbort(static_cast<ncclComm_t>(comm)));
  return DG_OK;
}

extern "C" int32_t dg_attn_merge_nccl(dg_ctx* c, void* comm, float* o_unnorm, float* m, float* l, void* out, uint32_t rows,
                                      uint32_t head_dim) {
  if (!c || !comm || !o_unnorm || !m || !l || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (!nccl().ok) return fail(DG_ERR_NCCL, "NCCL not loaded");
  DG_CUDA(cudaSetDevice(c->device));
  if (rows > c->nccl_rows || head_dim > c->nccl_d) {
    DG_CUDA(cudaStreamSynchronize(c->stream));
    cudaFree(c->nccl_pay);
    cudaFree(c->nccl_mg);
    c->nccl_pay = c->nccl_mg = nullptr;
    c->nccl_rows = c->nccl_d = 0;
    DG_CUDA(cudaMalloc(&c->nccl_pay, size_t(rows) * (head_dim + 1) * sizeof(float)));
    DG_CUDA(cudaMalloc(&c->nccl_mg, size_t(rows) * sizeof(float)));
    c->nccl_rows = rows;
    c->nccl_d = head_dim;
  }
  ncclComm_t cm = static_cast<ncclComm_t>(comm);
  // 1. global reference point   2. rescale [O | l] to it   3. sum across ranks   4. normalise
  DG_NCCL(nccl().AllReduce(m, c->nccl_mg, rows, ncclFloat32, ncclMax, cm, c->stream));
  launch_merge_pack(rows, head_dim, o_unnorm, m, c->nccl_mg, l, c->nccl_pay, c->stream);
  DG_CUDA(cudaGetLastError());
  DG_NCCL(nccl().AllReduce(c->nccl_pay, c->nccl_pay, size_t(rows) * (head_dim + 1), ncclFloat32, ncclSum, cm, c->stream));
  launch_merge_finalize(rows, head_dim, c->nccl_pay, static_cast<__nv_bfloat16*>(out), c->stream);
  DG_CUDA(cudaGetLastError());
  c->last_launches += 2;
  return DG_OK;
}

extern "C" int32_t dg_nccl_all_gather(dg_ctx* c, void* comm, const void* send, void* recv, uint64_t bytes_per_rank) {
  if (!c || !comm || !send || !recv) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (!nccl().ok) return fail(DG_ERR_NCCL, "NCCL not loaded");
  DG_CUDA(cudaSetDevice(c->device));
  DG_NCCL(nccl().AllGather(send, recv, bytes_per_rank, ncclUint8, static_cast<ncclComm_t>(comm), c->stream));
  return DG_OK;
}

// ------------------------------------------------------------------------------------------
// Stage 2 without any allocation
// ------------------------------------------------------------------------------------------
// Some hosts may not allocate device memory once they are running: a serving loop that has handed
// every free byte of HBM to its own pool, a step that is being recorded into a CUDA graph (stream
// capture forbids cudaMalloc), or a real-time thread that must not enter the allocator.  The regular
// entry points grow the split workspace with cudaMalloc the first time a launch needs more of it.
// dg_attention_static_scratch never does: its split workspace is the fixed array below, which every
// GPU that loads this library holds from module load until process exit.
//
// Layout of the array (floats): [partial O: kStaticSplits x kStaticRows x 256]
//                               [partial (m, l): kStaticSplits x kStaticRows x 2]
//                               [one counter per query tile: kStaticTiles words]
// = 4 x 4096 x 256 + 4 x 4096 x 2 + 128 floats = 16.13 MiB.
namespace {
constexpr uint32_t kStaticSplits = 4;      // at most 4 key splits per query tile
constexpr uint32_t kStaticRows = 4096;     // canvas * n_q_heads, e.g. 256 x 16
constexpr uint32_t kStaticTiles = 128;     // query tiles (counters)
constexpr size_t kStaticOFloats = size_t(kStaticSplits) * kStaticRows * 256;
constexpr size_t kStaticMlFloats = size_t(kStaticSplits) * kStaticRows * 2;
constexpr size_t kStaticFloats = kStaticOFloats + kStaticMlFloats + kStaticTiles;
constexpr int kMaxDevices = 64;
}  // namespace

static __device__ __align__(256) float g_static_scratch[kStaticFloats];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the address
// the kernels need comes from cudaGetSymbolAddress, asked once per device with that device current.
static float* g_static_scratch_addr[kMaxDevices] = {};
static std::mutex g_static_scratch_mutex;

static int32_t static_scratch_for_device(int device, float** out) {
  if (device < 0 || device >= kMaxDevices) return fail(DG_ERR_INVALID_ARG, "device index out of range");
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[device] == nullptr) {
    DG_CUDA(cudaSetDevice(device));
    void* ptr = nullptr;
    DG_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (ptr == nullptr) return fail(DG_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_static_scratch_addr[device] = static_cast<float*>(ptr);
  }
  *out = g_static_scratch_addr[device];
  return DG_OK;
}

extern "C" int32_t dg_attention_static_scratch(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint32_t kv_len, const void* q,
                                               void* out) {
  if (!c || !q || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  r = check_kv(*d, kv, uint64_t(kv_len) + d->canvas);
  if (r != DG_OK) return r;
  r = check_ptrs16({q, out});
  if (r != DG_OK) return r;
  DG_CUDA(cudaSetDevice(c->device));
  c->last_launches = 0;
  AttnCall a;
  a.q = q;
  a.q_prenormed = true;
  a.out = out;
  a.kv_len = kv_len;
  const bool tensor = tensor_path_ok(*d) && kv->has_tmap && !c->force_general;
  // the general kernel keeps all of its state in registers and shared memory: nothing to provide
  if (!tensor) return do_attention(c, *d, kv, a);
  const uint32_t rows = d->canvas * d->n_q_heads;
  const uint32_t q_tiles = sm100_query_tiles(d->canvas, d->n_q_heads / d->n_kv_heads, d->n_kv_heads) *
                           (d->head_dim == 512 ? 2u : 1u);
  const uint32_t row_limit = kStaticRows;
  if (rows > row_limit || q_tiles > kStaticTiles) {
    g_last_error = "dg_attention_static_scratch: canvas * n_q_heads = " + std::to_string(rows) + " rows (" +
                   std::to_string(q_tiles) + " query tiles) exceeds the built-in scratch of " +
                   std::to_string(row_limit) + " rows / " + std::to_string(kStaticTiles) +
                   " tiles; use dg_attention, which allocates its workspace";
    return DG_ERR_UNSUPPORTED;
  }
  float* scratch = nullptr;
  r = static_scratch_for_device(c->device, &scratch);
  if (r != DG_OK) return r;
  FixedWs ws;
  ws.o = scratch;
  ws.o_floats = kStaticOFloats;
  ws.ml = scratch + kStaticOFloats;
  ws.ml_floats = kStaticMlFloats;
  ws.counters = reinterpret_cast<uint32_t*>(scratch + kStaticOFloats + kStaticMlFloats);
  ws.n_counters = kStaticTiles;
  // The array keeps whatever the previous call left.  Partials are fully rewritten before they are
  // read, but the per-tile arrival counters must start at zero (a call that was cut short could have
  // left them half-counted), so they are cleared on the stream ahead of the launch.
  DG_CUDA(cudaMemsetAsync(ws.counters, 0, kStaticTiles * sizeof(uint32_t), launch_stream(c)));
  return do_attention(c, *d, kv, a, &ws);
}

// ------------------------------------------------------------------------------------------
// Split-KV over peer memory (one process per GPU, buffers shared through CUDA IPC)
// ------------------------------------------------------------------------------------------
struct dg_p2p {
  dg_ctx* ctx = nullptr;
  uint32_t world = 0, rank = 0, rows = 0, D = 0;
  uint8_t* local = nullptr;
  size_t bytes = 0;
  uint8_t* peer[8] = {};
  bool opened[8] = {};
  bool connected = false;
  uint32_t step = 0;
  uint32_t push_uses[3] = {0, 0, 0};   // push forms: steps that have used each receive slot since the last reset
  // pipelined push form: the step whose rows have been sent and whose slice is merged by the next call
  bool pend = false;
  uint32_t pend_slot = 0, pend_uses = 0;
  void* pend_out = nullptr;
  // host pipeline: every rank copies in its own row slice of Q and the slices are exchanged over peer memory
  bool share_q = false;
  uint32_t q_uses[8] = {};
  int32_t mode = 0;          // 0 automatic (all rows with two ranks, slices otherwise), 1 slices, 2 all rows, 3 push
  bool poisoned = false;     // a launch failed half-way through a step: the ranks may disagree until dg_p2p_reset
  unsigned long long* stamps = nullptr;   // caller-owned device buffer for the merge kernel's stamps
  P2pParams layout;
};

static bool p2p_is_push(const dg_p2p* x) { return x->mode == 3 || x->mode == 4; }
static void p2p_slice_bytes(const dg_p2p* x, size_t* off, size_t* bytes) {
  const size_t r0 = (size_t(x->rank) * x->rows) / x->world, r1 = (size_t(x->rank + 1) * x->rows) / x->world;
  *off = r0 * x->D * 2;
  *bytes = (r1 - r0) * x->D * 2;
}

static int32_t p2p_share_q(dg_p2p* x, uint32_t slot, const void* q_host, cudaStream_t st, __nv_bfloat16** q_dev) {
  *q_dev = nullptr;
  if (!x->share_q || x->world < 2 || slot >= 8) return DG_OK;
  size_t off = 0, bytes = 0;
  p2p_slice_bytes(x, &off, &bytes);
  uint8_t* stage = x->local + x->layout.off_qstage[slot];
  DG_CUDA(cudaMemcpyAsync(stage + off, static_cast<const uint8_t*>(q_host) + off, bytes, cudaMemcpyHostToDevice, st));
  x->q_uses[slot] += 1u;
  const cudaError_t e = launch_p2p_qgather(x->layout, slot, x->q_uses[slot], st);
  if (e != cudaSuccess) {
    x->poisoned = true;
    return fail_cuda(e, "launch_p2p_qgather");
  }
  *q_dev = reinterpret_cast<__nv_bfloat16*>(stage);
  return DG_OK;
}

static void p2p_layout(dg_p2p* x) {
  P2pParams& L = x->layout;
  std::memset(&L, 0, sizeof(L));
  size_t off = 0;
  auto take = [&](size_t n) { const size_t o = off; off = (off + n + 255) & ~size_t(255); return o; };
  for (int p = 0; p < 2; ++p) {
    L.off_o[p] = take(size_t(x->rows) * x->D * 4);
    L.off_m[p] = take(size_t(x->rows) * 4);
    L.off_l[p] = take(size_t(x->rows) * 4);
    L.off_res[p] = take(size_t(x->rows) * x->D * 2);
  }
  L.slice_cap = (x->rows + x->world - 1) / x->world;
  for (int p = 0; p < 3; ++p) {
    L.off_recv[p] = take(size_t(x->world) * L.slice_cap * x->D * 2);
    L.off_rml[p] = take(size_t(x->world) * L.slice_cap * 16);
  }
  for (int p = 0; p < 8; ++p) L.off_qstage[p] = take(size_t(x->rows) * x->D * 2);
  L.off_pflag = take(2 * 8 * 4);
  L.off_rflag = take(2 * 8 * 4);
  L.off_done = take(2 * 4);
  L.off_cnt = take(3 * 4);
  L.off_qcnt = take(8 * 4);
  x->bytes = off;
  L.world = x->world;
  L.rank = x->rank;
  L.rows = x->rows;
  L.D = x->D;
  L.status = x->ctx->d_status;
  L.wait_limit = 1000000000ll;
}

extern "C" int32_t dg_p2p_create(dg_ctx* c, uint32_t rows, uint32_t head_dim, int32_t world, int32_t rank, dg_p2p** out) {
  if (!c || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  *out = nullptr;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(DG_ERR_INVALID_ARG, "world must be 1..8 and rank inside it");
  if (rows == 0 || head_dim == 0 || head_dim % 8 != 0) return fail(DG_ERR_INVALID_ARG, "bad rows / head_dim");
  DG_CUDA(cudaSetDevice(c->device));
  dg_p2p* x = new (std::nothrow) dg_p2p();
  if (!x) return fail(DG_ERR_INVALID_ARG, "out of host memory");
  x->ctx = c;
  x->world = uint32_t(world);
  x->rank = uint32_t(rank);
  x->rows = rows;
  x->D = head_dim;
  p2p_layout(x);
  cudaError_t e = cudaMalloc(&x->local, x->bytes);
  if (e == cudaSuccess) e = cudaMemset(x->local, 0, x->bytes);
  if (e != cudaSuccess) {
    delete x;
    return fail_cuda(e, "dg_p2p_create");
  }
  x->peer[rank] = x->local;
  *out = x;
  return DG_OK;
}

extern "C" int32_t dg_p2p_set_mode(dg_p2p* x, int32_t mode) {
  if (!x) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (mode < 0 || mode > 4)
    return fail(DG_ERR_INVALID_ARG, "mode must be 0 (automatic), 1 (row slices), 2 (all rows), 3 (push) or 4 (push, pipelined)");
  if (x->pend) return fail(DG_ERR_INVALID_ARG, "a pipelined step is pending: call dg_p2p_flush first");
  x->mode = mode;
  return DG_OK;
}

extern "C" int32_t dg_p2p_set_wait_limit(dg_p2p* x, uint64_t limit_cycles) {
  if (!x) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (limit_cycles == 0 || limit_cycles > 20000000000ull) return fail(DG_ERR_INVALID_ARG, "limit must be in 1..2e10 cycles");
  x->layout.wait_limit = (long long)limit_cycles;
  return DG_OK;
}

extern "C" int32_t dg_p2p_slice(const dg_p2p* x, uint32_t* row0, uint32_t* n_rows) {
  if (!x || !row0 || !n_rows) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  const uint32_t r0 = uint32_t((uint64_t(x->rank) * x->rows) / x->world);
  const uint32_t r1 = uint32_t((uint64_t(x->rank + 1) * x->rows) / x->world);
  *row0 = r0;
  *n_rows = r1 - r0;
  return DG_OK;
}

extern "C" int32_t dg_p2p_set_share_q(dg_p2p* x, int32_t on) {
  if (!x) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  x->share_q = on != 0;
  return DG_OK;
}

extern "C" int32_t dg_p2p_flush(dg_p2p* x) {
  if (!x) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (!x->pend) return DG_OK;
  DG_CUDA(cudaSetDevice(x->ctx->device));
  P2pParams pp = x->layout;
  pp.stamps = nullptr;
  pp.send_on = 0u;
  pp.merge_on = 1u;
  pp.merge_first = 1u;
  pp.merge_slot = x->pend_slot;
  pp.merge_uses = x->pend_uses;
  const cudaError_t e = launch_p2p_push_merge(pp, x->pend_out, x->ctx->num_sms, x->ctx->stream);
  if (e != cudaSuccess) {
    x->poisoned = true;
    return fail_cuda(e, "launch_p2p_push_merge");
  }
  x->pend = false;
  return DG_OK;
}

extern "C" int32_t dg_p2p_phase_stamps(dg_p2p* x, void* device_buffer) {
  if (!x) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  x->stamps = static_cast<unsigned long long*>(device_buffer);
  return DG_OK;
}

extern "C" int32_t dg_p2p_reset(dg_p2p* x) {
  if (!x) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  DG_CUDA(cudaSetDevice(x->ctx->device));
  DG_CUDA(cudaStreamSynchronize(x->ctx->stream));
  // flags, counters and the step number start again; the caller holds every rank at a host barrier
  // before this call (no peer kernel may still be writing here) and after it
  const P2pParams& L = x->layout;
  DG_CUDA(cudaMemset(x->local + L.off_pflag, 0, x->bytes - L.off_pflag));
  x->step = 0;
  x->push_uses[0] = x->push_uses[1] = x->push_uses[2] = 0;
  for (uint32_t& u : x->q_uses) u = 0;
  x->pend = false;
  x->poisoned = false;
  return DG_OK;
}

extern "C" int32_t dg_p2p_handle(dg_p2p* x, uint8_t handle_out[64]) {
  if (!x || !handle_out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is 64 bytes");
  DG_CUDA(cudaSetDevice(x->ctx->device));
  cudaIpcMemHandle_t h;
  DG_CUDA(cudaIpcGetMemHandle(&h, x->local));
  std::memcpy(handle_out, &h, 64);
  return DG_OK;
}

extern "C" int32_t dg_p2p_connect(dg_p2p* x, const uint8_t* handles) {
  if (!x || !handles) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  DG_CUDA(cudaSetDevice(x->ctx->device));
  for (uint32_t w = 0; w < x->world; ++w) {
    if (w == x->rank) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handles + size_t(w) * 64, 64);
    void* ptr = nullptr;
    DG_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    x->peer[w] = static_cast<uint8_t*>(ptr);
    x->opened[w] = true;
  }
  for (uint32_t w = 0; w < 8; ++w) x->layout.peer[w] = x->peer[w < x->world ? w : x->rank];
  x->connected = true;
  return DG_OK;
}

extern "C" int32_t dg_p2p_destroy(dg_p2p* x) {
  if (!x) return DG_OK;
  cudaSetDevice(x->ctx->device);
  cudaStreamSynchronize(x->ctx->stream);
  for (uint32_t w = 0; w < x->world; ++w)
    if (x->opened[w]) cudaIpcCloseMemHandle(x->peer[w]);
  cudaFree(x->local);
  delete x;
  return DG_OK;
}

extern "C" int32_t dg_attn_denoise_split_p2p(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint32_t kv_len, uint32_t t0,
                                             uint32_t t1, int32_t include_canvas, dg_p2p* x, const void* q, const void* k,
                                             const void* v, const void* qw, const void* kw, void* out) {
  if (!c || !x || !q || !k || !v || !out) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  if (x->ctx != c) return fail(DG_ERR_INVALID_ARG, "the exchange buffer belongs to another context");
  if (!x->connected && x->world > 1) return fail(DG_ERR_INVALID_ARG, "dg_p2p_connect has not been called");
  if (x->poisoned) return fail(DG_ERR_INVALID_ARG, "an earlier step failed after its first launch: call dg_p2p_reset on every rank");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  if (x->rows != d->canvas * d->n_q_heads || x->D != d->head_dim) return fail(DG_ERR_INVALID_ARG, "exchange buffer geometry differs from desc");
  r = check_ptrs16({q, k, v, qw, kw, out});
  if (r != DG_OK) return r;
  DG_CUDA(cudaSetDevice(c->device));
  c->last_launches = 0;
  // The step number and the buffer parity advance only once every launch of the step has been
  // queued: a call that fails its checks (capacity, ring span, ...) leaves this rank in step with
  // its peers, and the caller may simply repeat it.
  const uint32_t step = x->step + 1u;
  const uint32_t par = step & 1u;
  if (x->world == 1) x->layout.peer[0] = x->local;
  AttnCall a;
  a.out = nullptr;
  a.out_o = reinterpret_cast<float*>(x->local + x->layout.off_o[par]);
  a.out_m = reinterpret_cast<float*>(x->local + x->layout.off_m[par]);
  a.out_l = reinterpret_cast<float*>(x->local + x->layout.off_l[par]);
  a.t0 = t0;
  a.t1 = t1;
  a.include_canvas = include_canvas ? 1 : 0;
  P2pParams pp = x->layout;
  pp.step = step;
  pp.parity = par;
  pp.stamps = x->stamps;
  r = denoise_one(c, *d, kv, kv_len, q, k, v, qw, kw, nullptr, a);
  if (r != DG_OK) {
    if (c->last_launches != 0) x->poisoned = true;   // part of the step is already queued
    return r;
  }

  if (x->mode == 3 || x->mode == 4) {
    const uint32_t slot = step % 3u;
    pp.send_on = 1u;
    pp.send_slot = slot;
    void* merge_out = out;
    if (x->mode == 3) {
      // this step's rows are sent, then this step's slice is merged
      pp.merge_on = 1u;
      pp.merge_first = 0u;
      pp.merge_slot = slot;
      pp.merge_uses = x->push_uses[slot] + 1u;
    } else {
      // pipelined: the slice of the previous step (its rows have had a whole step to arrive) is merged first, into
      // the output buffer that was given with THAT step; this step's rows are sent behind it
      pp.merge_on = x->pend ? 1u : 0u;
      pp.merge_first = 1u;
      pp.merge_slot = x->pend_slot;
      pp.merge_uses = x->pend_uses;
      merge_out = x->pend_out;
    }
    const cudaError_t e = launch_p2p_push_merge(pp, merge_out, c->num_sms, c->stream);
    if (e != cudaSuccess) {
      x->poisoned = true;
      return fail_cuda(e, "launch_p2p_push_merge");
    }
    x->push_uses[slot] += 1u;
    if (x->mode == 4) {
      x->pend = true;
      x->pend_slot = slot;
      x->pend_uses = x->push_uses[slot];
      x->pend_out = out;
    }
  } else {
    pp.all_rows = (x->mode == 2 || (x->mode == 0 && x->world == 2)) ? 1u : 0u;
    launch_p2p_merge(pp, out, c->num_sms, c->stream);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      x->poisoned = true;
      return fail_cuda(e, "launch_p2p_merge");
    }
  }
  x->step = step;
  c->last_launches += 1;
  return DG_OK;
}

// ------------------------------------------------------------------------------------------
// the attention stage with its neighbours: input norm -> Q|K|V projection -> attention -> output projection
// -> post-attention norm + residual (reference: encode_layer_qkv_gemm, encode_layer_qk_rope_kv_dispatch,
// encode_layer_attention_dispatch, encode_layer_o_proj_post_attn of src/metal/step_kernel/enc.rs:852-911,1560-1629)
// ------------------------------------------------------------------------------------------
constexpr uint32_t kBlockMaxSlices = 4;   // split-K slices of the output projection

static int32_t ensure_block_ws(dg_ctx* c, size_t rows, size_t hidden, size_t qe, size_t ke) {
  if (rows <= c->blk_rows && hidden <= c->blk_hidden && qe <= c->blk_qe && ke <= c->blk_ke) return DG_OK;
  DG_CUDA(cudaStreamSynchronize(c->stream));
  const size_t R = rows > c->blk_rows ? rows : c->blk_rows, H = hidden > c->blk_hidden ? hidden : c->blk_hidden;
  const size_t Q = qe > c->blk_qe ? qe : c->blk_qe, K = ke > c->blk_ke ? ke : c->blk_ke;
  for (void* ptr : {(void*)c->blk_xn, (void*)c->blk_q, (void*)c->blk_k, (void*)c->blk_v, (void*)c->blk_o, (void*)c->blk_part})
    cudaFree(ptr);
  c->blk_xn = c->blk_q = c->blk_k = c->blk_v = c->blk_o = nullptr;
  c->blk_part = nullptr;
  c->blk_rows = c->blk_hidden = c->blk_qe = c->blk_ke = 0;
  // rows are padded to whole 128-row tiles: the projections' loads of a ragged last tile stay inside the buffers
  const size_t Rp = (R + 127) / 128 * 128;
  DG_CUDA(cudaMalloc(&c->blk_xn, Rp * H * 2));
  DG_CUDA(cudaMalloc(&c->blk_q, Rp * Q * 2));
  DG_CUDA(cudaMalloc(&c->blk_k, Rp * K * 2));
  DG_CUDA(cudaMalloc(&c->blk_v, Rp * K * 2));
  DG_CUDA(cudaMalloc(&c->blk_o, Rp * Q * 2));
  DG_CUDA(cudaMalloc(&c->blk_part, kBlockMaxSlices * Rp * H * sizeof(float)));
  DG_CUDA(cudaMemset(c->blk_xn, 0, Rp * H * 2));
  DG_CUDA(cudaMemset(c->blk_o, 0, Rp * Q * 2));
  c->blk_rows = R;
  c->blk_hidden = H;
  c->blk_qe = Q;
  c->blk_ke = K;
  return DG_OK;
}

static int32_t weight_map(dg_ctx* c, const void* w, uint32_t n, uint32_t k, uint32_t bn, const CUtensorMap** out) {
  for (const dg_ctx::WMap& m : c->blk_wmaps)
    if (m.w == w && m.n == n && m.k == k && m.bn == bn) {
      *out = &m.tm;
      return DG_OK;
    }
  dg_ctx::WMap m;
  m.w = w;
  m.n = n;
  m.k = k;
  m.bn = bn;
  const int32_t r = make_kv_tmap(&m.tm, const_cast<void*>(w), n, 1, bn, k);
  if (r != DG_OK) return r;
  c->blk_wmaps.push_back(m);
  *out = &c->blk_wmaps.back().tm;
  return DG_OK;
}

extern "C" int32_t dg_attn_block(dg_ctx* c, const dg_layer_desc* d, const dg_block_weights* w, dg_kv* kv, uint32_t kv_len,
                                 const void* hidden_in, void* stream_out) {
  if (!c || !w || !kv || !hidden_in || !stream_out || !w->w_qkv || !w->w_o) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  r = check_ptrs16({hidden_in, stream_out, w->w_qkv, w->w_o, w->input_ln, w->post_attn_ln, w->q_norm, w->k_norm});
  if (r != DG_OK) return r;
  const uint32_t H = w->hidden, C = d->canvas;
  const uint32_t nq = d->n_q_heads * d->head_dim, nk = d->n_kv_heads * d->head_dim;
  const uint32_t n_qkv = nq + nk + (w->v_from_k ? 0u : nk);
  if (H == 0 || H % 64 != 0 || H > 8192 || nq % 128 != 0 || nk % 128 != 0)
    return fail(DG_ERR_UNSUPPORTED, "dg_attn_block: hidden must be a multiple of 64 up to 8192, n_heads * head_dim a multiple of 128");
  DG_CUDA(cudaSetDevice(c->device));
  const size_t old_rows = c->blk_rows, old_h = c->blk_hidden, old_q = c->blk_qe;
  const __nv_bfloat16* old_xn = c->blk_xn;
  r = ensure_block_ws(c, C, H, nq, nk);
  if (r != DG_OK) return r;
  if (c->blk_xn != old_xn || old_rows != c->blk_rows || old_h != c->blk_hidden || old_q != c->blk_qe || old_xn == nullptr) {
    // maps of the two activations the projections read, over whole 128-row tiles
    const size_t Rp = (c->blk_rows + 127) / 128 * 128;
    r = make_kv_tmap(&c->blk_tm_xn, c->blk_xn, Rp, 1, 128, uint32_t(c->blk_hidden));
    if (r == DG_OK) r = make_kv_tmap(&c->blk_tm_o, c->blk_o, Rp, 1, 128, uint32_t(c->blk_qe));
    if (r != DG_OK) return r;
  }
  // the maps above span the buffers' full width: this call's width must be the buffers'
  if (H != c->blk_hidden || nq != c->blk_qe)
    return fail(DG_ERR_UNSUPPORTED, "dg_attn_block: one context serves one (hidden, n_q_heads * head_dim) geometry");
  const CUtensorMap *tm_wqkv = nullptr, *tm_wo = nullptr;
  if (c->blk_wmaps.size() >= 4096) c->blk_wmaps.clear();   // before the look-ups of this call, never between them
  // Two row tiles (129..256 canvas rows) run as CTA pairs: each CTA stages half of every 128-column weight tile,
  // so the weight map then has 64-row boxes.
  const bool gemm_pair = c->pair_mode != 0 && C > 128 && C <= 256;
  r = weight_map(c, w->w_qkv, n_qkv, H, gemm_pair ? 64 : 128, &tm_wqkv);
  // output projection: 128 output columns per tile where hidden allows it, and as many slices of the contraction
  // as bring the grid to about one CTA per SM (hidden 2816, 256 rows: 22 x 2 tiles x 3 slices = 132 CTAs)
  const uint32_t bn_o = H % 128 == 0 ? 128u : 64u;
  const uint32_t tiles_o = (H / bn_o) * ((C + 127) / 128);
  uint32_t slices = (c->num_sms > 0 ? uint32_t(c->num_sms) : 148u) / tiles_o;
  slices = slices < 1 ? 1 : slices > kBlockMaxSlices ? kBlockMaxSlices : slices;
  if (slices > nq / 64) slices = nq / 64;
  const bool pair_o = gemm_pair && bn_o == 128;
  if (r == DG_OK) r = weight_map(c, w->w_o, H, nq, pair_o ? 64 : bn_o, &tm_wo);
  if (r != DG_OK) return r;
  cudaStream_t st = launch_stream(c);
  uint32_t launches = 0;
  // 1. input norm
  cudaError_t e = launch_rmsnorm_rows(hidden_in, w->input_ln, c->blk_xn, C, H, st);
  if (e != cudaSuccess) return fail_cuda(e, "launch_rmsnorm_rows");
  // 2. stacked projection: Q, K and V leave as three dense tensors
  GemmParams g = {};
  g.M = C;
  g.N = n_qkv;
  g.K = H;
  g.n_seg = w->v_from_k ? 2u : 3u;
  g.seg[0] = GemmSeg{c->blk_q, 0u, nq};
  g.seg[1] = GemmSeg{c->blk_k, nq, nk};
  g.seg[2] = GemmSeg{c->blk_v, nq + nk, nk};
  g.rowsq = nullptr;
  g.status = c->d_status;
  e = gemm_pair ? launch_gemm_sm100_pair(g, c->blk_tm_xn, *tm_wqkv, st) : launch_gemm_sm100(g, c->blk_tm_xn, *tm_wqkv, 128, st);
  if (e != cudaSuccess) return fail_cuda(e, "launch_gemm_sm100 (qkv)");
  launches += 2;
  // 3. per-head norm + RoPE + cache write + attention.  Q comes from the kernel queued just ahead, so the
  // attention kernel must not read it before its stream dependency has resolved.
  c->q_from_prev_kernel = 1;
  dg_kv* kvs[1] = {kv};
  const uint32_t lens[1] = {kv_len};
  r = dg_attn_denoise(c, d, kvs, lens, 1, c->blk_q, c->blk_k, w->v_from_k ? c->blk_k : c->blk_v, w->q_norm, w->k_norm, c->blk_o);
  c->q_from_prev_kernel = 0;
  if (r != DG_OK) return r;
  launches += c->last_launches;
  // 4. output projection: fp32 partial planes, one per slice of the contraction
  GemmParams go = {};
  go.M = C;
  go.N = H;
  go.K = nq;
  go.n_seg = 0;
  go.rowsq = nullptr;
  go.part = c->blk_part;
  go.k_slices = slices;
  go.status = c->d_status;
  e = pair_o ? launch_gemm_sm100_pair(go, c->blk_tm_o, *tm_wo, st) : launch_gemm_sm100(go, c->blk_tm_o, *tm_wo, bn_o, st);
  if (e != cudaSuccess) return fail_cuda(e, "launch_gemm_sm100 (o_proj)");
  // 5. planes added and stored as bf16, post-attention norm, residual
  e = launch_norm_residual(c->blk_part, slices, w->post_attn_ln, hidden_in, stream_out, C, H, st);
  if (e != cudaSuccess) return fail_cuda(e, "launch_norm_residual");
  c->last_launches = launches + 2;
  return DG_OK;
}

// ------------------------------------------------------------------------------------------
// top-k sparse attention of the reference's full layers (src/shaders/attn/attention_topk/, enc.rs:2125-2135):
// stage 1 -> score GEMM per KV head -> selection + gathered PV
// ------------------------------------------------------------------------------------------
extern "C" int32_t dg_attn_denoise_topk(dg_ctx* c, const dg_layer_desc* d, dg_kv* kv, uint32_t kv_len, const void* q,
                                        const void* k, const void* v, const void* qw, const void* kw, const dg_topk_cfg* cfg,
                                        void* out) {
  if (!c || !q || !k || !v || !out || !cfg) return fail(DG_ERR_INVALID_ARG, "NULL argument");
  int32_t r = check_desc(d);
  if (r != DG_OK) return r;
  r = check_kv(*d, kv, uint64_t(kv_len) + d->canvas);
  if (r != DG_OK) return r;
  r = check_ptrs16({q, k, v, qw, kw, out});
  if (r != DG_OK) return r;
  if (kv->ring_mask != 0 || kv->shard || !kv->has_tmap)
    return fail(DG_ERR_UNSUPPORTED, "dg_attn_denoise_topk: a linear, unsharded cache of head_dim 256 or 512");
  const uint32_t G = d->n_q_heads / d->n_kv_heads, D = d->head_dim, C = d->canvas;
  if (G > 128 || 128 % G != 0) return fail(DG_ERR_UNSUPPORTED, "dg_attn_denoise_topk: the GQA group must divide 128");
  if (cfg->k_div == 0 ? cfg->k_fixed == 0 : cfg->k_min > cfg->k_max)
    return fail(DG_ERR_INVALID_ARG, "dg_attn_denoise_topk: k_fixed >= 1, or k_min <= k_max with k_div");
  if ((cfg->k_div == 0 ? cfg->k_fixed : cfg->k_max) > 1024) return fail(DG_ERR_UNSUPPORTED, "dg_attn_denoise_topk: at most 1024 keys per row");
  DG_CUDA(cudaSetDevice(c->device));
  c->last_launches = 0;
  const size_t qe = size_t(C) * d->n_q_heads * D;
  r = ensure_stage(c, qe, 0);
  if (r != DG_OK) return r;
  // the score plane: keys padded to whole tiles of the score GEMM (128 keys at head_dim 256, 64 at 512)
  const uint32_t bn = D == 256 ? 128u : 64u;
  const uint32_t T = kv_len + C, ld = (T + bn - 1) / bn * bn;
  const size_t rows = size_t(C) * G, need = size_t(d->n_kv_heads) * ((rows + 127) / 128 * 128) * ld;
  if (need > c->topk_elems) {
    DG_CUDA(cudaStreamSynchronize(c->stream));
    cudaFree(c->topk_scores);
    c->topk_scores = nullptr;
    c->topk_elems = 0;
    DG_CUDA(cudaMalloc(&c->topk_scores, need * 2));
    c->topk_elems = need;
  }
  cudaStream_t st = launch_stream(c);
  // 1. stage 1: Q normed + roped into the staging tensor, canvas K/V into the cache
  r = do_append(c, *d, kv, kv_len, C, q, c->stage_q, k, nullptr, v, nullptr, qw, kw, nullptr);
  if (r != DG_OK) return r;
  // 2. scores of every (row, key) of one KV head: rows (i, g) of the staged Q against the cache's K
  CUtensorMap tm_q;
  {
    PFN_encodeTiled enc = get_encode_fn();
    if (!enc) return fail(DG_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    for (uint32_t h = 0; h < d->n_kv_heads; ++h) {
      const cuuint64_t dims[3] = {D, G, C};
      const cuuint64_t strides[2] = {cuuint64_t(D) * 2, cuuint64_t(d->n_q_heads) * D * 2};
      const cuuint32_t box[3] = {64, G, 128 / G};
      const cuuint32_t estr[3] = {1, 1, 1};
      const CUresult cr = enc(&tm_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, c->stage_q + size_t(h) * G * D, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (cr != CUDA_SUCCESS) return fail(DG_ERR_CUDA, "cuTensorMapEncodeTiled failed for the staged Q");
      GemmParams g = {};
      g.M = uint32_t(rows);
      g.N = ld;
      g.K = D;
      g.n_seg = 1;
      g.seg[0] = GemmSeg{c->topk_scores + size_t(h) * ((rows + 127) / 128 * 128) * ld, 0u, ld};
      g.a_inner = G;
      g.w_z = h;
      g.status = c->d_status;
      const cudaError_t e = launch_gemm_sm100(g, tm_q, kv->tm_k, bn, st);
      if (e != cudaSuccess) return fail_cuda(e, "launch_gemm_sm100 (scores)");
      c->last_launches += 1;
    }
  }
  // 3. selection + softmax over the kept keys + gathered PV
  TopkParams tp = {};
  tp.scores = c->topk_scores;
  tp.ld = ld;
  tp.head_rows = uint32_t((rows + 127) / 128 * 128);
  tp.q = c->stage_q;
  tp.k = kv->k;
  tp.v = kv->v;
  tp.out = static_cast<__nv_bfloat16*>(out);
  tp.C = C;
  tp.Hq = d->n_q_heads;
  tp.G = G;
  tp.D = D;
  tp.cap = kv->cap;
  tp.mask = make_mask(*d, kv_len, 0, 0xffffffffu, 1);
  tp.k_fixed = cfg->k_fixed;
  tp.k_div = cfg->k_div;
  tp.k_min = cfg->k_min;
  tp.k_max = cfg->k_max;
  tp.scale_log2 = d->softmax_scale * 1.4426950408889634f;
  const cudaError_t e = launch_topk_select_pv(tp, st);
  if (e != cudaSuccess) return fail_cuda(e, "launch_topk_select_pv");
  c->last_launches += 1;
  return DG_OK;
}
