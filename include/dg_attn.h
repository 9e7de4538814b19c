/* dg_attn.h - C ABI of the B200 (sm_100a) denoise-step canvas attention.
 *
 * This is the boundary a host written in any language binds (extern "C", plain pointers
 * and sizes).  It replaces the two per-layer dispatches the reference's step runtime issues
 * for attention (paths relative to the reference project):
 *
 *   stage LayerQkRopeKv  -> kernel qk_rope_kv      src/metal/step_kernel/enc.rs:1733-1806,
 *                                                  src/shaders/attn/qk_rope_kv/qk_rope_kv.metal:29-149
 *   stage LayerAttention -> kernels attention*     src/metal/step_kernel/enc.rs:2102-2296,
 *                                                  src/shaders/attn/attention/attention.metal:22-133
 *
 * Conventions
 *  - Every function returns an int32 status: 0 = OK, negative = host-side validation or CUDA
 *    error (nothing was launched, or the launch failed), positive = a device status code read
 *    back from the kernels (only reported by the synchronising calls).  Nothing aborts or traps.
 *  - All tensors are bf16 (IEEE bfloat16 bit patterns, round-to-nearest-even) unless stated.
 *  - A context owns a CUDA stream and a workspace; it is thread-compatible, not thread-safe:
 *    one context per host thread, calls on one context are ordered on its stream.  Calls are
 *    asynchronous with respect to the host unless stated; buffers must stay valid until
 *    dg_ctx_synchronize() (or a synchronising call) returns.
 *  - "device pointer" = memory of the context's GPU; "host pointer" = ordinary host memory.
 */
#ifndef DG_ATTN_H_
#define DG_ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ----------------------------------------------------------------------- */
enum {
  DG_OK = 0,
  DG_ERR_INVALID_ARG = -1,   /* NULL pointer, bad enum, size out of range                       */
  DG_ERR_UNSUPPORTED = -2,   /* geometry the kernels do not cover (e.g. head_dim > 512)         */
  DG_ERR_CAPACITY = -3,      /* kv_len + canvas exceeds the cache capacity                      */
  DG_ERR_CUDA = -4,          /* a CUDA runtime/driver call failed; see dg_last_error_message()  */
  DG_ERR_NO_DEVICE = -5,     /* no sm_100 GPU present / wrong architecture                      */
  DG_ERR_NCCL = -6,          /* NCCL not loadable or an NCCL call failed                        */
  DG_ERR_ALIGNMENT = -7,     /* a device pointer is not 16-byte aligned                         */
  DG_DEV_WAIT_TIMEOUT = 1,   /* a bounded device-side wait gave up (kernel unwound cleanly)     */
  DG_DEV_BAD_SHAPE = 2,      /* device-side shape assertion                                     */
  DG_DEV_SMEM_LAYOUT = 3     /* a kernel's shared-memory map did not fit its (unaligned) window; it
                              * returned without doing anything                                  */
};

/* mask modes: which keys a canvas row sees.  In the three denoise modes the canvas keys are visible
 * to every row, bidirectionally, and the mode only restricts the PREFIX keys
 * (src/shaders/attn/attention/attention.metal:52-63 with dims.causal == 0).  DG_MASK_CAUSAL is the
 * shader's dims.causal != 0 branch (attention.metal:51,57-62), which the reference uses when it
 * re-prefills a committed block (src/metal/step_generate/turn.rs:1235-1295): the query at position
 * kv_len+i sees keys [max(0, kv_len+i-(window-1)), kv_len+i], canvas keys included in that rule.
 * DG_MASK_WINDOW_PER_ROW is an extension for the benchmark's sliding-layer configuration (a window
 * that slides per row while the canvas stays bidirectional); the reference has no such mode.     */
enum {
  DG_MASK_NONE = 0,           /* all prefix keys (global layers)                                */
  DG_MASK_WINDOW_UNIFORM = 1, /* reference denoise rule: t >= max(0, kv_len-(window-1)), all rows */
  DG_MASK_WINDOW_PER_ROW = 2, /* row i (position kv_len+i): t >= max(0, kv_len+i-(window-1))    */
  DG_MASK_CAUSAL = 3          /* row i: max(0, kv_len+i-(window-1)) <= t <= kv_len+i (window 0: no lower bound) */
};

/* RoPE pairings.  src/shaders/attn/cpu.rs:31-65                                                */
enum {
  DG_ROPE_SPLIT_HALF = 0,     /* pairs (d, d + rotary_dim/2)                                    */
  DG_ROPE_PROPORTIONAL = 1    /* pairs (d, head_dim/2 + d), d < rotary_dim/2                    */
};

/* Per-layer geometry and semantics.  Mirrors what the reference spreads over LayerOffsets
 * {head_dim, n_kv_heads, is_full} (src/metal/step_kernel/mod.rs:132-167) and
 * AttnDims{canvas, n_q_heads, causal, window} (src/shaders/include/attention_device.metal:147-152). */
typedef struct dg_layer_desc {
  uint32_t n_q_heads;      /* 16                                                               */
  uint32_t n_kv_heads;     /* 8 (sliding) | 2 (global); must divide n_q_heads                  */
  uint32_t head_dim;       /* 256 on the tensor-core path; any multiple of 8 up to 512 otherwise */
  uint32_t canvas;         /* 1..256 query rows                                                */
  uint32_t rotary_dim;     /* <= head_dim, even                                                */
  float rope_theta;        /* 1e6 | 1e4                                                        */
  float rms_eps;           /* 1e-6                                                             */
  float softmax_scale;     /* 1/16 for the benchmark configs, 1.0 = reference semantics        */
  uint32_t window;         /* 0 = none                                                         */
  uint32_t mask_mode;      /* DG_MASK_*                                                        */
  uint32_t v_norm;         /* 1: V gets the no-scale RMSNorm before the cache write            */
  uint32_t rope_pairing;   /* DG_ROPE_*                                                        */
} dg_layer_desc;

typedef struct dg_ctx dg_ctx;
typedef struct dg_kv dg_kv;

/* ---- context ---------------------------------------------------------------------------- */
/* Replaces the reference's Metal device/queue/pipeline objects (src/metal/device.rs,
 * src/metal/step_kernel/build.rs:303-).  Creates a stream and a workspace on `device`.
 * Caches, host pipes and p2p groups made from a context keep a pointer to it: destroy them
 * before the context.                                                                          */
int32_t dg_ctx_create(int32_t device, dg_ctx** out);
int32_t dg_ctx_destroy(dg_ctx* ctx);
/* Use a caller-owned CUDA stream (cudaStream_t passed as void*) instead of the internal one.   */
int32_t dg_ctx_set_stream(dg_ctx* ctx, void* cuda_stream);
void* dg_ctx_stream(dg_ctx* ctx);
/* Wait for all work queued on the context, then return the first device status (0 = none).
 * Mirrors the reference's wait + DebugStatus check (src/metal/step_kernel/runtime.rs:565-632). */
int32_t dg_ctx_synchronize(dg_ctx* ctx);
/* {code, kernel_id, cta, value}, first-writer-wins; same convention as the reference's
 * DebugStatus (src/shaders/include/debug_status.metal:21-53).  Synchronises.                   */
int32_t dg_ctx_last_device_status(dg_ctx* ctx, uint32_t out[4]);
/* Reset the device status word to "no error" (ordered on the context's stream).                 */
int32_t dg_ctx_clear_device_status(dg_ctx* ctx);
/* Self-test of the failure path: launches a one-thread kernel that waits, with the given cycle
 * limit, on a flag nothing sets; it gives up and records DG_DEV_WAIT_TIMEOUT the way an attention
 * kernel whose barrier wait ran out does.  The context stays usable afterwards.                  */
int32_t dg_ctx_selftest_wait_timeout(dg_ctx* ctx, uint64_t limit_cycles);
const char* dg_status_str(int32_t status);
/* Text of the last CUDA/NCCL error seen by this thread ("" if none).                           */
const char* dg_last_error_message(void);
/* 1 when the tensor-core (tcgen05) kernel will serve this layer geometry, 0 when the general
 * kernel will.  No launch.                                                                     */
int32_t dg_uses_tensor_path(const dg_layer_desc* desc);
/* Force the general (CUDA-core) kernel for every geometry (1) or restore the default (0).
 * Used by tests to cross-check the two kernels.                                                */
int32_t dg_ctx_force_general(dg_ctx* ctx, int32_t on);
/* Select the tensor-path kernel form: 0 = one CTA per query tile, 1 = CTA pairs (tcgen05
 * cta_group::2: two query tiles of one KV head share every staged K/V tile, each CTA staging half
 * of it), 2 = automatic (default: pairs when a KV head has at least two query tiles and the key
 * range is at least 96 tiles of 128 keys).                                                        */
int32_t dg_ctx_set_pair_mode(dg_ctx* ctx, int32_t mode);
/* Number of thread-block clusters of the tensor-path kernel (pair = 0: (1, cluster_y, 1) CTAs,
 * pair = 1: (2, cluster_y, 1) CTAs) that can be resident on the device at once; negative on error. */
int32_t dg_ctx_max_active_clusters(dg_ctx* ctx, int32_t pair, uint32_t cluster_y);
/* Where the canvas K/V append of dg_attn_denoise runs once the RoPE table of the canvas positions is in
 * memory (every step after the first at those positions): 1 (default) = inside the attention launch - the
 * launch's own CTAs norm, rotate and store the canvas K/V before any of them loads a key tile that holds
 * canvas positions, one kernel per step; 0 = in the stand-alone append kernel ahead of the attention kernel
 * (the reference's two dispatches: src/metal/step_kernel/enc.rs:1733-1806, 2102-2296).  Same bits either way. */
int32_t dg_ctx_set_fused_append(dg_ctx* ctx, int32_t on);
/* A promise by the caller: the q, k, v, qw, kw buffers of the following hot-path calls are not written by any
 * work queued on the context's stream ahead of those calls (they were uploaded, or produced and waited for,
 * earlier).  With the append inside the attention launch (above) the library then lets the Q prologue of a
 * step start while the kernel ahead of it on the stream - normally the previous step's attention - is still
 * draining.  Off by default: without the promise every read waits for the kernel ahead.                       */
int32_t dg_ctx_set_inputs_stable(dg_ctx* ctx, int32_t on);
/* Override the number of key splits per query tile on the tensor path (0 = automatic).         */
int32_t dg_ctx_set_splits(dg_ctx* ctx, uint32_t n_splits);

/* ---- KV cache --------------------------------------------------------------------------- */
/* One layer's cache for one canvas stream: bf16 K[Hkv][cap][D] and V[Hkv][cap][D], head-major,
 * device-owned, zero-initialised.  Replaces the reference's per-layer kv_region inside its
 * monolithic buffer (src/metal/step_kv/mod.rs:1-25, src/metal/step_kernel/mod.rs:506-527).
 * `capacity_tokens` must cover prefix + canvas; it is rounded up to a multiple of 128.          */
int32_t dg_kv_create(dg_ctx* ctx, const dg_layer_desc* desc, uint64_t capacity_tokens, dg_kv** out);
/* Ring cache for sliding-window layers: `ring_slots` (a power of two, at least 256) slots per KV head,
 * position pos lives in slot pos & (ring_slots - 1), so only the last ring_slots positions are kept and
 * kv_len may grow without bound (up to 2^31).  The reference's LayerOffsets::kv_ring_mask
 * (src/metal/step_kernel/mod.rs:161-166; 2048 slots for a 1024 window + 256 canvas).  Every attention
 * call checks that what it can load - whole 128-key tiles from the first visible key of canvas row 0 to the
 * end of the canvas - still fits the ring and returns DG_ERR_CAPACITY otherwise (an unwindowed layer on a
 * ring works only while kv_len + canvas <= ring_slots).                                            */
int32_t dg_kv_create_ring(dg_ctx* ctx, const dg_layer_desc* desc, uint32_t ring_slots, dg_kv** out);
/* A linear cache that holds only the positions [pos_base, pos_base + capacity_tokens) (pos_base a multiple
 * of 128): one rank's shard of a long prefix under split-KV, so that a rank's cache costs shard + canvas
 * tokens instead of the whole prefix.  Positions keep their absolute values in every call; an attention
 * call whose visible keys (whole 128-key tiles) are not all inside the shard returns DG_ERR_CAPACITY, and
 * appends of positions outside the shard are dropped (a rank that does not own the canvas keys still
 * runs the step with the replicated canvas K/V).  No counterpart in the reference (single device).      */
int32_t dg_kv_create_shard(dg_ctx* ctx, const dg_layer_desc* desc, uint64_t pos_base, uint64_t capacity_tokens,
                           dg_kv** out);
uint64_t dg_kv_pos_base(const dg_kv* kv);
/* ring_slots - 1 of a ring cache, 0 for a linear one.                                            */
uint32_t dg_kv_ring_mask(const dg_kv* kv);
int32_t dg_kv_destroy(dg_kv* kv);
uint64_t dg_kv_capacity(const dg_kv* kv);
/* Copy `n` tokens of ready-to-use keys/values (K already normed + roped) into positions
 * [pos0, pos0+n).  k, v: token-major [n][Hkv][D] bf16, host or device pointers.  On a ring cache
 * only the last ring_slots positions of the run are stored (the older ones would be overwritten).  */
int32_t dg_kv_load_prefix(dg_kv* kv, const void* k, const void* v, uint64_t pos0, uint64_t n);
/* Read positions [pos0, pos0+n) back as token-major [n][Hkv][D] (snapshot/export; the
 * reference's compact gather: src/metal/step_kv/mod.rs:102-151).  Synchronises.                */
int32_t dg_kv_read(dg_kv* kv, void* k_out, void* v_out, uint64_t pos0, uint64_t n);
/* Norm (+weight) + RoPE raw keys, optional V norm, and write `n` tokens at [pos0, pos0+n):
 * the cache-write half of qk_rope_kv for an arbitrary run of tokens (a committed block, or a
 * synthetic prefill).  k, v: device pointers [n][Hkv][D]; kw: [D] or NULL.                      */
int32_t dg_kv_append(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* kv, uint64_t pos0, uint32_t n,
                     const void* k, const void* v, const void* kw);
/* dg_kv_append that leaves the cache untouched for positions >= write_end: the zero-padded tail of a
 * prefill chunk must not be stored, on a ring it would wrap onto live slots of the window.  The
 * reference's StepParams::kv_write_end (src/metal/step_kernel/mod.rs:203-212); 0xffffffff = no guard. */
int32_t dg_kv_append_guarded(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* kv, uint64_t pos0, uint32_t n,
                             const void* k, const void* v, const void* kw, uint32_t write_end);

/* ---- the hot path ----------------------------------------------------------------------- */
/* Stage 1 alone (reference stage LayerQkRopeKv): per-head RMSNorm(+weight) + RoPE on canvas
 * Q and K in place, V optionally normed in place, K/V written to the cache at
 * [kv_len, kv_len+canvas).  q: [C][Hq][D], k, v: [C][Hkv][D] device pointers (read-write).      */
int32_t dg_qk_rope_kv(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* kv, uint32_t kv_len, void* q, void* k,
                      void* v, const void* qw, const void* kw);
/* Stage 2 alone (reference stage LayerAttention): q is already normed + roped; the canvas
 * K/V are already in the cache.  out: [C][Hq][D] bf16 device pointer.                           */
int32_t dg_attention(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* kv, uint32_t kv_len, const void* q,
                     void* out);
/* Stage 2 for hosts that must not allocate device memory while they run (all HBM already given to
 * the host's own pool, a step being captured into a CUDA graph, a thread barred from the allocator).
 * Same arguments, checks (ring span included) and result as dg_attention, but the key-split workspace
 * is a 16.13 MiB array built into the library (every GPU that loads the library holds it until the
 * process exits) and the call performs no cudaMalloc / cudaFree.  It always runs the one-CTA-per-tile
 * form of the tensor kernels (head_dim 256 and 512) with every key split meeting in that array, so it
 * is a little slower than dg_attention on long key ranges; other geometries run the general kernel,
 * which needs no workspace.  Limits: canvas * n_q_heads <= 4096 rows, at most 128 query tiles (64 for
 * head_dim 512); the number of key splits is clamped to what the array holds for the call's row
 * count (4 at 4096 rows of head_dim 256, 2 at head_dim 512); beyond the row / tile limits the call
 * returns DG_ERR_UNSUPPORTED with an explanatory message.  The first call on each device looks up the
 * array's device address; make that first call before starting any stream capture.  All calls on a
 * device share the one array and it keeps the previous call's contents (the call clears the part
 * that must start at zero): two calls whose kernels overlap on the GPU (different streams, or
 * different contexts on one device) race on it and must be serialised by the caller.
 * This entry point has no counterpart in the reference.                                          */
int32_t dg_attention_static_scratch(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* kv, uint32_t kv_len,
                                    const void* q, void* out);
/* Both stages for `batch` independent canvases, Q prologue fused into the attention kernel.
 * q: [batch][C][Hq][D], k, v: [batch][C][Hkv][D] PRE-norm bf16 device pointers (not modified);
 * qw, kw: norm weights [D] or NULL (= unit); kv[b], kv_len[b]: cache and prefix length of canvas b
 * (kv_len is a host array).  Canvas K/V are written at [kv_len[b], kv_len[b]+C) (uncommitted,
 * overwritten by the next step: src/metal/step_kernel/runtime.rs:83-98).
 * out: [batch][C][Hq][D] bf16 device pointer.                                                   */
int32_t dg_attn_denoise(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* const* kv, const uint32_t* kv_len,
                        uint32_t batch, const void* q, const void* k, const void* v, const void* qw,
                        const void* kw, void* out);
/* Same call with HOST buffers for q, k, v and out: copies in, runs, copies out, synchronises.
 * This is the end-to-end call a host that keeps activations in host memory makes.              */
int32_t dg_attn_denoise_host(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* const* kv, const uint32_t* kv_len,
                             uint32_t batch, const void* q, const void* k, const void* v, const void* qw,
                             const void* kw, void* out);
/* Pipelined form of the host-buffer call for hosts that issue many steps: `depth` staging slots, a copy-in
 * and a copy-out stream beside the context's stream, so that the host-to-device copies of the next step and
 * the device-to-host copy of the previous one overlap the kernels of the current one.  submit() returns at
 * once with a ticket; the host buffers of a submit (q, k, v read, out written) belong to the library until
 * wait(ticket) returns (or until a later submit reuses the slot, which waits for it first).  Results are in
 * submission order.  q, k, v, out should be pinned host memory (pageable memory makes the copies synchronous).
 * Device-side conditions are reported by dg_ctx_synchronize / dg_ctx_last_device_status as for every other
 * call.  One pipe per context; other calls on the context may be interleaved, they are ordered on its stream.
 * No counterpart in the reference, whose activations never leave the device.                       */
typedef struct dg_host_pipe dg_host_pipe;
int32_t dg_host_pipe_create(dg_ctx* ctx, const dg_layer_desc* desc, uint32_t max_batch, uint32_t depth,
                            dg_host_pipe** out);
int32_t dg_host_pipe_submit(dg_host_pipe* pipe, const dg_layer_desc* desc, dg_kv* const* kv, const uint32_t* kv_len,
                            uint32_t batch, const void* q, const void* k, const void* v, const void* qw,
                            const void* kw, void* out, uint64_t* ticket);
int32_t dg_host_pipe_wait(dg_host_pipe* pipe, uint64_t ticket);
int32_t dg_host_pipe_destroy(dg_host_pipe* pipe);
/* Deferred launch (off by default).  With on = 1 dg_host_pipe_submit queues a step's copies in at once but its
 * kernels only at the NEXT submit (or at the wait for the step, or when the pipe is destroyed or this setting
 * changes), after the HOST has seen the copies complete.  No event wait then sits between consecutive steps'
 * kernels on the stream, their launches stay programmatic and a step's set-up overlaps the tail of the step before
 * it (measured on the 32k-prefix layer: 128 -> 117 us per step end to end, the device-resident step being 116).  The price: other calls on the context made between a submit and the next submit
 * are ordered BEFORE that step's kernels, errors of a step's launch are returned by the call that launches it, and
 * the caches and weights of a submitted step must stay valid until it has been waited for.                        */
int32_t dg_host_pipe_set_deferred_launch(dg_host_pipe* pipe, int32_t on);
/* General decoder bitmap (reference DecoderAttnMask, src/model/mask.rs:4-27): attend is a
 * device pointer to uint8 [C][kv_len+C], 1 = visible.  Served by the general kernel.            */
int32_t dg_attn_denoise_bitmap(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* kv, uint32_t kv_len,
                               const void* q, const void* k, const void* v, const void* qw, const void* kw,
                               const uint8_t* attend, void* out);

/* ---- the attention stage with its neighbours ------------------------------------------------
 * One decoder layer's attention block for the canvas rows of a denoise step, as the reference encodes it
 * (src/metal/step_kernel/enc.rs:852-911 encode_layer: encode_layer_qkv_gemm :1560-1629,
 * encode_layer_qk_rope_kv_dispatch, encode_layer_attention_dispatch, encode_layer_o_proj_post_attn :862-911):
 *   xn     = rms_norm(hidden) * input_ln                   (rms_norm_rows_tiled.metal:16-78, eps 1e-6)
 *   Q|K|V  = xn . w_qkv^T                                   (the stacked projection, one GEMM)
 *   O      = dg_attn_denoise(Q, K, V, q_norm, k_norm)       (per-head norm, RoPE, cache write, attention)
 *   t      = O . w_o^T
 *   stream = hidden + rms_norm(t) * post_attn_ln            (residual_half.metal:9-22 with no scalar)
 * every intermediate rounded to bf16 where the reference stores it in its activation arena.
 * Weights are row-major bf16 device tensors [out_features][in_features], 16-byte aligned, and must stay
 * valid and unchanged at their addresses while the context may use them (their TMA descriptors are
 * cached by address).  w_qkv rows: n_q_heads*head_dim of Q, then n_kv_heads*head_dim of K, then the same of V;
 * with v_from_k != 0 there are no V rows and V is the K projection before its norm (the reference's full
 * layers, v_proj == 0: src/shaders/attn/cpu.rs:110-121).  hidden must be a multiple of 64 and
 * n_kv_heads*head_dim of 128.  One context serves one (hidden, n_q_heads*head_dim) geometry.
 * The activations between the kernels live in buffers the context owns; the Q|K|V GEMM writes Q, K and V
 * as the three dense tensors the attention stage reads, the output projection's epilogue leaves each row's
 * sum of squares for the norm behind it, and every kernel is launched programmatically behind the one
 * before it.                                                                                      */
typedef struct dg_block_weights {
  const void* input_ln;     /* [hidden] or NULL (= unit) */
  const void* w_qkv;        /* [n_q*D + n_kv*D (+ n_kv*D)][hidden] */
  const void* q_norm;       /* [D] or NULL: per-head norm weights, as qw / kw of dg_attn_denoise */
  const void* k_norm;
  const void* w_o;          /* [hidden][n_q*D] */
  const void* post_attn_ln; /* [hidden] or NULL */
  uint32_t hidden;
  uint32_t v_from_k;
} dg_block_weights;
int32_t dg_attn_block(dg_ctx* ctx, const dg_layer_desc* desc, const dg_block_weights* w, dg_kv* kv, uint32_t kv_len,
                      const void* hidden_in, void* stream_out);

/* ---- top-k sparse attention (the reference's default on its full layers) ---------------------
 * The reference's DGQ_ATTN_TOPK_DECODE path (src/metal/step_kernel/enc.rs:2125-2135,
 * src/shaders/attn/attention_topk/, oracle attention_topk/cpu.rs:39-120): per (canvas row, query head) only the k
 * highest-scoring visible keys are kept (equal scores: lower index first), the softmax is renormalised over them and
 * O = sum_j p_j V[idx_j].  Its outputs differ from dense attention by construction; this call exists for hosts that
 * need the reference's default numerics, not for speed (on this GPU the exact dense step is faster).
 * k per row: with k_div != 0, k = clamp(n_visible / k_div, k_min, k_max) (the reference's kv-adaptive rule:
 * k_div 128, k_min 64, k_max 512), else k_fixed; never more than the row's visible keys, at most 1024.
 * Same q / k / v / qw / kw / out as dg_attn_denoise for one canvas; linear unsharded caches of head_dim 256 or 512,
 * GQA groups that divide 128.  Three stages: stage 1 as in dg_qk_rope_kv, a tensor-core GEMM that writes the scores
 * of every (row, key) as a 16-bit plane (the reference's u16 key plane), and a selection kernel: two 256-bin radix
 * levels find the k-th largest 16-bit score, keys that share it are ranked by their exact fp32 score, the winners'
 * exact scores are recomputed, softmax, gathered V.                                                              */
typedef struct dg_topk_cfg {
  uint32_t k_fixed, k_div, k_min, k_max;
} dg_topk_cfg;
int32_t dg_attn_denoise_topk(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* kv, uint32_t kv_len, const void* q,
                             const void* k, const void* v, const void* qw, const void* kw, const dg_topk_cfg* cfg,
                             void* out);

/* ---- split-KV building blocks (multi-GPU, and the block-continuation state of the reference:
 * AttnBlockRange / attn_state, src/shaders/include/attention_device.metal:154-165) ------------ */
/* Partial attention over prefix keys [t0, t1) (clipped to kv_len and to the layer's window)
 * plus the canvas keys iff include_canvas.  Canvas K/V are appended first exactly as in
 * dg_attn_denoise.  Outputs (device pointers, fp32): o_unnorm [C][Hq][D] = sum_t e^(s_t - m) v_t,
 * m [C][Hq] = reference point of the exponent (-inf when the row saw no key), l [C][Hq] =
 * sum_t e^(s_t - m); log-sum-exp = m + ln(l).                                                   */
int32_t dg_attn_partial(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* kv, uint32_t kv_len, uint32_t t0,
                        uint32_t t1, int32_t include_canvas, const void* q, const void* k, const void* v,
                        const void* qw, const void* kw, float* o_unnorm, float* m, float* l);
/* Merge `n_parts` partials that live on THIS device (o: [n_parts][rows][D], m, l: [n_parts][rows])
 * into bf16 out [rows][D].  rows = C*Hq.                                                        */
int32_t dg_attn_merge_local(dg_ctx* ctx, uint32_t n_parts, uint32_t rows, uint32_t head_dim, const float* o,
                            const float* m, const float* l, void* out);
/* Merge one partial per rank across an NCCL communicator (ncclComm_t passed as void*):
 * all-reduce(max) of m, local rescale, all-reduce(sum) of [O | l], normalise.  Every rank
 * receives the full bf16 out [rows][D].  o_unnorm, m, l are overwritten.                        */
int32_t dg_attn_merge_nccl(dg_ctx* ctx, void* nccl_comm, float* o_unnorm, float* m, float* l, void* out,
                           uint32_t rows, uint32_t head_dim);
/* NCCL bootstrap helpers for hosts without their own NCCL binding.  The 128-byte unique id is
 * created on rank 0 and must reach the other ranks by the host's own means.                    */
int32_t dg_nccl_unique_id(uint8_t id_out[128]);
int32_t dg_nccl_comm_create(dg_ctx* ctx, const uint8_t id[128], int32_t world_size, int32_t rank, void** comm_out);
int32_t dg_nccl_comm_destroy(void* comm);
/* Host-side watchdog between steps: DG_OK while the communicator is healthy, DG_ERR_NCCL (with NCCL's text in
 * dg_last_error_message) once a queued collective has failed asynchronously (ncclCommGetAsyncError); the host then
 * calls dg_nccl_comm_abort, which ends the communicator and lets its kernels that are still waiting return.  The
 * reference is single-device and has no counterpart; its own failure channel is DebugStatus (dg_ctx_last_device_status). */
int32_t dg_nccl_comm_check(void* comm);
int32_t dg_nccl_comm_abort(void* comm);
/* All-gather of per-rank output head slices (KV-head sharding): every rank contributes
 * `bytes_per_rank` bytes at send and receives world*bytes_per_rank at recv (device pointers).   */
int32_t dg_nccl_all_gather(dg_ctx* ctx, void* comm, const void* send, void* recv, uint64_t bytes_per_rank);

/* ---- split-KV over peer memory (NVLink), one process per GPU ------------------------------ */
/* The exchange of the per-rank (O, m, l) partials without NCCL: every rank owns an exchange buffer,
 * exports it with dg_p2p_handle (a 64-byte CUDA IPC handle the host carries to the other ranks),
 * maps the others with dg_p2p_connect (handles: [world][64] bytes, own entry ignored), and then
 * dg_attn_denoise_split_p2p = dg_attn_partial on this rank's shard + a merge kernel that reads the
 * partial rows of this rank's slice from the peers over NVLink, merges them and stores the bf16
 * result into every rank's buffer + a copy to `out` once all slices have arrived.  world <= 8;
 * every rank must make the same sequence of calls.  All device-side waits are bounded.          */
typedef struct dg_p2p dg_p2p;
int32_t dg_p2p_create(dg_ctx* ctx, uint32_t rows, uint32_t head_dim, int32_t world, int32_t rank, dg_p2p** out);
int32_t dg_p2p_handle(dg_p2p* x, uint8_t handle_out[64]);
/* How the merge is shared out.  Every rank must use the same mode.
 *   1 = every rank merges its slice of the rows and sends the finished rows to the others (two flag rounds);
 *   2 = every rank reads all partials and merges every row itself (one flag round; pays off with two ranks);
 *   0 = automatic (default: 2 with two ranks, 1 otherwise).  Modes 0-2 leave the full output on every rank.
 *   3 = push form (reduce-scatter): every rank STORES each row of its partial, as fp16 with a power-of-two
 *       scale per row, into the buffer of the rank that owns the row and bumps that rank's arrival counter;
 *       the owner waits on its own memory, merges and writes ONLY its row slice of `out` (dg_p2p_slice; the
 *       other rows of `out` are left untouched).  One exchange, no result scatter: the form for a host whose
 *       next operator is sharded by rows, or that gathers the slices itself.                                  */
/*   4 = mode 3 pipelined over consecutive steps, for hosts that keep several independent steps in flight (other
 *       canvases, other requests): a call sends the rows of ITS step, but first merges the slice of the PREVIOUS
 *       call's step - whose rows have had a whole step to arrive, so nobody waits for data that is still on its way
 *       or for a slower rank - into the `out` that was given with that previous call.  The slice of a step is
 *       therefore written by the NEXT call on the group (or by dg_p2p_flush); keep each `out` valid until then, and
 *       give consecutive calls different `out` buffers.                                                          */
int32_t dg_p2p_set_mode(dg_p2p* x, int32_t mode);
/* For dg_host_pipe_submit_split: with on = 1 a rank copies in only ITS row slice of the host's Q (the same rows it
 * owns of the output) and the ranks exchange the slices over peer memory, instead of every rank copying the whole
 * replicated Q over the host's PCIe links.  Every rank must use the same setting, the same pipe depth, and host
 * buffers q that hold the same values on every rank.  Off by default.                                            */
int32_t dg_p2p_set_share_q(dg_p2p* x, int32_t on);
/* Mode 4: merge the slice of the last step into its `out` (the call that a next step would have made).           */
int32_t dg_p2p_flush(dg_p2p* x);
/* The rows of the output this rank owns in modes 3 and 4: [*row0, *row0 + *n_rows) of the canvas * n_q_heads rows.    */
int32_t dg_p2p_slice(const dg_p2p* x, uint32_t* row0, uint32_t* n_rows);
/* Upper bound, in SM clock cycles, of every device-side wait of the exchange (default 1e9, about half a
 * second; at most 2e10).  The wait covers the peers' host-side launch skew as well as their GPU progress.       */
int32_t dg_p2p_set_wait_limit(dg_p2p* x, uint64_t limit_cycles);
/* After DG_DEV_WAIT_TIMEOUT on a p2p group (a peer never delivered: the step's output was left unwritten) or
 * after a call that failed half-way, the ranks no longer agree on the step number and a late peer may still
 * write into buffers of the abandoned step: the group must not be used again until every rank has (1) drained
 * its stream, (2) met the others at a host barrier, (3) called dg_p2p_reset, which zeroes the flags, counters
 * and the step number of this rank's buffer, and (4) met the others at a second host barrier.  Clear the
 * device status word (dg_ctx_clear_device_status) as well.                                                     */
int32_t dg_p2p_reset(dg_p2p* x);
/* Measurement aid for mode 3: with a non-NULL device buffer of 8 uint64, thread 0 of the merge kernel's first CTA
 * stores globaltimer stamps (ns, comparable with dg_ctx_phase_stamps on the same GPU): 0 kernel entered, 1 the
 * attention kernel ahead of it has completed, 2 this CTA's rows are sent, 3 its arrival count is published,
 * 4 every rank's rows have arrived here, 5 this CTA's share of the merge is written.  NULL switches them off.   */
int32_t dg_p2p_phase_stamps(dg_p2p* x, void* device_buffer);
int32_t dg_p2p_connect(dg_p2p* x, const uint8_t* handles);
int32_t dg_p2p_destroy(dg_p2p* x);
int32_t dg_attn_denoise_split_p2p(dg_ctx* ctx, const dg_layer_desc* desc, dg_kv* kv, uint32_t kv_len, uint32_t t0,
                                  uint32_t t1, int32_t include_canvas, dg_p2p* x, const void* q, const void* k,
                                  const void* v, const void* qw, const void* kw, void* out);
/* The same step with HOST buffers through a dg_host_pipe of this rank's context (one canvas): copies in,
 * kernels and the copy out of neighbouring steps overlap as in dg_host_pipe_submit.  A rank that does not
 * count the canvas keys (include_canvas = 0) and whose cache is a shard never stores the canvas K/V, so it
 * does not copy k and v at all; in mode 3 only this rank's row slice of `out` is copied back (to the same
 * offset in `out` that the rows have in the full output).                                                   */
int32_t dg_host_pipe_submit_split(dg_host_pipe* pipe, const dg_layer_desc* desc, dg_kv* kv, uint32_t kv_len, uint32_t t0,
                                  uint32_t t1, int32_t include_canvas, dg_p2p* x, const void* q, const void* k,
                                  const void* v, const void* qw, const void* kw, void* out, uint64_t* ticket);

/* ---- mask introspection (bit-exact mask parity) ----------------------------------------- */
/* Evaluate on the GPU the same visibility predicate the attention kernels use and write it as
 * uint8 [C][kv_len+C] to the device pointer `attend_out`.                                       */
int32_t dg_attn_visibility(dg_ctx* ctx, const dg_layer_desc* desc, uint32_t kv_len, uint32_t t0, uint32_t t1,
                           int32_t include_canvas, uint8_t* attend_out);

/* Algorithmic FLOPs of one dg_attn_denoise canvas: 4 * D * Hq * (visible (row, key) pairs).     */
double dg_attn_flops(const dg_layer_desc* desc, uint32_t kv_len);
/* Number of kernels the last hot-path call on this context launched.                           */
uint32_t dg_ctx_last_launch_count(const dg_ctx* ctx);
/* Measurement aid (the reference's per-stage profile: LayerEncodeSubProfile,
 * src/metal/step_kernel/mod.rs:399-429): with on = 1 every tensor-path attention launch is
 * bracketed by a CUDA event pair on the launching stream, up to max_launches launches;
 * dg_ctx_kernel_time synchronises and returns their summed duration and count.                  */
int32_t dg_ctx_kernel_timing(dg_ctx* ctx, int32_t on, uint32_t max_launches);
/* Measurement aid: with a non-NULL device buffer of CTAs x 16 uint64 (CTA index = (z * grid.y + y) * grid.x + x,
 * z = canvas of a batched call), thread 0 of every CTA of the
 * tensor-path kernel stores globaltimer stamps (ns) at its phase boundaries: 0 start, 1 set-up done,
 * 2 Q prologue done, 3 key loop done, 4 epilogue done, 5 merge done; slots 6-11 hold SM-clock
 * cycles single threads spent waiting inside the key loop (6 MMA issuer on K, 7 on V, 8 on P,
 * 9 the issuer's whole loop, 10 softmax thread 0 on S, 11 on the rescale barrier); slots 12-14 are
 * stamps inside the tail (12 last PV complete, 13 cluster's MMAs complete, 14 cluster's rows arrived).  The
 * stamps cost time; NULL switches them off.                                                             */
int32_t dg_ctx_phase_stamps(dg_ctx* ctx, void* device_buffer);
int32_t dg_ctx_kernel_time(dg_ctx* ctx, double* total_ms, uint32_t* launches);

#ifdef __cplusplus
}
#endif
#endif /* DG_ATTN_H_ */
