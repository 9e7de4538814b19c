"""Host-side mirror of the reference's two attention stages, over the C ABI.

The reference drives, per layer and per denoise step, the stages `LayerQkRopeKv` and
`LayerAttention` (src/metal/step_kernel/enc.rs:1733-1806, 2102-2296 in the reference project) with
the geometry in `LayerOffsets{head_dim, n_kv_heads, is_full}` and
`AttnDims{canvas, n_q_heads, causal, window}`.  The classes below carry the same information and
call the CUDA library; torch is used only to own device memory and streams.
"""
from __future__ import annotations

import ctypes as C
import weakref
from dataclasses import dataclass

import torch

from . import capi
from .capi import LayerDesc, check


@dataclass
class AttnLayer:
    """Geometry + semantics of one attention layer (dg_layer_desc)."""
    n_q_heads: int = 16
    n_kv_heads: int = 8
    head_dim: int = 256
    canvas: int = 256
    rotary_dim: int = 256
    rope_theta: float = 1.0e6
    rms_eps: float = 1.0e-6
    softmax_scale: float = 1.0 / 16.0
    window: int = 0
    mask_mode: int = capi.MASK_NONE
    v_norm: int = 0
    rope_pairing: int = capi.ROPE_SPLIT_HALF

    def c_desc(self) -> LayerDesc:
        return LayerDesc(self.n_q_heads, self.n_kv_heads, self.head_dim, self.canvas, self.rotary_dim,
                         self.rope_theta, self.rms_eps, self.softmax_scale, self.window, self.mask_mode,
                         self.v_norm, self.rope_pairing)

    @staticmethod
    def reference_sliding(window: int = 1024, canvas: int = 256) -> "AttnLayer":
        """A sliding layer with the reference's own semantics: no softmax scale, V normed, uniform
        denoise window (src/shaders/attn/attention/attention.metal:52-63)."""
        return AttnLayer(n_kv_heads=8, rope_theta=1.0e4, softmax_scale=1.0, window=window,
                         mask_mode=capi.MASK_WINDOW_UNIFORM, v_norm=1, canvas=canvas)

    def flops(self, kv_len: int) -> float:
        d = self.c_desc()
        return float(capi.load().dg_attn_flops(C.byref(d), kv_len))


def _ptr(t):
    if t is None:
        return None
    assert t.is_contiguous(), "tensors handed to the C ABI must be contiguous"
    return C.c_void_p(t.data_ptr())


class Context:
    """dg_ctx: one per host thread / stream."""

    def __init__(self, device: int = 0, make_current: bool = True):
        """With `make_current` a new torch stream becomes both torch's current stream on `device`
        and the context's launch stream, so tensor uploads, events and the library's kernels are
        ordered on one stream; otherwise the context keeps its own stream, wrapped by
        `torch_stream`."""
        self.lib = capi.load()
        h = C.c_void_p()
        check(self.lib.dg_ctx_create(device, C.byref(h)), "dg_ctx_create")
        self.h = h
        self.device = device
        self._made_current = make_current
        # caches and pipes made from this context refer to it natively: they are closed first
        self._dependents = weakref.WeakSet()
        if make_current:
            # torch owns the stream (so that nothing torch remembers about it can outlive it); the
            # context is told to launch on it
            torch.cuda.set_device(device)
            self.torch_stream = torch.cuda.Stream(device=device)
            check(self.lib.dg_ctx_set_stream(self.h, C.c_void_p(self.torch_stream.cuda_stream)), "dg_ctx_set_stream")
            torch.cuda.set_stream(self.torch_stream)
        else:
            self.torch_stream = torch.cuda.ExternalStream(int(self.lib.dg_ctx_stream(self.h)), device=device)

    def synchronize(self) -> None:
        check(self.lib.dg_ctx_synchronize(self.h), "dg_ctx_synchronize")

    def device_status(self):
        out = (C.c_uint32 * 4)()
        check(self.lib.dg_ctx_last_device_status(self.h, C.byref(out)), "dg_ctx_last_device_status")
        return tuple(out)

    def force_general(self, on: bool) -> None:
        check(self.lib.dg_ctx_force_general(self.h, int(on)), "dg_ctx_force_general")

    def set_pair_mode(self, on: bool | None) -> None:
        """True: CTA-pair form of the tensor kernel, False: single-CTA form, None: automatic (default)."""
        check(self.lib.dg_ctx_set_pair_mode(self.h, 2 if on is None else int(bool(on))), "dg_ctx_set_pair_mode")

    def set_fused_append(self, on: bool) -> None:
        """True (default): the canvas append runs inside the attention launch once the RoPE table is in memory."""
        check(self.lib.dg_ctx_set_fused_append(self.h, int(on)), "dg_ctx_set_fused_append")

    def set_inputs_stable(self, on: bool) -> None:
        """Promise that q/k/v/qw/kw of the following calls are not written by work queued ahead of them."""
        check(self.lib.dg_ctx_set_inputs_stable(self.h, int(on)), "dg_ctx_set_inputs_stable")

    def set_splits(self, n: int) -> None:
        check(self.lib.dg_ctx_set_splits(self.h, n), "dg_ctx_set_splits")

    @property
    def last_launch_count(self) -> int:
        return int(self.lib.dg_ctx_last_launch_count(self.h))

    def kernel_timing(self, on: bool, max_launches: int = 4096) -> None:
        check(self.lib.dg_ctx_kernel_timing(self.h, int(on), max_launches), "dg_ctx_kernel_timing")

    def kernel_time(self):
        """(summed ms, launches) of the attention-kernel launches since kernel_timing(True)."""
        ms = C.c_double()
        n = C.c_uint32()
        check(self.lib.dg_ctx_kernel_time(self.h, C.byref(ms), C.byref(n)), "dg_ctx_kernel_time")
        return ms.value, n.value

    def close(self) -> None:
        if self.h:
            for dep in list(self._dependents):
                dep.close()
            if self._made_current:
                # hand torch its default stream back before the context's stream is destroyed
                torch.cuda.synchronize(self.device)
                torch.cuda.set_stream(torch.cuda.default_stream(self.device))
            self.lib.dg_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KvCache:
    """dg_kv: one layer's head-major bf16 cache for one canvas stream."""

    def __init__(self, ctx: Context, layer: AttnLayer, capacity_tokens: int = 0, ring_slots: int | None = None,
                 pos_base: int | None = None):
        """Linear cache of `capacity_tokens` positions, or (sliding layers) a ring of `ring_slots` slots
        that keeps position pos in slot pos & (ring_slots - 1), or (pos_base given) one rank's shard of a
        long prefix: the positions [pos_base, pos_base + capacity_tokens) only."""
        self.ctx = ctx
        self.layer = layer
        h = C.c_void_p()
        d = layer.c_desc()
        if pos_base is not None:
            check(ctx.lib.dg_kv_create_shard(ctx.h, C.byref(d), pos_base, capacity_tokens, C.byref(h)),
                  "dg_kv_create_shard")
        elif ring_slots is None:
            check(ctx.lib.dg_kv_create(ctx.h, C.byref(d), capacity_tokens, C.byref(h)), "dg_kv_create")
        else:
            check(ctx.lib.dg_kv_create_ring(ctx.h, C.byref(d), ring_slots, C.byref(h)), "dg_kv_create_ring")
        self.h = h
        ctx._dependents.add(self)

    @property
    def ring_mask(self) -> int:
        return int(self.ctx.lib.dg_kv_ring_mask(self.h))

    @property
    def capacity(self) -> int:
        return int(self.ctx.lib.dg_kv_capacity(self.h))

    def load_prefix(self, k: torch.Tensor, v: torch.Tensor, pos0: int = 0) -> None:
        """k, v: [n, Hkv, D] bf16 (host or device), K already normed + roped."""
        assert k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and k.shape == v.shape
        check(self.ctx.lib.dg_kv_load_prefix(self.h, _ptr(k), _ptr(v), pos0, k.shape[0]), "dg_kv_load_prefix")
        if not k.is_cuda:
            self.ctx.synchronize()   # pageable host source must outlive the copy

    def append(self, k: torch.Tensor, v: torch.Tensor, pos0: int, kw: torch.Tensor | None = None,
               write_end: int | None = None) -> None:
        """Norm + RoPE raw keys and write them (and V) at [pos0, pos0+n).  Device tensors.  Positions at
        or past `write_end` (a padded chunk tail) are left out of the cache."""
        d = self.layer.c_desc()
        n = k.shape[0]
        done = 0
        we = 0xFFFFFFFF if write_end is None else int(write_end)
        while done < n:
            step = min(32768, n - done)
            check(self.ctx.lib.dg_kv_append_guarded(self.ctx.h, C.byref(d), self.h, pos0 + done, step,
                                                    _ptr(k[done:done + step]), _ptr(v[done:done + step]), _ptr(kw), we),
                  "dg_kv_append_guarded")
            done += step

    def read(self, pos0: int, n: int):
        lay = self.layer
        k = torch.empty((n, lay.n_kv_heads, lay.head_dim), dtype=torch.bfloat16, device=f"cuda:{self.ctx.device}")
        v = torch.empty_like(k)
        check(self.ctx.lib.dg_kv_read(self.h, _ptr(k), _ptr(v), pos0, n), "dg_kv_read")
        return k, v

    def close(self) -> None:
        if self.h:
            self.ctx.lib.dg_kv_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CanvasAttention:
    """The hot path for one layer: stage 1 (qk_rope_kv), stage 2 (attention), or both fused."""

    def __init__(self, ctx: Context, layer: AttnLayer):
        self.ctx = ctx
        self.layer = layer
        self.desc = layer.c_desc()
        self.lib = ctx.lib

    @property
    def uses_tensor_path(self) -> bool:
        return bool(self.lib.dg_uses_tensor_path(C.byref(self.desc)))

    # stage LayerQkRopeKv
    def qk_rope_kv(self, kv: KvCache, kv_len: int, q, k, v, qw=None, kw=None) -> None:
        check(self.lib.dg_qk_rope_kv(self.ctx.h, C.byref(self.desc), kv.h, kv_len, _ptr(q), _ptr(k), _ptr(v),
                                     _ptr(qw), _ptr(kw)), "dg_qk_rope_kv")

    # stage LayerAttention
    def attention(self, kv: KvCache, kv_len: int, q_normed, out=None):
        out = torch.empty_like(q_normed) if out is None else out
        check(self.lib.dg_attention(self.ctx.h, C.byref(self.desc), kv.h, kv_len, _ptr(q_normed), _ptr(out)),
              "dg_attention")
        return out

    def denoise_topk(self, kv: KvCache, kv_len: int, q, k, v, qw=None, kw=None, out=None, k_fixed: int = 0,
                     k_div: int = 128, k_min: int = 64, k_max: int = 512):
        """Top-k sparse attention of the reference's full layers for one canvas (dg_attn_denoise_topk).
        q: [C,Hq,D], k, v: [C,Hkv,D] pre-norm bf16 device tensors."""
        out = torch.empty_like(q) if out is None else out
        cfg = capi.TopkCfg(k_fixed, k_div, k_min, k_max)
        check(self.lib.dg_attn_denoise_topk(self.ctx.h, C.byref(self.desc), kv.h, kv_len, _ptr(q), _ptr(k), _ptr(v),
                                            _ptr(qw), _ptr(kw), C.byref(cfg), _ptr(out)), "dg_attn_denoise_topk")
        return out

    def denoise(self, kvs, kv_lens, q, k, v, qw=None, kw=None, out=None):
        """q: [B,C,Hq,D], k,v: [B,C,Hkv,D] pre-norm bf16 device tensors; kvs: list of KvCache."""
        B = len(kvs)
        out = torch.empty_like(q) if out is None else out
        kv_arr = (C.c_void_p * B)(*[kv.h for kv in kvs])
        len_arr = (C.c_uint32 * B)(*kv_lens)
        check(self.lib.dg_attn_denoise(self.ctx.h, C.byref(self.desc), kv_arr, len_arr, B, _ptr(q), _ptr(k), _ptr(v),
                                       _ptr(qw), _ptr(kw), _ptr(out)), "dg_attn_denoise")
        return out

    def denoise_host(self, kvs, kv_lens, q, k, v, out, qw=None, kw=None):
        """Same with HOST tensors q, k, v, out (pinned recommended); synchronous."""
        B = len(kvs)
        kv_arr = (C.c_void_p * B)(*[kv.h for kv in kvs])
        len_arr = (C.c_uint32 * B)(*kv_lens)
        check(self.lib.dg_attn_denoise_host(self.ctx.h, C.byref(self.desc), kv_arr, len_arr, B, _ptr(q), _ptr(k),
                                            _ptr(v), _ptr(qw), _ptr(kw), _ptr(out)), "dg_attn_denoise_host")
        return out

    def denoise_bitmap(self, kv: KvCache, kv_len: int, q, k, v, attend, qw=None, kw=None, out=None):
        out = torch.empty_like(q) if out is None else out
        check(self.lib.dg_attn_denoise_bitmap(self.ctx.h, C.byref(self.desc), kv.h, kv_len, _ptr(q), _ptr(k), _ptr(v),
                                              _ptr(qw), _ptr(kw), _ptr(attend), _ptr(out)), "dg_attn_denoise_bitmap")
        return out

    def partial(self, kv: KvCache, kv_len: int, t0: int, t1: int, include_canvas: bool, q, k, v, qw=None, kw=None):
        lay = self.layer
        dev = q.device
        o = torch.empty((lay.canvas, lay.n_q_heads, lay.head_dim), dtype=torch.float32, device=dev)
        m = torch.empty((lay.canvas, lay.n_q_heads), dtype=torch.float32, device=dev)
        l = torch.empty_like(m)
        check(self.lib.dg_attn_partial(self.ctx.h, C.byref(self.desc), kv.h, kv_len, t0, t1, int(include_canvas),
                                       _ptr(q), _ptr(k), _ptr(v), _ptr(qw), _ptr(kw), _ptr(o), _ptr(m), _ptr(l)),
              "dg_attn_partial")
        return o, m, l

    def merge_local(self, o, m, l):
        """o: [P,C,Hq,D], m,l: [P,C,Hq] fp32 -> bf16 [C,Hq,D]."""
        P = o.shape[0]
        rows = o.shape[1] * o.shape[2]
        out = torch.empty(o.shape[1:], dtype=torch.bfloat16, device=o.device)
        check(self.lib.dg_attn_merge_local(self.ctx.h, P, rows, o.shape[3], _ptr(o), _ptr(m), _ptr(l), _ptr(out)),
              "dg_attn_merge_local")
        return out

    def visibility(self, kv_len: int, t0: int = 0, t1: int = 0xFFFFFFFF, include_canvas: bool = True):
        T = kv_len + self.layer.canvas
        out = torch.empty((self.layer.canvas, T), dtype=torch.uint8, device=f"cuda:{self.ctx.device}")
        check(self.lib.dg_attn_visibility(self.ctx.h, C.byref(self.desc), kv_len, t0, t1, int(include_canvas),
                                          _ptr(out)), "dg_attn_visibility")
        return out


class AttnBlock:
    """One layer's attention block with its neighbours (dg_attn_block): input RMS norm, stacked Q|K|V projection,
    attention, output projection, post-attention norm + residual; the reference's encode_layer up to the dense
    FFN (src/metal/step_kernel/enc.rs:852-911).  Weights are bf16 device tensors [out_features, in_features];
    the object keeps them alive, the library caches their TMA descriptors by address."""

    def __init__(self, ctx: Context, layer: AttnLayer, w_qkv, w_o, input_ln=None, post_attn_ln=None, q_norm=None,
                 k_norm=None, v_from_k: bool = False):
        self.ctx, self.layer, self.lib = ctx, layer, ctx.lib
        self.desc = layer.c_desc()
        self.tensors = [t for t in (w_qkv, w_o, input_ln, post_attn_ln, q_norm, k_norm) if t is not None]
        for t in self.tensors:
            assert t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()
        self.hidden = int(w_qkv.shape[1])
        self.w = capi.BlockWeights(_ptr(input_ln), _ptr(w_qkv), _ptr(q_norm), _ptr(k_norm), _ptr(w_o), _ptr(post_attn_ln),
                                   self.hidden, int(v_from_k))

    def step(self, kv: KvCache, kv_len: int, hidden_in, out=None):
        """hidden_in: [canvas, hidden] bf16 device tensor; returns the residual stream after the block."""
        out = torch.empty_like(hidden_in) if out is None else out
        check(self.lib.dg_attn_block(self.ctx.h, C.byref(self.desc), C.byref(self.w), kv.h, kv_len, _ptr(hidden_in),
                                     _ptr(out)), "dg_attn_block")
        return out


class HostPipe:
    """dg_host_pipe: pipelined host-buffer steps (copies of neighbouring steps overlap the kernels)."""

    def __init__(self, ctx: Context, layer: AttnLayer, max_batch: int = 1, depth: int = 3):
        self.ctx, self.layer = ctx, layer
        self.desc = layer.c_desc()
        h = C.c_void_p()
        check(ctx.lib.dg_host_pipe_create(ctx.h, C.byref(self.desc), max_batch, depth, C.byref(h)), "dg_host_pipe_create")
        self.h = h
        self.depth = depth
        ctx._dependents.add(self)

    def submit(self, kvs, kv_lens, q, k, v, out, qw=None, kw=None) -> int:
        """Host tensors q, k, v (read) and out (written) stay in use until wait(ticket) returns."""
        B = len(kvs)
        kv_arr = (C.c_void_p * B)(*[kv.h for kv in kvs])
        len_arr = (C.c_uint32 * B)(*kv_lens)
        t = C.c_uint64()
        check(self.ctx.lib.dg_host_pipe_submit(self.h, C.byref(self.desc), kv_arr, len_arr, B, _ptr(q), _ptr(k), _ptr(v),
                                               _ptr(qw), _ptr(kw), _ptr(out), C.byref(t)), "dg_host_pipe_submit")
        return int(t.value)

    def submit_split(self, kv, kv_len: int, t0: int, t1: int, include_canvas: bool, p2p, q, k, v, out,
                     qw=None, kw=None) -> int:
        """One split-KV step of this rank with host tensors (dg_host_pipe_submit_split)."""
        t = C.c_uint64()
        check(self.ctx.lib.dg_host_pipe_submit_split(self.h, C.byref(self.desc), kv.h, kv_len, t0, t1,
                                                     int(include_canvas), p2p, _ptr(q), _ptr(k), _ptr(v), _ptr(qw),
                                                     _ptr(kw), _ptr(out), C.byref(t)), "dg_host_pipe_submit_split")
        return int(t.value)

    def wait(self, ticket: int) -> None:
        check(self.ctx.lib.dg_host_pipe_wait(self.h, ticket), "dg_host_pipe_wait")

    def set_deferred_launch(self, on: bool) -> None:
        """submit() queues a step's copies at once and its kernels at the next submit (dg_host_pipe_set_deferred_launch)."""
        check(self.ctx.lib.dg_host_pipe_set_deferred_launch(self.h, int(bool(on))), "dg_host_pipe_set_deferred_launch")

    def close(self) -> None:
        if self.h:
            self.ctx.lib.dg_host_pipe_destroy(self.h)
            self.h = None
