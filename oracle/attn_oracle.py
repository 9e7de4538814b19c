"""CPU oracle for the denoise-step canvas attention (TEST INFRASTRUCTURE ONLY).

This module is the checker, never the product: only the tests, the smoke entry
and the bench's CPU-baseline leg may import it.  It restates, in numpy fp32, the
arithmetic of the reference's own CPU code for this path (paths are relative to
the reference project):

* per-head RMSNorm           src/shaders/attn/cpu.rs:67-75, src/shaders/cpu/mod.rs:24-45
* split-half / proportional RoPE
                             src/shaders/attn/cpu.rs:31-65, src/shaders/cpu/mod.rs:205-252
* qk_rope_kv stage           src/shaders/attn/cpu.rs:78-145, src/model/attention.rs:718-743
* GQA attention + softmax    src/shaders/attn/cpu.rs:148-197, src/model/attention.rs:861-934,
                             src/shaders/cpu/mod.rs:175-190
* denoise window rule        src/shaders/attn/attention/attention.metal:52-63
* causal (re-prefill) rule   src/shaders/attn/attention/attention.metal:51,57-62
* general decoder bitmap     src/model/mask.rs:4-27, src/model/attention.rs:889-907
* (m, l, O) block state      src/shaders/include/attention_device.metal:154-165

Parity pin: the reference stores no golden output vectors for attention; this
oracle is pinned (1) against every known-answer value the reference's tests hold
for the path (RMSNorm, RoPE, softmax, masks - tests/test_oracle_pins.py) and the
structural properties they test (blocked online softmax == single pass), and
(2) against the reference's OWN shaders run on the CPU: attention.metal and
qk_rope_kv.metal compile as C++ through a <metal_stdlib> stand-in
(oracle/Makefile target `ref`, oracle/ref_attention.cpp, oracle/ref_qk_rope_kv.cpp),
and tests/test_ref_shader_pins.py holds this module to their outputs - the
visibility rule with a sliding window and the ring slot mapping bit for bit, both
RoPE pairings, the V-aliases-K form, and the softmax values - live where that
library is built and through the vectors stored in tests/golden/ elsewhere.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

MASK_NONE = 0          # every prefix key visible (global layers)
MASK_WINDOW_UNIFORM = 1  # reference denoise rule: one t_lo for every canvas row
MASK_WINDOW_PER_ROW = 2  # query at position p sees prefix keys [p-(W-1), p]
MASK_CAUSAL = 3        # prefill rule: query at position p sees keys [p-(W-1), p], canvas keys included

ROPE_SPLIT_HALF = 0    # pairs (d, d + rot/2)          (sliding layers)
ROPE_PROPORTIONAL = 1  # pairs (d, head_dim/2 + d)     (global layers, partial rotary)


@dataclass
class LayerDesc:
    n_q_heads: int = 16
    n_kv_heads: int = 8
    head_dim: int = 256
    canvas: int = 256
    rotary_dim: int = 256
    rope_theta: float = 1.0e6
    rms_eps: float = 1.0e-6
    softmax_scale: float = 1.0 / 16.0
    window: int = 0
    mask_mode: int = MASK_NONE
    v_norm: int = 0
    rope_pairing: int = ROPE_SPLIT_HALF


# ----------------------------------------------------------------------------
# bf16 helpers (round-to-nearest-even, the storage rounding of this build)
# ----------------------------------------------------------------------------
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    out = (rounded >> np.uint32(16)).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ----------------------------------------------------------------------------
# a1: per-head RMSNorm  (x * rsqrt(mean(x^2) + eps) * w)
# ----------------------------------------------------------------------------
def rms_norm_heads(x: np.ndarray, w: np.ndarray | None, eps: float) -> np.ndarray:
    """x: [..., D] fp32.  w: [D] or None (no-scale variant used for V)."""
    x = x.astype(np.float32)
    ss = np.sum(x * x, axis=-1, keepdims=True, dtype=np.float32)
    inv = (np.float32(1.0) / np.sqrt(ss / np.float32(x.shape[-1]) + np.float32(eps))).astype(np.float32)
    if w is not None:
        # x * (inv * w), the association of src/shaders/attn/cpu.rs:67-75
        y = x * (inv * w.astype(np.float32))
    else:
        y = x * inv
    return y.astype(np.float32)


# ----------------------------------------------------------------------------
# a2: RoPE.  angle = f32(pos) * theta^(-2d/head_dim), all in f32.
# ----------------------------------------------------------------------------
def rope_inv_freq(rotary_dim: int, head_dim: int, theta: float) -> np.ndarray:
    """f32 inverse frequencies, one per rotated pair.

    The reference evaluates `theta.powf(-2d/hd)` in f32.  A correctly rounded f32
    power is reproduced here by evaluating in f64 on the f32 operands and rounding
    once, which avoids depending on numpy's vectorised float32 `power` kernels.
    """
    half = rotary_dim // 2
    th = float(np.float32(theta))
    out = np.empty(half, dtype=np.float32)
    for d in range(half):
        e = float(np.float32(-2.0) * np.float32(d) / np.float32(head_dim))
        out[d] = np.float32(math.pow(th, e))
    return out


def rope_tables(positions: np.ndarray, rotary_dim: int, head_dim: int, theta: float):
    """cos/sin tables [n_pos, rotary_dim/2] in f32 (angle rounded to f32 first)."""
    inv = rope_inv_freq(rotary_dim, head_dim, theta)
    ang = (positions.astype(np.float32)[:, None] * inv[None, :]).astype(np.float32)
    a64 = ang.astype(np.float64)
    return np.cos(a64).astype(np.float32), np.sin(a64).astype(np.float32)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray, rotary_dim: int,
               pairing: int = ROPE_SPLIT_HALF) -> np.ndarray:
    """x: [n_pos, H, D];  cos/sin: [n_pos, rotary_dim/2]."""
    x = x.astype(np.float32).copy()
    d_model = x.shape[-1]
    half = rotary_dim // 2
    off = half if pairing == ROPE_SPLIT_HALF else d_model // 2
    c = cos[:, None, :]
    s = sin[:, None, :]
    x0 = x[..., :half].copy()
    x1 = x[..., off:off + half].copy()
    x[..., :half] = x0 * c - x1 * s
    x[..., off:off + half] = x0 * s + x1 * c
    return x


# ----------------------------------------------------------------------------
# a3: the qk_rope_kv stage on canvas Q/K/V
# ----------------------------------------------------------------------------
def qk_rope_kv(q, k, v, qw, kw, desc: LayerDesc, kv_len: int, round_out: bool = True):
    """q: [C,Hq,D], k,v: [C,Hkv,D] fp32 (bf16-representable).  Returns the normed+roped
    canvas Q, K and the (optionally normed) V, each rounded to bf16 when `round_out`
    (the reference rounds Q/K to 16 bit after this stage:
    src/shaders/attn/qk_rope_kv/mod.rs:251-258)."""
    C = q.shape[0]
    D = desc.head_dim
    qw = np.ones(D, np.float32) if qw is None else qw
    kw = np.ones(D, np.float32) if kw is None else kw
    pos = np.arange(kv_len, kv_len + C)
    cos, sin = rope_tables(pos, desc.rotary_dim, D, desc.rope_theta)
    qn = apply_rope(rms_norm_heads(q, qw, desc.rms_eps), cos, sin, desc.rotary_dim, desc.rope_pairing)
    kn = apply_rope(rms_norm_heads(k, kw, desc.rms_eps), cos, sin, desc.rotary_dim, desc.rope_pairing)
    vn = rms_norm_heads(v, None, desc.rms_eps) if desc.v_norm else v.astype(np.float32)
    if round_out:
        qn, kn, vn = round_bf16(qn), round_bf16(kn), round_bf16(vn)
    return qn, kn, vn


def prepare_prefix_k(k_raw: np.ndarray, desc: LayerDesc, pos0: int = 0, kw=None) -> np.ndarray:
    """Norm + RoPE prefix keys at positions pos0.. and round to bf16 (what a prefill
    would have left in the cache)."""
    n = k_raw.shape[0]
    kw = np.ones(desc.head_dim, np.float32) if kw is None else kw
    cos, sin = rope_tables(np.arange(pos0, pos0 + n), desc.rotary_dim, desc.head_dim, desc.rope_theta)
    return round_bf16(apply_rope(rms_norm_heads(k_raw, kw, desc.rms_eps), cos, sin,
                                 desc.rotary_dim, desc.rope_pairing))


# ----------------------------------------------------------------------------
# a5: visibility bitmap [C, T]  (T = kv_len + C; key t < kv_len is a prefix key)
# ----------------------------------------------------------------------------
def visibility(desc: LayerDesc, kv_len: int, t0: int = 0, t1: int | None = None,
               include_canvas: bool = True) -> np.ndarray:
    """Boolean bitmap attend[row, key].  Prefix keys are further restricted to the
    half-open shard [t0, t1) (split-KV); canvas keys are visible iff include_canvas."""
    C = desc.canvas
    T = kv_len + C
    t1 = kv_len if t1 is None else min(t1, kv_len)
    t = np.arange(T)[None, :]
    rows = np.arange(C)[:, None]
    if desc.mask_mode == MASK_NONE or desc.window == 0:
        t_lo = np.zeros((C, 1), dtype=np.int64)
    elif desc.mask_mode == MASK_WINDOW_UNIFORM:
        t_lo = np.full((C, 1), max(0, kv_len - (desc.window - 1)), dtype=np.int64)
    elif desc.mask_mode in (MASK_WINDOW_PER_ROW, MASK_CAUSAL):
        t_lo = np.maximum(0, kv_len + rows - (desc.window - 1)).astype(np.int64)
    else:
        raise ValueError("mask_mode")
    if desc.mask_mode not in (MASK_NONE, MASK_WINDOW_UNIFORM, MASK_WINDOW_PER_ROW, MASK_CAUSAL):
        raise ValueError("mask_mode")
    prefix = (t >= t_lo) & (t >= t0) & (t < t1) & (t < kv_len)
    canvas = (t >= kv_len) & bool(include_canvas)
    if desc.mask_mode == MASK_CAUSAL:
        # T = min(T_all, kv_len + tok + 1) and the window's lower bound also cuts canvas keys
        canvas = canvas & (t <= kv_len + rows) & (t >= t_lo)
    return prefix | canvas


# ----------------------------------------------------------------------------
# a4/a6: attention over [prefix | canvas] with a bitmap; optional partial state
# ----------------------------------------------------------------------------
def attention(qn, K, V, attend, desc: LayerDesc, return_partial: bool = False):
    """qn: [C,Hq,D] (normed+roped), K,V: [T,Hkv,D], attend: bool [C,T].
    Returns O [C,Hq,D] fp32; a fully masked row yields 0.
    With return_partial: (O_unnorm, m, l) where m is the row max of the scaled
    logits (-inf when nothing is visible), l = sum exp(s - m), O_unnorm = sum exp(s-m) v."""
    C, Hq, D = qn.shape
    Hkv = K.shape[1]
    G = Hq // Hkv
    scale = np.float32(desc.softmax_scale)
    out = np.zeros((C, Hq, D), np.float32)
    m_out = np.full((C, Hq), -np.inf, np.float32)
    l_out = np.zeros((C, Hq), np.float32)
    for h in range(Hq):
        kvh = h // G
        s = (qn[:, h, :].astype(np.float32) @ K[:, kvh, :].astype(np.float32).T) * scale
        s = np.where(attend, s, -np.inf).astype(np.float32)
        m = s.max(axis=1)
        m_safe = np.where(np.isfinite(m), m, 0.0).astype(np.float32)
        p = np.exp(s - m_safe[:, None]).astype(np.float32)
        p = np.where(attend, p, np.float32(0.0))
        l = p.sum(axis=1, dtype=np.float32)
        o = p @ V[:, kvh, :].astype(np.float32)
        m_out[:, h] = m
        l_out[:, h] = l
        if return_partial:
            out[:, h, :] = o
        else:
            out[:, h, :] = np.where(l[:, None] > 0, o / np.where(l > 0, l, 1.0)[:, None], 0.0)
    if return_partial:
        return out, m_out, l_out
    return out


def merge_partials(parts):
    """Log-sum-exp merge of [(O_unnorm, m, l), ...] -> normalised O.  Shards that saw
    no visible key carry m=-inf, l=0, O=0 and drop out without producing NaN."""
    m_g = parts[0][1].copy()
    for _, m, _ in parts[1:]:
        m_g = np.maximum(m_g, m)
    m_safe = np.where(np.isfinite(m_g), m_g, 0.0).astype(np.float32)
    o_acc = np.zeros_like(parts[0][0])
    l_acc = np.zeros_like(parts[0][2])
    for o, m, l in parts:
        w = np.where(np.isfinite(m), np.exp(m - m_safe), 0.0).astype(np.float32)
        o_acc += o * w[..., None]
        l_acc += l * w
    return np.where(l_acc[..., None] > 0, o_acc / np.where(l_acc > 0, l_acc, 1.0)[..., None], 0.0).astype(np.float32)


def attention_blocked(qn, K, V, attend, desc: LayerDesc, block: int):
    """Key-blocked online softmax (state carried as (m, l, O)); equals `attention`."""
    C = qn.shape[0]
    T = K.shape[0]
    parts = []
    for b0 in range(0, T, block):
        sub = np.zeros_like(attend)
        sub[:, b0:b0 + block] = attend[:, b0:b0 + block]
        parts.append(attention(qn, K, V, sub, desc, return_partial=True))
    return merge_partials(parts)


def denoise_attention(q, k, v, k_prefix, v_prefix, desc: LayerDesc, kv_len: int,
                      qw=None, kw=None, attend=None):
    """Whole hot path for one canvas: qk_rope_kv, append, masked GQA attention.
    k_prefix/v_prefix: [kv_len,Hkv,D] exactly as stored in the cache (bf16-representable)."""
    qn, kn, vn = qk_rope_kv(q, k, v, qw, kw, desc, kv_len)
    K = np.concatenate([k_prefix[:kv_len], kn], axis=0)
    V = np.concatenate([v_prefix[:kv_len], vn], axis=0)
    if attend is None:
        attend = visibility(desc, kv_len)
    return attention(qn, K, V, attend, desc)


# ----------------------------------------------------------------------------
# top-k sparse attention (src/shaders/attn/attention_topk/cpu.rs:39-120 of the reference)
# ----------------------------------------------------------------------------
def topk_k(n_valid: int, k_fixed: int = 0, k_div: int = 128, k_min: int = 64, k_max: int = 512) -> int:
    """Keys kept for a row with n_valid visible keys: the kv-adaptive rule of
    src/shaders/attn/attention_topk/attention_topk.metal:176-185 (k = clamp(n / k_div, k_min, k_max)) or a
    fixed k when k_div == 0; never more than n_valid."""
    k_req = int(np.clip(n_valid // k_div, k_min, k_max)) if k_div else max(int(k_fixed), 1)
    return min(k_req, n_valid)


def attention_topk(qn, K, V, attend, desc: LayerDesc, k_fixed: int = 0, k_div: int = 128, k_min: int = 64,
                   k_max: int = 512, return_gap: bool = False):
    """Per (row, head): scores over the visible keys, the top k by (score descending, index ascending)
    (cpu.rs:84-95), softmax renormalised over those (cpu.rs:96-106), O = sum p_j V[idx_j] (cpu.rs:107-115).
    qn: [C,Hq,D] normed+roped queries, K/V: [T,Hkv,D] as stored, attend: [C,T] bool.
    With return_gap also [C,Hq]: how far the last kept score lies above the first dropped one, relative to its
    magnitude (inf when every visible key is kept) - a row whose gap is within fp32 summation noise has no unique
    top-k set, and an implementation that sums the dot products in another order may keep the other key."""
    C, Hq, D = qn.shape
    G = Hq // desc.n_kv_heads
    out = np.zeros((C, Hq, D), np.float32)
    gap = np.full((C, Hq), np.inf, np.float32)
    scale = np.float32(desc.softmax_scale)
    for h in range(Hq):
        kvh = h // G
        s_all = (qn[:, h, :].astype(np.float32) @ K[:, kvh, :].astype(np.float32).T).astype(np.float32)   # [C, T]
        for i in range(C):
            vis = np.nonzero(attend[i])[0]
            k = topk_k(len(vis), k_fixed, k_div, k_min, k_max)
            if k == 0:
                continue
            sc = s_all[i, vis]
            full = np.argsort(-sc, kind="stable")               # equal scores: lower index first
            order = full[:k]
            if k < len(vis):
                gap[i, h] = (sc[full[k - 1]] - sc[full[k]]) / max(abs(float(sc[full[k - 1]])), 1e-30)
            idx, s = vis[order], sc[order] * scale
            p = np.exp(s - s.max()).astype(np.float32)
            out[i, h] = (p[:, None] * V[idx, kvh, :].astype(np.float32)).sum(axis=0) / p.sum()
    return (out, gap) if return_gap else out


TOPK_TIE_GAP = 5e-6      # relative score gap below which two fp32 summation orders may rank two keys differently


def topk_errors(got, ref, gap):
    """(max-abs over the (row, head) pairs whose kept set is unique, mean-abs over everything, share of pairs
    whose kept set is not unique).  A pair counts as not unique when its last kept and first dropped scores lie
    within TOPK_TIE_GAP of each other: either key may then be kept, and the outputs differ by that key's weight
    times the difference of two value rows (the reference's own GPU-vs-CPU test says the same of its kernels:
    src/shaders/attn/attention_topk/mod.rs:495-510)."""
    err = np.abs(np.asarray(got, np.float32) - ref)
    unique = gap >= TOPK_TIE_GAP
    mx = float(err[unique].max()) if unique.any() else 0.0
    return mx, float(err.mean()), float(1.0 - unique.mean())


def denoise_attention_topk(q, k, v, k_prefix, v_prefix, desc: LayerDesc, kv_len: int, qw=None, kw=None, **kcfg):
    """The hot path with the top-k stage 2: qk_rope_kv, append, top-k attention."""
    qn, kn, vn = qk_rope_kv(q, k, v, qw, kw, desc, kv_len)
    K = np.concatenate([k_prefix[:kv_len], kn], axis=0)
    V = np.concatenate([v_prefix[:kv_len], vn], axis=0)
    return attention_topk(qn, K, V, visibility(desc, kv_len), desc, **kcfg)


# ----------------------------------------------------------------------------
# the neighbours of the attention stage: input norm, stacked Q|K|V projection, output projection,
# post-attention norm + residual (src/metal/step_kernel/enc.rs:852-911, 1560-1629 of the reference)
# ----------------------------------------------------------------------------
def rms_norm_rows(x: np.ndarray, w: np.ndarray | None, eps: float = 1e-6) -> np.ndarray:
    """Row-wise RMS norm of the reference's activation planes
    (src/shaders/elementwise/rms_norm_rows/rms_norm_rows_tiled.metal:16-78): f32 sum of squares,
    inv = rsqrt(sum / dim + 1e-6), y = (x * inv) * w.  Not rounded here."""
    x = x.astype(np.float32)
    ss = np.sum(x.astype(np.float64) ** 2, axis=-1, keepdims=True)
    inv = (1.0 / np.sqrt(ss / x.shape[-1] + eps)).astype(np.float32)
    y = x * inv
    if w is not None:
        y = y * w.astype(np.float32)
    return y.astype(np.float32)


def linear_bf16(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """x [M,K] . w[N,K]^T on bf16-representable inputs, accumulated exactly, rounded once to bf16 (the
    reference's bf16 GEMMs accumulate in f32 and store to the bf16 arena)."""
    return round_bf16((x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32))


def attn_block(hidden, input_ln, w_qkv, qw, kw, w_o, post_ln, k_prefix, v_prefix, desc: LayerDesc, kv_len: int,
               v_from_k: bool = False):
    """One layer's attention block for the canvas rows of a step (enc.rs:852-911):
    stream = hidden + rms_norm(o_proj(attention(qkv_proj(rms_norm(hidden))))), every stored intermediate
    rounded to bf16.  hidden: [C, H]; w_qkv: [n_q*D + n_kv*D (+ n_kv*D), H]; w_o: [H, n_q*D]."""
    C, D = desc.canvas, desc.head_dim
    nq, nk = desc.n_q_heads * D, desc.n_kv_heads * D
    xn = round_bf16(rms_norm_rows(hidden, input_ln))
    qkv = linear_bf16(xn, w_qkv)
    q = qkv[:, :nq].reshape(C, desc.n_q_heads, D)
    k = qkv[:, nq:nq + nk].reshape(C, desc.n_kv_heads, D)
    v = k if v_from_k else qkv[:, nq + nk:nq + 2 * nk].reshape(C, desc.n_kv_heads, D)
    o = round_bf16(denoise_attention(q, k, v, k_prefix, v_prefix, desc, kv_len, qw, kw))
    t = linear_bf16(o.reshape(C, nq), w_o)
    tn = round_bf16(rms_norm_rows(t, post_ln))
    return round_bf16(hidden.astype(np.float32) + tn)


def algorithmic_flops(desc: LayerDesc, kv_len: int) -> float:
    """4*D flops per visible (row, q-head, key) triple."""
    vis = visibility(desc, kv_len).sum()
    return 4.0 * desc.head_dim * desc.n_q_heads * float(vis)
