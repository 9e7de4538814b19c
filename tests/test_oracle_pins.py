"""Pins the CPU oracle to every known-answer value and property the reference's own tests hold for
the canvas-attention path (paths are relative to the reference project)."""
import math

import numpy as np
import pytest

from oracle import attn_oracle as ao
from oracle import c_oracle as co


# --- src/shaders/cpu/mod.rs:304-313 (rms_norm_golden)
def test_rms_norm_golden():
    out = ao.rms_norm_heads(np.array([1, 2, 3, 4], np.float32), np.ones(4, np.float32), 1e-6)
    np.testing.assert_allclose(out, [0.36514835, 0.7302967, 1.0954450, 1.4605934], atol=1e-5)


# --- src/shaders/cpu/mod.rs:316-337 (default_rope_golden): hd=4, theta 1e4, pos 1
def test_rope_golden():
    cos, sin = ao.rope_tables(np.array([1]), 4, 4, 1e4)
    np.testing.assert_allclose([cos[0, 0], sin[0, 0], cos[0, 1], sin[0, 1]],
                               [0.5403023, 0.84147096, 0.99995, 0.01], atol=1e-5)
    v = ao.apply_rope(np.array([[[1.0, 0.0, 0.0, 1.0]]], np.float32), cos, sin, 4)
    np.testing.assert_allclose(v[0, 0], [0.5403023, -0.01, 0.84147096, 0.99995], atol=1e-4)


# --- src/shaders/attn/cpu.rs:203-209 (identity at position 0)
def test_rope_identity_at_zero():
    cos, sin = ao.rope_tables(np.array([0]), 4, 4, 1e4)
    v = ao.apply_rope(np.array([[[1.0, 0.0, 2.0, 0.0]]], np.float32), cos, sin, 4)
    np.testing.assert_allclose(v[0, 0], [1, 0, 2, 0], atol=1e-5)


# --- src/shaders/attn/cpu.rs:211-220 and src/shaders/cpu/mod.rs:363-381 (proportional / partial rotary)
def test_proportional_rope_pairs_across_halves():
    hd = 8
    v0 = (np.arange(hd) * 0.1).astype(np.float32)
    cos, sin = ao.rope_tables(np.array([1]), 4, hd, 1e6)
    v = ao.apply_rope(v0[None, None, :], cos, sin, 4, ao.ROPE_PROPORTIONAL)[0, 0]
    assert abs(v[0] - v0[0]) > 1e-6 or abs(v[4] - v0[4]) > 1e-6
    assert abs(v[2] - v0[2]) < 1e-6 and abs(v[6] - v0[6]) < 1e-6   # dims outside the rotated pairs
    assert abs(v[3] - v0[3]) < 1e-6 and abs(v[7] - v0[7]) < 1e-6


def test_partial_rotary_leaves_other_dims():
    # rotary_dim=4 on head_dim=6 with proportional pairing: pairs (0,3) and (1,4); 2 and 5 untouched
    cos, sin = ao.rope_tables(np.array([1]), 4, 4, 1e4)
    v = ao.apply_rope(np.array([[[1, 2, 3, 4, 5, 6]]], np.float32), cos, sin, 4, ao.ROPE_PROPORTIONAL)[0, 0]
    assert abs(v[2] - 3) < 1e-6 and abs(v[5] - 6) < 1e-6
    assert abs(v[0] - 1) > 1e-6 or abs(v[3] - 4) > 1e-6


def test_proportional_freqs_differ_from_default():
    a = ao.rope_inv_freq(4, 4, 1e6)
    b = ao.rope_inv_freq(4, 8, 1e6)
    assert abs(math.cos(a[1]) - math.cos(b[1])) > 1e-4 or abs(a[1] - b[1]) > 1e-4


# --- inverse frequencies: f32 power, identical in both oracles
@pytest.mark.parametrize("theta", [1e4, 1e6])
def test_inv_freq_twin_agrees(theta):
    np.testing.assert_array_equal(ao.rope_inv_freq(256, 256, theta), co.rope_inv_freq(256, 256, theta))


# --- src/shaders/cpu/mod.rs:390-398 (softmax rows sum to one) through the attention weights
def test_softmax_rows_sum_to_one():
    d = ao.LayerDesc(n_q_heads=2, n_kv_heads=1, head_dim=8, canvas=3, rotary_dim=8, softmax_scale=1.0)
    rng = np.random.default_rng(0)
    qn = rng.standard_normal((3, 2, 8)).astype(np.float32)
    K = rng.standard_normal((7, 1, 8)).astype(np.float32)
    V = np.ones((7, 1, 8), np.float32)
    out = ao.attention(qn, K, V, np.ones((3, 7), bool), d)
    np.testing.assert_allclose(out, 1.0, atol=1e-5)   # sum_t p_t * 1 == 1


# --- src/model/mask.rs:33-43 (all-valid mask is bidirectional over the canvas)
def test_all_valid_mask_bidirectional():
    d = ao.LayerDesc(canvas=4)
    m = ao.visibility(d, 3)
    assert m.shape == (4, 7) and m.all()
    assert m[0, 6] and m[3, 3] and m[2, 1]


# --- src/shaders/attn/attention/attention.metal:52-63 (denoise window rule, uniform over rows)
@pytest.mark.parametrize("kv_len,window", [(10, 4), (3, 8), (7, 8), (8, 8), (9, 8), (100, 1)])
def test_uniform_window_rule(kv_len, window):
    d = ao.LayerDesc(canvas=5, window=window, mask_mode=ao.MASK_WINDOW_UNIFORM)
    m = ao.visibility(d, kv_len)
    t_lo = max(0, kv_len - (window - 1))
    for r in range(5):
        for t in range(kv_len + 5):
            assert m[r, t] == (t >= t_lo), (r, t)
    np.testing.assert_array_equal(m, co.visibility(d, kv_len))


# --- per-row rule of the benchmark's sliding configuration: query at p sees prefix [p-(W-1), p]
@pytest.mark.parametrize("kv_len,window", [(10, 4), (3, 8), (300, 128)])
def test_per_row_window_rule(kv_len, window):
    d = ao.LayerDesc(canvas=6, window=window, mask_mode=ao.MASK_WINDOW_PER_ROW)
    m = ao.visibility(d, kv_len)
    for r in range(6):
        p = kv_len + r
        for t in range(kv_len + 6):
            want = True if t >= kv_len else (t >= max(0, p - (window - 1)))
            assert m[r, t] == want, (r, t)
    np.testing.assert_array_equal(m, co.visibility(d, kv_len))


# --- src/model/attention.rs:1042-1058: window=2 blocks the distant past (prefill form of the rule)
def test_window_two_blocks_distant_past():
    d = ao.LayerDesc(canvas=1, window=2, mask_mode=ao.MASK_WINDOW_PER_ROW)
    m = ao.visibility(d, 2)   # query at position 2 sees prefix key 1 only (+ itself)
    assert list(m[0]) == [False, True, True]


# --- the same Rust test as a whole 3 x 3 causal sliding mask (kv_len = 0, three tokens, window 2):
# the future and the distant past are both hidden
def test_causal_sliding_mask_blocks_future_and_distant_past():
    d = ao.LayerDesc(canvas=3, window=2, mask_mode=ao.MASK_CAUSAL)
    m = ao.visibility(d, 0)
    assert m.tolist() == [[True, False, False], [True, True, False], [False, True, True]]
    np.testing.assert_array_equal(m, co.visibility(d, 0))
    # without a window the causal mode is the plain lower triangle over [prefix | canvas]
    d = ao.LayerDesc(canvas=4, window=0, mask_mode=ao.MASK_CAUSAL)
    m = ao.visibility(d, 3)
    for r in range(4):
        assert m[r].tolist() == [t <= 3 + r for t in range(7)]
    np.testing.assert_array_equal(m, co.visibility(d, 3))


# --- src/shaders/attn/attention_flash/mod_tests.rs:21-36: blocked online softmax == single pass
@pytest.mark.parametrize("block", [1, 3, 8, 16, 64, 4096])
def test_blocked_equals_single_pass(block):
    d = ao.LayerDesc(n_q_heads=4, n_kv_heads=2, head_dim=32, canvas=5, rotary_dim=32, softmax_scale=1.0)
    rng = np.random.default_rng(block)
    qn = rng.standard_normal((5, 4, 32)).astype(np.float32)
    K = rng.standard_normal((70, 2, 32)).astype(np.float32)
    V = rng.standard_normal((70, 2, 32)).astype(np.float32)
    att = ao.visibility(d, 65)
    np.testing.assert_allclose(ao.attention_blocked(qn, K, V, att, d, block), ao.attention(qn, K, V, att, d), atol=1e-3)


def _scalar_online_attention(q, kv_k, kv_v, n_groups, scale=1.0):
    """Key-at-a-time online softmax, the shape of src/shaders/attn/cpu.rs:148-197 (all-valid)."""
    C, Hq, D = q.shape
    T = kv_k.shape[0]
    out = np.zeros_like(q)
    for tok in range(C):
        for qh in range(Hq):
            kvh = qh // n_groups
            m, l, acc = -np.inf, np.float32(0), np.zeros(D, np.float32)
            for t in range(T):
                dt = np.float32(np.dot(q[tok, qh], kv_k[t, kvh])) * np.float32(scale)
                mn = max(m, dt)
                corr = np.float32(math.exp(m - mn)) if np.isfinite(m) else np.float32(0)
                p = np.float32(math.exp(dt - mn))
                acc = acc * corr + p * kv_v[t, kvh]
                l = l * corr + p
                m = mn
            out[tok, qh] = acc / l
    return out


def _ref_fixture(canvas, hq, hkv, hd, kv_len, kind):
    """Closed-form inputs of the reference's attention fixtures
    (src/shaders/attn/attention/mod.rs:59-184)."""
    T = kv_len + canvas
    t, h, dd = np.meshgrid(np.arange(T), np.arange(hkv), np.arange(hd), indexing="ij")
    if kind == "tiny":
        K = np.sin((t * 17 + h * 3 + dd).astype(np.float32) * np.float32(0.05))
        V = np.cos((t * 13 + h * 5 + dd).astype(np.float32) * np.float32(0.04))
        i = np.arange(canvas * hq * hd, dtype=np.float32)
        q = np.sin(i * np.float32(0.11)) * np.float32(0.6)
    elif kind == "wide":
        idx = (t * hkv * hd * 2 + h * hd + dd).astype(np.float32)
        K = np.sin(idx * np.float32(0.031)) * np.float32(0.3)
        V = np.sin((idx + hkv * hd) * np.float32(0.031)) * np.float32(0.3)
        i = np.arange(canvas * hq * hd, dtype=np.float32)
        q = np.cos(i * np.float32(0.02)) * np.float32(0.5)
    else:  # model_attn_fixture
        K = np.sin((t * 19 + h * 7 + dd).astype(np.float32) * np.float32(0.0031)) * np.float32(0.4)
        V = np.cos((t * 23 + h * 11 + dd).astype(np.float32) * np.float32(0.0027)) * np.float32(0.35)
        i = np.arange(canvas * hq * hd)
        q = np.sin(i.astype(np.float32) * np.float32(0.017)) * np.float32(0.5) + np.float32(0.02) * (i % hd).astype(np.float32)
    return (ao.round_bf16(q.astype(np.float32).reshape(canvas, hq, hd)),
            ao.round_bf16(K.astype(np.float32)), ao.round_bf16(V.astype(np.float32)))


REF_FIXTURES = {
    "tiny": (2, 4, 2, 32, 2, "tiny"),
    "wide": (4, 8, 2, 64, 4, "wide"),
    "full_hd512": (4, 16, 8, 512, 28, "model"),
    "full_grp8_hd512": (16, 16, 2, 512, 28, "model"),
    "sliding_hd256": (4, 16, 8, 256, 128, "model"),
}


@pytest.mark.parametrize("name", ["tiny", "wide", "sliding_hd256"])
def test_reference_fixtures_vs_scalar_online(name):
    canvas, hq, hkv, hd, kv_len, kind = REF_FIXTURES[name]
    q, K, V = _ref_fixture(canvas, hq, hkv, hd, kv_len, kind)
    d = ao.LayerDesc(n_q_heads=hq, n_kv_heads=hkv, head_dim=hd, canvas=canvas, rotary_dim=hd, softmax_scale=1.0)
    want = _scalar_online_attention(q, K, V, hq // hkv)
    got = ao.attention(q, K, V, ao.visibility(d, kv_len), d)
    np.testing.assert_allclose(got, want, atol=2e-5)


def test_golden_vectors_match():
    """Committed vectors (tests/golden/attn_golden.npz, made by tests/golden/make_golden.py)."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "attn_golden.npz"))
    for name, (canvas, hq, hkv, hd, kv_len, kind) in REF_FIXTURES.items():
        q, K, V = _ref_fixture(canvas, hq, hkv, hd, kv_len, kind)
        d = ao.LayerDesc(n_q_heads=hq, n_kv_heads=hkv, head_dim=hd, canvas=canvas, rotary_dim=hd, softmax_scale=1.0)
        got = ao.attention(q, K, V, ao.visibility(d, kv_len), d)
        np.testing.assert_allclose(got, g[name], atol=1e-5, err_msg=name)


# --- C++ twin == numpy oracle (<= 1e-5 on identical normed inputs; prologue within one bf16 ulp)
@pytest.mark.parametrize("P,Hkv,W,mode,scale", [(300, 8, 0, 0, 1 / 16), (700, 2, 128, 1, 1.0), (700, 8, 128, 2, 1 / 16)])
def test_c_twin_matches_numpy(P, Hkv, W, mode, scale):
    d = ao.LayerDesc(n_kv_heads=Hkv, window=W, mask_mode=mode, softmax_scale=scale, rope_theta=1e4, v_norm=1)
    rng = np.random.default_rng(P)
    C, Hq, D = d.canvas, d.n_q_heads, d.head_dim
    B = ao.f32_to_bf16_bits
    q = ao.round_bf16(rng.standard_normal((C, Hq, D)).astype(np.float32))
    k = ao.round_bf16(rng.standard_normal((C, Hkv, D)).astype(np.float32))
    v = ao.round_bf16(rng.standard_normal((C, Hkv, D)).astype(np.float32))
    kp = ao.prepare_prefix_k(ao.round_bf16(rng.standard_normal((P, Hkv, D)).astype(np.float32)), d)
    vp = ao.round_bf16(rng.standard_normal((P, Hkv, D)).astype(np.float32))
    qn, kn, vn = ao.qk_rope_kv(q, k, v, None, None, d, P)
    cq, ck, cv = co.qk_rope_kv(d, P, B(q), B(k), B(v))
    for a, b in ((qn, cq), (kn, ck), (vn, cv)):
        bits = B(a).astype(np.int32)
        ulp_off = np.abs(bits - b.astype(np.int32))
        near_zero = np.abs(a - ao.bf16_bits_to_f32(b)) <= 1e-6       # cancellation in x0*c - x1*s
        assert ((ulp_off <= 1) | near_zero).all()                    # one bf16 ulp at most
        assert (bits != b).mean() < 1e-3
    ref = ao.attention(qn, np.concatenate([kp, kn]), np.concatenate([vp, vn]), ao.visibility(d, P), d)
    got = co.attention(d, P, B(qn), B(kn), B(vn), B(kp), B(vp))
    assert np.abs(got - ref).max() <= 1e-5
    # split partials merge back to the single-pass result
    parts = [co.attention(d, P, B(qn), B(kn), B(vn), B(kp), B(vp), t0=0, t1=P // 2, include_canvas=False, partial=True),
             co.attention(d, P, B(qn), B(kn), B(vn), B(kp), B(vp), t0=P // 2, t1=P, include_canvas=True, partial=True)]
    assert np.abs(ao.merge_partials(parts) - ref).max() <= 1e-5


def test_fully_masked_rows_give_zero_and_merge_without_nan():
    d = ao.LayerDesc(n_q_heads=2, n_kv_heads=1, head_dim=8, canvas=3, rotary_dim=8)
    rng = np.random.default_rng(5)
    qn = rng.standard_normal((3, 2, 8)).astype(np.float32)
    K = rng.standard_normal((8, 1, 8)).astype(np.float32)
    V = rng.standard_normal((8, 1, 8)).astype(np.float32)
    att = np.ones((3, 8), bool)
    att[1, :] = False
    out = ao.attention(qn, K, V, att, d)
    assert np.isfinite(out).all() and np.all(out[1] == 0)
    empty = ao.attention(qn, K, V, np.zeros((3, 8), bool), d, return_partial=True)
    full = ao.attention(qn, K, V, att, d, return_partial=True)
    merged = ao.merge_partials([empty, full])
    assert np.isfinite(merged).all()
    np.testing.assert_allclose(merged, out, atol=1e-6)


def test_decoder_bitmap_sparse_fixture_properties():
    """Shape of the reference's sparse decoder bitmap test
    (src/shaders/attn/gqa_attention/mod.rs:181-232): masked canvas keys where (q+k)%5==0 and rows
    q%7==0 that see no prefix.  Checked against the scalar key-at-a-time form."""
    canvas, kvc, hq, hkv, hd = 8, 14, 4, 2, 16
    T = kvc + canvas

    def fill(n, seed):
        i = np.arange(n, dtype=np.float32)
        return (np.sin(i * np.float32(seed)) * np.float32(0.29) + np.cos(i * np.float32(seed * 0.61)) * np.float32(0.17)).astype(np.float32)

    q = fill(canvas * hq * hd, 0.018).reshape(canvas, hq, hd)
    K = fill(T * hkv * hd, 0.015).reshape(T, hkv, hd)
    V = fill(T * hkv * hd, 0.015 * 1.3).reshape(T, hkv, hd)
    att = np.ones((canvas, T), bool)
    for qi in range(canvas):
        for k in range(kvc, T):
            if (qi + k) % 5 == 0:
                att[qi, k] = False
        if qi % 7 == 0:
            att[qi, :kvc] = False
    d = ao.LayerDesc(n_q_heads=hq, n_kv_heads=hkv, head_dim=hd, canvas=canvas, rotary_dim=hd, softmax_scale=1.0)
    got = ao.attention(q, K, V, att, d)
    # scalar form with -1e9 additive mask, like src/model/attention.rs:889-907
    for qi in range(canvas):
        for h in range(hq):
            s = K[:, h // 2, :] @ q[qi, h]
            s = np.where(att[qi], s, -1e9)
            p = np.exp(s - s.max())
            p /= p.sum()
            np.testing.assert_allclose(got[qi, h], p @ V[:, h // 2, :], atol=1e-5)


# --- the append kernels fold the K norm into the rotation: fma(x, w cos, x_partner (-/+ w_partner sin)) inv instead of
# the reference's (x inv w) rotated afterwards (src/shaders/attn/qk_rope_kv/qk_rope_kv.metal:58-149).  Restated here
# in fp32 (an fma = the exactly computed product-sum rounded once, taken through float64) the two orders must give
# the same bf16 value except where the exact result lies at a rounding boundary, and never differ by more than one
# bf16 step there.
def test_folded_k_rotation_matches_reference_order():
    rng = np.random.default_rng(11)
    C, H, D = 64, 4, 256
    half = D // 2
    x = ao.round_bf16(rng.standard_normal((C, H, D)).astype(np.float32))
    w = ao.round_bf16((1 + 0.1 * rng.standard_normal(D)).astype(np.float32))
    cos, sin = ao.rope_tables(np.arange(16384, 16384 + C), D, D, 1e4)
    ref = ao.round_bf16(ao.apply_rope(ao.rms_norm_heads(x, w, 1e-6), cos, sin, D))

    f32 = np.float32
    ss = np.sum(x * x, axis=-1, keepdims=True, dtype=np.float32)
    inv = (f32(1.0) / np.sqrt(ss / f32(D) + f32(1e-6))).astype(f32)
    c, s = cos[:, None, :], sin[:, None, :]
    x0, x1, w0, w1 = x[..., :half], x[..., half:], w[:half], w[half:]

    def fma(a, b, cc):
        return (a.astype(np.float64) * b.astype(np.float64) + cc.astype(np.float64)).astype(f32)

    lo = (fma(x0, (w0 * c).astype(f32), (x1 * (-(w1 * s).astype(f32))).astype(f32)) * inv).astype(f32)
    hi = (fma(x1, (w1 * c).astype(f32), (x0 * (w0 * s).astype(f32)).astype(f32)) * inv).astype(f32)
    got = ao.round_bf16(np.concatenate([lo, hi], axis=-1))

    differ = got != ref
    assert differ.mean() < 0.02, differ.mean()
    step = np.maximum(np.abs(ref), 2.0 ** -20) * 2.0 ** -7        # one bf16 step at the value's magnitude, at most
    assert np.all(np.abs(got - ref)[differ] <= step[differ])
