"""The CPU restatement of the attention block's neighbours (input norm, stacked Q|K|V projection, output
projection, post-attention norm + residual), pinned to the reference's known answers and checked for the
properties its composition must have (paths are relative to the reference project)."""
import numpy as np

from oracle import attn_oracle as ao


# --- src/shaders/elementwise/rms_norm_rows/mod.rs:34-42, 311-328 (tiny_fixture, golden_row_values)
def test_rms_norm_rows_golden():
    x = np.array([[1.0, 2.0, 3.0, 4.0], [-1.0, 0.5, 2.0, -0.5]], np.float32)
    w = np.array([1.0, 0.5, 2.0, 1.5], np.float32)
    out = ao.rms_norm_rows(x, w, 1e-6)
    np.testing.assert_allclose(out.ravel(), [0.36514835, 0.36514835, 2.19089, 2.19089,
                                             -0.8528026, 0.21320064, 3.4112102, -0.6396019], atol=1e-4)


# --- src/shaders/cpu/mod.rs:24-45: the unscaled normalise, then the per-lane weight
def test_rms_norm_rows_is_the_head_norm_of_the_same_row():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 64)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(64)).astype(np.float32)
    np.testing.assert_allclose(ao.rms_norm_rows(x, w), ao.rms_norm_heads(x, w, 1e-6), rtol=2e-6, atol=1e-6)
    np.testing.assert_allclose(ao.rms_norm_rows(x, None), ao.rms_norm_heads(x, None, 1e-6), rtol=2e-6, atol=1e-6)


# --- src/shaders/cpu/mod.rs:80-100 (linear: y = x @ W^T, PyTorch weight layout)
def test_linear_layout_and_rounding():
    x = np.array([[1.0, 2.0], [0.5, -1.0]], np.float32)
    w = np.array([[1.0, 0.0], [0.0, 1.0], [2.0, 3.0]], np.float32)
    np.testing.assert_array_equal(ao.linear_bf16(x, w), [[1.0, 2.0, 8.0], [0.5, -1.0, -2.0]])
    # one rounding to bf16 at the store
    y = ao.linear_bf16(np.array([[1.0, 1.0]], np.float32), np.array([[1.0, 2.0 ** -9]], np.float32))
    assert y[0, 0] == 1.0


def _tiny_block(w_o_scale, v_from_k=False):
    rng = np.random.default_rng(11)
    d = ao.LayerDesc(4, 2, 16, 6, 16, 1e4, 1e-6, 0.25, 0, ao.MASK_NONE, 1, ao.ROPE_SPLIT_HALF)
    H, P = 32, 9
    nq, nk = d.n_q_heads * d.head_dim, d.n_kv_heads * d.head_dim
    r = lambda *s: ao.round_bf16(rng.standard_normal(s).astype(np.float32))
    hidden = r(d.canvas, H)
    w_qkv = ao.round_bf16(r(nq + nk * (1 if v_from_k else 2), H) / np.sqrt(H))
    w_o = ao.round_bf16(w_o_scale * r(H, nq) / np.sqrt(nq))
    kp, vp = r(P, d.n_kv_heads, d.head_dim), r(P, d.n_kv_heads, d.head_dim)
    ln = ao.round_bf16(1 + 0.1 * rng.standard_normal(H).astype(np.float32))
    return d, hidden, ln, w_qkv, w_o, kp, vp, P


# enc.rs:888-911: with a zero output projection the normed term is zero and the residual passes through
def test_block_with_zero_output_projection_is_the_identity():
    d, hidden, ln, w_qkv, w_o, kp, vp, P = _tiny_block(0.0)
    out = ao.attn_block(hidden, ln, w_qkv, None, None, w_o, ln, kp, vp, d, P)
    np.testing.assert_array_equal(out, hidden)


# enc.rs:852-911: the block is the composition of its stages with a bf16 store between them
def test_block_is_the_composition_of_its_stages():
    for v_from_k in (False, True):
        d, hidden, ln, w_qkv, w_o, kp, vp, P = _tiny_block(1.0, v_from_k)
        nq, nk = d.n_q_heads * d.head_dim, d.n_kv_heads * d.head_dim
        xn = ao.round_bf16(ao.rms_norm_rows(hidden, ln))
        q = ao.linear_bf16(xn, w_qkv[:nq]).reshape(d.canvas, d.n_q_heads, d.head_dim)
        k = ao.linear_bf16(xn, w_qkv[nq:nq + nk]).reshape(d.canvas, d.n_kv_heads, d.head_dim)
        v = k if v_from_k else ao.linear_bf16(xn, w_qkv[nq + nk:]).reshape(d.canvas, d.n_kv_heads, d.head_dim)
        o = ao.round_bf16(ao.denoise_attention(q, k, v, kp, vp, d, P))
        t = ao.linear_bf16(o.reshape(d.canvas, nq), w_o)
        ref = ao.round_bf16(hidden + ao.round_bf16(ao.rms_norm_rows(t, None)))
        out = ao.attn_block(hidden, ln, w_qkv, None, None, w_o, None, kp, vp, d, P, v_from_k=v_from_k)
        np.testing.assert_array_equal(out, ref)
        assert np.abs(out - hidden).max() > 0.1
