"""The CPU restatement of the reference's top-k sparse attention, checked for the properties the reference's own
tests hold for it (paths are relative to the reference project)."""
import numpy as np

from oracle import attn_oracle as ao


def _case(seed=5, C=6, Hq=4, Hkv=2, D=16, P=40):
    rng = np.random.default_rng(seed)
    d = ao.LayerDesc(Hq, Hkv, D, C, D, 1e4, 1e-6, 0.25, 0, ao.MASK_NONE, 1, ao.ROPE_SPLIT_HALF)
    r = lambda *s: ao.round_bf16(rng.standard_normal(s).astype(np.float32))
    return d, r(C, Hq, D), r(C, Hkv, D), r(C, Hkv, D), r(P, Hkv, D), r(P, Hkv, D), P


# --- src/shaders/attn/attention_topk/cpu.rs:127-236: top-k with k >= n_valid equals dense attention
def test_topk_with_k_at_least_n_is_dense():
    d, q, k, v, kp, vp, P = _case()
    dense = ao.denoise_attention(q, k, v, kp, vp, d, P)
    for kcfg in (dict(k_fixed=P + d.canvas, k_div=0), dict(k_fixed=10 ** 6, k_div=0), dict(k_div=1, k_min=1, k_max=10 ** 6)):
        np.testing.assert_allclose(ao.denoise_attention_topk(q, k, v, kp, vp, d, P, **kcfg), dense, rtol=1e-5, atol=1e-6)


# --- cpu.rs:84-115: k = 1 returns the value of the best key
def test_top1_returns_the_value_of_the_best_key():
    d, q, k, v, kp, vp, P = _case(seed=6)
    qn, kn, vn = ao.qk_rope_kv(q, k, v, None, None, d, P)
    K, V = np.concatenate([kp, kn]), np.concatenate([vp, vn])
    out = ao.denoise_attention_topk(q, k, v, kp, vp, d, P, k_fixed=1, k_div=0)
    G = d.n_q_heads // d.n_kv_heads
    for i in range(d.canvas):
        for h in range(d.n_q_heads):
            best = int(np.argmax(qn[i, h] @ K[:, h // G].T))
            np.testing.assert_allclose(out[i, h], V[best, h // G], rtol=1e-6)


# --- cpu.rs:15-17, 87-93: equal scores are broken by index, lower first
def test_ties_go_to_the_lower_index():
    d, q, k, v, kp, vp, P = _case(seed=7)
    q = np.zeros_like(q)                              # every score is 0: the first k keys win
    out = ao.denoise_attention_topk(q, k, v, kp, vp, d, P, k_fixed=5, k_div=0)
    G = d.n_q_heads // d.n_kv_heads
    for h in range(d.n_q_heads):
        np.testing.assert_allclose(out[0, h], vp[:5, h // G].mean(axis=0), rtol=1e-5, atol=1e-6)


# --- src/shaders/attn/attention_topk/attention_topk.metal:176-185: the kv-adaptive k
def test_adaptive_k_rule():
    assert ao.topk_k(33024) == 258 and ao.topk_k(100256) == 512 and ao.topk_k(2000) == 64 and ao.topk_k(40) == 40
    assert ao.topk_k(500, k_fixed=64, k_div=0) == 64 and ao.topk_k(10, k_fixed=64, k_div=0) == 10


# a row whose last kept and first dropped scores coincide has no unique kept set: the comparison helper says so
def test_near_tie_rows_are_reported():
    d, q, k, v, kp, vp, P = _case(seed=8)
    qn, kn, vn = ao.qk_rope_kv(q, k, v, None, None, d, P)
    K, V = np.concatenate([kp, kn]), np.concatenate([vp, vn])
    K[3] = K[7]                                         # two identical keys: identical scores
    out, gap = ao.attention_topk(qn, K, V, ao.visibility(d, P), d, k_fixed=5, k_div=0, return_gap=True)
    assert gap.shape == (d.canvas, d.n_q_heads) and (gap >= 0).all()
    mx, mean, ties = ao.topk_errors(out, out, gap)
    assert mx == 0.0 and mean == 0.0 and 0.0 <= ties <= 1.0
