"""The numpy oracle held to the reference's OWN shaders.

`oracle/_ref/libdg_ref_shaders.so` is attention.metal and qk_rope_kv.metal of the reference project
compiled as C++ (see oracle/Makefile).  tests/golden/ref_shader_golden.npz holds their outputs on seeded
inputs (generator: tests/golden/make_ref_shader_golden.py), so these pins also hold where the reference
tree is absent; where the compiled library is present the stored vectors are additionally checked
against a live run.

What is pinned: the denoise visibility rule with and without a sliding window, bit for bit
(attention.metal:52-63: t_lo = kv_len - (window - 1), uniform over canvas rows), the causal rule of the
same shader (attention.metal:51,57-62: the committed-block re-prefill), the ring slot mapping
(attention_device.metal:27-33), both RoPE pairings with their rotary extents and thetas and the
V-aliases-raw-K form of full layers (qk_rope_kv.metal:58-101), and the streaming softmax values."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

import make_ref_shader_golden as G  # noqa: E402
from oracle import attn_oracle as ao  # noqa: E402
from oracle import ref_shader as rs  # noqa: E402

GOLD = np.load(os.path.join(ROOT, "tests", "golden", "ref_shader_golden.npz"))


def oracle_desc(hd, n_q, n_kv, canvas, is_full, window, causal=0):
    # what qk_rope_kv.metal:58-60 and attention.metal hard-wire per layer kind
    mode = ao.MASK_CAUSAL if causal else (ao.MASK_WINDOW_UNIFORM if window else ao.MASK_NONE)
    return ao.LayerDesc(n_q_heads=n_q, n_kv_heads=n_kv, head_dim=hd, canvas=canvas,
                        rotary_dim=hd // 4 if is_full else hd, rope_theta=1e6 if is_full else 1e4, rms_eps=1e-6,
                        softmax_scale=1.0, window=window, mask_mode=mode, v_norm=1,
                        rope_pairing=1 if is_full else 0)


@pytest.mark.parametrize("idx", range(len(G.MASK_CASES)))
def test_visibility_rule_matches_the_reference_shader_bit_for_bit(idx):
    kv_len, window, ring = G.MASK_CASES[idx]
    canvas, hd = 16, 256
    d = oracle_desc(hd, 4, 2, canvas, 0, window)
    mine = ao.visibility(d, kv_len)                      # [canvas][kv_len + canvas]
    expect = np.zeros((canvas, hd), bool)
    for t in range(kv_len + canvas):
        expect[:, t % hd] |= mine[:, t]
    # one key per output dimension among the keys the probe stored (the last 300 + canvas)
    assert np.array_equal(GOLD[f"mask{idx}_visible"], expect), (kv_len, window, ring)


@pytest.mark.parametrize("idx", range(len(G.CAUSAL_MASK_CASES)))
def test_causal_rule_matches_the_reference_shader_bit_for_bit(idx):
    """dims.causal = 1 (attention.metal:51,57-62): query kv_len+i sees [kv_len+i-(window-1), kv_len+i]."""
    kv_len, window, ring = G.CAUSAL_MASK_CASES[idx]
    canvas, hd = 16, 256
    d = oracle_desc(hd, 4, 2, canvas, 0, window, causal=1)
    mine = ao.visibility(d, kv_len)
    expect = np.zeros((canvas, hd), bool)
    for t in range(kv_len + canvas):
        expect[:, t % hd] |= mine[:, t]
    assert np.array_equal(GOLD[f"cmask{idx}_visible"], expect), (kv_len, window, ring)
    # the C++ twin evaluates the same rule
    from oracle import c_oracle as co
    assert np.array_equal(co.visibility(d, kv_len), mine)


def ulp_bf16(x):
    return np.maximum(np.abs(x), 2.0 ** -20) * 2.0 ** -7


ALL_VALUE_CASES = {**G.VALUE_CASES, **G.CAUSAL_VALUE_CASES}


@pytest.mark.parametrize("name", list(ALL_VALUE_CASES))
def test_stage1_and_attention_values_match_the_reference_shaders(name):
    hd, n_q, n_kv, canvas, kv_len, is_full, window, ring, valias, seed = ALL_VALUE_CASES[name]
    q, k, v, kp, vp, qw, kw = G.value_inputs(*ALL_VALUE_CASES[name])
    d = oracle_desc(hd, n_q, n_kv, canvas, is_full, window, causal=int(name in G.CAUSAL_VALUE_CASES))
    qn, kn, vn = ao.qk_rope_kv(q, k, k if valias else v, qw, kw, d, kv_len)
    # stage 1: the shader truncates Q to bf16 and keeps K / V in f16; the oracle rounds all three to bf16
    assert (np.abs(qn - GOLD[f"{name}_q_out"]) <= 2.0 * ulp_bf16(qn) + 1e-6).all()
    assert (np.abs(kn - GOLD[f"{name}_k_cache"]) <= 1.5 * ulp_bf16(kn) + 1e-5).all()
    assert (np.abs(vn - GOLD[f"{name}_v_cache"]) <= 1.5 * ulp_bf16(vn) + 1e-5).all()
    # whole path
    out = ao.denoise_attention(q, k, k if valias else v, kp, vp, d, kv_len, qw, kw)
    ref = GOLD[f"{name}_out"]
    # the shader TRUNCATES its output to bf16 (arena.metal:13-15): up to one bf16 ulp of the difference is its
    # own quantisation; what remains is held to the gate the GPU path is held to
    err = np.maximum(np.abs(out - ref) - ulp_bf16(ref), 0.0)
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (name, float(err.max()), float(err.mean()))


def test_wrong_rules_would_be_caught():
    """The pins have teeth: a window bound off by one key, or the other RoPE pairing, fails them."""
    kv_len, window, ring = G.MASK_CASES[1]
    d = oracle_desc(256, 4, 2, 16, 0, window + 1)          # one more visible prefix key
    mine = ao.visibility(d, kv_len)
    expect = np.zeros((16, 256), bool)
    for t in range(kv_len + 16):
        expect[:, t % 256] |= mine[:, t]
    assert not np.array_equal(GOLD["mask1_visible"], expect)
    name = "full_hd512_valias"
    hd, n_q, n_kv, canvas, kv_len, is_full, window, ring, valias, seed = G.VALUE_CASES[name]
    q, k, v, kp, vp, qw, kw = G.value_inputs(*G.VALUE_CASES[name])
    d = oracle_desc(hd, n_q, n_kv, canvas, is_full, window)
    d.rope_pairing = 0                                     # split-half instead of proportional
    qn, _, _ = ao.qk_rope_kv(q, k, k, qw, kw, d, kv_len)
    assert not (np.abs(qn - GOLD[f"{name}_q_out"]) <= 2.0 * ulp_bf16(qn) + 1e-6).all()


@pytest.mark.skipif(not rs.available(), reason="compiled reference shaders not present (built where the reference tree is)")
def test_stored_vectors_equal_a_live_run_of_the_compiled_shaders():
    for i, (kv_len, window, ring) in enumerate(G.MASK_CASES[:6]):
        q, cache = G.mask_inputs(kv_len, window, ring)
        out = rs.attention(q, cache, kv_len, window, 0, ring)
        assert np.array_equal(out[:, 0, :] > 0, GOLD[f"mask{i}_visible"])
    for i, (kv_len, window, ring) in enumerate(G.CAUSAL_MASK_CASES[:4]):
        q, cache = G.mask_inputs(kv_len, window, ring)
        out = rs.attention(q, cache, kv_len, window, 1, ring)
        assert np.array_equal(out[:, 0, :] > 0, GOLD[f"cmask{i}_visible"])
    live = G.run_value_case(*G.CAUSAL_VALUE_CASES["causal_sliding"], causal=1)
    for key, val in live.items():
        assert np.array_equal(val.astype(np.float32), GOLD[f"causal_sliding_{key}"]), key
    for name in ("sliding_short", "full_hd512_valias"):
        live = G.run_value_case(*G.VALUE_CASES[name])
        for key, val in live.items():
            assert np.array_equal(val.astype(np.float32), GOLD[f"{name}_{key}"]), (name, key)
