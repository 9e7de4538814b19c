"""dg_attn_denoise_topk (the reference's top-k sparse attention: score GEMM, radix selection, gathered PV) against
the CPU restatement of src/shaders/attn/attention_topk/cpu.rs, through the C ABI."""
import numpy as np
import pytest
import torch

from diffgemma_b200 import capi
from diffgemma_b200.step_attn import AttnLayer, CanvasAttention, Context, KvCache
from oracle import attn_oracle as ao
from tests import util

pytestmark = pytest.mark.gpu


def _run(ctx, case, **kcfg):
    kv, att = util.gpu_setup(ctx, case)
    try:
        out = att.denoise_topk(kv, case["prefix"], util.dev(case, "q"), util.dev(case, "kc"), util.dev(case, "vc"),
                               util.dev(case, "qw"), util.dev(case, "kw"), **kcfg)
        ctx.synchronize()
        return util.t2f(out)
    finally:
        kv.close()


def _oracle(case, **kcfg):
    f = util.t2f
    qw = None if case["qw"] is None else f(case["qw"])
    kw = None if case["kw"] is None else f(case["kw"])
    return ao.denoise_attention_topk(f(case["q"]), f(case["kc"]), f(case["vc"]), f(case["kp"]), f(case["vp"]), case["desc"],
                                     case["prefix"], qw, kw, **kcfg)


CASES = [
    ("global256 adaptive k (64)", dict(n_q_heads=16, n_kv_heads=2, head_dim=256, canvas=256, rope_theta=1e6), 3000, {}),
    ("global256 k=300", dict(n_q_heads=16, n_kv_heads=2, head_dim=256, canvas=256, rope_theta=1e6), 3000,
     dict(k_fixed=300, k_div=0)),
    ("full512, no scale", dict(n_q_heads=16, n_kv_heads=2, head_dim=512, canvas=256, rotary_dim=128, rope_theta=1e6,
                               softmax_scale=1.0, v_norm=1, rope_pairing=capi.ROPE_PROPORTIONAL), 2000, {}),
    ("Hkv 8, ragged canvas, ragged keys", dict(n_q_heads=16, n_kv_heads=8, head_dim=256, canvas=100, rope_theta=1e4), 1111,
     dict(k_div=16, k_min=8, k_max=100)),
    # masked rows: only the window's keys are candidates, and k follows each row's own visible count
    ("sliding window, per row", dict(n_q_heads=16, n_kv_heads=8, head_dim=256, canvas=128, rope_theta=1e4, window=512,
                                     mask_mode=capi.MASK_WINDOW_PER_ROW), 2000, dict(k_div=8, k_min=16, k_max=128)),
    ("causal block", dict(n_q_heads=8, n_kv_heads=2, head_dim=256, canvas=64, rope_theta=1e6, mask_mode=capi.MASK_CAUSAL), 500,
     dict(k_fixed=48, k_div=0)),
]


@pytest.mark.parametrize("name,lk,P,kcfg", CASES, ids=[c[0] for c in CASES])
def test_topk_matches_oracle(ctx, name, lk, P, kcfg):
    layer = AttnLayer(**lk)
    case = util.make_case(layer, P, seed=P, weights=True)
    got = _run(ctx, case, **kcfg)
    ref, gap = _oracle(case, return_gap=True, **kcfg)
    # rows whose k-th and (k+1)-th scores coincide to fp32 summation noise have no unique kept set: they are left
    # out of the max-abs gate (there may only be a handful) and stay inside the mean-abs gate
    mx, mean, ties = ao.topk_errors(got, ref, gap)
    tol = util.max_abs_tol(ref) if layer.softmax_scale == 1.0 else util.MAX_ABS_TOL
    assert mx <= tol and mean <= util.MEAN_ABS_TOL and ties <= 0.02, (name, mx, mean, ties)
    assert ctx.device_status()[0] == 0
    # same bits on a second run: the kept keys are summed in index order
    assert np.array_equal(got, _run(ctx, case, **kcfg))


# src/shaders/attn/attention_topk/cpu.rs:127-236: with k >= the number of visible keys top-k IS dense attention
def test_topk_with_all_keys_is_dense(ctx):
    layer = AttnLayer(n_q_heads=16, n_kv_heads=2, head_dim=256, canvas=256, rope_theta=1e6)
    case = util.make_case(layer, 700, seed=9)
    dense = util.run_gpu(ctx, case)
    got = _run(ctx, case, k_fixed=1024, k_div=0)
    util.assert_close(got, dense, "top-k with k >= n against the dense kernel")
    util.assert_close(got, util.run_oracle(case), "top-k with k >= n against the dense oracle")


# cpu.rs:15-17: identical scores are broken by index.  With Q = 0 every score is 0, every key shares the threshold
# value (the bulk path of the selection) and the first k keys of the row win.
def test_topk_ties_take_the_lowest_indices(ctx):
    layer = AttnLayer(n_q_heads=16, n_kv_heads=2, head_dim=256, canvas=64, rope_theta=1e6)
    case = util.make_case(layer, 3000, seed=10)
    case["q"] = torch.zeros_like(case["q"])
    got = _run(ctx, case, k_fixed=37, k_div=0)
    want = util.t2f(case["vp"])[:37].mean(axis=0)                  # [Hkv, D]
    G = layer.n_q_heads // layer.n_kv_heads
    for h in range(layer.n_q_heads):
        np.testing.assert_allclose(got[:, h], np.broadcast_to(want[h // G], got[:, h].shape), atol=4e-3)


def test_topk_argument_errors(ctx):
    layer = AttnLayer(n_q_heads=16, n_kv_heads=2, head_dim=256, canvas=64, rope_theta=1e6)
    case = util.make_case(layer, 300, seed=11)
    with pytest.raises(capi.DgError):
        _run(ctx, case, k_fixed=0, k_div=0)
    with pytest.raises(capi.DgError):
        _run(ctx, case, k_fixed=2000, k_div=0)
