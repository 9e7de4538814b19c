"""The allocation-free stage-2 entry point, dg_attention_static_scratch.

It exists for hosts that cannot allocate device memory once they are running (HBM fully owned by the
host's pool, a step under stream capture, a thread that may not enter the allocator): its key-split
workspace is a fixed array inside the library instead of a cudaMalloc'd buffer.  The test calls it
through the C ABI twice in a row with different queries and compares each result with the regular
dg_attention call on the same inputs, within the suite's usual tolerance.  This file is collected
last so that a run stopping at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import util
from diffgemma_b200 import capi
from diffgemma_b200.step_attn import AttnLayer, CanvasAttention, KvCache
from oracle import attn_oracle as ao

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_static_scratch_matches_regular_entry_point_twice(ctx):
    layer = AttnLayer(n_kv_heads=2, rope_theta=1e6)
    P = 5000                                   # 42 key tiles -> several key splits per query tile
    case = util.make_case(layer, P, seed=4242)
    d = case["desc"]
    kv, att = util.gpu_setup(ctx, case)
    lib = ctx.lib
    # stage 1 once: canvas K/V into the cache, normed + roped Q for stage 2
    q1, k1, v1 = util.dev(case, "q").clone(), util.dev(case, "kc").clone(), util.dev(case, "vc").clone()
    att.qk_rope_kv(kv, P, q1, k1, v1)
    q2 = torch.roll(q1, shifts=3, dims=0).contiguous()     # a second, different query block
    qn_ref, kn_ref, vn_ref = ao.qk_rope_kv(util.t2f(case["q"]), util.t2f(case["kc"]), util.t2f(case["vc"]), None, None, d, P)
    K = np.concatenate([util.t2f(case["kp"]), kn_ref])
    V = np.concatenate([util.t2f(case["vp"]), vn_ref])
    for q in (q1, q2):
        want = att.attention(kv, P, q)                      # existing entry point
        got = torch.empty_like(q)
        st = lib.dg_attention_static_scratch(ctx.h, C.byref(att.desc), kv.h, P, C.c_void_p(q.data_ptr()),
                                             C.c_void_p(got.data_ptr()))
        assert st == capi.DG_OK, lib.dg_last_error_message()
        ctx.synchronize()
        util.assert_close(util.t2f(got), util.t2f(want), "static scratch vs dg_attention")
        oracle = ao.attention(util.t2f(q), K, V, ao.visibility(d, P), d)
        util.assert_close(util.t2f(got), oracle, "static scratch vs oracle")
    assert ctx.device_status()[0] == 0
    kv.close()


def test_static_scratch_rejects_sizes_beyond_its_array(ctx):
    layer = AttnLayer(n_q_heads=32, n_kv_heads=2)           # 256 x 32 = 8192 rows > 4096
    kv = KvCache(ctx, layer, 512)
    att = CanvasAttention(ctx, layer)
    q = torch.zeros(256, 32, 256, dtype=torch.bfloat16, device=DEV)
    out = torch.empty_like(q)
    st = ctx.lib.dg_attention_static_scratch(ctx.h, C.byref(att.desc), kv.h, 0, C.c_void_p(q.data_ptr()),
                                             C.c_void_p(out.data_ptr()))
    assert st == capi.DG_ERR_UNSUPPORTED
    assert b"exceeds the built-in scratch" in ctx.lib.dg_last_error_message()
    kv.close()


def _static(ctx, att, kv, kv_len, q, out):
    return ctx.lib.dg_attention_static_scratch(ctx.h, C.byref(att.desc), kv.h, kv_len, C.c_void_p(q.data_ptr()),
                                               C.c_void_p(out.data_ptr()))


@pytest.mark.parametrize("splits", [3, 4, 8])
def test_static_scratch_merges_forced_split_counts_in_the_array(ctx, splits):
    """With the split count forced the merge through the built-in array runs whatever the cost model would
    choose: 3 (the general last-arriver merge), 4 (what the array holds at 4096 rows) and 8 (clamped to 4)."""
    layer = AttnLayer(n_kv_heads=2, rope_theta=1e6)
    P = 2300
    case = util.make_case(layer, P, seed=4300 + splits)
    kv, att = util.gpu_setup(ctx, case)
    q, k, v = util.dev(case, "q").clone(), util.dev(case, "kc").clone(), util.dev(case, "vc").clone()
    att.qk_rope_kv(kv, P, q, k, v)
    ctx.set_splits(0)
    want = att.attention(kv, P, q)
    ctx.set_splits(splits)
    try:
        for _ in range(2):
            got = torch.zeros_like(q)
            assert _static(ctx, att, kv, P, q, got) == capi.DG_OK, ctx.lib.dg_last_error_message()
            ctx.synchronize()
            util.assert_close(util.t2f(got), util.t2f(want), f"static scratch, {splits} splits forced")
    finally:
        ctx.set_splits(0)
    assert ctx.device_status()[0] == 0
    kv.close()


def test_static_scratch_on_a_ring_cache_and_its_span_check(ctx):
    """Sliding layer on a ring: same result as dg_attention, and the same refusal when the visible span
    (window + canvas, tile aligned) no longer fits the ring."""
    layer = AttnLayer(n_kv_heads=8, rope_theta=1e4, window=1024, mask_mode=capi.MASK_WINDOW_UNIFORM)
    P = 5000
    case = util.make_case(layer, P, seed=4400)
    att = CanvasAttention(ctx, layer)
    ring = KvCache(ctx, layer, ring_slots=2048)
    n0 = P - 1500
    ring.load_prefix(case["kp"][n0:].contiguous().to(DEV), case["vp"][n0:].contiguous().to(DEV), n0)
    q, k, v = util.dev(case, "q").clone(), util.dev(case, "kc").clone(), util.dev(case, "vc").clone()
    att.qk_rope_kv(ring, P, q, k, v)
    want = att.attention(ring, P, q)
    got = torch.zeros_like(q)
    assert _static(ctx, att, ring, P, q, got) == capi.DG_OK, ctx.lib.dg_last_error_message()
    ctx.synchronize()
    util.assert_close(util.t2f(got), util.t2f(want), "static scratch on a ring")
    util.assert_close(util.t2f(got), util.run_oracle(case), "static scratch on a ring vs oracle")
    # a window of 4096 on the same 2048-slot ring: both entry points refuse, nothing is launched
    wide = AttnLayer(n_kv_heads=8, rope_theta=1e4, window=4096, mask_mode=capi.MASK_WINDOW_UNIFORM)
    att_w = CanvasAttention(ctx, wide)
    with pytest.raises(capi.DgError) as ei:
        att_w.attention(ring, P, q)
    assert ei.value.status == capi.DG_ERR_CAPACITY
    assert _static(ctx, att_w, ring, P, q, got) == capi.DG_ERR_CAPACITY
    assert ctx.device_status()[0] == 0
    ring.close()


def test_static_scratch_head_dim_512_runs_the_tensor_kernel(ctx):
    """head_dim 512 (the reference's full layers): the tensor kernel with its splits in the built-in array."""
    layer = AttnLayer(n_kv_heads=2, head_dim=512, rotary_dim=128, rope_theta=1e6, v_norm=1,
                      rope_pairing=capi.ROPE_PROPORTIONAL)
    P = 4000
    case = util.make_case(layer, P, seed=4500)
    kv, att = util.gpu_setup(ctx, case)
    q, k, v = util.dev(case, "q").clone(), util.dev(case, "kc").clone(), util.dev(case, "vc").clone()
    att.qk_rope_kv(kv, P, q, k, v)
    want = att.attention(kv, P, q)
    for splits in (0, 2):
        ctx.set_splits(splits)
        got = torch.zeros_like(q)
        assert _static(ctx, att, kv, P, q, got) == capi.DG_OK, ctx.lib.dg_last_error_message()
        ctx.synchronize()
        assert ctx.last_launch_count == 1
        util.assert_close(util.t2f(got), util.t2f(want), "static scratch, head_dim 512")
    ctx.set_splits(0)
    util.assert_close(util.t2f(got), util.run_oracle(case), "static scratch, head_dim 512 vs oracle")
    assert ctx.device_status()[0] == 0
    kv.close()
