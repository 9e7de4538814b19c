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
