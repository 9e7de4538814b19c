"""Parity of the CUDA path with the CPU oracle, through the C ABI (all tests need a B200).

Tolerances: bf16 outputs vs the fp32 oracle on identical seeded inputs must satisfy max-abs <= 2e-2
and mean-abs <= 2e-3 (tests/util.py); masks and integer outputs are compared bit-exactly."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import util
from diffgemma_b200 import capi
from diffgemma_b200.step_attn import AttnLayer, CanvasAttention, KvCache
from oracle import attn_oracle as ao
from test_oracle_pins import REF_FIXTURES, _ref_fixture

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ------------------------------------------------------------------------------------------
# stage 1: qk_rope_kv  (reference fixtures: src/shaders/attn/qk_rope_kv/mod.rs:82-185)
# ------------------------------------------------------------------------------------------
def _bits(t):
    return t.detach().cpu().view(torch.int16).numpy().astype(np.int32) & 0xFFFF


def _assert_bf16_close(got_t, want_f32, what):
    got = util.t2f(got_t)
    want = ao.round_bf16(want_f32)
    ulp = np.abs(_bits(got_t) - ao.f32_to_bf16_bits(want).astype(np.int32))
    ok = (ulp <= 1) | (np.abs(got - want) <= 2e-6)
    assert ok.all(), f"{what}: {np.count_nonzero(~ok)} values differ by more than one bf16 ulp"
    assert (ulp != 0).mean() < 5e-3, f"{what}: too many one-ulp differences"


@pytest.mark.parametrize("canvas,hq,hkv,hd,kv_len,rot,pairing,vnorm,weights", [
    (2, 4, 2, 32, 2, 32, 0, 1, False),        # tiny
    (2, 4, 2, 64, 2, 16, 1, 1, False),        # full_layer: rotary = hd/4, proportional pairing
    (1, 16, 2, 512, 22, 128, 1, 1, True),     # full_hd512 with non-unit weights
    (256, 16, 8, 256, 8192, 256, 0, 0, True),
    (256, 16, 2, 256, 131072, 256, 0, 1, False),
])
def test_qk_rope_kv_stage(ctx, canvas, hq, hkv, hd, kv_len, rot, pairing, vnorm, weights):
    layer = AttnLayer(n_q_heads=hq, n_kv_heads=hkv, head_dim=hd, canvas=canvas, rotary_dim=rot,
                      rope_theta=1e6 if pairing else 1e4, v_norm=vnorm, rope_pairing=pairing)
    d = util.oracle_desc(layer)
    g = torch.Generator().manual_seed(hd + kv_len)
    q = torch.randn(canvas, hq, hd, generator=g).to(torch.bfloat16)
    k = torch.randn(canvas, hkv, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(canvas, hkv, hd, generator=g).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(hd, generator=g)).to(torch.bfloat16) if weights else None
    kw = (1 + 0.1 * torch.randn(hd, generator=g)).to(torch.bfloat16) if weights else None
    qn, kn, vn = ao.qk_rope_kv(util.t2f(q), util.t2f(k), util.t2f(v), None if qw is None else util.t2f(qw),
                               None if kw is None else util.t2f(kw), d, kv_len, round_out=False)
    kv = KvCache(ctx, layer, kv_len + canvas)
    att = CanvasAttention(ctx, layer)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    att.qk_rope_kv(kv, kv_len, qd, kd, vd, None if qw is None else qw.to(DEV), None if kw is None else kw.to(DEV))
    ctx.synchronize()
    _assert_bf16_close(qd, qn, "q")
    _assert_bf16_close(kd, kn, "k")
    ck, cv = kv.read(kv_len, canvas)
    _assert_bf16_close(ck, kn, "cache k")
    _assert_bf16_close(cv, vn, "cache v")
    if vnorm:
        _assert_bf16_close(vd, vn, "v written back")
    kv.close()


# ------------------------------------------------------------------------------------------
# stage 2 on the reference's closed-form fixtures (src/shaders/attn/attention/mod.rs:59-184);
# tolerance of the reference's own GPU-vs-CPU gate: max-abs 2e-2, cosine >= 0.9999 (:842-946)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(REF_FIXTURES))
def test_attention_stage_reference_fixtures(ctx, name):
    canvas, hq, hkv, hd, kv_len, kind = REF_FIXTURES[name]
    q, K, V = _ref_fixture(canvas, hq, hkv, hd, kv_len, kind)
    layer = AttnLayer(n_q_heads=hq, n_kv_heads=hkv, head_dim=hd, canvas=canvas, rotary_dim=hd, softmax_scale=1.0)
    kv = KvCache(ctx, layer, kv_len + canvas)
    kv.load_prefix(util.f2t(K, DEV), util.f2t(V, DEV), 0)
    att = CanvasAttention(ctx, layer)
    out = att.attention(kv, kv_len, util.f2t(q, DEV))
    ctx.synchronize()
    got = util.t2f(out)
    want = np.load(os.path.join(os.path.dirname(__file__), "golden", "attn_golden.npz"))[name]
    assert np.abs(got - want).max() <= 2e-2
    cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
    assert cos >= 0.9999
    kv.close()


# ------------------------------------------------------------------------------------------
# the fused hot path vs the oracle
# ------------------------------------------------------------------------------------------
PARITY_CASES = [
    # prefix, Hkv, window, mask_mode, scale, canvas, weights, v_norm
    (0, 8, 0, 0, 1 / 16, 256, False, 0),        # empty prefix
    (1, 8, 0, 0, 1 / 16, 256, False, 0),
    (100, 8, 0, 0, 1 / 16, 256, False, 0),      # below one key tile
    (127, 2, 0, 0, 1 / 16, 256, False, 0),
    (128, 2, 0, 0, 1 / 16, 256, True, 0),       # exactly one tile
    (129, 2, 0, 0, 1 / 16, 256, False, 1),      # tile + 1
    (1000, 8, 0, 0, 1.0, 256, True, 1),         # reference semantics: no scale, V normed
    (2048, 8, 0, 0, 1 / 16, 256, False, 0),     # configuration 0
    (700, 8, 1024, 1, 1 / 16, 256, False, 0),   # kv_len < window
    (1023, 8, 1024, 1, 1 / 16, 256, False, 0),  # kv_len = window - 1
    (1024, 8, 1024, 2, 1 / 16, 256, False, 0),  # kv_len = window
    (3000, 8, 1024, 1, 1.0, 256, False, 1),     # uniform window (reference rule), > window
    (3000, 8, 1024, 2, 1 / 16, 256, False, 0),  # per-row window
    (8192, 8, 1024, 2, 1 / 16, 256, False, 0),  # configuration 1
    (8192, 8, 1024, 1, 1 / 16, 256, False, 0),
    (500, 16, 0, 0, 1 / 16, 256, False, 0),     # GQA group 1
    (500, 4, 0, 0, 1 / 16, 256, False, 0),      # GQA group 4
    (500, 8, 0, 0, 1 / 16, 128, False, 0),      # narrower active canvases
    (500, 2, 0, 0, 1 / 16, 64, True, 0),
    (333, 8, 64, 2, 1 / 16, 100, False, 0),     # ragged canvas, tiny window
    (0, 8, 0, 3, 1 / 16, 256, False, 0),        # causal re-prefill of a block on an empty cache
    (700, 8, 0, 3, 1.0, 256, True, 1),          # causal, no window, reference semantics
    (3000, 8, 1024, 3, 1.0, 256, False, 1),     # causal sliding: query p sees [p - 1023, p]
    (3000, 2, 1024, 3, 1 / 16, 256, False, 0),  # the same with 16 query tiles per KV head (tile-range trimming)
    (333, 8, 64, 3, 1 / 16, 100, False, 0),     # causal window shorter than the canvas: it cuts canvas keys too
]


@pytest.mark.parametrize("P,Hkv,W,mode,scale,canvas,weights,vnorm", PARITY_CASES)
def test_denoise_parity(ctx, P, Hkv, W, mode, scale, canvas, weights, vnorm):
    layer = AttnLayer(n_kv_heads=Hkv, window=W, mask_mode=mode, softmax_scale=scale, canvas=canvas,
                      rope_theta=1e4 if W else 1e6, v_norm=vnorm)
    case = util.make_case(layer, P, seed=P * 7 + Hkv, weights=weights)
    ref = util.run_oracle(case)
    assert CanvasAttention(ctx, layer).uses_tensor_path
    ctx.force_general(False)
    try:
        for pair in (None, False):   # automatic choice (CTA pairs where they apply), then the single-CTA form
            ctx.set_pair_mode(pair)
            for splits in (0, 1, 3, 8):     # 8: one cluster of eight CTAs in the single-CTA form (clamped to the key tiles)
                ctx.set_splits(splits)
                got = util.run_gpu(ctx, case)
                util.assert_close(got, ref, f"tensor path pair={pair} splits={splits}", stress=(scale == 1.0))
    finally:
        ctx.set_splits(0)
        ctx.set_pair_mode(None)
    ctx.force_general(True)
    got = util.run_gpu(ctx, case)
    ctx.force_general(False)
    util.assert_close(got, ref, "general path", stress=(scale == 1.0))
    assert ctx.device_status()[0] == 0


@pytest.mark.parametrize("cfg_prefix,Hkv", [(32768, 2), (131072, 2)])
def test_full_size_parity_and_split_invariance(ctx, cfg_prefix, Hkv):
    """Configurations 2 and 4 at full size against the oracle, plus properties that do not depend
    on the size: the result must not depend on the number of key splits, rows of softmax weights sum
    to one (V = 1 gives O = 1), and the output is linear in V."""
    layer = AttnLayer(n_kv_heads=Hkv, rope_theta=1e6)
    case = util.make_case(layer, cfg_prefix, seed=20261125 + cfg_prefix)
    ref = util.run_oracle(case)
    kv, att = util.gpu_setup(ctx, case)
    q, kc, vc = util.dev(case, "q")[None], util.dev(case, "kc")[None], util.dev(case, "vc")[None]
    outs = {}
    for splits in (0, 1, 4, 7):
        ctx.set_splits(splits)
        outs[splits] = util.t2f(att.denoise([kv], [cfg_prefix], q, kc, vc)[0])
        util.assert_close(outs[splits], ref, f"P={cfg_prefix} splits={splits}")
    ctx.set_splits(0)
    assert np.abs(outs[1] - outs[4]).max() <= 2e-3 and np.abs(outs[1] - outs[7]).max() <= 2e-3
    # V = 1 everywhere -> every output element is exactly the sum of the weights = 1
    ones_p = torch.ones_like(case["vp"]).to(DEV)
    kv.load_prefix(case["kp"].to(DEV), ones_p, 0)
    o1 = util.t2f(att.denoise([kv], [cfg_prefix], q, kc, torch.ones_like(vc))[0])
    assert np.abs(o1 - 1.0).max() <= 8e-3
    # linearity in V: O(V) + O(1) == O(V + 1) up to bf16 rounding of the outputs
    kv.load_prefix(case["kp"].to(DEV), (case["vp"].float() + 1).to(torch.bfloat16).to(DEV), 0)
    o2 = util.t2f(att.denoise([kv], [cfg_prefix], q, kc, (vc.float() + 1).to(torch.bfloat16))[0])
    assert np.abs(o2 - (outs[0] + 1.0)).max() <= 3e-2
    assert np.abs(o2 - (outs[0] + 1.0)).mean() <= 4e-3
    kv.close()


def test_run_twice_is_bitwise_identical(ctx):
    layer = AttnLayer(n_kv_heads=2)
    case = util.make_case(layer, 5000, seed=11)
    kv, att = util.gpu_setup(ctx, case)
    q, kc, vc = util.dev(case, "q")[None], util.dev(case, "kc")[None], util.dev(case, "vc")[None]
    a = att.denoise([kv], [5000], q, kc, vc).clone()
    b = att.denoise([kv], [5000], q, kc, vc).clone()
    ctx.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    kv.close()


def test_batch_of_independent_canvases(ctx):
    """Four canvases with their own caches and ragged prefix lengths (configuration 3's shape)."""
    layer = AttnLayer(n_kv_heads=8, window=1024, mask_mode=capi.MASK_WINDOW_UNIFORM, rope_theta=1e4)
    lens = [2048 - 64 * b for b in range(4)]
    cases = [util.make_case(layer, lens[b], seed=300 + b) for b in range(4)]
    kvs = []
    for c in cases:
        kv, att = util.gpu_setup(ctx, c)
        kvs.append(kv)
    q = torch.stack([c["q"] for c in cases]).to(DEV)
    k = torch.stack([c["kc"] for c in cases]).to(DEV)
    v = torch.stack([c["vc"] for c in cases]).to(DEV)
    out = att.denoise(kvs, lens, q, k, v)
    ctx.synchronize()
    for b, c in enumerate(cases):
        util.assert_close(util.t2f(out[b]), util.run_oracle(c), f"canvas {b}")
    for kv in kvs:
        kv.close()


@pytest.mark.parametrize("Hkv,W,weights", [(8, 0, True), (2, 0, False), (8, 1024, True)])
def test_append_with_cached_rope_table_writes_the_same_bits(ctx, Hkv, W, weights):
    """The first step at a position computes the RoPE table and runs the general append kernel; later
    steps at the same positions read the table in a shorter kernel.  Cache contents and output must
    be the same, bit for bit."""
    layer = AttnLayer(n_kv_heads=Hkv, window=W, mask_mode=capi.MASK_WINDOW_UNIFORM if W else 0,
                      rope_theta=1e4 if W else 1e6)
    P = 1300
    case = util.make_case(layer, P, seed=71 + Hkv, weights=weights)
    kv, att = util.gpu_setup(ctx, case)
    args = ([kv], [P], util.dev(case, "q")[None], util.dev(case, "kc")[None], util.dev(case, "vc")[None],
            util.dev(case, "qw"), util.dev(case, "kw"))
    # another position first (on a scratch cache), so that the table of position P is certainly not cached
    scratch = KvCache(ctx, layer, 100 + layer.canvas)
    scratch.load_prefix(util.dev(case, "kp")[:100].contiguous(), util.dev(case, "vp")[:100].contiguous(), 0)
    att.denoise([scratch], [100], *args[2:])
    scratch.close()
    first = att.denoise(*args).clone()
    k1, v1 = kv.read(P, layer.canvas)
    second = att.denoise(*args).clone()
    k2, v2 = kv.read(P, layer.canvas)
    ctx.synchronize()
    assert torch.equal(k1.view(torch.int16), k2.view(torch.int16))
    assert torch.equal(v1.view(torch.int16), v2.view(torch.int16))
    assert torch.equal(first.view(torch.int16), second.view(torch.int16))
    util.assert_close(util.t2f(second[0]), util.run_oracle(case), "cached-table step")
    kv.close()


def test_host_buffer_call_matches_device_call(ctx):
    layer = AttnLayer(n_kv_heads=8)
    case = util.make_case(layer, 777, seed=5)
    kv, att = util.gpu_setup(ctx, case)
    dev_out = att.denoise([kv], [777], util.dev(case, "q")[None], util.dev(case, "kc")[None], util.dev(case, "vc")[None])
    q, k, v = (case[n][None].contiguous().pin_memory() for n in ("q", "kc", "vc"))
    host_out = torch.empty_like(q).pin_memory()
    att.denoise_host([kv], [777], q, k, v, host_out)
    assert torch.equal(host_out.view(torch.int16), dev_out.cpu().view(torch.int16))
    assert ctx.last_launch_count in (1, 2)      # 1: the canvas append ran inside the attention launch
    kv.close()


# ------------------------------------------------------------------------------------------
# masks: bit-exact
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("P,W,mode,canvas", [(0, 0, 0, 256), (300, 0, 0, 256), (700, 1024, 1, 256), (1023, 1024, 2, 256),
                                             (1024, 1024, 2, 256), (1025, 1024, 1, 256), (3000, 1024, 2, 256),
                                             (8192, 1024, 2, 256), (8192, 1024, 1, 256), (333, 64, 2, 100),
                                             (0, 0, 3, 256), (300, 0, 3, 256), (1025, 1024, 3, 256), (333, 64, 3, 100),
                                             (5, 8, 3, 16)])
def test_visibility_bitmap_bit_exact(ctx, P, W, mode, canvas):
    layer = AttnLayer(window=W, mask_mode=mode, canvas=canvas)
    att = CanvasAttention(ctx, layer)
    d = util.oracle_desc(layer)
    shards = [(0, P, True), (0, P // 2, False), (P // 2, P, True), (P // 3, P // 3, True)]
    for t0, t1, inc in shards:
        got = att.visibility(P, t0, t1, inc).cpu().numpy().astype(bool)
        np.testing.assert_array_equal(got, ao.visibility(d, P, t0, t1, inc))


@pytest.mark.parametrize("force_general", [False, True])
@pytest.mark.parametrize("P,W,mode,t0,t1,inc", [
    (100, 0, 0, 0, 100, True), (100, 64, 1, 0, 100, True), (100, 64, 2, 0, 100, True),
    (100, 64, 2, 30, 80, False), (100, 0, 0, 50, 50, True), (90, 32, 2, 0, 90, True),
    (100, 0, 3, 0, 100, True), (100, 64, 3, 0, 100, True), (100, 16, 3, 20, 100, True), (0, 8, 3, 0, 0, True),
])
def test_kernel_mask_bit_exact_through_indicator_values(ctx, force_general, P, W, mode, t0, t1, inc):
    """With Q = 0 every visible key has weight exactly 1, so l counts the visible keys of a row and,
    with V[t] = one-hot(t), the un-normalised output IS the row of the visibility bitmap.  T <= 256
    so each key has its own output column: the kernels' mask is compared bit for bit."""
    canvas = 256 - P if P >= 100 else 128
    canvas = min(canvas, 256 - P)
    layer = AttnLayer(n_kv_heads=8, window=W, mask_mode=mode, canvas=canvas)
    T = P + canvas
    assert T <= 256
    onehot = torch.zeros(T, 8, 256, dtype=torch.bfloat16)
    for t in range(T):
        onehot[t, :, t] = 1.0
    kv = KvCache(ctx, layer, T)
    if P > 0:
        kv.load_prefix(torch.zeros(P, 8, 256, dtype=torch.bfloat16).to(DEV), onehot[:P].to(DEV), 0)
    att = CanvasAttention(ctx, layer)
    q = torch.zeros(canvas, 16, 256, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(canvas, 8, 256, dtype=torch.bfloat16, device=DEV)
    vc = onehot[P:].to(DEV).contiguous()
    ctx.force_general(force_general)
    o, m, l = att.partial(kv, P, t0, t1, inc, q, kc, vc)
    ctx.synchronize()
    ctx.force_general(False)
    want = ao.visibility(util.oracle_desc(layer), P, t0, t1, inc)        # [canvas, T]
    o = o.cpu().numpy()
    l = l.cpu().numpy()
    for h in (0, 7, 15):
        np.testing.assert_array_equal(o[:, h, :T] != 0, want)
        np.testing.assert_array_equal(o[:, h, :T][want], 1.0)
        np.testing.assert_array_equal(l[:, h], want.sum(axis=1).astype(np.float32))
    kv.close()


def test_sparse_decoder_bitmap(ctx):
    """Shape of the reference's sparse decoder-bitmap fixture (src/shaders/attn/gqa_attention/mod.rs:
    181-232): 32 canvas rows, 14 prefix keys, 16Q/8KV, head_dim 256; canvas keys with (q+k)%5==0
    masked and rows q%7==0 blind to the prefix."""
    layer = AttnLayer(n_kv_heads=8, canvas=32, softmax_scale=1.0)
    P = 14
    case = util.make_case(layer, P, seed=99)
    att_map = np.ones((32, P + 32), bool)
    for qi in range(32):
        for k in range(P, P + 32):
            if (qi + k) % 5 == 0:
                att_map[qi, k] = False
        if qi % 7 == 0:
            att_map[qi, :P] = False
    ref = util.run_oracle(case, attend=att_map)
    kv, att = util.gpu_setup(ctx, case)
    out = att.denoise_bitmap(kv, P, util.dev(case, "q"), util.dev(case, "kc"), util.dev(case, "vc"),
                             torch.from_numpy(att_map.astype(np.uint8)).to(DEV))
    ctx.synchronize()
    util.assert_close(util.t2f(out), ref, "bitmap")
    kv.close()


# ------------------------------------------------------------------------------------------
# split-KV partials and merges
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("P,W,mode,cuts", [(5000, 0, 0, [0, 1280, 2560, 5000]), (3000, 1024, 1, [0, 1024, 2048, 3000]),
                                           (3000, 1024, 2, [0, 1500, 3000])])
def test_partials_merge_to_single_shot(ctx, P, W, mode, cuts):
    layer = AttnLayer(n_kv_heads=2, window=W, mask_mode=mode)
    case = util.make_case(layer, P, seed=P + W)
    ref = util.run_oracle(case)
    kv, att = util.gpu_setup(ctx, case)
    q, kc, vc = util.dev(case, "q"), util.dev(case, "kc"), util.dev(case, "vc")
    parts = []
    for i in range(len(cuts) - 1):
        inc = i == len(cuts) - 2
        o, m, l = att.partial(kv, P, cuts[i], cuts[i + 1], inc, q, kc, vc)
        want_o, want_m, want_l = util.run_oracle(case, partial=(cuts[i], cuts[i + 1], inc))
        # same log-sum-exp and same normalised partial output as the oracle's shard
        lse = (m + torch.log(l)).cpu().numpy()
        want_lse = want_m + np.log(np.where(want_l > 0, want_l, 1.0))
        seen = want_l > 0
        if seen.any():
            assert np.abs(lse[seen] - want_lse[seen]).max() <= 2e-3
        assert np.all(np.isneginf(m.cpu().numpy()[~seen])) and np.all(l.cpu().numpy()[~seen] == 0)
        norm = (o / torch.where(l > 0, l, torch.ones_like(l))[..., None]).cpu().numpy()
        want_norm = want_o / np.where(want_l > 0, want_l, 1.0)[..., None]
        assert np.abs(norm - want_norm).max() <= 2e-2
        parts.append((o, m, l))
    merged = att.merge_local(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]),
                             torch.stack([p[2] for p in parts]))
    ctx.synchronize()
    util.assert_close(util.t2f(merged), ref, "merged partials")
    kv.close()


# ------------------------------------------------------------------------------------------
# errors: reported, never raised as faults
# ------------------------------------------------------------------------------------------
def test_argument_errors(ctx):
    layer = AttnLayer(n_kv_heads=8)
    att = CanvasAttention(ctx, layer)
    kv = KvCache(ctx, layer, 512)
    q = torch.zeros(1, 256, 16, 256, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(1, 256, 8, 256, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(capi.DgError) as e:
        att.denoise([kv], [400], q, k, k)              # 400 + 256 > capacity 512
    assert e.value.status == capi.DG_ERR_CAPACITY
    lib = ctx.lib
    arr = (C.c_void_p * 1)(kv.h)
    lens = (C.c_uint32 * 1)(0)
    st = lib.dg_attn_denoise(ctx.h, C.byref(att.desc), arr, lens, 1, C.c_void_p(q.data_ptr() + 2), C.c_void_p(k.data_ptr()),
                             C.c_void_p(k.data_ptr()), None, None, C.c_void_p(q.data_ptr()))
    assert st == capi.DG_ERR_ALIGNMENT
    st = lib.dg_attn_denoise(ctx.h, C.byref(att.desc), arr, lens, 1, None, None, None, None, None, None)
    assert st == capi.DG_ERR_INVALID_ARG
    other = AttnLayer(n_kv_heads=2)
    with pytest.raises(capi.DgError) as e:
        CanvasAttention(ctx, other).denoise([kv], [0], q, k[:, :, :2].contiguous(), k[:, :, :2].contiguous())
    assert e.value.status == capi.DG_ERR_INVALID_ARG   # cache geometry differs from the layer
    assert ctx.device_status()[0] == 0
    kv.close()


def test_output_guard_rows_untouched(ctx):
    """Canary rows before and after the output must survive (no out-of-bounds stores), also for a
    ragged canvas whose last query tile is partly padding."""
    layer = AttnLayer(n_kv_heads=8, canvas=100)
    case = util.make_case(layer, 300, seed=8)
    kv, att = util.gpu_setup(ctx, case)
    n = 100 * 16 * 256
    guard = 4096
    buf = torch.full((n + 2 * guard,), 7.0, dtype=torch.bfloat16, device=DEV)
    out = buf[guard:guard + n].view(1, 100, 16, 256)
    for splits in (1, 3):
        ctx.set_splits(splits)
        att.denoise([kv], [300], util.dev(case, "q")[None], util.dev(case, "kc")[None], util.dev(case, "vc")[None], out=out)
    ctx.set_splits(0)
    ctx.synchronize()
    assert torch.all(buf[:guard] == 7.0) and torch.all(buf[guard + n:] == 7.0)
    util.assert_close(util.t2f(out[0]), util.run_oracle(case), "ragged canvas")
    kv.close()


@pytest.mark.parametrize("v_scale", [2.0 ** 14, 2.0 ** -10, 2.0 ** -100])
def test_split_exchange_is_range_independent(ctx, v_scale):
    """Inside a cluster the partial rows cross between CTAs as fp16 with one power-of-two scale per
    row.  V scaled by a power of two (exact in bf16) must give the same output scaled by it, bit for
    bit after rescaling, with and without key splits, and stay within tolerance of the oracle."""
    layer = AttnLayer(n_kv_heads=2, rope_theta=1e6)
    case = util.make_case(layer, 3000, seed=4242)
    ref = util.run_oracle(case)
    scaled = dict(case)
    scaled["vp"] = (case["vp"].float() * v_scale).to(torch.bfloat16)
    scaled["vc"] = (case["vc"].float() * v_scale).to(torch.bfloat16)
    assert torch.equal(scaled["vp"].float() / v_scale, case["vp"].float())     # the scaling was exact
    try:
        for pair in (False, True):
            ctx.set_pair_mode(pair)
            for splits in (1, 2, 4):
                ctx.set_splits(splits)
                base = util.run_gpu(ctx, case)
                got = util.run_gpu(ctx, scaled).astype(np.float64) / v_scale
                assert np.array_equal(got.astype(np.float32), base), f"pair={pair} splits={splits} scale={v_scale}"
                util.assert_close(got.astype(np.float32), ref, f"pair={pair} splits={splits} scale={v_scale}")
    finally:
        ctx.set_splits(0)
        ctx.set_pair_mode(None)
    assert ctx.device_status()[0] == 0


# ------------------------------------------------------------------------------------------
# CTA-pair kernel variant (tcgen05 cta_group::2)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("P,Hkv,W,mode,scale,canvas", [(300, 8, 0, 0, 1 / 16, 256), (1000, 2, 0, 0, 1 / 16, 256),
                                                       (3000, 8, 1024, 2, 1 / 16, 256), (3000, 8, 1024, 1, 1.0, 256),
                                                       (500, 8, 0, 0, 1 / 16, 100), (500, 2, 0, 0, 1 / 16, 64)])
def test_pair_kernel_parity(ctx, P, Hkv, W, mode, scale, canvas):
    layer = AttnLayer(n_kv_heads=Hkv, window=W, mask_mode=mode, softmax_scale=scale, canvas=canvas,
                      rope_theta=1e4 if W else 1e6, v_norm=1 if scale == 1.0 else 0)
    case = util.make_case(layer, P, seed=P + 13 * Hkv)
    ref = util.run_oracle(case)
    ctx.set_pair_mode(True)
    try:
        for splits in (0, 1, 2, 3, 4):
            ctx.set_splits(splits)
            util.assert_close(util.run_gpu(ctx, case), ref, f"pair kernel splits={splits}", stress=(scale == 1.0))
    finally:
        ctx.set_splits(0)
        ctx.set_pair_mode(None)
    assert ctx.device_status()[0] == 0


# ------------------------------------------------------------------------------------------
# failure path: a bounded wait that runs out is reported through the status word, nothing faults
# ------------------------------------------------------------------------------------------
def test_wait_timeout_is_reported_and_context_survives(ctx):
    lib = ctx.lib
    assert lib.dg_ctx_selftest_wait_timeout(ctx.h, 200000) == capi.DG_OK      # ~0.1 ms
    assert lib.dg_ctx_synchronize(ctx.h) == capi.DG_DEV_WAIT_TIMEOUT
    st = ctx.device_status()
    assert st[0] == capi.DG_DEV_WAIT_TIMEOUT and st[1] == 6
    assert lib.dg_ctx_clear_device_status(ctx.h) == capi.DG_OK
    assert lib.dg_ctx_synchronize(ctx.h) == capi.DG_OK
    # the context still computes correctly
    layer = AttnLayer(n_kv_heads=8)
    case = util.make_case(layer, 300, seed=21)
    util.assert_close(util.run_gpu(ctx, case), util.run_oracle(case), "after a reported timeout")


# ------------------------------------------------------------------------------------------
# the CUDA path against the reference's OWN shaders (vectors stored by tests/golden/make_ref_shader_golden.py
# from attention.metal / qk_rope_kv.metal compiled for the CPU)
# ------------------------------------------------------------------------------------------
def _ref_golden():
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "tests", "golden"))
    import make_ref_shader_golden as G
    return G, np.load(os.path.join(root, "tests", "golden", "ref_shader_golden.npz"))


@pytest.mark.parametrize("name", ["sliding_short", "sliding_window_cuts", "sliding_ring", "full_hd512_valias",
                                  "full_hd256_vproj", "causal_sliding", "causal_full_hd256"])
def test_gpu_matches_reference_shader_vectors(ctx, name):
    G, gold = _ref_golden()
    cases = {**G.VALUE_CASES, **G.CAUSAL_VALUE_CASES}
    hd, n_q, n_kv, canvas, kv_len, is_full, window, ring, valias, seed = cases[name]
    q, k, v, kp, vp, qw, kw = G.value_inputs(*cases[name])
    mode = capi.MASK_CAUSAL if name in G.CAUSAL_VALUE_CASES else (capi.MASK_WINDOW_UNIFORM if window else capi.MASK_NONE)
    layer = AttnLayer(n_q_heads=n_q, n_kv_heads=n_kv, head_dim=hd, canvas=canvas,
                      rotary_dim=hd // 4 if is_full else hd, rope_theta=1e6 if is_full else 1e4, rms_eps=1e-6,
                      softmax_scale=1.0, window=window, mask_mode=mode,
                      v_norm=1, rope_pairing=capi.ROPE_PROPORTIONAL if is_full else capi.ROPE_SPLIT_HALF)
    kv = KvCache(ctx, layer, ring_slots=ring + 1) if ring else KvCache(ctx, layer, kv_len + canvas)
    t = lambda a: util.f2t(a).to(DEV)
    kv.load_prefix(t(kp), t(vp), 0)
    att = CanvasAttention(ctx, layer)
    kc = t(k)
    out = att.denoise([kv], [kv_len], t(q)[None], kc[None], (kc if valias else t(v))[None], t(qw), t(kw))
    ctx.synchronize()
    got = util.t2f(out[0])
    ref = gold[f"{name}_out"]
    # the shader truncates its output to bf16: one bf16 ulp of the difference is its own quantisation
    err = np.maximum(np.abs(got - ref) - np.maximum(np.abs(ref), 2.0 ** -20) * 2.0 ** -7, 0.0)
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (name, float(err.max()), float(err.mean()))
    assert ctx.device_status()[0] == 0
    kv.close()


# ------------------------------------------------------------------------------------------
# head_dim 512 (the reference's full-attention layers) on the tensor path
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("P,Hq,Hkv,canvas,W,mode,scale,vnorm", [
    (60, 4, 2, 4, 0, 0, 1.0, 1),            # tiny: one partial tile
    (700, 16, 2, 256, 0, 0, 1 / 16, 0),     # 16 query tiles per KV head, ragged last key tile
    (4096, 16, 2, 256, 0, 0, 1 / 16, 1),    # aligned prefix
    (3000, 8, 8, 100, 0, 0, 1 / 16, 1),     # no GQA stacking, ragged canvas
    (5000, 16, 4, 256, 1024, 1, 1 / 16, 1), # sliding window on a 512-wide head (not a reference layer; mask logic)
    (700, 16, 2, 256, 0, 3, 1.0, 1),        # causal re-prefill of a block on a full layer
    (8192 + 64, 16, 2, 256, 0, 0, 1.0, 1),  # odd number of 64-key tiles, unscaled logits: the reference moves often
    (1, 16, 2, 256, 0, 0, 1.0, 1),          # one prefix key: the canvas tiles carry everything
])
def test_hd512_tensor_path_parity(ctx, P, Hq, Hkv, canvas, W, mode, scale, vnorm):
    """All three tensor forms: one CTA per value half with the scores computed twice (pair mode off), the two-CTA
    cluster that splits the score work and exchanges P (pair mode on), and the four-CTA cluster that also shares the
    K and V stages between two query tiles (automatic, taken when a KV head has an even number of query tiles)."""
    layer = AttnLayer(n_q_heads=Hq, n_kv_heads=Hkv, head_dim=512, canvas=canvas, rotary_dim=128, rope_theta=1e6,
                      softmax_scale=scale, window=W, mask_mode=mode, v_norm=vnorm, rope_pairing=capi.ROPE_PROPORTIONAL)
    case = util.make_case(layer, P, seed=P + Hq, weights=True)
    ref = util.run_oracle(case)
    assert CanvasAttention(ctx, layer).uses_tensor_path
    try:
        for pair in (None, True, False):
            ctx.set_pair_mode(pair)
            for splits in (0, 1, 2, 5):
                ctx.set_splits(splits)
                util.assert_close(util.run_gpu(ctx, case), ref, f"hd512 tensor path pair={pair} splits={splits}",
                                  stress=(scale == 1.0))
                assert ctx.device_status()[0] == 0
    finally:
        ctx.set_splits(0)
        ctx.set_pair_mode(None)
    ctx.force_general(True)
    got = util.run_gpu(ctx, case)
    ctx.force_general(False)
    util.assert_close(got, ref, "hd512 general path", stress=(scale == 1.0))
    assert ctx.device_status()[0] == 0


# ------------------------------------------------------------------------------------------
# host-buffer pipeline
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("deferred", [False, True])
def test_host_pipe_matches_the_synchronous_host_call(ctx, deferred):
    """Also with the deferred launch: a step's kernels are queued one submit after its copies, or at its wait."""
    from diffgemma_b200.step_attn import HostPipe
    layer = AttnLayer(n_kv_heads=2)
    cases = [util.make_case(layer, 3000, seed=400 + i) for i in range(7)]
    kv, att = util.gpu_setup(ctx, cases[0])
    pin = lambda t: t[None].contiguous().pin_memory()
    ins = [(pin(c["q"]), pin(c["kc"]), pin(c["vc"])) for c in cases]
    want = []
    for q, k, v in ins:                                   # synchronous reference, one step at a time
        o = torch.empty_like(q).pin_memory()
        att.denoise_host([kv], [3000], q, k, v, o)
        want.append(o.clone())
    pipe = HostPipe(ctx, layer, 1, depth=3)
    pipe.set_deferred_launch(deferred)
    outs = [torch.empty_like(ins[0][0]).pin_memory() for _ in cases]
    tickets = [pipe.submit([kv], [3000], q, k, v, o) for (q, k, v), o in zip(ins, outs)]   # more submits than slots
    for t in reversed(tickets):                           # collected out of order
        pipe.wait(t)
    for o, w in zip(outs, want):
        assert torch.equal(o.view(torch.int16), w.view(torch.int16))
    pipe.close()
    kv.close()
    assert ctx.device_status()[0] == 0


# ------------------------------------------------------------------------------------------
# a warmed-up step can be captured into a CUDA graph and replayed (what a 48-step denoise loop does)
# ------------------------------------------------------------------------------------------
def test_step_is_capturable_into_a_cuda_graph(ctx):
    layer = AttnLayer(n_kv_heads=8, window=1024, mask_mode=capi.MASK_WINDOW_UNIFORM, rope_theta=1e4)
    cases = [util.make_case(layer, 3000 - 64 * b, seed=500 + b) for b in range(3)]
    kvs = [util.gpu_setup(ctx, c)[0] for c in cases]
    att = CanvasAttention(ctx, layer)
    lens = [c["prefix"] for c in cases]
    q = torch.stack([c["q"] for c in cases]).to(DEV)
    k = torch.stack([c["kc"] for c in cases]).to(DEV)
    v = torch.stack([c["vc"] for c in cases]).to(DEV)
    out = torch.empty_like(q)
    for _ in range(2):                                     # warm-up: workspaces, side streams, RoPE tables
        att.denoise(kvs, lens, q, k, v, out=out)
    ctx.synchronize()
    want = out.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=ctx.torch_stream):
        att.denoise(kvs, lens, q, k, v, out=out)
    out.zero_()
    g.replay()
    ctx.synchronize()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    for b, c in enumerate(cases):
        util.assert_close(util.t2f(out[b]), util.run_oracle(c), f"graph replay, canvas {b}")
    for kv in kvs:
        kv.close()


def test_graph_replay_survives_eager_calls_at_other_positions(ctx):
    """A captured step reads the RoPE table of its own cache.  Eager calls on OTHER caches at other
    positions between capture and replay, and a step captured before its cache's table was ever written
    (the recorded launches then write and read a table of their own), must both replay correctly."""
    layer = AttnLayer(n_kv_heads=8, rope_theta=1e4)
    a = util.make_case(layer, 700, seed=811)
    b = util.make_case(layer, 1500, seed=812)
    c = util.make_case(layer, 300, seed=813)
    att = CanvasAttention(ctx, layer)
    kv_a, _ = util.gpu_setup(ctx, a)
    kv_b, _ = util.gpu_setup(ctx, b)
    kv_c, _ = util.gpu_setup(ctx, c)
    dv = lambda case, n: util.dev(case, n)[None]
    out_a = torch.empty_like(dv(a, "q"))
    out_c = torch.empty_like(dv(c, "q"))
    # warm the workspaces on cache B only, so that A's table is valid (eager step) and C's is not
    att.denoise([kv_b], [b["prefix"]], dv(b, "q"), dv(b, "kc"), dv(b, "vc"))
    att.denoise([kv_a], [a["prefix"]], dv(a, "q"), dv(a, "kc"), dv(a, "vc"), out=out_a)
    ctx.synchronize()
    want_a = out_a.clone()
    qa, ka, va = dv(a, "q"), dv(a, "kc"), dv(a, "vc")
    qc, kc, vc = dv(c, "q"), dv(c, "kc"), dv(c, "vc")
    g_a, g_c = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_a, stream=ctx.torch_stream):      # table of A already holds these positions
        att.denoise([kv_a], [a["prefix"]], qa, ka, va, out=out_a)
    with torch.cuda.graph(g_c, stream=ctx.torch_stream):      # C has never run: the graph carries its own table
        att.denoise([kv_c], [c["prefix"]], qc, kc, vc, out=out_c)
    # eager calls at other positions on another cache, and an eager call on C AFTER its capture
    got_b = att.denoise([kv_b], [b["prefix"]], dv(b, "q"), dv(b, "kc"), dv(b, "vc"))
    got_c_eager = att.denoise([kv_c], [c["prefix"]], qc, kc, vc)
    out_a.zero_()
    out_c.zero_()
    g_a.replay()
    g_c.replay()
    got_c_eager2 = att.denoise([kv_c], [c["prefix"]], qc, kc, vc)   # eager again after the replay
    ctx.synchronize()
    assert torch.equal(out_a.view(torch.int16), want_a.view(torch.int16))
    util.assert_close(util.t2f(out_a[0]), util.run_oracle(a), "graph replay after eager calls elsewhere")
    ref_c = util.run_oracle(c)
    util.assert_close(util.t2f(out_c[0]), ref_c, "graph captured before the cache's table existed")
    util.assert_close(util.t2f(got_c_eager[0]), ref_c, "eager call between capture and replay")
    util.assert_close(util.t2f(got_c_eager2[0]), ref_c, "eager call after the replay")
    util.assert_close(util.t2f(got_b[0]), util.run_oracle(b), "eager call on the other cache")
    assert ctx.device_status()[0] == 0
    for kv in (kv_a, kv_b, kv_c):
        kv.close()


# ------------------------------------------------------------------------------------------
# shard caches and the peer-memory exchange on ONE rank (the multi-rank forms need >= 2 GPUs)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("P,t0,t1,inc", [(6000, 2560, 4224, False), (6000, 4224, 6000, True), (5000, 0, 1280, False)])
def test_shard_cache_partial_matches_full_cache(ctx, P, t0, t1, inc):
    """A cache that holds only positions [t0, t1) (+ the canvas on the rank that counts it) gives the same
    partial as a full-size cache, bit for bit, and refuses calls whose keys lie outside it."""
    layer = AttnLayer(n_kv_heads=2)
    case = util.make_case(layer, P, seed=P + t0)
    att = CanvasAttention(ctx, layer)
    full, _ = util.gpu_setup(ctx, case)
    cap = t1 - t0 + (layer.canvas if inc else 0)
    shard = KvCache(ctx, layer, cap, pos_base=t0)
    shard.load_prefix(case["kp"][t0:t1].contiguous().to(DEV), case["vp"][t0:t1].contiguous().to(DEV), t0)
    q, kc, vc = util.dev(case, "q"), util.dev(case, "kc"), util.dev(case, "vc")
    want = att.partial(full, P, t0, t1, inc, q, kc, vc)
    got = att.partial(shard, P, t0, t1, inc, q, kc, vc)
    ctx.synchronize()
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    o, m, l = util.run_oracle(case, partial=(t0, t1, inc))
    lg = np.where(l > 0, l, 1.0)
    util.assert_close(got[0].cpu().numpy() / got[2].cpu().numpy().clip(min=1e-30)[..., None], o / lg[..., None], "shard partial")
    # keys outside the shard: refused before anything is launched
    with pytest.raises(capi.DgError) as ei:
        att.partial(shard, P, 0 if t0 else t1, t1 + 1024, inc, q, kc, vc)
    assert ei.value.status == capi.DG_ERR_CAPACITY
    k_back, _ = shard.read(t0, 128)
    assert torch.equal(k_back, case["kp"][t0:t0 + 128].to(DEV))
    full.close()
    shard.close()


def test_pipelined_push_exchange_on_one_rank(ctx):
    """Mode 4 with this rank as the only peer: the slice of a step is written by the next call or by the flush."""
    import ctypes as C
    layer = AttnLayer(n_kv_heads=2)
    P = 3000
    cases = [util.make_case(layer, P, seed=520 + i) for i in range(4)]
    kv, att = util.gpu_setup(ctx, cases[0])          # same prefix for all steps; canvas inputs differ per step
    lib = ctx.lib
    x = C.c_void_p()
    capi.check(lib.dg_p2p_create(ctx.h, layer.canvas * layer.n_q_heads, layer.head_dim, 1, 0, C.byref(x)), "dg_p2p_create")
    capi.check(lib.dg_p2p_set_mode(x, 4), "dg_p2p_set_mode")
    outs = [torch.zeros_like(util.dev(cases[0], "q")) for _ in range(4)]
    ins = [(util.dev(c, "q"), util.dev(c, "kc"), util.dev(c, "vc")) for c in cases]
    for i in range(4):
        q, kc, vc = ins[i]
        capi.check(lib.dg_attn_denoise_split_p2p(ctx.h, C.byref(att.desc), kv.h, P, 0, P, 1, x, util_ptr(q), util_ptr(kc),
                                                 util_ptr(vc), None, None, util_ptr(outs[i])), "dg_attn_denoise_split_p2p")
        if i == 0:
            ctx.synchronize()
            assert not outs[0].any()                 # nothing has been merged yet
    assert lib.dg_p2p_set_mode(x, 3) == capi.DG_ERR_INVALID_ARG      # a step is pending
    capi.check(lib.dg_p2p_flush(x), "dg_p2p_flush")
    ctx.synchronize()
    for i, c in enumerate(cases):
        cc = dict(c)
        cc["kp"], cc["vp"] = cases[0]["kp"], cases[0]["vp"]
        util.assert_close(util.t2f(outs[i]), util.run_oracle(cc), f"pipelined exchange, step {i}")
    capi.check(lib.dg_p2p_set_mode(x, 3), "dg_p2p_set_mode")
    assert ctx.device_status()[0] == 0
    lib.dg_p2p_destroy(x)
    kv.close()


@pytest.mark.parametrize("mode", [0, 1, 3])
def test_peer_exchange_forms_on_one_rank(ctx, mode):
    """world = 1: the exchange kernels run with this rank as the only peer (the push form stores its rows
    into its own receive area and merges them from there) and must reproduce the plain call."""
    import ctypes as C
    layer = AttnLayer(n_kv_heads=2)
    P = 3000
    case = util.make_case(layer, P, seed=515)
    kv, att = util.gpu_setup(ctx, case)
    lib = ctx.lib
    x = C.c_void_p()
    capi.check(lib.dg_p2p_create(ctx.h, layer.canvas * layer.n_q_heads, layer.head_dim, 1, 0, C.byref(x)), "dg_p2p_create")
    capi.check(lib.dg_p2p_set_mode(x, mode), "dg_p2p_set_mode")
    q, kc, vc = util.dev(case, "q"), util.dev(case, "kc"), util.dev(case, "vc")
    ref = util.run_oracle(case)
    for step in range(3):
        out = torch.zeros_like(q)
        capi.check(lib.dg_attn_denoise_split_p2p(ctx.h, C.byref(att.desc), kv.h, P, 0, P, 1, x, util_ptr(q), util_ptr(kc),
                                                 util_ptr(vc), None, None, util_ptr(out)), "dg_attn_denoise_split_p2p")
        ctx.synchronize()
        util.assert_close(util.t2f(out), ref, f"one-rank exchange mode {mode} step {step}")
    r0, n = C.c_uint32(), C.c_uint32()
    capi.check(lib.dg_p2p_slice(x, C.byref(r0), C.byref(n)), "dg_p2p_slice")
    assert (r0.value, n.value) == (0, layer.canvas * layer.n_q_heads)
    capi.check(lib.dg_p2p_reset(x), "dg_p2p_reset")
    out = torch.zeros_like(q)
    capi.check(lib.dg_attn_denoise_split_p2p(ctx.h, C.byref(att.desc), kv.h, P, 0, P, 1, x, util_ptr(q), util_ptr(kc),
                                             util_ptr(vc), None, None, util_ptr(out)), "dg_attn_denoise_split_p2p")
    ctx.synchronize()
    util.assert_close(util.t2f(out), ref, "after reset")
    assert ctx.device_status()[0] == 0
    lib.dg_p2p_destroy(x)
    kv.close()


def util_ptr(t):
    import ctypes as C
    return C.c_void_p(t.data_ptr())


# ------------------------------------------------------------------------------------------
# canvas append inside the attention launch
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("P,Hkv,W,mode,weights,vnorm,ring", [
    (3000, 2, 0, 0, True, 1, 0),                 # 16 query tiles per head, splits in clusters
    (20000, 2, 0, 0, False, 0, 0),               # long key range: the CTA-pair form
    (2048, 8, 0, 0, False, 0, 0),                # configuration 0
    (8192, 8, 1024, 2, True, 0, 0),              # configuration 1
    (10000, 8, 1024, 1, False, 1, 2048),         # sliding layer on a ring
    (100, 8, 0, 0, False, 0, 0),                 # canvas tiles only: every CTA waits for the append at once
    (2048, 4, 0, 0, False, 0, 0),                # 8 query heads on 4 KV heads: 16 query tiles, 8 splits = 16 clusters of
                                                 # 8 CTAs, one more than fit on the device at once
])
def test_in_launch_append_matches_the_two_kernel_step(ctx, P, Hkv, W, mode, weights, vnorm, ring):
    """Steps after the first at the same positions append the canvas K/V inside the attention launch.  Output and
    cache contents must equal, bit for bit, those of the stand-alone append kernel + attention kernel, with every
    split count, with and without the caller's promise of stable inputs, over repeated launches (the append's
    control words reset themselves)."""
    layer = AttnLayer(n_q_heads=8 if Hkv == 4 else 16, n_kv_heads=Hkv, window=W, mask_mode=mode,
                      rope_theta=1e4 if W else 1e6, v_norm=vnorm)
    case = util.make_case(layer, P, seed=P + 5 * Hkv, weights=weights)
    ref = util.run_oracle(case)
    att = CanvasAttention(ctx, layer)
    split_list = (0, 1, 3, 4, 8)

    def fresh():
        if ring:
            kv = KvCache(ctx, layer, ring_slots=ring)
            n0 = max(0, P - (ring - layer.canvas))
            kv.load_prefix(case["kp"][n0:].contiguous().to(DEV), case["vp"][n0:].contiguous().to(DEV), n0)
        else:
            kv, _ = util.gpu_setup(ctx, case)
        return kv

    args = [util.dev(case, n) for n in ("q", "kc", "vc")]
    qw, kw = util.dev(case, "qw"), util.dev(case, "kw")
    # a second input set: the in-launch append must really write what the step was given
    kc2 = torch.roll(args[1], 7, dims=0).contiguous()
    vc2 = torch.roll(args[2], 3, dims=0).contiguous()
    results = {}
    try:
        for fused in (False, True):
            ctx.set_fused_append(fused)
            for stable in ((False, True) if fused else (False,)):
                ctx.set_inputs_stable(stable)
                for splits in split_list:
                    ctx.set_splits(splits)
                    kv = fresh()
                    outs = []
                    att.denoise([kv], [P], args[0][None], args[1][None], args[2][None], qw, kw)     # writes the table
                    for kc, vc in ((args[1], args[2]), (kc2, vc2), (args[1], args[2])):
                        outs.append(att.denoise([kv], [P], args[0][None], kc[None], vc[None], qw, kw)[0].clone())
                    ctx.synchronize()
                    lo = max(P, 0)
                    kk, vv = kv.read(P, layer.canvas)
                    results[(fused, stable, splits)] = (outs, kk.clone(), vv.clone())
                    kv.close()
    finally:
        ctx.set_fused_append(True)
        ctx.set_inputs_stable(False)
        ctx.set_splits(0)
    for splits in split_list:
        base = results[(False, False, splits)]
        util.assert_close(util.t2f(base[0][0]), ref, f"two-kernel step splits={splits}")
        assert torch.equal(base[0][0], base[0][2]) and not torch.equal(base[0][0], base[0][1])
        for stable in (False, True):
            got = results[(True, stable, splits)]
            for a, b in zip(got[0], base[0]):
                assert torch.equal(a, b), f"in-launch append, output differs (stable={stable}, splits={splits})"
            assert torch.equal(got[1], base[1]) and torch.equal(got[2], base[2]), "cache contents differ"
    assert ctx.device_status()[0] == 0
