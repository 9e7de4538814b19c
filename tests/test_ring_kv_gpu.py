"""Ring KV cache for sliding-window layers (slot = pos & mask) and the guarded append.

Reference behaviour: LayerOffsets::kv_ring_mask (src/metal/step_kernel/mod.rs:161-166) and
StepParams::kv_write_end (src/metal/step_kernel/mod.rs:203-212).  A ring is transparent: the attention
result must equal the oracle's on the same logical keys, whatever the prefix length."""
import ctypes as C

import numpy as np
import pytest
import torch

import util
from diffgemma_b200 import capi
from diffgemma_b200.step_attn import AttnLayer, CanvasAttention, KvCache

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_ring(ctx, case, ring_slots, via_append=False, pair=None, general=False):
    layer, P = case["layer"], case["prefix"]
    kv = KvCache(ctx, layer, ring_slots=ring_slots)
    assert kv.ring_mask == ring_slots - 1
    if P > 0:
        kv.load_prefix(case["kp"].to(DEV), case["vp"].to(DEV), 0)   # only the last ring_slots positions are kept
    att = CanvasAttention(ctx, layer)
    ctx.set_pair_mode(pair)
    ctx.force_general(general)
    try:
        out = att.denoise([kv], [P], util.dev(case, "q")[None], util.dev(case, "kc")[None], util.dev(case, "vc")[None],
                          util.dev(case, "qw"), util.dev(case, "kw"))
        ctx.synchronize()
    finally:
        ctx.set_pair_mode(None)
        ctx.force_general(False)
    res = util.t2f(out[0])
    kv.close()
    return res


@pytest.mark.parametrize("P,Hkv,W,mode,ring,canvas", [
    (300, 8, 1024, capi.MASK_WINDOW_UNIFORM, 2048, 256),      # shorter than the ring: no wrap yet
    (1900, 8, 1024, capi.MASK_WINDOW_UNIFORM, 2048, 256),     # the canvas wraps around the end of the ring
    (3000, 8, 1024, capi.MASK_WINDOW_UNIFORM, 2048, 256),     # prefix longer than the ring
    (10000, 8, 1024, capi.MASK_WINDOW_PER_ROW, 2048, 256),    # several turns of the ring, per-row windows
    (70001, 2, 1024, capi.MASK_WINDOW_UNIFORM, 2048, 256),    # odd length, Hkv = 2 (four query tiles per head)
    (5000, 8, 512, capi.MASK_WINDOW_UNIFORM, 1024, 100),      # smaller ring, ragged canvas
])
def test_ring_cache_matches_oracle(ctx, P, Hkv, W, mode, ring, canvas):
    layer = AttnLayer(n_kv_heads=Hkv, window=W, mask_mode=mode, canvas=canvas, rope_theta=1e4)
    case = util.make_case(layer, P, seed=P + ring)
    ref = util.run_oracle(case)
    util.assert_close(run_ring(ctx, case, ring), ref, "ring, tensor path")
    util.assert_close(run_ring(ctx, case, ring, pair=False), ref, "ring, single-CTA form")
    util.assert_close(run_ring(ctx, case, ring, general=True), ref, "ring, general kernel")
    assert ctx.device_status()[0] == 0


def test_ring_equals_linear_bitwise(ctx):
    """Same keys, same kernel, same tile order: a ring and a linear cache give identical bits."""
    layer = AttnLayer(n_kv_heads=8, window=1024, mask_mode=capi.MASK_WINDOW_UNIFORM, rope_theta=1e4)
    case = util.make_case(layer, 6000, seed=5)
    lin = util.run_gpu(ctx, case)
    ring = run_ring(ctx, case, 2048)
    assert np.array_equal(lin.view(np.uint32), ring.view(np.uint32))


def test_ring_append_and_read_back(ctx):
    """Appending in chunks wraps slot = pos & mask; read() returns positions in order across the wrap."""
    layer = AttnLayer(n_kv_heads=2, window=1024, mask_mode=capi.MASK_WINDOW_UNIFORM, rope_theta=1e4)
    ring = 1024
    n = 2500
    g = torch.Generator(device=DEV).manual_seed(3)
    k = torch.randn(n, 2, 256, generator=g, device=DEV).to(torch.bfloat16)
    v = torch.randn(n, 2, 256, generator=g, device=DEV).to(torch.bfloat16)
    kv_ring = KvCache(ctx, layer, ring_slots=ring)
    kv_lin = KvCache(ctx, layer, n)
    for pos0 in range(0, n, 700):
        kv_ring.append(k[pos0:pos0 + 700], v[pos0:pos0 + 700], pos0)
        kv_lin.append(k[pos0:pos0 + 700], v[pos0:pos0 + 700], pos0)
    # the last `ring` positions, read across the wrap point, equal the linear cache's
    kr, vr = kv_ring.read(n - ring, ring)
    kl, vl = kv_lin.read(n - ring, ring)
    assert torch.equal(kr.view(torch.int16), kl.view(torch.int16))
    assert torch.equal(vr.view(torch.int16), vl.view(torch.int16))
    kv_ring.close()
    kv_lin.close()


def test_guarded_append_skips_the_padded_tail(ctx):
    """Positions >= write_end must not reach the cache: on a ring they would overwrite live slots."""
    layer = AttnLayer(n_kv_heads=2, window=1024, mask_mode=capi.MASK_WINDOW_UNIFORM, rope_theta=1e4)
    ring = 1024
    g = torch.Generator(device=DEV).manual_seed(4)
    k = torch.randn(1200, 2, 256, generator=g, device=DEV).to(torch.bfloat16)
    v = torch.randn(1200, 2, 256, generator=g, device=DEV).to(torch.bfloat16)
    kv = KvCache(ctx, layer, ring_slots=ring)
    kv.append(k[:1000], v[:1000], 0)
    before_k, before_v = kv.read(0, 1000)
    # a padded chunk of 200 tokens at position 1000 of which only 24 are real: 1024.. would wrap onto 0..
    kv.append(k[1000:], v[1000:], 1000, write_end=1024)
    after_k, after_v = kv.read(176, 848)         # slots 176..1023 = positions 176..1023, untouched or newly written
    assert torch.equal(after_k[:824].view(torch.int16), before_k[176:1000].view(torch.int16))
    low_k, low_v = kv.read(1024, 176)            # positions 1024..1199 map to slots 0..175: must still hold 0..175
    assert torch.equal(low_k.view(torch.int16), before_k[:176].view(torch.int16))
    assert torch.equal(low_v.view(torch.int16), before_v[:176].view(torch.int16))
    kv.close()


def test_ring_too_small_is_refused(ctx):
    layer = AttnLayer(n_kv_heads=8, window=1024, mask_mode=capi.MASK_WINDOW_UNIFORM, rope_theta=1e4)
    case = util.make_case(layer, 3000, seed=6)
    with pytest.raises(capi.DgError) as e:
        run_ring(ctx, case, 1024)                # window 1023 + canvas 256 (+ tile alignment) > 1024 slots
    assert e.value.status == capi.DG_ERR_CAPACITY
    lay0 = AttnLayer(n_kv_heads=2)               # all prefix visible: only fits while kv_len + canvas <= ring
    case0 = util.make_case(lay0, 3000, seed=7)
    with pytest.raises(capi.DgError):
        run_ring(ctx, case0, 2048)
    h = C.c_void_p()
    d = layer.c_desc()
    assert ctx.lib.dg_kv_create_ring(ctx.h, C.byref(d), 1000, C.byref(h)) == capi.DG_ERR_INVALID_ARG
