"""dg_attn_block (input norm, stacked Q|K|V projection, attention, output projection, post-attention norm +
residual) against the CPU restatement of the same stages, through the C ABI."""
import numpy as np
import pytest
import torch

from diffgemma_b200 import capi
from diffgemma_b200.step_attn import AttnBlock, AttnLayer, KvCache
from oracle import attn_oracle as ao
from tests import util

pytestmark = pytest.mark.gpu

# The residual stream is hidden + normed projection, |values| up to about 6: one bf16 step there is 2^-6..2^-5, and a
# projection output that lands on the other side of a rounding boundary moves the result by one such step.
BLOCK_MAX_ABS = 6.3e-2
BLOCK_MEAN_ABS = 4e-3


def _weights(layer, hidden, seed, v_from_k):
    g = torch.Generator().manual_seed(seed)
    nq, nk = layer.n_q_heads * layer.head_dim, layer.n_kv_heads * layer.head_dim
    n_qkv = nq + nk * (1 if v_from_k else 2)
    bf = lambda t: t.to(torch.bfloat16)
    return dict(w_qkv=bf(torch.randn(n_qkv, hidden, generator=g) / hidden ** 0.5),
                w_o=bf(torch.randn(hidden, nq, generator=g) / nq ** 0.5),
                input_ln=bf(1 + 0.1 * torch.randn(hidden, generator=g)),
                post_attn_ln=bf(1 + 0.1 * torch.randn(hidden, generator=g)),
                q_norm=bf(1 + 0.1 * torch.randn(layer.head_dim, generator=g)),
                k_norm=bf(1 + 0.1 * torch.randn(layer.head_dim, generator=g)))


CASES = [
    # the reference's sliding layer: 256 x 2816 -> 4096 + 2048 + 2048, window per row
    ("sliding", dict(n_q_heads=16, n_kv_heads=8, head_dim=256, canvas=256, rope_theta=1e4, window=1024,
                     mask_mode=capi.MASK_WINDOW_PER_ROW), 2816, 3000, False),
    # the benchmark's global layer geometry (head_dim 256, 2 KV heads)
    ("global256", dict(n_q_heads=16, n_kv_heads=2, head_dim=256, canvas=256, rope_theta=1e6), 2816, 2000, False),
    # the reference's full layer: head_dim 512, partial proportional rotary, V = the K projection
    ("full512", dict(n_q_heads=16, n_kv_heads=2, head_dim=512, canvas=256, rotary_dim=128, rope_theta=1e6,
                     softmax_scale=1.0, v_norm=1, rope_pairing=capi.ROPE_PROPORTIONAL), 2816, 1500, True),
    # ragged: 100 canvas rows (one partial 128-row tile), a narrow model
    ("ragged", dict(n_q_heads=4, n_kv_heads=2, head_dim=256, canvas=100, rope_theta=1e4), 256, 300, False),
    # 200 canvas rows: two row tiles, the second partial (the projections run as CTA pairs)
    ("ragged_pair", dict(n_q_heads=4, n_kv_heads=2, head_dim=256, canvas=200, rope_theta=1e4), 512, 700, False),
]


@pytest.mark.parametrize("name,lk,hidden,P,v_from_k", CASES, ids=[c[0] for c in CASES])
def test_attn_block_matches_oracle(name, lk, hidden, P, v_from_k):
    from diffgemma_b200.step_attn import Context
    ctx = Context(0)       # one context serves one geometry
    layer = AttnLayer(**lk)
    case = util.make_case(layer, P, seed=P + hidden)
    w = _weights(layer, hidden, seed=P, v_from_k=v_from_k)
    g = torch.Generator().manual_seed(P + 5)
    h = torch.randn(layer.canvas, hidden, generator=g).to(torch.bfloat16)
    f = util.t2f
    ref = ao.attn_block(f(h), f(w["input_ln"]), f(w["w_qkv"]), f(w["q_norm"]), f(w["k_norm"]), f(w["w_o"]),
                        f(w["post_attn_ln"]), f(case["kp"]), f(case["vp"]), case["desc"], P, v_from_k=v_from_k)
    kv = KvCache(ctx, layer, P + layer.canvas)
    kv.load_prefix(case["kp"].cuda(), case["vp"].cuda(), 0)      # the prefix as the cache holds it
    blk = AttnBlock(ctx, layer, **{k: t.cuda() for k, t in w.items()}, v_from_k=v_from_k)
    hd = h.cuda()
    out = blk.step(kv, P, hd)
    ctx.synchronize()
    got = f(out)
    assert ctx.device_status()[0] == 0
    assert np.isfinite(got).all()
    err = np.abs(got - ref)
    assert err.max() <= BLOCK_MAX_ABS and err.mean() <= BLOCK_MEAN_ABS, (name, float(err.max()), float(err.mean()))
    # the block did something, and the same call gives the same bits
    assert np.abs(got - f(h)).mean() > 0.3
    out2 = blk.step(kv, P, hd)
    ctx.synchronize()
    assert torch.equal(out, out2)
    if 128 < layer.canvas <= 256:
        # the same step with the projections as single-CTA tiles: split-K planes and bf16 rounding are the same
        ctx.set_pair_mode(False)
        out3 = blk.step(kv, P, hd)
        ctx.synchronize()
        ctx.set_pair_mode(None)
        err3 = np.abs(f(out3) - ref)
        assert err3.max() <= BLOCK_MAX_ABS and err3.mean() <= BLOCK_MEAN_ABS, (name, "single", float(err3.max()))
    kv.close()
    ctx.close()
