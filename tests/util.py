"""Shared helpers of the parity tests: seeded cases, oracle runs, library runs, error metrics."""
from __future__ import annotations

import numpy as np
import torch

from diffgemma_b200 import synthetic
from diffgemma_b200.step_attn import AttnLayer, CanvasAttention, KvCache
from oracle import attn_oracle as ao

# acceptance for bf16 I/O with fp32 accumulation against the fp32 oracle
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3


def t2f(t: torch.Tensor) -> np.ndarray:
    """bf16 torch tensor -> float32 numpy (exact)."""
    return t.detach().cpu().to(torch.float32).numpy()


def f2t(a: np.ndarray, device="cpu") -> torch.Tensor:
    """float32 numpy (bf16-representable) -> bf16 torch tensor."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).to(device)


def oracle_desc(layer: AttnLayer) -> ao.LayerDesc:
    return ao.LayerDesc(layer.n_q_heads, layer.n_kv_heads, layer.head_dim, layer.canvas, layer.rotary_dim,
                        layer.rope_theta, layer.rms_eps, layer.softmax_scale, layer.window, layer.mask_mode,
                        layer.v_norm, layer.rope_pairing)


def make_case(layer: AttnLayer, prefix: int, seed: int, weights: bool = False):
    """Seeded case: raw canvas q/k/v, cache-ready prefix K (normed + roped by the oracle) and V."""
    q, kc, vc, kp_raw, vp = synthetic.draw(layer, prefix, seed)
    d = oracle_desc(layer)
    qw = kw = None
    if weights:
        g = torch.Generator().manual_seed(seed + 77)
        qw = (1.0 + 0.1 * torch.randn(layer.head_dim, generator=g)).to(torch.bfloat16)
        kw = (1.0 + 0.1 * torch.randn(layer.head_dim, generator=g)).to(torch.bfloat16)
    kp = ao.prepare_prefix_k(t2f(kp_raw), d, 0, None if kw is None else t2f(kw)) if prefix > 0 else \
        np.zeros((0, layer.n_kv_heads, layer.head_dim), np.float32)
    return dict(layer=layer, desc=d, prefix=prefix, q=q, kc=kc, vc=vc, kp=f2t(kp), vp=vp, qw=qw, kw=kw)


def run_oracle(case, attend=None, partial=None):
    d = case["desc"]
    qw = None if case["qw"] is None else t2f(case["qw"])
    kw = None if case["kw"] is None else t2f(case["kw"])
    P = case["prefix"]
    if partial is None:
        return ao.denoise_attention(t2f(case["q"]), t2f(case["kc"]), t2f(case["vc"]), t2f(case["kp"]),
                                    t2f(case["vp"]), d, P, qw, kw, attend)
    t0, t1, inc = partial
    qn, kn, vn = ao.qk_rope_kv(t2f(case["q"]), t2f(case["kc"]), t2f(case["vc"]), qw, kw, d, P)
    K = np.concatenate([t2f(case["kp"])[:P], kn], axis=0)
    V = np.concatenate([t2f(case["vp"])[:P], vn], axis=0)
    return ao.attention(qn, K, V, ao.visibility(d, P, t0, t1, inc), d, return_partial=True)


def gpu_setup(ctx, case, extra_capacity: int = 0):
    layer = case["layer"]
    kv = KvCache(ctx, layer, case["prefix"] + layer.canvas + extra_capacity)
    if case["prefix"] > 0:
        kv.load_prefix(case["kp"].cuda(), case["vp"].cuda(), 0)
    return kv, CanvasAttention(ctx, layer)


def dev(case, name):
    t = case[name]
    return None if t is None else t.cuda()


def run_gpu(ctx, case):
    kv, att = gpu_setup(ctx, case)
    out = att.denoise([kv], [case["prefix"]], dev(case, "q")[None], dev(case, "kc")[None], dev(case, "vc")[None],
                      dev(case, "qw"), dev(case, "kw"))
    ctx.synchronize()
    res = t2f(out[0])
    kv.close()
    return res


def errors(got: np.ndarray, ref: np.ndarray):
    diff = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    return float(diff.max()), float(diff.mean())


def max_abs_tol(ref: np.ndarray) -> float:
    """The bound of the STRESS cases only (unscaled logits, huge or tiny values): 2e-2 for outputs of
    magnitude <= 2.  bf16 has 8 significant bits, so rounding the OUTPUT alone costs up to
    2^-9 * 2^ceil(log2|o|): 7.8e-3 below 2, 1.6e-2 in [2, 4), 3.1e-2 in [4, 8); there the bound grows in
    proportion to the largest reference magnitude beyond 2."""
    return MAX_ABS_TOL * max(1.0, float(np.abs(ref).max()) / 2.0)


# every comparison that needed more than the flat 2e-2: (what, max-abs, bound used)
RELAXED = []


def assert_close(got, ref, what="", stress=False):
    """max-abs <= 2e-2 and mean-abs <= 2e-3, flat.  Only a test that declares itself a stress case
    (softmax_scale = 1 on N(0,1) inputs, values scaled by 2^14, ...) may use the bound that grows with the
    output magnitude; such comparisons are recorded in RELAXED when they really exceeded 2e-2."""
    mx, mean = errors(got, ref)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    tol = max_abs_tol(ref) if stress else MAX_ABS_TOL
    if mx > MAX_ABS_TOL and stress:
        RELAXED.append((what, mx, tol))
    assert mx <= tol and mean <= MEAN_ABS_TOL, f"{what}: max-abs {mx:.3e} (tol {tol:.2e}) mean-abs {mean:.3e}"
    return mx, mean
