"""Regenerates tests/golden/ref_shader_golden.npz from the reference's OWN shaders.

`make -C oracle ref` compiles src/shaders/attn/attention/attention.metal and
src/shaders/attn/qk_rope_kv/qk_rope_kv.metal of the reference project as C++ (oracle/ref_attention.cpp,
oracle/ref_qk_rope_kv.cpp, oracle/ref_shim/) and this script runs them on seeded inputs.  The stored
outputs are what tests/test_ref_shader_pins.py holds the numpy oracle to, also where the reference tree
(and so the compiled library) is absent.

Run from the repository root, where the reference tree is present:
    make -C oracle ref REF=<reference tree> && python tests/golden/make_ref_shader_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import ref_shader as rs  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_shader_golden.npz")

# visibility cases: (kv_len, window, ring_mask), canvas 16, one key per output dimension
MASK_CASES = [(200, 0, 0), (200, 64, 0), (30, 64, 0), (63, 64, 0), (64, 64, 0), (65, 64, 0), (200, 64, 255),
              (1000, 64, 255), (5000, 100, 255), (100000, 128, 255), (240, 1, 0), (240, 2, 0)]
# the same probe with dims.causal = 1 (the re-prefill of a committed block): plain causal, causal with a
# window, a window shorter than the canvas (its lower bound then cuts canvas keys too), an empty prefix, a ring
CAUSAL_MASK_CASES = [(200, 0, 0), (200, 64, 0), (30, 64, 0), (5, 8, 0), (0, 0, 0), (0, 4, 0), (1000, 64, 255),
                     (240, 1, 0), (240, 2, 0)]
# value cases: name -> (hd, n_q, n_kv, canvas, kv_len, is_full, window, ring_mask, v_aliases_k, seed)
VALUE_CASES = {
    "sliding_short": (256, 8, 2, 8, 40, 0, 1024, 0, 0, 1),
    "sliding_window_cuts": (256, 8, 2, 8, 300, 0, 128, 0, 0, 2),
    "sliding_ring": (256, 8, 2, 8, 2500, 0, 128, 511, 0, 3),
    "full_hd512_valias": (512, 4, 2, 4, 60, 1, 0, 0, 1, 4),
    "full_hd256_vproj": (256, 4, 1, 4, 33, 1, 0, 0, 0, 5),
}
# value cases run with dims.causal = 1, same tuple layout
CAUSAL_VALUE_CASES = {
    "causal_sliding": (256, 8, 2, 8, 300, 0, 128, 0, 0, 6),
    "causal_full_hd256": (256, 4, 1, 8, 33, 1, 0, 0, 0, 7),
}


def grid(rng, shape, step=1 / 64, lim=3.0):
    """Values exactly representable in bf16 and f16: multiples of `step` in [-lim, lim]."""
    n = int(lim / step)
    return (rng.integers(-n, n + 1, size=shape) * step).astype(np.float32)


def mask_inputs(kv_len, window, ring, canvas=16, hd=256, n_q=4, n_kv=2):
    T = kv_len + canvas
    cache = rs.make_cache(ring + 1 if ring else T, n_kv, hd)
    for t in range(max(0, kv_len - 300), T):
        k = np.zeros((1, n_kv, hd), np.float32)
        v = np.zeros((1, n_kv, hd), np.float32)
        v[0, :, t % hd] = 1.0
        rs.cache_store(cache, t, k, v, ring)
    return np.zeros((canvas, n_q, hd), np.uint16), cache


def value_inputs(hd, n_q, n_kv, canvas, kv_len, is_full, window, ring, valias, seed):
    rng = np.random.default_rng(seed)
    q = grid(rng, (canvas, n_q, hd))
    k = grid(rng, (canvas, n_kv, hd))
    v = grid(rng, (canvas, n_kv, hd))
    kp = grid(rng, (kv_len, n_kv, hd), lim=2.0)      # cache-ready prefix K and V
    vp = grid(rng, (kv_len, n_kv, hd), lim=2.0)
    # norm weights: 1/16 on Q keeps the logits O(1) (the reference applies no softmax scale), K near one
    qw = np.full(hd, 1 / 16, np.float32)
    kw = (1.0 + grid(rng, (hd,), step=1 / 32, lim=0.25)).astype(np.float32)
    return q, k, v, kp, vp, qw, kw


def run_value_case(hd, n_q, n_kv, canvas, kv_len, is_full, window, ring, valias, seed, causal=0):
    q, k, v, kp, vp, qw, kw = value_inputs(hd, n_q, n_kv, canvas, kv_len, is_full, window, ring, valias, seed)
    T = kv_len + canvas
    cache = rs.make_cache(ring + 1 if ring else T, n_kv, hd)
    lo = max(0, kv_len - (ring + 1 - canvas)) if ring else 0     # older positions no longer have a slot
    rs.cache_store(cache, lo, kp[lo:], vp[lo:], ring)
    bits = rs.bf16_bits_trunc
    qb, kb, vb = rs.qk_rope_kv(bits(q), bits(k), bits(v), cache, bits(qw), bits(kw), kv_len, is_full, valias,
                               ring_mask=ring)
    out = rs.attention(qb, cache, kv_len, window, causal, ring)
    # the canvas K / V the stage left in the cache (f16), in position order
    slots = [((kv_len + i) & ring) if ring else kv_len + i for i in range(canvas)]
    kc = cache[slots, 0].view(np.float16).astype(np.float32)
    vc = cache[slots, 1].view(np.float16).astype(np.float32)
    return dict(q_out=rs.bf16_to_f32(qb), k_cache=kc, v_cache=vc, out=out)


def main():
    assert rs.available(), "build the reference shaders first: make -C oracle ref REF=<reference tree>"
    store = {}
    for i, (kv_len, window, ring) in enumerate(MASK_CASES):
        q, cache = mask_inputs(kv_len, window, ring)
        out = rs.attention(q, cache, kv_len, window, 0, ring)
        store[f"mask{i}_visible"] = out[:, 0, :] > 0
        print("mask", kv_len, window, ring, "visible per row", int((out[0, 0] > 0).sum()))
    for i, (kv_len, window, ring) in enumerate(CAUSAL_MASK_CASES):
        q, cache = mask_inputs(kv_len, window, ring)
        out = rs.attention(q, cache, kv_len, window, 1, ring)
        store[f"cmask{i}_visible"] = out[:, 0, :] > 0
        print("causal mask", kv_len, window, ring, "visible per row", (out[:, 0] > 0).sum(axis=1).tolist())
    for cases, causal in ((VALUE_CASES, 0), (CAUSAL_VALUE_CASES, 1)):
        for name, cfg in cases.items():
            for key, val in run_value_case(*cfg, causal=causal).items():
                store[f"{name}_{key}"] = val.astype(np.float32)
            print("value", name, "max |out|", float(np.abs(store[f"{name}_out"]).max()))
    np.savez_compressed(OUT, **store)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
