"""Regenerates tests/golden/attn_golden.npz.

The reference stores no output vectors for its attention fixtures (their expected values are
recomputed by its CPU oracle at test time) and its code cannot be built in this environment, so
these vectors are produced by this repository's numpy oracle on the reference's closed-form fixture
inputs (src/shaders/attn/attention/mod.rs:59-184 in the reference project).  They pin the oracle
against regressions; the independent pins are the known-answer tests in tests/test_oracle_pins.py.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import attn_oracle as ao  # noqa: E402
from test_oracle_pins import REF_FIXTURES, _ref_fixture  # noqa: E402


def main():
    out = {}
    for name, (canvas, hq, hkv, hd, kv_len, kind) in REF_FIXTURES.items():
        q, K, V = _ref_fixture(canvas, hq, hkv, hd, kv_len, kind)
        d = ao.LayerDesc(n_q_heads=hq, n_kv_heads=hkv, head_dim=hd, canvas=canvas, rotary_dim=hd, softmax_scale=1.0)
        out[name] = ao.attention(q, K, V, ao.visibility(d, kv_len), d)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz"), **out)
    for k, v in out.items():
        print(k, v.shape, float(np.abs(v).max()))


if __name__ == "__main__":
    main()
