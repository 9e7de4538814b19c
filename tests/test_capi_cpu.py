"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, validates
arguments, counts FLOPs like the benchmark tables, and refuses to run without a GPU."""
import ctypes as C
import os
import re

import pytest
import torch

from diffgemma_b200 import capi
from diffgemma_b200.step_attn import AttnLayer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dg_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dg_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(capi.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/dg_attn.h but not exported"
    assert set(names) == set(capi.SIGNATURES), set(names) ^ set(capi.SIGNATURES)


def test_status_strings():
    lib = capi.load()
    assert lib.dg_status_str(0) == b"ok"
    assert b"capacity" in lib.dg_status_str(capi.DG_ERR_CAPACITY)
    assert b"timed out" in lib.dg_status_str(capi.DG_DEV_WAIT_TIMEOUT)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_gpu_fails_loudly():
    lib = capi.load()
    h = C.c_void_p()
    st = lib.dg_ctx_create(0, C.byref(h))
    assert st == capi.DG_ERR_NO_DEVICE and not h
    assert b"no CPU path" in lib.dg_last_error_message()
    with pytest.raises(capi.DgError):
        capi.check(st, "dg_ctx_create")


def test_flops_match_benchmark_tables():
    """4*C*Hq*T_vis*D per layer-step (masked keys not counted)."""
    cases = [
        (AttnLayer(n_kv_heads=8), 2048, 9.664e9),
        (AttnLayer(n_kv_heads=8, window=1024, mask_mode=capi.MASK_WINDOW_PER_ROW), 8192, 4.830e9),
        (AttnLayer(n_kv_heads=8, window=1024, mask_mode=capi.MASK_WINDOW_UNIFORM), 8192, 5.365e9),
        (AttnLayer(n_kv_heads=2), 32768, 138.51e9),
        (AttnLayer(n_kv_heads=2), 131072, 550.83e9),
        (AttnLayer(n_kv_heads=2), 16384, 69.79e9),
    ]
    for layer, P, want in cases:
        assert abs(layer.flops(P) - want) / want < 2e-3, (P, layer.flops(P), want)


def test_desc_validation_needs_no_gpu():
    lib = capi.load()
    bad = AttnLayer(n_q_heads=16, n_kv_heads=3).c_desc()
    assert lib.dg_attn_flops(C.byref(bad), 10) == 0.0
    assert lib.dg_uses_tensor_path(C.byref(bad)) == 0
    assert lib.dg_uses_tensor_path(C.byref(AttnLayer().c_desc())) == 1
    assert lib.dg_uses_tensor_path(C.byref(AttnLayer(head_dim=512, rotary_dim=128).c_desc())) == 1   # full layers
    assert lib.dg_uses_tensor_path(C.byref(AttnLayer(head_dim=128, rotary_dim=128).c_desc())) == 0
    assert lib.dg_ctx_synchronize(None) == capi.DG_ERR_INVALID_ARG
    assert lib.dg_kv_destroy(None) == capi.DG_OK
