"""ctypes access to the reference's own shaders compiled for the CPU (oracle/_ref/libdg_ref_shaders.so).

Test infrastructure only: used by tests and by tests/golden/make_ref_shader_golden.py to pin the
oracle against the reference itself.  The library is built by `make -C oracle ref` where the reference
tree is present.

Data conventions of the reference (src/shaders/include/attention_device.metal, arena.metal):
activations (q, k, v, out) are bf16 bit patterns and stores TRUNCATE f32 to bf16; the KV cache holds
f16, slot-major: slot s = [K heads: n_kv x hd][V heads: n_kv x hd], slot of position t = t or
t & ring_mask."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libdg_ref_shaders.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(LIB_PATH)
        u16p, u32 = C.POINTER(C.c_uint16), C.c_uint32
        L.ref_attention.restype = C.c_int
        L.ref_attention.argtypes = [u16p, u16p, u16p] + [u32] * 9
        L.ref_qk_rope_kv.restype = C.c_int
        L.ref_qk_rope_kv.argtypes = [u16p] * 6 + [u32] * 9
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint16))


def bf16_bits_trunc(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns by truncation (the reference's arena store)."""
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def make_cache(n_slots: int, n_kv: int, hd: int) -> np.ndarray:
    """Zeroed cache region [slot][K|V][n_kv][hd] of f16 bit patterns."""
    return np.zeros((n_slots, 2, n_kv, hd), np.uint16)


def cache_store(cache: np.ndarray, pos0: int, k: np.ndarray, v: np.ndarray, ring_mask: int = 0) -> None:
    """Write k, v [n][n_kv][hd] (f32, rounded to f16) at positions pos0.. (slot = pos or pos & ring_mask)."""
    for i in range(k.shape[0]):
        s = (pos0 + i) & ring_mask if ring_mask else pos0 + i
        cache[s, 0] = k[i].astype(np.float16).view(np.uint16)
        cache[s, 1] = v[i].astype(np.float16).view(np.uint16)


def attention(q_bits: np.ndarray, cache: np.ndarray, kv_len: int, window: int = 0, causal: int = 0,
              ring_mask: int = 0) -> np.ndarray:
    """The reference's `attention` kernel.  q_bits: [canvas][n_q][hd] bf16 bits.  Returns f32 [canvas][n_q][hd]
    (the kernel's bf16 output widened)."""
    canvas, n_q, hd = q_bits.shape
    n_kv = cache.shape[2]
    q_bits = np.ascontiguousarray(q_bits, np.uint16)
    cache = np.ascontiguousarray(cache, np.uint16)
    out = np.zeros_like(q_bits)
    lanes = 32 if hd <= 256 else 64
    r = lib().ref_attention(_p(q_bits), _p(cache), _p(out), canvas, n_q, n_kv, hd, kv_len, window, causal, ring_mask, lanes)
    assert r == 0, "ref_attention refused the geometry"
    return bf16_to_f32(out)


def qk_rope_kv(q_bits, k_bits, v_bits, cache, q_norm_bits, k_norm_bits, kv_len: int, is_full: int, v_aliases_k: int,
               kv_write_end: int = 0xFFFFFFFF, ring_mask: int = 0):
    """The reference's `qk_rope_kv` kernel, in place on copies.  Returns (q, k, v) bf16 bits after the call; the
    cache is updated in place."""
    canvas, n_q, hd = q_bits.shape
    n_kv = k_bits.shape[1]
    q = np.ascontiguousarray(q_bits, np.uint16).copy()
    k = np.ascontiguousarray(k_bits, np.uint16).copy()
    v = np.ascontiguousarray(v_bits, np.uint16).copy()
    assert cache.flags["C_CONTIGUOUS"] and cache.dtype == np.uint16
    qn = np.ascontiguousarray(q_norm_bits, np.uint16)
    kn = np.ascontiguousarray(k_norm_bits, np.uint16)
    r = lib().ref_qk_rope_kv(_p(q), _p(k), _p(v), _p(cache), _p(qn), _p(kn), canvas, n_q, n_kv, hd, is_full, v_aliases_k,
                             kv_len, kv_write_end, ring_mask)
    assert r == 0
    return q, k, v
