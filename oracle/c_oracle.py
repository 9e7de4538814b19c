"""ctypes binding of the C++/OpenMP oracle twin (oracle/attn_oracle.cpp).

TEST INFRASTRUCTURE ONLY - the checker and the timed CPU baseline; the shipped library
never loads it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libdg_oracle.so")


class DgoDesc(C.Structure):
    _fields_ = [("n_q_heads", C.c_uint32), ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("canvas", C.c_uint32), ("rotary_dim", C.c_uint32), ("rope_theta", C.c_float),
                ("rms_eps", C.c_float), ("softmax_scale", C.c_float), ("window", C.c_uint32),
                ("mask_mode", C.c_uint32), ("v_norm", C.c_uint32), ("rope_pairing", C.c_uint32)]


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "attn_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libdg_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        L.dgo_rope_inv_freq.argtypes = [C.c_uint32, C.c_uint32, C.c_float, C.c_void_p]
        L.dgo_qk_rope_kv.argtypes = [C.POINTER(DgoDesc), C.c_uint32] + [C.c_void_p] * 8
        L.dgo_visibility.argtypes = [C.POINTER(DgoDesc), C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, C.c_void_p]
        L.dgo_attention.argtypes = ([C.POINTER(DgoDesc), C.c_uint32] + [C.c_void_p] * 6 +
                                    [C.c_uint32, C.c_uint32, C.c_int, C.c_uint32, C.c_uint32] +
                                    [C.c_void_p] * 3 + [C.c_int])
        L.dgo_attention.restype = C.c_int
        L.dgo_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _desc(d) -> DgoDesc:
    return DgoDesc(d.n_q_heads, d.n_kv_heads, d.head_dim, d.canvas, d.rotary_dim, d.rope_theta,
                   d.rms_eps, d.softmax_scale, d.window, d.mask_mode, d.v_norm, d.rope_pairing)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def rope_inv_freq(rotary_dim, head_dim, theta):
    out = np.empty(max(1, rotary_dim // 2), np.float32)
    lib().dgo_rope_inv_freq(rotary_dim, head_dim, theta, _p(out))
    return out[: rotary_dim // 2]


def qk_rope_kv(desc, kv_len, q_bits, k_bits, v_bits, qw_bits=None, kw_bits=None):
    """All arrays are uint16 bf16 bit patterns, [C,H,D]."""
    qn = np.empty_like(q_bits)
    kn = np.empty_like(k_bits)
    vn = np.empty_like(v_bits)
    dd = _desc(desc)
    lib().dgo_qk_rope_kv(C.byref(dd), kv_len, _p(q_bits), _p(k_bits), _p(v_bits), _p(qw_bits),
                         _p(kw_bits), _p(qn), _p(kn), _p(vn))
    return qn, kn, vn


def visibility(desc, kv_len, t0=0, t1=None, include_canvas=True):
    T = kv_len + desc.canvas
    out = np.empty((desc.canvas, T), np.uint8)
    dd = _desc(desc)
    lib().dgo_visibility(C.byref(dd), kv_len, t0, kv_len if t1 is None else t1, int(include_canvas), _p(out))
    return out.astype(bool)


def attention(desc, kv_len, qn, kn, vn, kp, vp, attend=None, t0=0, t1=None, include_canvas=True,
              row_begin=0, row_end=None, partial=False, n_threads=0):
    """bf16-bit inputs; kp/vp are [kv_len,Hkv,D].  Returns O fp32 (or (O_unnorm, m, l))."""
    Cn, Hq, D = desc.canvas, desc.n_q_heads, desc.head_dim
    out = np.zeros((Cn, Hq, D), np.float32)
    m = np.full((Cn, Hq), -np.inf, np.float32) if partial else None
    l = np.zeros((Cn, Hq), np.float32) if partial else None
    att = None if attend is None else np.ascontiguousarray(attend, dtype=np.uint8)
    dd = _desc(desc)
    lib().dgo_attention(C.byref(dd), kv_len, _p(qn), _p(kn), _p(vn), _p(kp), _p(vp), _p(att), t0,
                        kv_len if t1 is None else t1, int(include_canvas), row_begin,
                        Cn if row_end is None else row_end, _p(out), _p(m), _p(l), n_threads)
    return (out, m, l) if partial else out


def num_threads() -> int:
    return lib().dgo_num_threads()
