"""ctypes binding of libdg_attn.so - the C ABI declared in include/dg_attn.h.

Nothing here computes: every call goes to the CUDA library.  If the library is missing the
import of this module fails loudly (there is no CPU fallback).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdg_attn.so")

# status codes / enums (include/dg_attn.h)
DG_OK = 0
DG_ERR_INVALID_ARG = -1
DG_ERR_UNSUPPORTED = -2
DG_ERR_CAPACITY = -3
DG_ERR_CUDA = -4
DG_ERR_NO_DEVICE = -5
DG_ERR_NCCL = -6
DG_ERR_ALIGNMENT = -7
DG_DEV_WAIT_TIMEOUT = 1
DG_DEV_SMEM_LAYOUT = 3
DG_DEV_BAD_SHAPE = 2

MASK_NONE, MASK_WINDOW_UNIFORM, MASK_WINDOW_PER_ROW, MASK_CAUSAL = 0, 1, 2, 3
ROPE_SPLIT_HALF, ROPE_PROPORTIONAL = 0, 1


class LayerDesc(C.Structure):
    """dg_layer_desc"""
    _fields_ = [("n_q_heads", C.c_uint32), ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("canvas", C.c_uint32), ("rotary_dim", C.c_uint32), ("rope_theta", C.c_float),
                ("rms_eps", C.c_float), ("softmax_scale", C.c_float), ("window", C.c_uint32),
                ("mask_mode", C.c_uint32), ("v_norm", C.c_uint32), ("rope_pairing", C.c_uint32)]


_vp = C.c_void_p
_u32 = C.c_uint32
_i32 = C.c_int32
_u64 = C.c_uint64
_pd = C.POINTER(LayerDesc)


class TopkCfg(C.Structure):
    """dg_topk_cfg"""
    _fields_ = [("k_fixed", C.c_uint32), ("k_div", C.c_uint32), ("k_min", C.c_uint32), ("k_max", C.c_uint32)]


class BlockWeights(C.Structure):
    """dg_block_weights of include/dg_attn.h (field for field)."""
    _fields_ = [("input_ln", C.c_void_p), ("w_qkv", C.c_void_p), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("w_o", C.c_void_p), ("post_attn_ln", C.c_void_p), ("hidden", C.c_uint32), ("v_from_k", C.c_uint32)]

# name -> (restype, argtypes); must list every symbol of include/dg_attn.h
SIGNATURES = {
    "dg_ctx_create": (_i32, [_i32, C.POINTER(_vp)]),
    "dg_ctx_destroy": (_i32, [_vp]),
    "dg_ctx_set_stream": (_i32, [_vp, _vp]),
    "dg_ctx_stream": (_vp, [_vp]),
    "dg_ctx_synchronize": (_i32, [_vp]),
    "dg_ctx_last_device_status": (_i32, [_vp, C.POINTER(_u32 * 4)]),
    "dg_ctx_clear_device_status": (_i32, [_vp]),
    "dg_ctx_selftest_wait_timeout": (_i32, [_vp, _u64]),
    "dg_status_str": (C.c_char_p, [_i32]),
    "dg_last_error_message": (C.c_char_p, []),
    "dg_uses_tensor_path": (_i32, [_pd]),
    "dg_ctx_force_general": (_i32, [_vp, _i32]),
    "dg_ctx_set_splits": (_i32, [_vp, _u32]),
    "dg_ctx_set_fused_append": (_i32, [_vp, _i32]),
    "dg_ctx_set_inputs_stable": (_i32, [_vp, _i32]),
    "dg_ctx_set_pair_mode": (_i32, [_vp, _i32]),
    "dg_ctx_max_active_clusters": (_i32, [_vp, _i32, _u32]),
    "dg_attn_denoise_topk": (_i32, [_vp, _pd, _vp, _u32, _vp, _vp, _vp, _vp, _vp, C.POINTER(TopkCfg), _vp]),
    "dg_attn_block": (_i32, [_vp, _pd, C.POINTER(BlockWeights), _vp, _u32, _vp, _vp]),
    "dg_kv_create": (_i32, [_vp, _pd, _u64, C.POINTER(_vp)]),
    "dg_kv_create_ring": (_i32, [_vp, _pd, _u32, C.POINTER(_vp)]),
    "dg_kv_create_shard": (_i32, [_vp, _pd, _u64, _u64, C.POINTER(_vp)]),
    "dg_kv_pos_base": (_u64, [_vp]),
    "dg_kv_ring_mask": (_u32, [_vp]),
    "dg_kv_destroy": (_i32, [_vp]),
    "dg_kv_capacity": (_u64, [_vp]),
    "dg_kv_load_prefix": (_i32, [_vp, _vp, _vp, _u64, _u64]),
    "dg_kv_read": (_i32, [_vp, _vp, _vp, _u64, _u64]),
    "dg_kv_append": (_i32, [_vp, _pd, _vp, _u64, _u32, _vp, _vp, _vp]),
    "dg_kv_append_guarded": (_i32, [_vp, _pd, _vp, _u64, _u32, _vp, _vp, _vp, _u32]),
    "dg_qk_rope_kv": (_i32, [_vp, _pd, _vp, _u32, _vp, _vp, _vp, _vp, _vp]),
    "dg_attention": (_i32, [_vp, _pd, _vp, _u32, _vp, _vp]),
    "dg_attention_static_scratch": (_i32, [_vp, _pd, _vp, _u32, _vp, _vp]),
    "dg_attn_denoise": (_i32, [_vp, _pd, C.POINTER(_vp), C.POINTER(_u32), _u32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dg_attn_denoise_host": (_i32, [_vp, _pd, C.POINTER(_vp), C.POINTER(_u32), _u32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dg_host_pipe_create": (_i32, [_vp, _pd, _u32, _u32, C.POINTER(_vp)]),
    "dg_host_pipe_submit": (_i32, [_vp, _pd, C.POINTER(_vp), C.POINTER(_u32), _u32, _vp, _vp, _vp, _vp, _vp, _vp,
                                   C.POINTER(_u64)]),
    "dg_host_pipe_wait": (_i32, [_vp, _u64]),
    "dg_host_pipe_destroy": (_i32, [_vp]),
    "dg_host_pipe_set_deferred_launch": (_i32, [_vp, _i32]),
    "dg_attn_denoise_bitmap": (_i32, [_vp, _pd, _vp, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dg_attn_partial": (_i32, [_vp, _pd, _vp, _u32, _u32, _u32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dg_attn_merge_local": (_i32, [_vp, _u32, _u32, _u32, _vp, _vp, _vp, _vp]),
    "dg_attn_merge_nccl": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32]),
    "dg_nccl_unique_id": (_i32, [_vp]),
    "dg_nccl_comm_create": (_i32, [_vp, _vp, _i32, _i32, C.POINTER(_vp)]),
    "dg_nccl_comm_destroy": (_i32, [_vp]),
    "dg_nccl_comm_check": (_i32, [_vp]),
    "dg_nccl_comm_abort": (_i32, [_vp]),
    "dg_nccl_all_gather": (_i32, [_vp, _vp, _vp, _vp, _u64]),
    "dg_p2p_create": (_i32, [_vp, _u32, _u32, _i32, _i32, C.POINTER(_vp)]),
    "dg_p2p_set_mode": (_i32, [_vp, _i32]),
    "dg_p2p_slice": (_i32, [_vp, C.POINTER(_u32), C.POINTER(_u32)]),
    "dg_p2p_set_wait_limit": (_i32, [_vp, _u64]),
    "dg_p2p_reset": (_i32, [_vp]),
    "dg_p2p_flush": (_i32, [_vp]),
    "dg_p2p_set_share_q": (_i32, [_vp, _i32]),
    "dg_p2p_phase_stamps": (_i32, [_vp, _vp]),
    "dg_p2p_handle": (_i32, [_vp, _vp]),
    "dg_p2p_connect": (_i32, [_vp, _vp]),
    "dg_p2p_destroy": (_i32, [_vp]),
    "dg_attn_denoise_split_p2p": (_i32, [_vp, _pd, _vp, _u32, _u32, _u32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "dg_host_pipe_submit_split": (_i32, [_vp, _pd, _vp, _u32, _u32, _u32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                         C.POINTER(_u64)]),
    "dg_attn_visibility": (_i32, [_vp, _pd, _u32, _u32, _u32, _i32, _vp]),
    "dg_attn_flops": (C.c_double, [_pd, _u32]),
    "dg_ctx_last_launch_count": (_u32, [_vp]),
    "dg_ctx_kernel_timing": (_i32, [_vp, _i32, _u32]),
    "dg_ctx_phase_stamps": (_i32, [_vp, _vp]),
    "dg_ctx_kernel_time": (_i32, [_vp, C.POINTER(C.c_double), C.POINTER(_u32)]),
}

_lib = None


def load():
    """Load libdg_attn.so and attach signatures.  Raises if the library is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m diffgemma_b200.build` "
            "(this package has no CPU fallback)")
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class DgError(RuntimeError):
    def __init__(self, status: int, where: str):
        lib = load()
        msg = lib.dg_status_str(status).decode()
        detail = lib.dg_last_error_message().decode()
        super().__init__(f"{where}: status {status} ({msg})" + (f": {detail}" if detail else ""))
        self.status = status


def check(status: int, where: str) -> None:
    if status != DG_OK:
        raise DgError(status, where)
