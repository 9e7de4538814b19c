"""Seeded synthetic inputs and the benchmark configurations for the canvas-attention path.

The reference measures this op on no public dataset; the five configurations below are the
benchmark's own shapes.  Inputs are i.i.d. N(0,1) drawn on the CPU by a seeded torch generator in
the order q, k_canvas, v_canvas, k_prefix, v_prefix, then rounded to bf16.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import capi
from .step_attn import AttnLayer

SEED_BASE = 20261125


@dataclass
class BenchConfig:
    name: str
    prefix: int
    layer: AttnLayer
    batch: int = 1
    note: str = ""


def configs() -> dict[int, BenchConfig]:
    return {
        0: BenchConfig("cfg0_global_p2048", 2048, AttnLayer(n_kv_heads=8, rope_theta=1e6)),
        1: BenchConfig("cfg1_sliding_p8192_w1024", 8192,
                       AttnLayer(n_kv_heads=8, rope_theta=1e4, window=1024, mask_mode=capi.MASK_WINDOW_PER_ROW)),
        2: BenchConfig("cfg2_global_p32768", 32768, AttnLayer(n_kv_heads=2, rope_theta=1e6)),
        4: BenchConfig("cfg4_global_p131072", 131072, AttnLayer(n_kv_heads=2, rope_theta=1e6)),
        # not one of the benchmark's configurations: the reference's real full-attention layer geometry
        # (head_dim 512, rotary on 128 dims with proportional pairing, V normed without weight)
        5: BenchConfig("ref_full_layer_hd512_p32768", 32768,
                       AttnLayer(n_kv_heads=2, head_dim=512, rotary_dim=128, rope_theta=1e6, v_norm=1,
                                 rope_pairing=capi.ROPE_PROPORTIONAL)),
    }


def stack_layers() -> list[AttnLayer]:
    """The 30-layer pattern of configuration 3: global layers at indices 5, 11, 17, 23, 29
    (src/metal/step_kernel/mod.rs:127 in the reference project), sliding layers elsewhere."""
    out = []
    for i in range(30):
        if i % 6 == 5:
            out.append(AttnLayer(n_kv_heads=2, rope_theta=1e6))
        else:
            out.append(AttnLayer(n_kv_heads=8, rope_theta=1e4, window=1024, mask_mode=capi.MASK_WINDOW_UNIFORM))
    return out


def draw(layer: AttnLayer, prefix: int, seed: int, with_prefix: bool = True):
    """Returns bf16 CPU tensors q [C,Hq,D], k_c, v_c [C,Hkv,D], k_p, v_p [P,Hkv,D] (raw, pre-norm)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    C, Hq, Hkv, D = layer.canvas, layer.n_q_heads, layer.n_kv_heads, layer.head_dim

    def n(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float32).to(torch.bfloat16)

    q = n(C, Hq, D)
    k_c = n(C, Hkv, D)
    v_c = n(C, Hkv, D)
    if not with_prefix:
        return q, k_c, v_c, None, None
    k_p = n(prefix, Hkv, D)
    v_p = n(prefix, Hkv, D)
    return q, k_c, v_c, k_p, v_p


def config_seed(cfg: int, canvas_idx: int = 0, step: int = 0) -> int:
    return SEED_BASE + 1000 * cfg + canvas_idx + step
