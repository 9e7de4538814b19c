"""Host logic of the multi-GPU paths on CPU: shard planning, canvas ownership, and the two-step
merge protocol (all-reduce max of m, rescale, all-reduce sum of [O | l]) run by two gloo ranks on
oracle partials.  The CUDA/NCCL implementation of the same protocol is tested with -m gpu."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from diffgemma_b200 import split_kv
from oracle import attn_oracle as ao

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plan_shards_properties():
    for kv_len in [0, 1, 127, 128, 129, 1000, 32768, 131072, 16384 - 64]:
        for world in [1, 2, 4, 8]:
            b = split_kv.plan_shards(kv_len, world)
            assert len(b) == world + 1 and b[0] == 0 and b[-1] == kv_len
            assert all(b[i] <= b[i + 1] for i in range(world))
            assert all(x % 128 == 0 for x in b[1:-1])
    assert split_kv.plan_shards(32768, 8) == [4096 * i for i in range(9)]
    # with the canvas keys of the last rank counted, every rank sweeps a near-equal number of keys
    for kv_len in (32768, 131072, 6000):
        for world in (2, 4, 8):
            b = split_kv.plan_shards(kv_len, world, canvas=256)
            assert b[0] == 0 and b[-1] == kv_len and all(x % 128 == 0 for x in b[1:-1])
            shares = [b[i + 1] - b[i] + (256 if i == world - 1 else 0) for i in range(world)]
            assert max(shares) - min(shares) <= 256, shares
    assert split_kv.canvas_owner(8) == 7


def test_head_shards():
    assert split_kv.head_shards(8, 2) == [(0, 4), (4, 4)]
    assert split_kv.head_shards(8, 8) == [(i, 1) for i in range(8)]
    assert split_kv.head_shards(2, 4) == [(0, 1), (1, 1), (0, 0), (0, 0)]


def _case(seed=3, P=600, Hkv=2, W=0, mode=0):
    d = ao.LayerDesc(n_q_heads=8, n_kv_heads=Hkv, head_dim=64, canvas=16, rotary_dim=64, rope_theta=1e4,
                     window=W, mask_mode=mode)
    rng = np.random.default_rng(seed)
    qn = rng.standard_normal((16, 8, 64)).astype(np.float32)
    K = rng.standard_normal((P + 16, Hkv, 64)).astype(np.float32)
    V = rng.standard_normal((P + 16, Hkv, 64)).astype(np.float32)
    return d, P, qn, K, V


def _rank_main(rank, world, port, W, mode, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d, P, qn, K, V = _case(W=W, mode=mode)
        b = split_kv.plan_shards(P, world)
        inc = rank == split_kv.canvas_owner(world)
        o, m, l = ao.attention(qn, K, V, ao.visibility(d, P, b[rank], b[rank + 1], inc), d, return_partial=True)
        o, m, l = torch.from_numpy(o), torch.from_numpy(m), torch.from_numpy(l)
        # protocol of dg_attn_merge_nccl
        mg = m.clone()
        dist.all_reduce(mg, op=dist.ReduceOp.MAX)
        w = torch.where(torch.isinf(m), torch.zeros_like(m), torch.exp(m - mg))
        pay = torch.cat([o * w[..., None], (l * w)[..., None]], dim=-1)
        dist.all_reduce(pay, op=dist.ReduceOp.SUM)
        lg = pay[..., -1:]
        out = torch.where(lg > 0, pay[..., :-1] / torch.where(lg > 0, lg, torch.ones_like(lg)), torch.zeros_like(lg))
        ref = ao.attention(qn, K, V, ao.visibility(d, P), d)
        ret[rank] = float(np.abs(out.numpy() - ref).max())
    finally:
        dist.destroy_process_group()


def _run(world, W, mode, port):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, port, W, mode, ret), nprocs=world, join=True)
    assert len(ret) == world
    assert max(ret.values()) < 1e-5, dict(ret)


def test_split_merge_two_ranks_global():
    _run(2, 0, 0, 29611)


def test_split_merge_two_ranks_window_leaves_empty_shard():
    # window 64 on a 600-key prefix: rank 0's shard [0, 256) is entirely masked -> m = -inf partial
    _run(2, 64, ao.MASK_WINDOW_UNIFORM, 29612)


def test_stack_units_cover_every_canvas_head_pair_once():
    """KV-head sharding of the batched stack (bench.py: stack_units): over the ranks, every (canvas, KV head)
    pair of a layer is computed exactly once, and every rank gets the same amount of work."""
    sys.path.insert(0, ROOT)
    import bench
    for n_kv in (8, 2):
        for world in (1, 2, 4, 8):
            seen = {}
            sizes = set()
            for r in range(world):
                h0, nh, canv = bench.stack_units(n_kv, 4, world, r)
                sizes.add(nh * len(canv))
                for b in canv:
                    for h in range(h0, h0 + nh):
                        assert (b, h) not in seen, (n_kv, world, r, b, h)
                        seen[(b, h)] = r
            assert len(seen) == 4 * n_kv and len(sizes) == 1, (n_kv, world, sizes)
