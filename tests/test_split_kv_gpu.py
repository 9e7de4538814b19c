"""Split-KV across GPUs over NCCL: every rank holds one prefix shard, the per-rank (O, m, l) partials
are merged by dg_attn_merge_nccl, and the result must equal the single-GPU oracle.  Needs >= 2 GPUs
(skipped otherwise); ranks are child processes, one per GPU."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, P, W, mode, exchange, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import util
    from diffgemma_b200.split_kv import SplitKvGroup, plan_shards
    from diffgemma_b200.step_attn import AttnLayer, Context, KvCache
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = Context(rank)
        layer = AttnLayer(n_kv_heads=2, window=W, mask_mode=mode)
        case = util.make_case(layer, P, seed=77)          # same seed on every rank: replicated inputs
        dev = f"cuda:{rank}"
        b = plan_shards(P, world)
        kv = KvCache(ctx, layer, P + layer.canvas)
        t0, t1 = b[rank], b[rank + 1]
        if t1 > t0:                                        # only this rank's shard is resident
            kv.load_prefix(case["kp"][t0:t1].contiguous().to(dev), case["vp"][t0:t1].contiguous().to(dev), t0)
        mode = {"p2p": 0, "p2p-slices": 1, "p2p-allrows": 2}.get(exchange, 0)
        grp = SplitKvGroup(ctx, layer, exchange="nccl" if exchange == "nccl" else "p2p", p2p_mode=mode)
        out = None
        for _ in range(3):                                 # several steps: buffer parities and flags are reused
            out = grp.denoise(kv, P, case["q"].to(dev), case["kc"].to(dev), case["vc"].to(dev))
        ctx.synchronize()
        ref = util.run_oracle(case)
        ret[rank] = util.errors(util.t2f(out), ref) + (float(util.max_abs_tol(ref)),)
        grp.close()
        kv.close()
        ctx.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["p2p", "p2p-slices", "p2p-allrows", "nccl"])
@pytest.mark.parametrize("P,W,mode,port", [(6000, 0, 0, 29721), (3000, 1024, 1, 29722)])
def test_split_kv_matches_oracle(P, W, mode, port, exchange):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    port += {"p2p": 0, "nccl": 10, "p2p-slices": 20, "p2p-allrows": 30}[exchange]
    mp.spawn(_rank_main, args=(world, port, P, W, mode, exchange, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank, (mx, mean, tol) in ret.items():
        assert mx <= tol and mean <= 2e-3, (rank, mx, mean)


def _head_shard_main(rank, world, port, P, W, mode, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import util
    from diffgemma_b200.split_kv import HeadShardGroup
    from diffgemma_b200.step_attn import AttnLayer, Context, KvCache
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = Context(rank)
        layer = AttnLayer(n_kv_heads=8, window=W, mask_mode=mode, rope_theta=1e4 if W else 1e6)
        case = util.make_case(layer, P, seed=91)          # same seed on every rank: replicated inputs
        dev = f"cuda:{rank}"
        grp = HeadShardGroup(ctx, layer)
        h0, h1 = grp.kv_heads()
        kv = KvCache(ctx, grp.local, P + layer.canvas)     # this rank's KV heads only
        kv.load_prefix(case["kp"][:, h0:h1].contiguous().to(dev), case["vp"][:, h0:h1].contiguous().to(dev), 0)
        out = None
        for _ in range(2):
            out = grp.denoise(kv, P, case["q"].to(dev), case["kc"].to(dev), case["vc"].to(dev))
        ctx.synchronize()
        ref = util.run_oracle(case)
        ret[rank] = util.errors(util.t2f(out), ref) + (float(util.max_abs_tol(ref)),)
        grp.close()
        kv.close()
        ctx.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("P,W,mode,port", [(2048, 0, 0, 29741), (8192, 1024, 1, 29742)])
def test_kv_head_sharding_matches_oracle(P, W, mode, port):
    """Rank r owns KV heads [r*Hkv/N, (r+1)*Hkv/N): no softmax merge, one all-gather of output head slices."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_head_shard_main, args=(world, port, P, W, mode, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        mx, mean, tol = ret[rank]
        assert mx <= tol and mean <= 2e-3, (rank, mx, mean)
