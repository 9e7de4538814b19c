"""Split-KV across GPUs: every rank holds one prefix shard, the per-rank (O, m, l) partials are merged
over peer memory (four forms) or by dg_attn_merge_nccl, and the result must equal the single-GPU oracle.
Also KV-head sharding, and the failure path of the peer-memory exchange (a rank that skips a step makes
the other's bounded wait give up; the group is resynchronised and carries on).  Needs >= 2 GPUs (skipped
otherwise); ranks are child processes, one per GPU, NVLS off, plain peer loads and stores only."""
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
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = Context(rank)
        layer = AttnLayer(n_kv_heads=2, window=W, mask_mode=mode)
        case = util.make_case(layer, P, seed=77)          # same seed on every rank: replicated inputs
        dev = f"cuda:{rank}"
        mode = {"p2p": 0, "p2p-slices": 1, "p2p-allrows": 2, "p2p-push": 3, "p2p-push-pipelined": 4}.get(exchange, 0)
        grp = SplitKvGroup(ctx, layer, exchange="nccl" if exchange == "nccl" else "p2p", p2p_mode=mode)
        t0, t1 = grp.shard_bounds(P)                       # the cuts count the canvas keys of the last rank
        # the push form runs on shard caches (shard + canvas tokens per rank), the others on full-size ones
        kv = grp.make_shard_cache(P) if exchange.startswith("p2p-push") else KvCache(ctx, layer, P + layer.canvas)
        if t1 > t0:                                        # only this rank's shard is resident
            kv.load_prefix(case["kp"][t0:t1].contiguous().to(dev), case["vp"][t0:t1].contiguous().to(dev), t0)
        out = None
        if exchange == "p2p-push-pipelined":
            # the slice of a step is written by the NEXT call: five steps into three rotating outputs, then the flush;
            # every output must then hold the same result (the steps have the same inputs)
            outs = [torch.zeros_like(case["q"].to(dev)) for _ in range(3)]
            q, kc, vc = case["q"].to(dev), case["kc"].to(dev), case["vc"].to(dev)
            for i in range(5):
                grp.denoise(kv, P, q, kc, vc, out=outs[i % 3])
            grp.flush()
            ctx.synchronize()
            r0, n = grp.row_slice()
            flat = [o.reshape(-1, layer.head_dim) for o in outs]
            assert torch.equal(flat[0][r0:r0 + n], flat[1][r0:r0 + n]) and torch.equal(flat[0][r0:r0 + n], flat[2][r0:r0 + n])
            out = grp.gather_rows(outs[1])
        else:
            for _ in range(3):                             # several steps: buffer parities and flags are reused
                out = grp.denoise(kv, P, case["q"].to(dev), case["kc"].to(dev), case["vc"].to(dev))
        if exchange == "p2p-push":
            out = grp.gather_rows(out)                     # every rank holds its row slice only
        ctx.synchronize()
        ref = util.run_oracle(case)
        ret[rank] = util.errors(util.t2f(out), ref) + (float(util.max_abs_tol(ref)),)
        grp.close()
        kv.close()
        ctx.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["p2p", "p2p-slices", "p2p-allrows", "p2p-push", "p2p-push-pipelined", "nccl"])
@pytest.mark.parametrize("P,W,mode,port", [(6000, 0, 0, 29721), (3000, 1024, 1, 29722)])
def test_split_kv_matches_oracle(P, W, mode, port, exchange):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    port += {"p2p": 0, "nccl": 10, "p2p-slices": 20, "p2p-allrows": 30, "p2p-push": 40, "p2p-push-pipelined": 50}[exchange]
    mp.spawn(_rank_main, args=(world, port, P, W, mode, exchange, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank, (mx, mean, tol) in ret.items():
        assert mx <= tol and mean <= 2e-3, (rank, mx, mean)


def _failure_main(rank, world, port, ret):
    """Rank 1 skips one step: rank 0's bounded wait gives up and reports it; both ranks resynchronise;
    a failed host-side call on one rank must not desynchronise the group; clean steps follow."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import util
    from diffgemma_b200 import capi
    from diffgemma_b200.split_kv import SplitKvGroup, plan_shards
    from diffgemma_b200.step_attn import AttnLayer, Context, KvCache
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = Context(rank)
        layer = AttnLayer(n_kv_heads=2)
        P = 3000
        case = util.make_case(layer, P, seed=78)
        dev = f"cuda:{rank}"
        grp = SplitKvGroup(ctx, layer, exchange="p2p", p2p_mode=3)
        kv = grp.make_shard_cache(P)
        t0, t1 = grp.shard_bounds(P)
        kv.load_prefix(case["kp"][t0:t1].contiguous().to(dev), case["vp"][t0:t1].contiguous().to(dev), t0)
        q, kc, vc = case["q"].to(dev), case["kc"].to(dev), case["vc"].to(dev)
        ref = util.run_oracle(case)
        res = {}
        out = grp.gather_rows(grp.denoise(kv, P, q, kc, vc))
        ctx.synchronize()
        res["first"] = util.errors(util.t2f(out), ref)
        # -- a host-side failure on rank 0 only (the visible keys lie outside its shard): nothing is launched,
        #    the step number does not advance, and the repeated call merges with the peer's
        if rank == 0:
            with pytest.raises(capi.DgError) as ei:
                grp.denoise(kv, P + 4096, q, kc, vc)
            res["host_error"] = ei.value.status
        out = grp.gather_rows(grp.denoise(kv, P, q, kc, vc))
        ctx.synchronize()
        res["after_host_error"] = util.errors(util.t2f(out), ref)
        # -- rank 1 sits one step out (between steps, nothing of its own in flight)
        dist.barrier()
        grp.set_wait_limit(40_000_000)                     # about 20 ms
        if rank == 0:
            grp.denoise(kv, P, q, kc, vc)
            st = ctx.device_status()
            res["timeout_status"] = (st[0], st[1])
        dist.barrier()
        grp.set_wait_limit(1_000_000_000)
        grp.reset()                                        # drain, barrier, zero flags, barrier
        res["status_after_reset"] = ctx.device_status()[0]
        for _ in range(3):
            out = grp.gather_rows(grp.denoise(kv, P, q, kc, vc))
        ctx.synchronize()
        res["after_reset"] = util.errors(util.t2f(out), ref)
        res["tol"] = float(util.max_abs_tol(ref))
        ret[rank] = res
        grp.close()
        kv.close()
        ctx.close()
    finally:
        dist.destroy_process_group()


def test_push_exchange_timeout_is_reported_and_group_recovers():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_failure_main, args=(2, 29761, ret), nprocs=2, join=True)
    assert len(ret) == 2
    from diffgemma_b200 import capi
    assert ret[0]["host_error"] == capi.DG_ERR_CAPACITY
    assert ret[0]["timeout_status"] == (capi.DG_DEV_WAIT_TIMEOUT, 4)      # kernel id 4: the merge kernel
    for rank in range(2):
        r = ret[rank]
        assert r["status_after_reset"] == 0
        for key in ("first", "after_host_error", "after_reset"):
            mx, mean = r[key]
            assert mx <= r["tol"] and mean <= 2e-3, (rank, key, mx, mean)


def _pipe_main(rank, world, port, share_q, deferred, ret):
    """The host-buffer pipeline of one rank under split-KV: several steps in flight, each with its own host inputs;
    every rank ends with its row slice of every step's output in host memory."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import util
    from diffgemma_b200.split_kv import SplitKvGroup
    from diffgemma_b200.step_attn import AttnLayer, Context, HostPipe
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = Context(rank)
        layer = AttnLayer(n_kv_heads=2)
        P = 4000
        cases = [util.make_case(layer, P, seed=600 + i) for i in range(7)]     # same seeds on every rank
        dev = f"cuda:{rank}"
        grp = SplitKvGroup(ctx, layer, exchange="p2p", p2p_mode=3)
        grp.set_share_q(share_q)
        kv = grp.make_shard_cache(P)
        t0, t1 = grp.shard_bounds(P)
        kv.load_prefix(cases[0]["kp"][t0:t1].contiguous().to(dev), cases[0]["vp"][t0:t1].contiguous().to(dev), t0)
        pipe = HostPipe(ctx, layer, 1, 3)
        pipe.set_deferred_launch(deferred)
        hosts = [tuple(c[n].contiguous().pin_memory() for n in ("q", "kc", "vc")) + (torch.zeros_like(c["q"]).pin_memory(),)
                 for c in cases]
        tickets = [pipe.submit_split(kv, P, t0, t1, grp.owns_canvas, grp.p2p, q, k, v, o) for q, k, v, o in hosts]
        for t in tickets:
            pipe.wait(t)
        ctx.synchronize()
        r0, n = grp.row_slice()
        worst = (0.0, 0.0)
        for c, (_, _, _, o) in zip(cases, hosts):
            cc = dict(c)
            cc["kp"], cc["vp"] = cases[0]["kp"], cases[0]["vp"]
            ref = util.run_oracle(cc).reshape(-1, layer.head_dim)[r0:r0 + n]
            got = util.t2f(o).reshape(-1, layer.head_dim)
            assert not got[:r0].any() and not got[r0 + n:].any()          # only this rank's slice is copied back
            e = util.errors(got[r0:r0 + n], ref)
            worst = (max(worst[0], e[0]), max(worst[1], e[1]))
        ret[rank] = worst
        pipe.close()
        grp.close()
        kv.close()
        ctx.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("share_q,deferred,port", [(False, False, 29771), (True, False, 29772), (False, True, 29773)])
def test_host_pipe_split_step(share_q, deferred, port):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_pipe_main, args=(2, port, share_q, deferred, ret), nprocs=2, join=True)
    assert len(ret) == 2
    for rank in range(2):
        mx, mean = ret[rank]
        assert mx <= 2e-2 and mean <= 2e-3, (rank, mx, mean)


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
