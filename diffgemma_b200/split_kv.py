"""Multi-GPU partitioning of the canvas attention: split-KV (SplitKvGroup) and KV-head sharding
(HeadShardGroup).

One process per GPU.  torch.distributed is used only for rendezvous (to carry the NCCL unique id
to the other ranks); the data path is the CUDA library's own NCCL communicator.

Split-KV: rank r owns the contiguous prefix shard [bounds[r], bounds[r+1]) in its local cache, at
the same absolute key positions; Q and the canvas K/V are replicated.  The canvas keys are counted
by exactly one rank (the last one) so the log-sum-exp merge does not double-count them.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import capi
from .capi import check
from .step_attn import AttnLayer, CanvasAttention, Context, KvCache, _ptr


def plan_shards(kv_len: int, world: int, align: int = 128, canvas: int = 0) -> list[int]:
    """Shard bounds [b_0=0, ..., b_world=kv_len]: contiguous, tile-aligned interior cuts.  With `canvas` keys
    counted by the last rank, the cuts give every rank a near-equal share of ALL keys (prefix + canvas), so the
    rank that also sweeps the canvas gets a shorter prefix shard and the ranks finish together."""
    assert world >= 1 and kv_len >= 0
    total = kv_len + canvas
    bounds = [0]
    for r in range(1, world):
        cut = min(kv_len, (total * r) // world)
        cut = (cut // align) * align
        bounds.append(max(cut, bounds[-1]))
    bounds.append(kv_len)
    return bounds


def canvas_owner(world: int) -> int:
    """The rank whose partial includes the canvas keys."""
    return world - 1


def head_shards(n_kv_heads: int, world: int) -> list[tuple[int, int]]:
    """KV-head sharding: (first_head, n_heads) per rank; ranks beyond n_kv_heads get (0, 0)."""
    per = max(1, n_kv_heads // world) if world <= n_kv_heads else 1
    out = []
    for r in range(world):
        h0 = r * per
        out.append((h0, per) if h0 + per <= n_kv_heads else (0, 0))
    return out


class SplitKvGroup:
    """Split-KV attention over the ranks of a torch.distributed process group.

    exchange="p2p" (default): partials are merged by a kernel over the peers' exchange buffers (CUDA IPC
    mappings, NVLink); p2p_mode 0-2 leave the full output on every rank, p2p_mode 3 (push form) leaves
    every rank with its own row slice (`row_slice`) only, p2p_mode 4 is the push form pipelined over
    consecutive steps (the slice of a step is written by the next `denoise` or by `flush`).  exchange="nccl": two NCCL all-reduces (max of
    m, sum of [O | l]).
    """

    def __init__(self, ctx: Context, layer: AttnLayer, group=None, exchange: str = "p2p", p2p_mode: int = 0):
        assert exchange in ("p2p", "nccl")
        self.ctx = ctx
        self.layer = layer
        self.group = group
        self.exchange = exchange
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.att = CanvasAttention(ctx, layer)
        self.comm = None
        self.p2p = None
        self._bounds = {}             # kv_len -> this rank's (t0, t1): steps repeat at the same positions
        lib = ctx.lib
        on_gpu = dist.get_backend(group) == "nccl"
        xdev = torch.device("cuda", ctx.device) if on_gpu else torch.device("cpu")
        if exchange == "p2p":
            h = C.c_void_p()
            rows = layer.canvas * layer.n_q_heads
            check(lib.dg_p2p_create(ctx.h, rows, layer.head_dim, self.world, self.rank, C.byref(h)), "dg_p2p_create")
            self.p2p = h
            check(lib.dg_p2p_set_mode(h, p2p_mode), "dg_p2p_set_mode")   # 0 automatic, 1 row slices, 2 all rows, 3 push
            self.p2p_mode = p2p_mode
            buf = (C.c_uint8 * 64)()
            check(lib.dg_p2p_handle(h, C.cast(buf, C.c_void_p)), "dg_p2p_handle")
            mine = torch.tensor(list(buf), dtype=torch.uint8, device=xdev)
            gathered = [torch.zeros(64, dtype=torch.uint8, device=xdev) for _ in range(self.world)]
            dist.all_gather(gathered, mine, group=group)   # rendezvous only: carries the IPC handles
            flat = (C.c_uint8 * (64 * self.world))(*[int(b) for t in gathered for b in t.cpu().tolist()])
            check(lib.dg_p2p_connect(h, C.cast(flat, C.c_void_p)), "dg_p2p_connect")
            dist.barrier(group=group)
            return
        self.comm = _nccl_comm(ctx, group)

    def shard_bounds(self, kv_len: int):
        hit = self._bounds.get(kv_len)
        if hit is None:
            b = plan_shards(kv_len, self.world, canvas=self.layer.canvas)
            hit = self._bounds[kv_len] = (b[self.rank], b[self.rank + 1])
        return hit

    @property
    def owns_canvas(self) -> bool:
        return self.rank == canvas_owner(self.world)

    def make_shard_cache(self, kv_len: int, canvas_room: bool = True) -> KvCache:
        """A cache that holds this rank's prefix shard only (plus, on the rank that counts the canvas
        keys, room for the canvas): shard + canvas tokens of HBM instead of the whole prefix."""
        t0, t1 = self.shard_bounds(kv_len)
        cap = max(128, t1 - t0 + (self.layer.canvas if self.owns_canvas and canvas_room else 0))
        return KvCache(self.ctx, self.layer, cap, pos_base=t0)

    def row_slice(self):
        """(first row, number of rows) of the canvas * n_q_heads output rows this rank owns in p2p_mode 3."""
        r0, n = C.c_uint32(), C.c_uint32()
        check(self.ctx.lib.dg_p2p_slice(self.p2p, C.byref(r0), C.byref(n)), "dg_p2p_slice")
        return int(r0.value), int(n.value)

    def set_mode(self, p2p_mode: int) -> None:
        """Switch the exchange form (every rank, between steps; a pipelined step must have been flushed)."""
        check(self.ctx.lib.dg_p2p_set_mode(self.p2p, p2p_mode), "dg_p2p_set_mode")
        self.p2p_mode = p2p_mode

    def set_share_q(self, on: bool) -> None:
        """Host pipeline: every rank copies in only its row slice of Q, the ranks exchange the slices over NVLink."""
        check(self.ctx.lib.dg_p2p_set_share_q(self.p2p, int(on)), "dg_p2p_set_share_q")

    def flush(self) -> None:
        """p2p_mode 4: merge the slice of the last step into the `out` that was given with it."""
        check(self.ctx.lib.dg_p2p_flush(self.p2p), "dg_p2p_flush")

    def set_wait_limit(self, cycles: int) -> None:
        check(self.ctx.lib.dg_p2p_set_wait_limit(self.p2p, cycles), "dg_p2p_set_wait_limit")

    def reset(self) -> None:
        """Resynchronise the group after a timed-out or failed step: drain, barrier, zero this rank's flags
        and step number, barrier (every rank must call it)."""
        try:
            self.ctx.synchronize()
        except capi.DgError:
            pass                      # the device status that led here
        dist.barrier(group=self.group)
        check(self.ctx.lib.dg_p2p_reset(self.p2p), "dg_p2p_reset")
        check(self.ctx.lib.dg_ctx_clear_device_status(self.ctx.h), "dg_ctx_clear_device_status")
        self.ctx.synchronize()
        dist.barrier(group=self.group)

    def gather_rows(self, out):
        """p2p_mode 3 leaves each rank with its row slice of `out` [C,Hq,D]; this collects all slices on every
        rank with one all-gather over the process group (not part of the timed path)."""
        flat = out.reshape(self.layer.canvas * self.layer.n_q_heads, self.layer.head_dim)
        r0, n = self.row_slice()
        cap = (flat.shape[0] + self.world - 1) // self.world
        mine = torch.zeros((cap, flat.shape[1]), dtype=flat.dtype, device=flat.device)
        mine[:n] = flat[r0:r0 + n]
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        full = torch.empty_like(flat)
        for w, part in enumerate(parts):
            a, b = (w * flat.shape[0]) // self.world, ((w + 1) * flat.shape[0]) // self.world
            full[a:b] = part[:b - a]
        return full.reshape(out.shape)

    def denoise(self, kv: KvCache, kv_len: int, q, k, v, qw=None, kw=None, out=None):
        """q: [C,Hq,D], k, v: [C,Hkv,D] (replicated inputs).  Every rank gets the full bf16 output."""
        t0, t1 = self.shard_bounds(kv_len)
        out = torch.zeros_like(q) if out is None else out
        if self.exchange == "p2p":
            check(self.ctx.lib.dg_attn_denoise_split_p2p(self.ctx.h, C.byref(self.att.desc), kv.h, kv_len, t0, t1,
                                                         int(self.owns_canvas), self.p2p,
                                                         _ptr(q), _ptr(k), _ptr(v), _ptr(qw), _ptr(kw), _ptr(out)),
                  "dg_attn_denoise_split_p2p")
            return out
        o, m, l = self.att.partial(kv, kv_len, t0, t1, self.rank == canvas_owner(self.world), q, k, v, qw, kw)
        rows = self.layer.canvas * self.layer.n_q_heads
        check(self.ctx.lib.dg_attn_merge_nccl(self.ctx.h, self.comm, _ptr(o), _ptr(m), _ptr(l), _ptr(out), rows,
                                              self.layer.head_dim), "dg_attn_merge_nccl")
        self._keep = (o, m, l)   # keep the partial buffers alive until the stream has consumed them
        return out

    def close(self):
        if self.p2p:
            self.ctx.synchronize()
            if dist.is_initialized():
                dist.barrier(group=self.group)   # nobody unmaps a buffer a peer's kernel may still read
            self.ctx.lib.dg_p2p_destroy(self.p2p)
            self.p2p = None
        if self.comm:
            self.ctx.synchronize()
            self.ctx.lib.dg_nccl_comm_destroy(self.comm)
            self.comm = None


def _nccl_comm(ctx: Context, group):
    """The library's own NCCL communicator over the ranks of `group` (torch.distributed carries the id)."""
    lib = ctx.lib
    rank = dist.get_rank(group)
    ident = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = (C.c_uint8 * 128)()
        check(lib.dg_nccl_unique_id(C.cast(buf, C.c_void_p)), "dg_nccl_unique_id")
        ident = torch.tensor(list(buf), dtype=torch.uint8)
    dev = torch.device("cuda", ctx.device) if dist.get_backend(group) == "nccl" else torch.device("cpu")
    ident = ident.to(dev)
    dist.broadcast(ident, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    idb = (C.c_uint8 * 128)(*ident.cpu().tolist())
    comm = C.c_void_p()
    check(lib.dg_nccl_comm_create(ctx.h, C.cast(idb, C.c_void_p), dist.get_world_size(group), rank, C.byref(comm)),
          "dg_nccl_comm_create")
    return comm


class HeadShardGroup:
    """KV-head sharding over the ranks of a process group: rank r owns KV heads [r*Hkv/N, (r+1)*Hkv/N) and their
    query heads, with its own cache of those heads.  No softmax merge is needed; one all-gather of the output
    head slices gives every rank the full result.  n_kv_heads must be a multiple of the world size."""

    def __init__(self, ctx: Context, layer: AttnLayer, group=None):
        self.ctx, self.group = ctx, group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        assert layer.n_kv_heads % self.world == 0, "n_kv_heads must be a multiple of the number of ranks"
        self.full = layer
        self.G = layer.n_q_heads // layer.n_kv_heads
        self.kv_per = layer.n_kv_heads // self.world
        self.q_per = self.kv_per * self.G
        from dataclasses import replace
        self.local = replace(layer, n_q_heads=self.q_per, n_kv_heads=self.kv_per)   # what this rank computes
        self.att = CanvasAttention(ctx, self.local)
        self.comm = _nccl_comm(ctx, group)

    def kv_heads(self):
        h0 = self.rank * self.kv_per
        return h0, h0 + self.kv_per

    def denoise(self, kv: KvCache, kv_len: int, q, k, v, qw=None, kw=None):
        """q: [C,Hq,D], k, v: [C,Hkv,D] (full, replicated).  kv: this rank's cache (its KV heads only).
        Returns the full [C,Hq,D] output on every rank."""
        h0, h1 = self.kv_heads()
        ql = q[:, h0 * self.G:h1 * self.G].contiguous()
        kl = k[:, h0:h1].contiguous()
        vl = v[:, h0:h1].contiguous()
        ol = self.att.denoise([kv], [kv_len], ql[None], kl[None], vl[None], qw, kw)[0]     # [C, q_per, D]
        gathered = torch.empty((self.world,) + tuple(ol.shape), dtype=ol.dtype, device=ol.device)
        check(self.ctx.lib.dg_nccl_all_gather(self.ctx.h, self.comm, _ptr(ol), _ptr(gathered), ol.numel() * 2),
              "dg_nccl_all_gather")
        # [N, C, q_per, D] -> [C, N * q_per, D]
        return gathered.permute(1, 0, 2, 3).reshape(ol.shape[0], self.world * self.q_per, ol.shape[2])

    def close(self):
        if self.comm:
            self.ctx.synchronize()
            self.ctx.lib.dg_nccl_comm_destroy(self.comm)
            self.comm = None
