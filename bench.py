"""Benchmark of the denoise-step canvas attention.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--cfg 2]

A "step" is one pass of the hot path (qk_rope_kv append + fused attention) over one canvas of the
32k-prefix global-layer configuration (Hq=16, Hkv=2, head_dim=256, canvas 256, prefix 32768).  With
N > 1 (launched by torchrun, one rank per GPU) the prefix is split across the ranks (split-KV): every
rank holds its shard in a shard-sized cache, computes a partial (O, m, l) over it and the partials are
merged over peer memory (NVLink); every rank ends the step owning its row slice of the output (the
reduce-scatter form).  Total work is fixed: scaling is "strong".

Inputs are seeded synthetic N(0,1) bf16 tensors.  Between timed steps the working set is rotated
over several KV caches whose total size per GPU exceeds the 126 MB L2, as the layers of a model would.

Every arm checks what it times: outside the timed region one step runs on the seeded case and a sample
of its output rows (on every rank, rows of that rank's slice) is compared with the C++ port of the
reference's CPU attention; the line carries the errors and the run fails if they leave the gate
(max-abs 2e-2, mean-abs 2e-3).  Rank 0 prints ONE JSON line; with the default configuration it also
carries, under "extra", short measurements of the other benchmark configurations.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "canvas-attn TFLOP/s @32k prefix"
UNIT = "TFLOP/s"
L2_BYTES = 126e6
MAX_ABS_GATE, MEAN_ABS_GATE = 2e-2, 2e-3

# dram__bytes_read.sum + dram__bytes_write.sum of one attention-kernel launch of the headline
# workload on one GPU, from an ncu capture of this kernel (read 70.32 MB + write 4.32 MB)
NCU_TRAFFIC_BYTES_PER_LAUNCH = {2: 74.64e6}


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"bf16_tflops": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]), "source": "measured",
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)) or None}
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback", "bf16_tflops_sustained": 1400.0}


class ClockSampler:
    """Samples SM clocks and throttle reasons with one long-running nvidia-smi (-lms 20) while the
    timed region runs; the process is ended by its own PID afterwards."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self._t = None

    def _reader(self):
        try:
            for line in self.proc.stdout:
                parts = [x.strip() for x in line.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
        except Exception:
            pass

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._reader, daemon=True)
            self._t.start()
            time.sleep(0.3)     # let the first samples arrive before the timed region
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        if self._t is not None:
            self._t.join(timeout=5)

    def mark(self) -> int:
        return len(self.samples)

    def summary(self, first: int = 0):
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples[first:]:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except ValueError:
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


_T0 = time.time()


def log(msg: str) -> None:
    """Progress on stderr (every rank; the JSON line on stdout stays alone)."""
    print(f"[bench {time.time() - _T0:7.1f}s rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


def _cfg(idx: int):
    from diffgemma_b200 import synthetic
    return synthetic.configs()[idx]


def _rot_count(kv_bytes_per_gpu: float) -> int:
    """How many KV caches a GPU rotates over so that their total exceeds twice the L2."""
    return int(min(40, max(2, int(L2_BYTES * 2 // max(1.0, kv_bytes_per_gpu)) + 1)))


def _shard_tokens(prefix: int, canvas: int, world: int) -> int:
    """Tokens of the largest per-rank cache under split-KV (the last rank also holds the canvas)."""
    from diffgemma_b200.split_kv import plan_shards
    b = plan_shards(prefix, world, canvas=canvas)
    return max((b[r + 1] - b[r]) + (canvas if r == world - 1 else 0) for r in range(world))


def config_dict(cfg_idx: int, world: int, exchange: str = "p2p"):
    """The `config` object of the JSON line; identical in both arms for the same command line."""
    cfg = _cfg(cfg_idx)
    lay = cfg.layer
    P = cfg.prefix
    tokens = P + lay.canvas if world == 1 else _shard_tokens(P, lay.canvas, world)
    kv_bytes = 2 * lay.n_kv_heads * tokens * lay.head_dim * 2
    n_rot = _rot_count(kv_bytes)
    if lay.window:
        mask = f"prefix window {lay.window} " + ("per row" if lay.mask_mode == 2 else "uniform") + ", canvas bidirectional"
    else:
        mask = "all prefix visible, canvas bidirectional"
    if world == 1:
        part = "single GPU"
    elif exchange == "nccl":
        part = f"split-KV over {world} GPUs + NCCL LSE merge, full output on every rank"
    else:
        part = (f"split-KV over {world} GPUs, shard-sized caches, LSE merge over peer memory (NVLink), "
                f"every rank keeps its row slice of the output; consecutive steps are independent and the exchange is "
                f"pipelined over them (every rank runs two contexts that take alternate steps, so that one step's exchange "
                f"runs beside the next step's attention; a step's rows are sent in that step, its slice is merged by the "
                f"context's next call: throughput of a stream of steps; latency_ms_per_step is one step alone on one "
                f"context, merged at once)")
    out = {"workload": cfg.name, "prefix": P, "n_q_heads": lay.n_q_heads, "n_kv_heads": lay.n_kv_heads,
           "head_dim": lay.head_dim, "canvas": lay.canvas, "mask": mask, "partition": part,
           "l2": f"steps rotate over {n_rot} KV caches per GPU ({n_rot * kv_bytes / 1e6:.0f} MB > 126 MB L2)",
           "algorithmic_gflop_per_step": lay.flops(P) / 1e9}
    if cfg_idx == 4:
        out["inputs"] = "a block of 48 denoise steps: canvas Q/K/V re-drawn for every step, prefix KV frozen"
    return out


# ----------------------------------------------------------------------------------------------
# CPU side: the C++/OpenMP port of the reference's CPU attention (checker and timed baseline)
# ----------------------------------------------------------------------------------------------
class CpuOracle:
    """The oracle port on the seeded case of a configuration.  Inputs are prepared once; the prefix keys
    are used as drawn (norm + RoPE of the prefix is prefill work, not this path)."""

    def __init__(self, cfg_idx: int | None, n_threads: int = 0, case=None, layer=None, prefix=None):
        import numpy as np
        import torch
        from oracle import attn_oracle as ao
        from oracle import c_oracle as co
        from diffgemma_b200 import synthetic
        self.ao, self.co, self.np = ao, co, np
        if cfg_idx is None:
            cfg = synthetic.BenchConfig("custom", prefix, layer)
        else:
            cfg = _cfg(cfg_idx)
        lay = cfg.layer
        self.cfg, self.lay = cfg, lay
        self.d = ao.LayerDesc(lay.n_q_heads, lay.n_kv_heads, lay.head_dim, lay.canvas, lay.rotary_dim, lay.rope_theta,
                              lay.rms_eps, lay.softmax_scale, lay.window, lay.mask_mode, lay.v_norm, lay.rope_pairing)
        if case is None:
            case = synthetic.draw(lay, cfg.prefix, synthetic.config_seed(cfg_idx))
        self.t = [x.contiguous().view(torch.int16).numpy().view(np.uint16) for x in case]
        self.n_threads = n_threads
        self.cores = n_threads or co.num_threads()
        self._stage1 = None
        self._vis = None

    def stage1(self):
        if self._stage1 is None:
            q, kc, vc, _, _ = self.t
            self._stage1 = self.co.qk_rope_kv(self.d, self.cfg.prefix, q, kc, vc)
        return self._stage1

    def rows(self, row_begin: int, row_end: int):
        """fp32 output [row_end - row_begin, Hq, D] of the canvas rows [row_begin, row_end)."""
        qn, kn, vn = self.stage1()
        out = self.co.attention(self.d, self.cfg.prefix, qn, kn, vn, self.t[3], self.t[4], row_begin=row_begin,
                                row_end=row_end, n_threads=self.n_threads)
        return out[row_begin:row_end]

    def timed(self, rows: int):
        """(TFLOP/s, seconds, flops) of stage 1 + the first `rows` canvas rows."""
        if self._vis is None:
            self._vis = self.ao.visibility(self.d, self.cfg.prefix).sum(axis=1)
        q, kc, vc, kp, vp = self.t
        t0 = time.perf_counter()
        qn, kn, vn = self.co.qk_rope_kv(self.d, self.cfg.prefix, q, kc, vc)
        self.co.attention(self.d, self.cfg.prefix, qn, kn, vn, kp, vp, row_begin=0, row_end=rows, n_threads=self.n_threads)
        dt = time.perf_counter() - t0
        flops = 4.0 * self.lay.head_dim * self.lay.n_q_heads * float(self._vis[:rows].sum())
        return flops / dt / 1e12, dt, flops


def run_reference(args):
    """Reference arm: the reference's CPU implementation of the path (its own CPU code is Rust and
    cannot be built in this image, so this is the C++/OpenMP port of it), all host threads, each
    step a bounded sample of the workload sized so that the whole run takes about two minutes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = _cfg(args.cfg)
    # all host threads this process may use: the launcher of a multi-rank run exports
    # OMP_NUM_THREADS=1, which must not shrink the CPU arm to one core
    smp = CpuOracle(args.cfg, n_threads=len(os.sched_getaffinity(0)))
    smp.timed(1)
    _, dt8, _ = smp.timed(8)
    n_steps = args.warmup + args.steps
    rows = int(max(1, min(cfg.layer.canvas, 8 * (120.0 / n_steps) / dt8)))
    vals = []
    for i in range(n_steps):
        v, dt, flops = smp.timed(rows)
        if i >= args.warmup:
            vals.append((v, dt))
    value = sum(v for v, _ in vals) / len(vals)
    ms = 1e3 * sum(dt for _, dt in vals) / len(vals)
    sample = f"first {rows} of {cfg.layer.canvas} canvas rows x all {cfg.layer.n_q_heads} heads x all keys per step"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(args.cfg, args.gpus, args.exchange),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": smp.cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# one configuration resident on this rank
# ----------------------------------------------------------------------------------------------
class Workload:
    """Rotating KV caches, inputs and step functions of one benchmark configuration on this rank.
    Cache 0 and input set 0 are the seeded case (CPU generator, the same on every rank), so that one
    step on them can be checked against the CPU oracle; the other caches and input sets are drawn on
    the device."""

    def __init__(self, ctx, cfg_idx, world, rank, args, redraw=1, n_rot=None):
        import torch
        from diffgemma_b200 import synthetic
        from diffgemma_b200.split_kv import SplitKvGroup
        from diffgemma_b200.step_attn import CanvasAttention, KvCache
        self.torch = torch
        self.ctx, self.cfg_idx, self.world, self.rank, self.args = ctx, cfg_idx, world, rank, args
        cfg = _cfg(cfg_idx)
        self.cfg, self.lay, self.P = cfg, cfg.layer, cfg.prefix
        lay, P = self.lay, self.P
        dev = torch.device("cuda", ctx.device)
        self.dev = dev
        self.flops = lay.flops(P)
        self.att = CanvasAttention(ctx, lay)
        self.group = None
        self.pipelined = world > 1 and args.exchange == "p2p" and not args.no_pipelined_exchange
        if world > 1:
            self.group = SplitKvGroup(ctx, lay, exchange=args.exchange,
                                      p2p_mode=(4 if self.pipelined else 3) if args.exchange == "p2p" else 0)
            self.t0, self.t1 = self.group.shard_bounds(P)
        else:
            self.t0, self.t1 = 0, P
        tokens = P + lay.canvas if world == 1 else _shard_tokens(P, lay.canvas, world)
        self.kv_bytes = 2 * lay.n_kv_heads * tokens * lay.head_dim * 2
        self.n_rot = n_rot or _rot_count(self.kv_bytes)
        # the seeded case
        self.case = synthetic.draw(lay, P, synthetic.config_seed(cfg_idx))
        q0, kc0, vc0, kp0, vp0 = self.case
        lo = self.t0
        if lay.window:
            lo = max(lo, P - lay.window - 256)      # older positions are outside every row's window
        self.kvs = []
        g = torch.Generator(device=dev).manual_seed(synthetic.config_seed(cfg_idx) + 17 + 1000 * rank)
        for j in range(self.n_rot):
            kv = self.group.make_shard_cache(P) if self.group is not None and args.exchange == "p2p" \
                else KvCache(ctx, lay, P + lay.canvas)
            n = self.t1 - lo
            if n > 0:
                if j == 0:
                    kv.load_prefix(kp0[lo:self.t1].contiguous().to(dev), vp0[lo:self.t1].contiguous().to(dev), lo)
                else:
                    kv.load_prefix(torch.randn(n, lay.n_kv_heads, lay.head_dim, generator=g, device=dev).to(torch.bfloat16),
                                   torch.randn(n, lay.n_kv_heads, lay.head_dim, generator=g, device=dev).to(torch.bfloat16), lo)
            self.kvs.append(kv)
        ctx.synchronize()
        # input sets: [0] the seeded case, the others re-drawn on the device (configuration 4 draws a new
        # canvas Q/K/V for every step of a block)
        self.ins = [(q0[None].to(dev), kc0[None].to(dev), vc0[None].to(dev))]
        for s in range(1, redraw):
            self.ins.append(tuple(torch.randn(1, lay.canvas, h, lay.head_dim, generator=g, device=dev).to(torch.bfloat16)
                                  for h in (lay.n_q_heads, lay.n_kv_heads, lay.n_kv_heads)))
        self.out = torch.zeros_like(self.ins[0][0])
        # pipelined exchange: the slice of a step is written by the NEXT call, so consecutive steps get different
        # output buffers
        self.outs = [self.out] + ([torch.zeros_like(self.out) for _ in range(2)] if self.pipelined else [])
        self.pipe = None
        # A second lane on several GPUs: a second context (own stream, workspace, exchange buffers, caches) that
        # takes every other step, so that the exchange kernel of one step (latency: a grid boundary, posted stores,
        # one NVLink round trip) runs beside the attention kernel of the next.  Consecutive steps are independent -
        # the situation of a host with several canvases or requests in flight.
        self.lane2 = None
        self.two_lanes = False
        if self.pipelined and not args.one_lane:
            from diffgemma_b200.step_attn import Context
            torch.cuda.synchronize()
            ctx2 = Context(ctx.device, make_current=False)
            ctx2.set_inputs_stable(True)
            if args.kernel_form != "auto":
                ctx2.set_pair_mode(args.kernel_form == "pair")
            grp2 = SplitKvGroup(ctx2, lay, exchange="p2p", p2p_mode=4)
            kvs2 = []
            for j in range(self.n_rot):
                kv = grp2.make_shard_cache(P)
                n = self.t1 - lo
                if n > 0:
                    kr = torch.randn(n, lay.n_kv_heads, lay.head_dim, generator=g, device=dev).to(torch.bfloat16)
                    vr = torch.randn(n, lay.n_kv_heads, lay.head_dim, generator=g, device=dev).to(torch.bfloat16)
                    torch.cuda.synchronize()           # the copy below runs on the second context's stream
                    kv.load_prefix(kr, vr, lo)
                    ctx2.synchronize()
                kvs2.append(kv)
            self.lane2 = {"ctx": ctx2, "group": grp2, "kvs": kvs2, "outs": [torch.zeros_like(self.out) for _ in range(3)]}
            self.two_lanes = True
            torch.cuda.synchronize()

    @property
    def extra_streams(self):
        return [self.lane2["ctx"].torch_stream] if (self.lane2 is not None and self.two_lanes) else []

    # ---- device-resident step
    def step_dev(self, i, kv=None, ins=None):
        if kv is None and self.lane2 is not None and self.two_lanes and (i & 1):
            L = self.lane2
            j = i >> 1
            q, kc, vc = self.ins[i % len(self.ins)] if ins is None else ins
            L["group"].denoise(L["kvs"][j % self.n_rot], self.P, q[0], kc[0], vc[0], out=L["outs"][j % 3][0])
            return
        if kv is None and self.lane2 is not None and self.two_lanes:
            kv = self.kvs[(i >> 1) % self.n_rot]
            q, kc, vc = self.ins[i % len(self.ins)] if ins is None else ins
            self.group.denoise(kv, self.P, q[0], kc[0], vc[0], out=self.outs[(i >> 1) % len(self.outs)][0])
            return
        kv = self.kvs[i % self.n_rot] if kv is None else kv
        q, kc, vc = self.ins[i % len(self.ins)] if ins is None else ins
        if self.group is None:
            self.att.denoise([kv], [self.P], q, kc, vc, out=self.out)
        else:
            self.group.denoise(kv, self.P, q[0], kc[0], vc[0], out=self.outs[i % len(self.outs)][0])

    def drain(self):
        """Pipelined exchange: merge the slice of the last step (what a next step would have done)."""
        if self.pipelined and self.group.p2p_mode == 4:
            self.group.flush()
        if self.lane2 is not None:
            self.lane2["group"].flush()

    # ---- end-to-end step: host buffers through the library's pipeline, several steps in flight (more with several
    # ranks, whose steps are short and coupled: a host thread that falls behind stalls every rank)
    PIPE_DEPTH = 3

    def host_setup(self):
        from diffgemma_b200.step_attn import HostPipe
        torch = self.torch
        if self.pipelined:
            # the host pipe copies a step's slice back right behind that step's kernels: the plain push form, one lane
            self.drain()
            self.two_lanes = False
            self.group.set_mode(3)
        if self.group is not None and self.args.exchange == "p2p" and self.args.share_q:
            self.group.set_share_q(True)       # every rank copies in its row slice of Q; the slices cross NVLink
        self.PIPE_DEPTH = 3 if self.world == 1 else 6
        self.pipe = HostPipe(self.ctx, self.lay, 1, self.PIPE_DEPTH)
        if self.group is None and not self.args.no_deferred_launch:   # measured slower on a split-KV rank (host-bound)
            # a step's kernel is launched one submit after its copies: no event wait between consecutive kernels
            self.pipe.set_deferred_launch(True)
        self.pending = []
        q0, kc0, vc0 = (t[None].contiguous() for t in self.case[:3])
        self.host_sets = [tuple(t.clone().pin_memory() for t in (q0, kc0, vc0, torch.zeros_like(q0)))
                          for _ in range(self.PIPE_DEPTH)]
        owner = self.group is None or self.group.owns_canvas
        stores_canvas = owner or self.args.exchange != "p2p"
        q_bytes = q0.numel() * 2
        if self.group is not None and self.args.exchange == "p2p" and self.args.share_q:
            q_bytes = self.group.row_slice()[1] * self.lay.head_dim * 2
        self.h2d_bytes = q_bytes + (kc0.numel() * 2 + vc0.numel() * 2 if stores_canvas else 0)
        if self.group is not None and self.args.exchange == "p2p":
            self.d2h_bytes = self.group.row_slice()[1] * self.lay.head_dim * 2
        else:
            self.d2h_bytes = q0.numel() * 2

    def step_host(self, i):
        kv = self.kvs[i % self.n_rot]
        qs, ks, vs, os_ = self.host_sets[i % self.PIPE_DEPTH]
        if self.group is None:
            self.pending.append(self.pipe.submit([kv], [self.P], qs, ks, vs, os_))
        elif self.args.exchange == "p2p":
            self.pending.append(self.pipe.submit_split(kv, self.P, self.t0, self.t1, self.group.owns_canvas,
                                                       self.group.p2p, qs[0], ks[0], vs[0], os_[0]))
        else:
            q, kc, vc = self.ins[0]
            q.copy_(qs, non_blocking=True)
            kc.copy_(ks, non_blocking=True)
            vc.copy_(vs, non_blocking=True)
            self.group.denoise(kv, self.P, q[0], kc[0], vc[0], out=self.out[0])
            os_.copy_(self.out, non_blocking=True)
            self.ctx.synchronize()
            return
        if len(self.pending) >= self.PIPE_DEPTH:
            self.pipe.wait(self.pending.pop(0))

    def finish_host(self):
        while self.pending:
            self.pipe.wait(self.pending.pop(0))

    # ---- what one step produced on the seeded case against the CPU oracle
    def parity(self, rows_per_range: int = 2):
        """Runs one step on cache 0 with the seeded inputs and compares a sample of this rank's output rows
        (all heads, all keys) with the oracle.  Returns the errors over all ranks."""
        torch = self.torch
        import numpy as np
        import torch.distributed as dist
        self.out.zero_()
        self.step_dev(0, kv=self.kvs[0], ins=self.ins[0])
        self.drain()
        self.ctx.synchronize()
        got = self.out[0].float().cpu().numpy()                   # [C, Hq, D]
        C, Hq = self.lay.canvas, self.lay.n_q_heads
        if self.group is not None and self.args.exchange == "p2p":
            r0, n = self.group.row_slice()
            c0, c1 = (r0 + Hq - 1) // Hq, (r0 + n) // Hq         # canvas rows wholly inside this rank's slice
        else:
            c0, c1 = 0, C
        k = min(rows_per_range, max(1, (c1 - c0) // 2))
        ranges = [(c0, c0 + k), (c1 - k, c1)] if c1 - c0 >= 2 * k else [(c0, c1)]
        oracle = CpuOracle(self.cfg_idx, n_threads=min(8, len(os.sched_getaffinity(0))), case=self.case)
        mx, tot, cnt = 0.0, 0.0, 0
        for a, b in ranges:
            ref = oracle.rows(a, b)
            diff = np.abs(got[a:b].astype(np.float64) - ref.astype(np.float64))
            mx = max(mx, float(diff.max()))
            tot += float(diff.sum())
            cnt += diff.size
        finite = bool(np.isfinite(got[c0:c1]).all())
        stats = torch.tensor([mx, tot, float(cnt), 0.0 if finite else 1.0], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            mxt = stats[[0, 3]].clone()
            dist.all_reduce(mxt, op=dist.ReduceOp.MAX)
            dist.all_reduce(stats, op=dist.ReduceOp.SUM)
            stats[0], stats[3] = mxt[0], mxt[1]
        mx, tot, cnt, bad = (float(x) for x in stats.tolist())
        res = {"max_abs": mx, "mean_abs": tot / max(1.0, cnt), "vs": "oracle (C++ port of the reference's CPU attention)",
               "rows": f"{int(cnt) // (Hq * self.lay.head_dim)} canvas rows x {Hq} heads x all keys"
                       + (f", {sum(b - a for a, b in ranges)} of every rank's own row slice" if self.world > 1 else ""),
               "gate": {"max_abs": MAX_ABS_GATE, "mean_abs": MEAN_ABS_GATE}}
        res["ok"] = bool(bad == 0.0 and res["max_abs"] <= MAX_ABS_GATE and res["mean_abs"] <= MEAN_ABS_GATE)
        return res

    def close(self):
        if self.pipe is not None:
            self.pipe.close()
        if self.lane2 is not None:
            self.lane2["group"].flush()
            self.lane2["group"].close()
            for kv in self.lane2["kvs"]:
                kv.close()
            self.lane2["ctx"].close()
        if self.group is not None:
            self.group.close()
        for kv in self.kvs:
            kv.close()


def _timer(world, dev, stream):
    import torch
    import torch.distributed as dist

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, finish=None, extra_streams=()):
        for i in range(warmup):
            fn(i)
        if finish:
            finish()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for s in extra_streams:           # work on the other lanes starts after the clock does ...
            s.wait_event(e0)
        for i in range(steps):
            fn(warmup + i)
        if finish:
            finish()          # every result is complete (back in host memory, end to end) before the clock stops
        for s in extra_streams:           # ... and ends before it stops
            ev = torch.cuda.Event()
            ev.record(s)
            stream.wait_event(ev)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    return timed


def _kernel_pass(ctx, timed, fn, steps, finish=None, wl=None):
    """The same steps once more with a CUDA event pair around every launch of the dominant kernel (on its
    own stream): a separate pass, because an event record between the append and the attention launch
    keeps the two from overlapping (programmatic dependent launch) and so changes the step time."""
    lanes = wl.two_lanes if wl is not None else False
    if wl is not None:
        wl.two_lanes = False              # the kernel's own duration: one lane, nothing running beside it
    ctx.kernel_timing(True, steps + 8)
    timed(fn, steps, 0, finish)
    k_ms, k_n = ctx.kernel_time()
    ctx.kernel_timing(False)
    if wl is not None:
        wl.two_lanes = lanes
    return (k_ms / k_n if k_n else None), k_n


def exchange_timeline(ctx, wl, world):
    """In-kernel time stamps of one unpipelined split-KV step on every rank (the library's measurement aids
    dg_ctx_phase_stamps and dg_p2p_phase_stamps): when the merge kernel was resident, saw its predecessor complete,
    had sent its rows, had published its count, had every rank's rows, had merged its slice - in microseconds
    relative to the end of the rank's own attention kernel.  The stamps cost time: read the intervals, not the step."""
    import ctypes as C
    import numpy as np
    import torch
    import torch.distributed as dist
    wl.drain()
    wl.two_lanes = False
    wl.group.set_mode(3)
    dev = wl.dev
    st = torch.zeros(4096 * 16, dtype=torch.int64, device=dev)
    ms = torch.zeros(8, dtype=torch.int64, device=dev)
    ctx.lib.dg_ctx_phase_stamps(ctx.h, C.c_void_p(st.data_ptr()))
    ctx.lib.dg_p2p_phase_stamps(wl.group.p2p, C.c_void_p(ms.data_ptr()))
    for i in range(5):
        wl.step_dev(i)
    ctx.synchronize()
    ctx.lib.dg_ctx_phase_stamps(ctx.h, None)
    ctx.lib.dg_p2p_phase_stamps(wl.group.p2p, None)
    a = st.cpu().numpy().reshape(4096, 16)
    a = a[a[:, 0] != 0]
    m = ms.cpu().numpy()
    t_end = a[:, 5].max()
    mine = {"attention_us": float(t_end - a[:, 0].min()) / 1e3, "ctas": int(len(a)),
            "merge_kernel_resident": float(m[0] - t_end) / 1e3, "predecessor_complete": float(m[1] - t_end) / 1e3,
            "rows_sent": float(m[2] - t_end) / 1e3, "count_published": float(m[3] - t_end) / 1e3,
            "all_rows_arrived": float(m[4] - t_end) / 1e3, "slice_merged": float(m[5] - t_end) / 1e3}
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    return {"unit": "us after the end of the rank's own attention kernel (stamps on)", "ranks": everyone}


def measure_block(ctx, cfg_idx, world, rank, args, steps, timed, peaks, redraw=1, want_e2e=False):
    """A short measurement of one configuration for the `extra` object of the line."""
    log(f"extra block: cfg {cfg_idx}")
    wl = Workload(ctx, cfg_idx, world, rank, args, redraw=redraw)
    try:
        par = wl.parity()
        ms = timed(wl.step_dev, steps, max(3, min(20, steps)), wl.drain, wl.extra_streams)
        if ctx.last_launch_count == 1:
            k_ms = ms                       # one kernel per step, back to back
        else:
            k_ms, _ = _kernel_pass(ctx, timed, wl.step_dev, min(steps, 200), wl.drain, wl)
        value = wl.flops / (ms * 1e-3) / 1e12
        lay = wl.lay
        io_bytes = 2 * lay.n_kv_heads * (wl.P + lay.canvas) * lay.head_dim * 2 + 2 * lay.canvas * lay.n_q_heads * lay.head_dim * 2
        if lay.window:
            io_bytes = 2 * lay.n_kv_heads * (lay.window + 2 * lay.canvas) * lay.head_dim * 2 + 2 * lay.canvas * lay.n_q_heads * lay.head_dim * 2
        blk = {"config": config_dict(cfg_idx, world, args.exchange), "value": value, "unit": UNIT, "ms_per_step": ms,
               "steps": steps, "steps_per_s": 1e3 / ms, "kernel_ms_rank0": k_ms,
               "frac_of_measured_bf16_peak": value / (peaks["bf16_tflops"] * world),
               "achieved_hbm_gbs": io_bytes / (ms * 1e-3) / 1e9,
               "frac_of_measured_hbm_peak": io_bytes / (ms * 1e-3) / 1e9 / (peaks["hbm_gbs"] * world), "parity": par}
        return blk
    finally:
        wl.close()


BLOCK_HIDDEN = 2816        # the reference's model width (enc.rs:1560-1629: 256 x 2816 -> 4096 + 2048 + 2048)


def measure_attn_block(cfg_idx, args, timed_of, peaks, steps=200, v_from_k=False):
    """One layer's attention block with its neighbours (dg_attn_block: input norm, stacked Q|K|V projection,
    attention, output projection, post-attention norm + residual) on the geometry of a configuration, beside the
    attention stage alone on the same caches.  Three weight sets (207 MB at the sliding geometry, more than L2) and
    three caches rotate, as the layers of a model would; parity of the first canvas rows against the CPU restatement."""
    import numpy as np
    import torch
    from diffgemma_b200 import synthetic
    from diffgemma_b200.step_attn import AttnBlock, CanvasAttention, Context, KvCache
    from oracle import attn_oracle as ao
    log(f"extra block: attention block with neighbours, cfg {cfg_idx}")
    cfg = _cfg(cfg_idx)
    lay, P, H = cfg.layer, cfg.prefix, BLOCK_HIDDEN
    C, D = lay.canvas, lay.head_dim
    nq, nk = lay.n_q_heads * D, lay.n_kv_heads * D
    n_qkv = nq + nk * (1 if v_from_k else 2)
    ctx = Context(0)
    ctx.set_inputs_stable(True)
    dev = torch.device("cuda", 0)
    timed = timed_of(ctx)
    try:
        g = torch.Generator().manual_seed(synthetic.config_seed(cfg_idx) + 9)
        bf = lambda t: t.to(torch.bfloat16)
        def wset():
            return dict(w_qkv=bf(torch.randn(n_qkv, H, generator=g) / H ** 0.5), w_o=bf(torch.randn(H, nq, generator=g) / nq ** 0.5),
                        input_ln=bf(1 + 0.1 * torch.randn(H, generator=g)), post_attn_ln=bf(1 + 0.1 * torch.randn(H, generator=g)))
        w0 = wset()
        blocks = [AttnBlock(ctx, lay, **{k: t.to(dev) for k, t in w0.items()}, v_from_k=v_from_k)]
        for _ in range(2):
            blocks.append(AttnBlock(ctx, lay, **{k: t.to(dev) for k, t in wset().items()}, v_from_k=v_from_k))
        hidden = bf(torch.randn(C, H, generator=g))
        _, _, _, kp, vp = synthetic.draw(lay, P, synthetic.config_seed(cfg_idx))
        kvs = []
        for j in range(3):
            kv = KvCache(ctx, lay, P + C)
            if j == 0:
                kv.load_prefix(kp.to(dev), vp.to(dev), 0)
            else:
                gd = torch.Generator(device=dev).manual_seed(100 + j)
                kv.load_prefix(torch.randn(P, lay.n_kv_heads, D, generator=gd, device=dev).to(torch.bfloat16),
                               torch.randn(P, lay.n_kv_heads, D, generator=gd, device=dev).to(torch.bfloat16), 0)
            kvs.append(kv)
        h_dev = hidden.to(dev)
        out = torch.empty_like(h_dev)
        # parity: the first rows of the seeded case
        R = 4
        f = lambda t: t.to(torch.float32).numpy()
        xn = ao.round_bf16(ao.rms_norm_rows(f(hidden), f(w0["input_ln"])))
        qkv = ao.linear_bf16(xn, f(w0["w_qkv"]))
        tq = torch.from_numpy(qkv[:, :nq].reshape(C, lay.n_q_heads, D).copy()).to(torch.bfloat16)
        tk = torch.from_numpy(qkv[:, nq:nq + nk].reshape(C, lay.n_kv_heads, D).copy()).to(torch.bfloat16)
        tv = tk if v_from_k else torch.from_numpy(qkv[:, nq + nk:].reshape(C, lay.n_kv_heads, D).copy()).to(torch.bfloat16)
        orc = CpuOracle(None, n_threads=0, case=(tq, tk, tv, kp, vp), layer=lay, prefix=P)
        o_rows = ao.round_bf16(orc.rows(0, R).reshape(R, nq))
        t_rows = ao.linear_bf16(o_rows, f(w0["w_o"]))
        ref = ao.round_bf16(f(hidden)[:R] + ao.round_bf16(ao.rms_norm_rows(t_rows, f(w0["post_attn_ln"]))))
        blocks[0].step(kvs[0], P, h_dev, out=out)
        ctx.synchronize()
        err = np.abs(f(out.cpu())[:R] - ref)
        gate = {"max_abs": 6.3e-2, "mean_abs": 4e-3}
        par = {"max_abs": float(err.max()), "mean_abs": float(err.mean()), "rows": f"{R} canvas rows x {H} columns",
               "vs": "CPU restatement of the block's stages (attention rows by the C++ port)", "gate": gate,
               "ok": bool(err.max() <= gate["max_abs"] and err.mean() <= gate["mean_abs"])}
        att = CanvasAttention(ctx, lay)
        q4, k4, v4 = (t.to(dev)[None].contiguous() for t in (tq, tk, tv))
        o4 = torch.empty_like(q4)
        ms_blk = timed(lambda i: blocks[i % 3].step(kvs[i % 3], P, h_dev, out=out), steps, 5)
        launches = ctx.last_launch_count
        ms_att = timed(lambda i: att.denoise([kvs[i % 3]], [P], q4, k4, v4, out=o4), steps, 5)
        st = ctx.device_status()
        assert st[0] == 0, f"device status {st}"
        fl_att = ao.algorithmic_flops(orc.d, P)
        fl_gemm = 2.0 * C * H * (n_qkv + nq)
        w_bytes = 2.0 * H * (n_qkv + nq)
        nb = max(ms_blk - ms_att, 1e-6)
        return {"workload": f"{cfg.name}: rms norm + Q|K|V projection ({C}x{H} -> {n_qkv}) + attention + output projection "
                            f"({nq} -> {H}) + norm + residual", "ms_per_step": ms_blk, "ms_attention_alone": ms_att,
                "ms_neighbours": ms_blk - ms_att, "launches_per_step": launches, "steps": steps,
                "value": (fl_att + fl_gemm) / (ms_blk * 1e-3) / 1e12, "unit": UNIT,
                "projection_flops": fl_gemm, "weight_bytes": w_bytes,
                "neighbours_tflops": fl_gemm / (nb * 1e-3) / 1e12,
                "neighbours_weight_gbs": w_bytes / (nb * 1e-3) / 1e9,
                "neighbours_frac_of_measured_hbm_peak": w_bytes / (nb * 1e-3) / 1e9 / peaks["hbm_gbs"], "parity": par}
    finally:
        ctx.close()


def measure_topk(cfg_idx, args, timed_of, peaks, steps=50):
    """The reference's top-k sparse attention (dg_attn_denoise_topk, kv-adaptive k = clamp(T / 128, 64, 512)) on the
    geometry of a configuration, beside the exact dense step on the same caches; parity of the first canvas rows
    against the CPU restatement of the reference's top-k oracle."""
    import numpy as np
    import torch
    from diffgemma_b200 import synthetic
    from diffgemma_b200.step_attn import CanvasAttention, Context, KvCache
    from oracle import attn_oracle as ao
    log(f"extra block: top-k sparse attention, cfg {cfg_idx}")
    cfg = _cfg(cfg_idx)
    lay, P = cfg.layer, cfg.prefix
    ctx = Context(0)
    ctx.set_inputs_stable(True)
    dev = torch.device("cuda", 0)
    timed = timed_of(ctx)
    try:
        q, kc, vc, kp, vp = synthetic.draw(lay, P, synthetic.config_seed(cfg_idx))
        kvs = []
        for j in range(2):
            kv = KvCache(ctx, lay, P + lay.canvas)
            if j == 0:
                kv.load_prefix(kp.to(dev), vp.to(dev), 0)
            else:
                gd = torch.Generator(device=dev).manual_seed(200 + j)
                kv.load_prefix(torch.randn(P, lay.n_kv_heads, lay.head_dim, generator=gd, device=dev).to(torch.bfloat16),
                               torch.randn(P, lay.n_kv_heads, lay.head_dim, generator=gd, device=dev).to(torch.bfloat16), 0)
            kvs.append(kv)
        att = CanvasAttention(ctx, lay)
        qd, kd, vd = q.to(dev), kc.to(dev), vc.to(dev)
        out = torch.empty_like(qd)
        att.denoise_topk(kvs[0], P, qd, kd, vd, out=out)
        ctx.synchronize()
        R = 2
        f = lambda t: t.to(torch.float32).numpy()
        d = ao.LayerDesc(lay.n_q_heads, lay.n_kv_heads, lay.head_dim, lay.canvas, lay.rotary_dim, lay.rope_theta, lay.rms_eps,
                         lay.softmax_scale, lay.window, lay.mask_mode, lay.v_norm, lay.rope_pairing)
        qn, kn, vn = ao.qk_rope_kv(f(q), f(kc), f(vc), None, None, d, P)
        K = np.concatenate([f(kp), kn], axis=0)
        V = np.concatenate([f(vp), vn], axis=0)
        ref, gap = ao.attention_topk(qn[:R], K, V, ao.visibility(d, P)[:R], d, return_gap=True)
        mx, mean, ties = ao.topk_errors(f(out.cpu())[:R], ref, gap)
        par = {"max_abs": mx, "mean_abs": mean, "rows_without_a_unique_kept_set": ties,
               "rows": f"{R} canvas rows x {lay.n_q_heads} heads",
               "vs": "CPU restatement of the reference's top-k oracle (max-abs over the rows whose kept set is unique)",
               "gate": {"max_abs": MAX_ABS_GATE, "mean_abs": MEAN_ABS_GATE},
               "ok": bool(mx <= MAX_ABS_GATE and mean <= MEAN_ABS_GATE and ties <= 0.1)}
        ms_topk = timed(lambda i: att.denoise_topk(kvs[i % 2], P, qd, kd, vd, out=out), steps, 3)
        launches = ctx.last_launch_count
        q4, k4, v4 = qd[None].contiguous(), kd[None].contiguous(), vd[None].contiguous()
        o4 = torch.empty_like(q4)
        ms_dense = timed(lambda i: att.denoise([kvs[i % 2]], [P], q4, k4, v4, out=o4), steps, 3)
        st = ctx.device_status()
        assert st[0] == 0, f"device status {st}"
        T = P + lay.canvas
        rows = lay.canvas * lay.n_q_heads
        return {"workload": f"{cfg.name}: top-k sparse attention, k = {ao.topk_k(T)} of {T} keys per row", "ms_per_step": ms_topk,
                "ms_dense_attention": ms_dense, "launches_per_step": launches, "steps": steps,
                "score_plane_bytes": 2.0 * rows * T, "score_gemm_flops": 2.0 * rows * T * lay.head_dim, "parity": par}
    finally:
        ctx.close()


def stack_units(n_kv_heads: int, n_canvases: int, world: int, rank: int):
    """KV-head sharding of one layer of the stack over `world` ranks.  The sharded unit is the KV head; where a
    layer has fewer KV heads than there are ranks (the global layers: 2), the (canvas, KV head) pairs are the
    units, so that every rank still owns an equal share and no softmax merge is needed anywhere.
    Returns (first KV head, number of KV heads, canvases) of this rank."""
    per = max(1, n_kv_heads // world)
    groups = n_kv_heads // per                 # ranks that differ in their heads
    share = max(1, world // groups)            # ranks that share the same heads and split the canvases
    assert n_canvases % share == 0, "canvases must divide over the ranks that share a KV head"
    return (rank % groups) * per, per, [b for b in range(n_canvases) if b % share == rank // groups]


def run_stack(args, as_block=False):
    """Configuration 3: one denoise step of attention over the 30-layer stack (global layers at 5, 11, 17, 23, 29,
    sliding layers with a 1024 window on ring caches elsewhere) for 4 independent canvases at a 16,384-token prefix.
    Only attention runs per layer; the canvases of a layer go through one batched call.  On N > 1 GPUs the KV heads
    are sharded (stack_units): every rank computes its heads (and, on the global layers, its canvases) from caches
    that hold only those heads, and one all-gather per layer leaves the layer's full output on every rank.  The step
    is captured once into a CUDA graph and replayed.  Not the headline metric: printed in the same JSON shape."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from dataclasses import replace
    from diffgemma_b200 import synthetic
    from diffgemma_b200.capi import check
    from diffgemma_b200.split_kv import _nccl_comm
    from diffgemma_b200.step_attn import CanvasAttention, Context, KvCache, _ptr
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    own_pg = False
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        own_pg = True
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    dev = torch.device("cuda", local)
    ctx = Context(local)
    if args.kernel_form != "auto":
        ctx.set_pair_mode(args.kernel_form == "pair")
    ctx.set_inputs_stable(True)        # resident inputs, written before the timed region
    comm = _nccl_comm(ctx, None) if world > 1 else None
    P, B = 16384, 4
    layers = synthetic.stack_layers()
    PARITY_LAYERS = {0: 31, 5: 32}            # layer index -> seed offset of its seeded canvas 0
    g = torch.Generator(device=dev).manual_seed(synthetic.config_seed(3) + 1000 * rank)
    kvs, atts, units, flops = [], [], [], 0.0
    seeded = {}
    for li, lay in enumerate(layers):
        h0, nh, canv = stack_units(lay.n_kv_heads, B, world, rank)
        G = lay.n_q_heads // lay.n_kv_heads
        loc = replace(lay, n_kv_heads=nh, n_q_heads=nh * G)
        units.append((h0, nh, canv, G))
        row = []
        n0 = P - 1100 if lay.window else 0                 # older positions have left the window (and the ring)
        for b in canv:
            kv = KvCache(ctx, loc, ring_slots=2048) if lay.window else KvCache(ctx, loc, P + lay.canvas)
            if li in PARITY_LAYERS and b == 0:
                case = synthetic.draw(lay, P, synthetic.config_seed(3) + PARITY_LAYERS[li])
                seeded[li] = case
                kv.load_prefix(case[3][n0:, h0:h0 + nh].contiguous().to(dev), case[4][n0:, h0:h0 + nh].contiguous().to(dev), n0)
            else:
                kv.load_prefix(torch.randn(P - n0, nh, lay.head_dim, generator=g, device=dev).to(torch.bfloat16),
                               torch.randn(P - n0, nh, lay.head_dim, generator=g, device=dev).to(torch.bfloat16), n0)
            row.append(kv)
        if li in PARITY_LAYERS and li not in seeded:       # this rank does not hold canvas 0 of the layer: same draw, unused
            seeded[li] = synthetic.draw(lay, P, synthetic.config_seed(3) + PARITY_LAYERS[li], with_prefix=False)
        kvs.append(row)
        atts.append(CanvasAttention(ctx, loc))
        flops += B * lay.flops(P)
    ctx.synchronize()
    # per-layer inputs are independent draws in the configuration; here one draw per layer kind is reused by the
    # layers of that kind.  Canvas 0 of each kind carries the seeded case that the parity check reads.
    ins, outs, gath = {}, {}, {}
    for li in (0, 5):
        lay = layers[li]
        h0, nh, canv, G = units[li]
        q = torch.randn(len(canv), 256, nh * G, 256, generator=g, device=dev).to(torch.bfloat16)
        k = torch.randn(len(canv), 256, nh, 256, generator=g, device=dev).to(torch.bfloat16)
        v = torch.randn(len(canv), 256, nh, 256, generator=g, device=dev).to(torch.bfloat16)
        if 0 in canv:
            j = canv.index(0)
            q[j] = seeded[li][0][:, h0 * G:(h0 + nh) * G].to(dev)
            k[j] = seeded[li][1][:, h0:h0 + nh].to(dev)
            v[j] = seeded[li][2][:, h0:h0 + nh].to(dev)
        ins[lay.n_kv_heads] = (q, k, v)
        outs[lay.n_kv_heads] = torch.zeros_like(q)
        gath[lay.n_kv_heads] = torch.zeros((world,) + tuple(q.shape), dtype=q.dtype, device=dev)

    def step(upto=len(layers), gather=True):
        for li, lay in enumerate(layers[:upto]):
            q, k, v = ins[lay.n_kv_heads]
            o = outs[lay.n_kv_heads]
            atts[li].denoise(kvs[li], [P] * len(kvs[li]), q, k, v, out=o)
            if comm is not None and gather:
                check(ctx.lib.dg_nccl_all_gather(ctx.h, comm, _ptr(o), _ptr(gath[lay.n_kv_heads]), o.numel() * 2),
                      "dg_nccl_all_gather")

    # ---- parity: the seeded canvas 0 of layers 0 and 5, every rank's block of the gathered output against the oracle
    mx, tot, cnt = 0.0, 0.0, 0
    log("stack: caches built; parity of layers 0 and 5")
    for li in (0, 5):
        lay = layers[li]
        step(upto=li + 1)                                   # the shared output buffers then hold layer li
        ctx.synchronize()
        full = gath[lay.n_kv_heads] if comm is not None else outs[lay.n_kv_heads][None]
        full = full.float().cpu().numpy()                   # [world, canvases, C, q_per, D]
        if rank == 0:
            oracle = CpuOracle(None, n_threads=min(8, len(os.sched_getaffinity(0))), case=seeded[li] if len(seeded[li]) == 5 and
                               seeded[li][3] is not None else synthetic.draw(lay, P, synthetic.config_seed(3) + PARITY_LAYERS[li]),
                               layer=lay, prefix=P)
            for a, b in ((0, 2), (254, 256)):
                ref = oracle.rows(a, b)                     # [rows, Hq, D]
                for w in range(world):
                    h0, nh, canv = stack_units(lay.n_kv_heads, B, world, w)
                    if 0 not in canv:
                        continue
                    G = lay.n_q_heads // lay.n_kv_heads
                    diff = np.abs(full[w, canv.index(0), a:b].astype(np.float64) - ref[:, h0 * G:(h0 + nh) * G].astype(np.float64))
                    mx = max(mx, float(diff.max()))
                    tot += float(diff.sum())
                    cnt += diff.size
    parity = {"max_abs": mx, "mean_abs": tot / max(1, cnt), "vs": "oracle (C++ port of the reference's CPU attention)",
              "rows": "canvas 0 of layers 0 (sliding) and 5 (global): 4 canvas rows x 16 heads x all keys, every rank's heads "
                      "as they arrive in rank 0's gathered output",
              "gate": {"max_abs": MAX_ABS_GATE, "mean_abs": MEAN_ABS_GATE}}
    parity["ok"] = bool(cnt > 0 and mx <= MAX_ABS_GATE and parity["mean_abs"] <= MEAN_ABS_GATE) if rank == 0 else True

    log(f"stack: parity {parity['max_abs']:.3e} / {parity['mean_abs']:.3e}; warm-up")
    warm = max(3, args.warmup)
    for _ in range(warm):
        step()
    ctx.synchronize()
    # The timed step is the attention of the 30 layers on this rank's heads, captured once into a CUDA graph: under
    # KV-head sharding the path needs no collective when the o_proj that follows is sharded by heads the same way
    # (its all-reduce lies behind this path).  The variant that leaves every layer's full output on every rank - one
    # all-gather per layer - is timed beside it with eager launches (ms_per_step_with_gather).
    graph = None
    if not args.stack_eager:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=ctx.torch_stream):
            step(gather=False)
    run = graph.replay if graph is not None else (lambda: step(gather=False))
    launches = 0                                     # kernels of one steady-state step, counted by the library
    for li, lay in enumerate(layers):
        q, k, v = ins[lay.n_kv_heads]
        atts[li].denoise(kvs[li], [P] * len(kvs[li]), q, k, v, out=outs[lay.n_kv_heads])
        launches += ctx.last_launch_count
    steps = args.steps if not as_block else min(args.steps, 100)

    def time_steps(fn, n):
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ctx.torch_stream)
        for _ in range(n):
            fn()
        e1.record(ctx.torch_stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t_ms = e0.elapsed_time(e1) / n
        if world > 1:
            t = torch.tensor([t_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_ms = float(t.item())
        return t_ms

    with ClockSampler(local) as clk:
        ms = time_steps(run, steps)
        ms_gather = time_steps(step, min(steps, 50)) if comm is not None else None
    st = ctx.device_status()
    assert st[0] == 0, f"device status {st}"
    peaks = _peaks()
    value = flops / (ms * 1e-3) / 1e12
    config = {"workload": "cfg3_stack30_p16384_batch4", "prefix": P, "canvases": B, "layers": 30,
              "sliding_layers": "25 x (Hkv 8, window 1024 uniform, ring cache of 2048 slots)",
              "global_layers": "5 x (Hkv 2, all prefix visible)", "head_dim": 256, "canvas": 256,
              "partition": "single GPU" if world == 1 else
              (f"KV heads sharded over {world} GPUs (sliding layers: {max(1, 8 // world)} of 8 KV heads per rank; global layers: "
               f"the 8 (canvas, KV head) pairs, {8 // world} per rank); no softmax merge and no collective in the timed step "
               "(the output stays sharded by heads for a head-sharded o_proj); ms_per_step_with_gather adds one NCCL "
               "all-gather of the output slices per layer"),
              "launch": ("one CUDA graph replay per step" if graph is not None else "eager launches") +
                        "; the canvases of a layer in one batched call",
              "l2": f"30 layers x 4 canvases of KV per step ({761 / world:.0f} MB per GPU > 126 MB L2)" if world <= 4 else
                    f"30 layers x 4 canvases of KV per step ({761 / world:.0f} MB per GPU: below the 126 MB L2 at this GPU count, "
                    "the sharded stack is L2-resident by construction)",
              "algorithmic_gflop_per_step": flops / 1e9}
    if comm is not None:
        ctx.synchronize()
        ctx.lib.dg_nccl_comm_destroy(comm)
    for row in kvs:
        for kv in row:
            kv.close()
    ctx.close()
    blk = {"config": config, "value": value, "unit": UNIT, "ms_per_step": ms, "steps": steps,
           "frac_of_measured_bf16_peak": value / (peaks["bf16_tflops"] * world), "gpu_launches_per_step": launches,
           "ms_per_step_with_gather": ms_gather, "parity": parity}
    if as_block:
        return blk
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warm,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": config,
                "pct_of_measured_bf16_peak": 100.0 * value / (peaks["bf16_tflops"] * world),
                "parity": parity, "parity_ok": parity["ok"],
                "roofline": {"bound": "tensor", "achieved": value / world, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                             "frac": value / world / peaks["bf16_tflops"], "traffic": None,
                             "peak_source": peaks["source"] + " burst", "kernel": f"whole step ({launches} launches per rank)"},
                "e2e": None, "gpu_launches": int(launches * steps), "clocks": clk.summary()}
        print(json.dumps(line), flush=True)
    if own_pg:
        dist.destroy_process_group()
    if rank == 0 and not parity["ok"]:
        sys.exit("parity gate failed: " + json.dumps(parity))


def run_ours(args):
    import torch
    import torch.distributed as dist
    from diffgemma_b200.step_attn import Context

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    dev = torch.device("cuda", local)
    ctx = Context(local)
    if args.kernel_form != "auto":
        ctx.set_pair_mode(args.kernel_form == "pair")
    # the inputs of the timed steps are resident tensors written before the timed region, never by work queued
    # ahead of a step: the library may start a step's Q prologue while the previous step drains
    ctx.set_inputs_stable(True)
    peaks = _peaks()
    redraw = 48 if args.cfg == 4 else 1          # configuration 4: a block of 48 steps, Q/K/V re-drawn per step
    log(f"building workload cfg {args.cfg} on {world} GPU(s)")
    wl = Workload(ctx, args.cfg, world, rank, args, redraw=redraw)
    lay, P, flops = wl.lay, wl.P, wl.flops
    timed = _timer(world, dev, ctx.torch_stream)
    log("parity check of one step against the oracle")
    parity = wl.parity()
    log(f"parity {parity['max_abs']:.3e} / {parity['mean_abs']:.3e}; timing {args.steps} steps")

    warm = max(3, args.warmup)
    with ClockSampler(local) as clk:
        # device-resident arm
        ms_dev = timed(wl.step_dev, args.steps, warm, wl.drain, wl.extra_streams)
        launches_per_step = ctx.last_launch_count
        log(f"device-resident: {ms_dev * 1e3:.1f} us per step, {launches_per_step} launch(es) per step")
        mark = clk.mark()
        if launches_per_step == 1:
            # one kernel per step (the append runs inside the attention launch): the launches of the timed region run
            # back to back, so the region's CUDA-event time divided by its launches IS the kernel's average duration
            # (gaps between launches included, which can only make it longer)
            k_avg_ms, k_n, k_how = ms_dev, args.steps, "timed region / launches (one kernel per step, back to back)"
        else:
            k_avg_ms, k_n = _kernel_pass(ctx, timed, wl.step_dev, args.steps, wl.drain, wl)
            k_how = "CUDA event pair around every launch of the kernel, in a separate pass of the same steps" 
        clocks = clk.summary()
        # a timed region of less than a second is a burst at the boost clock: the same steps for at least
        # 1.2 s show what the kernel sustains under the power cap
        sustained = None
        if ms_dev * args.steps < 1000.0 and not args.no_sustained:
            n_sus = int(min(60000, math.ceil(1200.0 / ms_dev)))
            log(f"sustained loop of {n_sus} steps")
            timed(wl.step_dev, max(1, n_sus // 3), 0, wl.drain, wl.extra_streams)          # reach the steady clock first
            mark = clk.mark()
            ms_sus = timed(wl.step_dev, n_sus, 0, wl.drain, wl.extra_streams)
            if launches_per_step == 1:
                ks_ms = ms_sus
            else:
                ks_ms, _ = _kernel_pass(ctx, timed, wl.step_dev, min(n_sus, 4000), wl.drain, wl)
            cs = clk.summary(mark)
            ach = (flops / world) / (ks_ms * 1e-3) / 1e12 if ks_ms else None
            sustained = {"steps": n_sus, "ms_per_step": ms_sus, "value": flops / (ms_sus * 1e-3) / 1e12,
                         "kernel_ms": ks_ms, "achieved": ach, "frac": ach / peaks["bf16_tflops"] if ach else None,
                         "frac_of_sustained_peak": (ach / peaks["bf16_tflops_sustained"])
                         if (ach and peaks["bf16_tflops_sustained"]) else None,
                         "sm_mhz_median": cs["sm_mhz"], "reasons": cs["reasons"],
                         "kernel_ms_x_sm_mhz": ks_ms * cs["sm_mhz"] if (ks_ms and cs["sm_mhz"]) else None}
        # one step alone: rows sent and slice merged inside the step (what a host that cannot keep a second step
        # in flight sees)
        ms_latency = None
        if wl.pipelined:
            wl.drain()
            wl.two_lanes = False
            wl.group.set_mode(3)
            ms_latency = timed(wl.step_dev, min(args.steps, 300), 5)
            log(f"one step alone (unpipelined exchange): {ms_latency * 1e3:.1f} us")
        timeline = None
        if args.exchange_timeline and wl.group is not None and args.exchange == "p2p":
            timeline = exchange_timeline(ctx, wl, world)
        # end-to-end arm: host buffers, H2D + kernels + D2H every step
        log("end-to-end arm (host buffers)")
        wl.host_setup()
        ms_e2e = timed(wl.step_host, args.steps, warm, wl.finish_host)
        log(f"end to end: {ms_e2e * 1e3:.1f} us per step")
    st = ctx.device_status()
    assert st[0] == 0, f"device status {st}"

    # bytes every rank moves per step, summed over the ranks
    io = torch.tensor([float(wl.h2d_bytes), float(wl.d2h_bytes)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(io, op=dist.ReduceOp.SUM)
    h2d_total, d2h_total = (int(x) for x in io.tolist())

    extra = {}
    if args.cfg == 2 and not args.no_extra:
        short = max(50, min(args.steps, 300))
        if world == 1:
            for idx, name in ((0, "cfg0_global_p2048"), (1, "cfg1_sliding_p8192_w1024")):
                extra[name] = measure_block(ctx, idx, world, rank, args, short, timed, peaks)
            extra["ref_full_layer_hd512_p32768"] = measure_block(ctx, 5, world, rank, args, min(short, 100), timed, peaks)
        extra["cfg4_global_p131072"] = measure_block(ctx, 4, world, rank, args, 48, timed, peaks, redraw=48)
        if world == 1:
            timed_of = lambda c: _timer(1, dev, c.torch_stream)
            extra["attn_block_cfg1_sliding"] = measure_attn_block(1, args, timed_of, peaks)
            extra["attn_block_cfg2_global"] = measure_attn_block(2, args, timed_of, peaks)
            extra["attn_block_ref_full_layer_hd512"] = measure_attn_block(5, args, timed_of, peaks, steps=100, v_from_k=True)
            extra["topk_cfg2_global"] = measure_topk(2, args, timed_of, peaks)
            extra["topk_ref_full_layer_hd512"] = measure_topk(5, args, timed_of, peaks)

    if rank == 0:
        value = flops / (ms_dev * 1e-3) / 1e12
        e2e = flops / (ms_e2e * 1e-3) / 1e12
        achieved = (flops / world) / (k_avg_ms * 1e-3) / 1e12 if k_avg_ms else None
        if world > 1 and k_avg_ms:
            # per-rank kernel work: rank 0's shard (the canvas keys are counted by the last rank)
            vis = (wl.t1 - wl.t0) + (lay.canvas if rank == world - 1 else 0)
            achieved = 4.0 * lay.head_dim * lay.n_q_heads * lay.canvas * vis / (k_avg_ms * 1e-3) / 1e12
        io_bytes = 2 * lay.n_kv_heads * (P + lay.canvas) * lay.head_dim * 2 + 2 * lay.canvas * lay.n_q_heads * lay.head_dim * 2
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_dev, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(args.cfg, world, args.exchange),
            "steps_per_s": 1e3 / ms_dev, "latency_ms_per_step": ms_latency if ms_latency is not None else ms_dev,
            "pct_of_measured_bf16_peak": 100.0 * value / (peaks["bf16_tflops"] * world),
            "pct_of_nominal_bf16_peak": 100.0 * value / (2250.0 * world),
            "achieved_hbm_gbs": io_bytes / (ms_dev * 1e-3) / 1e9,
            "parity": parity,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": (achieved / peaks["bf16_tflops"]) if achieved else None,
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH.get(args.cfg) if world == 1 else None,
                         "peak_source": peaks["source"] + " burst",
                         # the cuBLAS figure measured in a seconds-long loop, beside the burst one
                         "peak_sustained": peaks["bf16_tflops_sustained"],
                         "frac_of_sustained": (achieved / peaks["bf16_tflops_sustained"])
                         if (achieved and peaks["bf16_tflops_sustained"]) else None,
                         "kernel": {"single": "dg_attn_sm100_hd512_kernel", "pair": "dg_attn_sm100_hd512x_kernel"}.get(args.kernel_form, "dg_attn_sm100_hd512q_kernel")
                         if lay.head_dim == 512 else "dg_attn_sm100_kernel",
                         "kernel_ms": k_avg_ms, "kernel_launches_timed": k_n, "kernel_ms_how": k_how, "sustained": sustained},
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": ms_e2e,
                    "how": (f"dg_host_pipe, {wl.PIPE_DEPTH} steps in flight on every rank: every step copies its inputs "
                            "from pinned host memory and its result back; copies of neighbouring steps overlap the kernels"
                            + (("; a rank copies in " + ("its row slice of Q (the ranks exchange the slices over NVLink)"
                                                         if args.share_q else "all of Q (every rank needs every row)")
                                + " and the canvas K/V only where they are stored, and copies back its own row slice of the output")
                               if world > 1 and args.exchange == "p2p" else "")),
                    "h2d_bytes_per_step": h2d_total, "d2h_bytes_per_step": d2h_total},
            "gpu_launches": int(launches_per_step * args.steps),
            "clocks": clocks,
        }
        if extra:
            line["extra"] = extra
        if timeline is not None:
            line["exchange_timeline"] = timeline
        if world == 1 and not args.no_cpu:
            smp = CpuOracle(args.cfg)
            smp.timed(1)
            v, dt, fl = smp.timed(args.ref_rows)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": smp.cores, "kind": "port",
                                    "sample": f"first {args.ref_rows} of {lay.canvas} canvas rows x {lay.n_q_heads} heads x all keys "
                                              f"({fl / 1e9:.1f} GFLOP in {dt:.2f} s), C++/OpenMP fp32 port"}
    wl.close()
    ctx.close()
    stack_blk = None
    if args.cfg == 2 and not args.no_extra and not args.no_stack:
        log("extra block: 30-layer stack")
        stack_blk = run_stack(args, as_block=True)          # builds its own context; every rank takes part
    log("done")
    if rank == 0:
        if stack_blk is not None:
            line.setdefault("extra", {})["cfg3_stack30_p16384_batch4"] = stack_blk
        ok = parity["ok"] and all(b.get("parity", {}).get("ok", True) for b in line.get("extra", {}).values())
        line["parity_ok"] = bool(ok)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if rank == 0 and not line["parity_ok"]:
        sys.exit("parity gate failed: " + json.dumps({"main": parity, **{k: v.get("parity") for k, v in line.get("extra", {}).items()}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cfg", type=int, default=2, choices=[0, 1, 2, 3, 4, 5])
    ap.add_argument("--ref-rows", type=int, default=256, help="canvas rows in the bounded CPU sample")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="leave out the short runs of the other configurations")
    ap.add_argument("--no-stack", action="store_true", help="leave out the 30-layer stack from the extra runs")
    ap.add_argument("--no-sustained", action="store_true", help="leave out the >= 1.2 s sustained loop")
    ap.add_argument("--stack-eager", action="store_true", help="configuration 3: launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"], help="multi-GPU partial exchange")
    ap.add_argument("--exchange-timeline", action="store_true",
                    help="multi-GPU: add in-kernel time stamps of one split-KV step on every rank to the line")
    ap.add_argument("--share-q", action="store_true",
                    help="multi-GPU end-to-end arm: every rank copies in only its row slice of Q and the ranks "
                         "exchange the slices over NVLink (for hosts whose PCIe links are the bottleneck)")
    ap.add_argument("--no-deferred-launch", action="store_true",
                    help="end-to-end arm on one GPU: launch every step's kernels inside its own submit")
    ap.add_argument("--one-lane", action="store_true",
                    help="multi-GPU: one context per rank instead of two that take alternate steps")
    ap.add_argument("--no-pipelined-exchange", action="store_true",
                    help="multi-GPU: merge every step's slice inside that step instead of one step later")
    ap.add_argument("--kernel-form", default="auto", choices=["auto", "pair", "single"],
                    help="tensor-kernel form: CTA pairs, one CTA per query tile, or the library's choice")
    ap.add_argument("--topk", type=int, default=None, choices=[2, 5],
                    help="only the top-k sparse attention (dg_attn_denoise_topk) on this configuration's geometry, 1 GPU; "
                         "prints that block's record, not the benchmark line")
    ap.add_argument("--attn-block", type=int, default=None, choices=[1, 2, 5],
                    help="only the attention block with its neighbours (dg_attn_block) on this configuration's geometry, "
                         "1 GPU; prints that block's record, not the benchmark line")
    args = ap.parse_args()
    if args.topk is not None:
        import torch
        from diffgemma_b200 import build as _build
        _build.build()
        dev = torch.device("cuda", 0)
        blk = measure_topk(args.topk, args, lambda c: _timer(1, dev, c.torch_stream), _peaks(), steps=min(args.steps, 50))
        print(json.dumps(blk), flush=True)
        if not blk["parity"]["ok"]:
            sys.exit("parity gate failed: " + json.dumps(blk["parity"]))
        return
    if args.attn_block is not None:
        import torch
        from diffgemma_b200 import build as _build
        _build.build()
        dev = torch.device("cuda", 0)
        blk = measure_attn_block(args.attn_block, args, lambda c: _timer(1, dev, c.torch_stream), _peaks(),
                                 steps=min(args.steps, 200), v_from_k=args.attn_block == 5)
        print(json.dumps(blk), flush=True)
        if not blk["parity"]["ok"]:
            sys.exit("parity gate failed: " + json.dumps(blk["parity"]))
        return
    if args.impl == "reference":
        if args.cfg == 3:
            args.cfg = 2      # the CPU arm times the headline workload
        run_reference(args)
    elif args.cfg == 3:
        run_stack(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
