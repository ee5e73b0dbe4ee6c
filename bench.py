#!/usr/bin/env python
"""W8A8 (i8i8) linear benchmark: quantize + int8 GEMM + dequant(+bias)(+re-quantize).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c0..c4]
                    [--extras]

One "step" = one pass of the whole path over one batch of synthetic input of the chosen
configuration.  Prints ONE JSON line on rank 0.  metric = TOPS = 2*M*N*K / t.

  value     device-resident: inputs already in HBM, CUDA-event time over K steps (max over ranks)
  e2e       same path with the step's activations copied from pinned host memory and the step's
            outputs copied back to pinned host memory inside the timed region (weights stay
            resident in HBM, as they do in the reference's deployment)
  roofline  dominant kernel (the tcgen05 GEMM with fused epilogue) timed alone with CUDA events
  cpu_baseline  the scalar host oracle on the box's cores (a reported baseline, not a target)

--impl reference runs the reference's own kernels (compiled unmodified into oracle/_ref:
minmax_quantize_fp16 -> cuBLASLt gemm_i8i8i32 -> minmax_dequantize_fp16 [-> minmax_quantize_fp16])
for the same workload; if that library is absent it times the host oracle port instead.

Multi-GPU (torchrun, one rank per GPU): the default workload c1 does not shard ("replicas only",
weak scaling: every rank runs its own batch).  With --workload c2/c4 the N dimension is split
(column parallel, no communication), with --workload c3 the K dimension is split and the int32
partial accumulators are all-reduced before the dequant epilogue (row parallel); these report
"scaling": "strong".  --extras appends those sharded configurations to the default line.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "ppl.llm.kernel.cuda_b200"))

L2_BYTES_FALLBACK = 126 * 1024 * 1024

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (bytes).
TRAFFIC_NCU = {"c1": 50973952 + 129792, "c2": 107780608 + 138983424}


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def _dist_setup(n):
    import torch
    if n <= 1:
        return 0, 1
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    return rank, world


def _barrier(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def _max_over_ranks(ms, world):
    import torch
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _time_steps(runner, steps, warmup, world):
    """runner.run(first, count) enqueues `count` steps on the current stream.  Returns ms for exactly
    `steps` steps after `warmup` untimed ones (CUDA events, max over ranks)."""
    import torch
    runner.run(0, warmup)
    _barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    # start the timed region on a round boundary so that whole-round graphs can be used
    first = -(-warmup // getattr(runner, "nsets", 1)) * getattr(runner, "nsets", 1)
    runner.run(first, steps)
    e1.record()
    _barrier(world)
    return _max_over_ranks(e0.elapsed_time(e1), world)


class _Captured:
    """CUDA-graph form of fn(s): one graph per buffer set plus one "round" graph that runs all the
    sets back to back.  run(first, count) enqueues exactly `count` consecutive steps starting at
    step index `first`, using round graphs where a whole round fits, so the host's launch cost
    is paid once per round instead of once per microsecond-scale step."""

    def __init__(self, fn, nsets):
        import torch
        self.fn, self.nsets = fn, nsets  # fn owns the buffers the graphs point into
        self.single = []
        for s in range(nsets):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn(s)
            self.single.append(g)
        self.round = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.round):
            for s in range(nsets):
                fn(s)

    def run(self, first, count):
        i, end = first, first + count
        while i < end:
            if i % self.nsets == 0 and end - i >= self.nsets:
                self.round.replay()
                i += self.nsets
            else:
                self.single[i % self.nsets].replay()
                i += 1


class StatusWordSet(RuntimeError):
    """A device status word was non-zero.  Raised from values that were max-reduced over the ranks, so every
    rank raises it at the same place (the only exception run_config's callers may swallow and carry on after)."""


def _round_stats(runner, nsets, reps, world):
    """Per-step median and minimum over `reps` separately timed rounds (one round = one step on every
    buffer set), in ms; rank-local CUDA events, max over ranks of each statistic."""
    import torch
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    _barrier(world)
    evs[0].record()
    for r in range(reps):
        runner.run(0, nsets)
        evs[r + 1].record()
    torch.cuda.synchronize()
    per_step = sorted(evs[r].elapsed_time(evs[r + 1]) / nsets for r in range(reps))
    med = per_step[len(per_step) // 2] if len(per_step) % 2 else 0.5 * (per_step[len(per_step) // 2 - 1] + per_step[len(per_step) // 2])
    return _max_over_ranks(med, world), _max_over_ranks(per_step[0], world)


class _SameSet:
    """Replays the graph of buffer set 0 only: operands stay in L2 (the "L2-warm" figure)."""

    def __init__(self, captured):
        self.captured, self.nsets = captured, 1

    def run(self, first, count):
        for _ in range(count):
            self.captured.single[0].replay()


class _Eager:
    def __init__(self, fn):
        self.fn = fn

    def run(self, first, count):
        for i in range(first, first + count):
            self.fn(i)


class Workload:
    """Device-resident inputs of one configuration (one rank's shard), rotated over `nsets` distinct
    copies so that consecutive steps do not hit each other's data in L2."""

    def __init__(self, name, rank, world, sharded):
        import numpy as np
        import torch
        import pplb200
        from pplb200 import workloads as wl
        self.name, self.cfg = name, wl.CONFIGS[name]
        c = self.cfg
        self.M, self.K, self.N = c["M"], c["K"], c["N"]
        self.rank, self.world = rank, world
        self.shard = c["shard"] if (sharded and world > 1) else None
        x = wl.make_activations(name)
        w = wl.make_weights(name)
        sn = wl.make_column_scales(name)
        bias = wl.make_bias(name)
        self.Kw, self.Nw = self.K, self.N
        if self.shard == "column":
            n0, n1 = wl.shard_rows(self.N, world, rank)
            w, sn = w[n0:n1], sn[n0:n1]
            bias = None if bias is None else bias[n0:n1]
            self.Nw = n1 - n0
        elif self.shard == "row":
            k0, k1 = wl.shard_rows(self.K, world, rank)
            w = np.ascontiguousarray(w[:, k0:k1])
            self.Kw, self.k0, self.k1 = k1 - k0, k0, k1
        self.x_host = torch.from_numpy(x).pin_memory()
        bytes_per_set = x.nbytes + w.nbytes + 2 * self.M * self.Nw
        l2 = torch.cuda.get_device_properties(0).L2_cache_size or L2_BYTES_FALLBACK
        self.l2 = l2
        self.nsets = max(2, min(16, -(-3 * l2 // bytes_per_set))) if bytes_per_set < 3 * l2 else 1
        dev = "cuda"
        self.x = [torch.from_numpy(x).to(dev) for _ in range(self.nsets)]
        self.w = [torch.from_numpy(w).to(dev) for _ in range(self.nsets)]
        self.sn = torch.from_numpy(sn).to(dev)
        self.bias = None if bias is None else torch.from_numpy(bias).to(dev)
        self.set_bytes = bytes_per_set
        self.l2_note = ("rotating %d distinct weight/activation/output sets, %.0f MB in total > L2 %.0f MB"
                        % (self.nsets, self.nsets * bytes_per_set / 1e6, l2 / 1e6)) if self.nsets > 1 else \
                       ("one set of %.0f MB per step > L2 %.0f MB" % (bytes_per_set / 1e6, l2 / 1e6))
        self.ops = 2 * self.M * self.N * self.K  # whole-job ops of one step of the unsharded problem


def build_ours(wk):
    """Returns (step(i), e2e_step(i), kernel_only(i), launches_per_step, h2d, d2h, gemm_bytes)."""
    import torch
    import pplb200
    M, K, N, Kw, Nw = wk.M, wk.K, wk.N, wk.Kw, wk.Nw
    requant = wk.cfg["requant"]
    dev = "cuda"
    if wk.shard is None or wk.shard == "column":
        lins = [pplb200.W8A8Linear(wk.w[s], wk.sn, wk.bias, max_tokens=M, requant=requant) for s in range(wk.nsets)]

        def step(i):
            s = i % wk.nsets
            lins[s](wk.x[s])

        x_stage = torch.empty_like(wk.x[0])
        y_host = torch.empty((M, Nw), dtype=torch.float16).pin_memory()
        yq_host = torch.empty((M, Nw), dtype=torch.int8).pin_memory() if requant else None
        ys_host = torch.empty((M,), dtype=torch.float16).pin_memory() if requant else None

        def e2e(i):
            s = i % wk.nsets
            x_stage.copy_(wk.x_host, non_blocking=True)
            lins[s](x_stage)
            y_host.copy_(lins[s].y, non_blocking=True)
            if requant:
                yq_host.copy_(lins[s].yq, non_blocking=True)
                ys_host.copy_(lins[s].ys, non_blocking=True)

        h2d = wk.x_host.numel() * 2
        d2h = M * Nw * 2 + ((M * Nw + M * 2) if requant else 0)

        # dominant kernel alone: GEMM + fused epilogue on pre-quantized activations
        xq, sm = pplb200.minmax_quantize_fp16(wk.x[0])
        mode = pplb200.EPI_DEQUANT_F16
        ys = [l.y for l in lins]

        def kernel_only(i):
            s = i % wk.nsets
            pplb200.gemm_i8i8(xq, wk.w[s], mode=mode, scale_m=sm, scale_n=wk.sn, bias=wk.bias, out=ys[s])

        gemm_bytes = M * K + Nw * K + 2 * Nw + (2 * Nw if wk.bias is not None else 0) + 2 * M + 2 * M * Nw
        launches = 2 + (1 if requant else 0)
        return step, e2e, kernel_only, launches, h2d, d2h, gemm_bytes

    # row parallel: quantize the full activation rows (full-K absmax), GEMM on this rank's K shard,
    # exact int32 reduction, dequant epilogue.  Default: the reduction over peer-mapped memory (GEMM
    # epilogue pushes tiles to the row owner); --row-reduce nccl selects reduce-scatter / all-gather.
    import torch.distributed as dist
    uid = [pplb200.nccl_unique_id() if wk.rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    comm = pplb200.nccl_comm_init(uid[0], wk.rank, wk.world)
    wk.comm = comm
    xq_full = torch.empty((M, K), dtype=torch.int8, device=dev)
    sm = torch.empty((M,), dtype=torch.float16, device=dev)
    y = torch.empty((M, N), dtype=torch.float16, device=dev)
    wk.row_reduce = "nccl"
    qbuf = None
    if wk.row_reduce_wanted == "p2p" and M % wk.world == 0:
        ok, p2p = 1, None
        try:
            p2p = pplb200.P2PContext(wk.rank, wk.world, M, N)
            mine = p2p.handle()
        except pplb200.PplError as e:
            ok, mine = 0, b"\0" * 64
            sys.stderr.write("rank %d: peer buffer not available (%s)\n" % (wk.rank, e))
        handles = [None] * wk.world
        dist.all_gather_object(handles, (ok, mine))
        if all(h[0] for h in handles):
            try:
                p2p.connect([h[1] for h in handles])
            except pplb200.PplError as e:
                ok = 0
                sys.stderr.write("rank %d: mapping the peers' buffers failed (%s)\n" % (wk.rank, e))
        else:
            ok = 0
        oks = [None] * wk.world
        dist.all_gather_object(oks, ok)
        if all(oks):
            wk.row_reduce, wk.p2p = "p2p", p2p
        elif p2p is not None:
            p2p.destroy()
    if wk.row_reduce == "nccl":
        qbuf = torch.empty((M, N), dtype=torch.int32, device=dev)

    x_stage = torch.empty_like(wk.x[0])
    y_host = torch.empty((M, N), dtype=torch.float16).pin_memory()
    if wk.row_reduce == "p2p":
        # every rank holds (and quantizes) only its K shard; the row maxima are exchanged inside the quantizer
        xs = [wk.x[s][:, wk.k0:wk.k1].contiguous() for s in range(wk.nsets)]
        xs_host = wk.x_host[:, wk.k0:wk.k1].contiguous().pin_memory()
        xs_stage = torch.empty_like(xs[0])
        xq_shard = torch.empty((M, Kw), dtype=torch.int8, device=dev)

        def step(i):
            s = i % wk.nsets
            pplb200.minmax_quantize_fp16_p2p(wk.p2p, xs[s], out=xq_shard, scale=sm)
            pplb200.row_parallel_linear_p2p(wk.p2p, xq_shard, wk.w[s], sm, wk.sn, wk.bias, K, N, out=y)

        def e2e(i):
            s = i % wk.nsets
            xs_stage.copy_(xs_host, non_blocking=True)
            pplb200.minmax_quantize_fp16_p2p(wk.p2p, xs_stage, out=xq_shard, scale=sm)
            pplb200.row_parallel_linear_p2p(wk.p2p, xq_shard, wk.w[s], sm, wk.sn, wk.bias, K, N, out=y)
            y_host.copy_(y, non_blocking=True)

        h2d = xs_host.numel() * 2
        # the step's parts, timed one by one with --row-pieces (phases = 1 runs the GEMM and its pushes only)
        wk.pieces = {
            "sharded_quantizer": lambda i: pplb200.minmax_quantize_fp16_p2p(wk.p2p, xs[i % wk.nsets], out=xq_shard, scale=sm),
            "gemm_with_push": lambda i: pplb200.row_parallel_linear_p2p(wk.p2p, xq_shard, wk.w[i % wk.nsets], sm, wk.sn,
                                                                        wk.bias, K, N, out=y, phases=1),
            "linear_over_peer_memory": lambda i: pplb200.row_parallel_linear_p2p(wk.p2p, xq_shard, wk.w[i % wk.nsets], sm,
                                                                                 wk.sn, wk.bias, K, N, out=y),
        }
    else:
        def step(i):
            s = i % wk.nsets
            pplb200.minmax_quantize_fp16(wk.x[s], out=xq_full, scale=sm)
            pplb200.row_parallel_linear(xq_full[:, wk.k0:wk.k1], wk.w[s], sm, wk.sn, wk.bias, K, N, rank=wk.rank,
                                        size=wk.world, comm=comm, quant_buffer=qbuf, out=y)

        def e2e(i):
            s = i % wk.nsets
            x_stage.copy_(wk.x_host, non_blocking=True)
            pplb200.minmax_quantize_fp16(x_stage, out=xq_full, scale=sm)
            pplb200.row_parallel_linear(xq_full[:, wk.k0:wk.k1], wk.w[s], sm, wk.sn, wk.bias, K, N, rank=wk.rank,
                                        size=wk.world, comm=comm, quant_buffer=qbuf, out=y)
            y_host.copy_(y, non_blocking=True)

        h2d = wk.x_host.numel() * 2

    raw = torch.empty((M, N), dtype=torch.int32, device=dev) if qbuf is None else qbuf
    pplb200.minmax_quantize_fp16(wk.x[0], out=xq_full, scale=sm)  # real operand values for the GEMM timed alone

    def kernel_only(i):
        s = i % wk.nsets
        pplb200.gemm_i8i8(xq_full[:, wk.k0:wk.k1], wk.w[s], out=raw)

    gemm_bytes = M * Kw + N * Kw + 4 * M * N
    launches = 6 if wk.row_reduce == "p2p" else 3  # quantizer, GEMM, 2 flag kernels, reduce + dequant, row fetch
    return step, e2e, kernel_only, launches, h2d, M * N * 2, gemm_bytes


class RefLib:
    """The reference's own kernels (oracle/_ref/libref_i8i8.so), for the reference arm only."""

    def __init__(self):
        path = os.path.join(ROOT, "oracle", "_ref", "libref_i8i8.so")
        self.lib = ctypes.CDLL(path)
        vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float
        self.lib.ref_minmax_quantize_fp16.argtypes = [vp, vp, i64, i64, f32, i32, vp, vp]
        self.lib.ref_minmax_dequantize_fp16.argtypes = [vp, vp, vp, vp, vp, i64, i64, f32, f32, i32, vp]
        self.lib.ref_gemm_i8i8i32.argtypes = [vp, vp, vp, i64, i64, i64, vp, i64, vp]
        self.lib.ref_column_parallel_linear.argtypes = [vp, vp, vp, vp, vp, vp, f32, f32, i64, i64, i64, i32, vp, vp, i64, vp]


def build_reference(wk):
    """Reference arm: minmax_quantize_fp16 -> column_parallel_linear(gather_output=true, size 1)
    [-> minmax_quantize_fp16 of the output], all the reference's own code."""
    import torch
    ref = RefLib().lib
    M, K, N = wk.M, wk.K, wk.Nw
    requant = wk.cfg["requant"]
    dev = "cuda"
    xq = torch.empty((M, K), dtype=torch.int8, device=dev)
    sm = torch.empty((M,), dtype=torch.float16, device=dev)
    acc = torch.empty((M, N), dtype=torch.int32, device=dev)
    ys = [torch.empty((M, N), dtype=torch.float16, device=dev) for _ in range(wk.nsets)]
    yq = torch.empty((M, N), dtype=torch.int8, device=dev) if requant else None
    yqs = torch.empty((M,), dtype=torch.float16, device=dev) if requant else None
    ws = torch.empty((64 << 20,), dtype=torch.uint8, device=dev)
    P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    S = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run(x, s):
        rc = ref.ref_minmax_quantize_fp16(S(), P(x), M, K, 4096.0, 0, P(xq), P(sm))
        rc |= ref.ref_column_parallel_linear(S(), P(xq), P(wk.w[s]), P(wk.bias), P(sm), P(wk.sn), 1.0 / 4096, 1.0 / 8192,
                                             M, N, K, 1, P(acc), P(ws), ws.numel(), P(ys[s]))
        if requant:
            rc |= ref.ref_minmax_quantize_fp16(S(), P(ys[s]), M, N, 4096.0, 0, P(yq), P(yqs))
        if rc:
            raise RuntimeError("reference call failed rc=%d" % rc)

    def step(i):
        s = i % wk.nsets
        run(wk.x[s], s)

    x_stage = torch.empty_like(wk.x[0])
    y_host = torch.empty((M, N), dtype=torch.float16).pin_memory()
    yq_host = torch.empty((M, N), dtype=torch.int8).pin_memory() if requant else None
    ys_host = torch.empty((M,), dtype=torch.float16).pin_memory() if requant else None

    def e2e(i):
        s = i % wk.nsets
        x_stage.copy_(wk.x_host, non_blocking=True)
        run(x_stage, s)
        y_host.copy_(ys[s], non_blocking=True)
        if requant:
            yq_host.copy_(yq, non_blocking=True)
            ys_host.copy_(yqs, non_blocking=True)

    h2d = wk.x_host.numel() * 2
    d2h = M * N * 2 + ((M * N + M * 2) if requant else 0)
    return step, e2e, None, 3 + (1 if requant else 0), h2d, d2h, None


def cpu_baseline(name, budget_s=12.0):
    """Times the scalar host oracle (all host cores) on a bounded sample of the workload: the first
    `rows` token rows with the full N and K, repeated until about `budget_s` seconds of CPU work
    have been spent.  Returns the cpu_baseline object (TOPS from the fastest repetition)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as orc
    from pplb200 import workloads as wl
    c = wl.CONFIGS[name]
    cores = os.cpu_count() or 1
    orc.set_threads(cores)
    w = wl.make_weights(name)
    sn = wl.make_column_scales(name)
    bias = wl.make_bias(name)
    rows = min(c["M"], max(cores, 16))
    x = wl.make_activations(name, rows)
    t0 = time.perf_counter()
    orc.linear(x, w, sn, bias, requant=c["requant"])
    t_probe = time.perf_counter() - t0
    # grow the sample towards ~2 s per repetition, capped at the full batch
    while rows < c["M"] and t_probe * (2 * rows) / rows < 2.0:
        rows = min(c["M"], rows * 2)
        t_probe *= 2
    x = wl.make_activations(name, rows)
    best, spent, reps = float("inf"), 0.0, 0
    while spent < budget_s and reps < 1000:
        t0 = time.perf_counter()
        orc.linear(x, w, sn, bias, requant=c["requant"])
        dt = time.perf_counter() - t0
        best, spent, reps = min(best, dt), spent + dt, reps + 1
    tops = 2.0 * rows * c["N"] * c["K"] / best / 1e12
    return {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port",
            "sample": "%d of %d token rows, full N=%d K=%d, %d repetitions, %.1f s of CPU work, best %.3f s"
                      % (rows, c["M"], c["N"], c["K"], reps, spent, best)}


def run_config(name, args, rank, world, impl, sharded, want_cpu):
    import torch
    import pplb200
    from pplb200 import workloads as wl
    peaks = _peaks()
    wk = Workload(name, rank, world, sharded)
    wk.row_reduce_wanted = args.row_reduce
    if impl == "ours":
        step, e2e, kernel_only, launches, h2d, d2h, gemm_bytes = build_ours(wk)
    else:
        step, e2e, kernel_only, launches, h2d, d2h, gemm_bytes = build_reference(wk)

    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    # Eager passes first (one-time set-up, the reference's autotuner), then one CUDA graph per
    # buffer set so that the host's launch cost does not bound these microsecond-scale steps.
    # The row-parallel step contains NCCL collectives on a side stream; it is launched eagerly.
    use_graphs = wk.shard != "row" and not args.no_graphs
    for s in range(wk.nsets):
        step(s)
        e2e(s)
        if kernel_only:
            kernel_only(s)
    torch.cuda.synchronize()
    wrap = (lambda f: _Captured(f, wk.nsets)) if use_graphs else _Eager
    step, e2e = wrap(step), wrap(e2e)
    if kernel_only:
        kernel_only = wrap(kernel_only)
    ms = _time_steps(step, args.steps, args.warmup, world)
    ms_e2e = _time_steps(e2e, args.steps, args.warmup, world)
    ms_k = _time_steps(kernel_only, args.steps, args.warmup, 1) if kernel_only else None
    reps = max(5, min(20, args.steps // max(1, wk.nsets)))
    med_ms, min_ms = _round_stats(step, wk.nsets, reps, world)
    warm_ms = None
    if use_graphs and wk.nsets > 1 and wk.cfg["bound"] == "hbm":
        warm_ms = _time_steps(_SameSet(step), args.steps, args.warmup, world) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    if impl == "ours":
        st = int(_max_over_ranks(float(pplb200.gemm_status()), world))  # same verdict on every rank
        if st != 0:
            raise StatusWordSet("GEMM kernel reported a timed-out wait (status %d)" % st)

    replicas = world if (wk.shard is None and world > 1) else 1
    ops_per_step = wk.ops * replicas
    per_step = ms / args.steps
    line = {
        "metric": "W8A8 linear TOPS (quant+GEMM+dequant)",
        "value": ops_per_step / (per_step * 1e-3) / 1e12,
        "unit": "TOPS",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_step,
        "higher_is_better": True,
        "scaling": "weak" if wk.shard is None else "strong",
        "vs_baseline": None,
        "dtype": "int8 (int32 accumulate, fp16 in/out)",
        "data": "synthetic",
        "config": {
            "workload": "%s: %s" % (name, wk.cfg["desc"]),
            "M": wk.M, "K": wk.K, "N": wk.N,
            "sharding": ("replicas only (x%d)" % world) if wk.shard is None and world > 1 else
                        ("none" if wk.shard is None else "%s-parallel over %d GPUs" % (wk.shard, world)),
            "l2": wk.l2_note,
            "launch": ("CUDA graph replay, %d steps (one per buffer set) per graph" % wk.nsets) if use_graphs else "eager launches",
            "ms_per_step_median": med_ms, "ms_per_step_min": min_ms,
            "ms_per_step_stat": "over %d separately timed rounds of %d step(s)" % (reps, wk.nsets),
            "l2_warm_ms_per_step": warm_ms,  # one buffer set replayed: operands served from L2, NOT the headline
            "algorithmic_bytes_per_step": wl.algorithmic_bytes(name),
            "gb_per_s": wl.algorithmic_bytes(name) * replicas / (per_step * 1e-3) / 1e9 if wk.shard is None else None,
        },
        "e2e": {"value": ops_per_step / (ms_e2e / args.steps * 1e-3) / 1e12, "unit": "TOPS",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "note": "activations in / outputs out through pinned host memory each step; weights resident"},
        "gpu_launches": launches * args.steps,
        "clocks": clocks,
    }
    if impl == "reference":
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "TOPS", "cores": 0, "kind": "reference",
                                "sample": "full workload; the reference path is CUDA-only, so its own kernels "
                                          "(compute_80 PTX JIT + cuBLASLt int8) run on the same GPU"}
    if args.row_pieces and getattr(wk, "pieces", None):
        pieces = {}
        for name_, fn_ in wk.pieces.items():
            pieces[name_ + "_us"] = _time_steps(_Eager(fn_), args.steps, args.warmup, world) / args.steps * 1e3
        if ms_k is not None:
            pieces["gemm_local_us"] = ms_k / args.steps * 1e3
        line["row_parallel_pieces"] = pieces
    if ms_k is not None and rank == 0:
        kt = ms_k / args.steps * 1e-3
        if wk.cfg["bound"] == "hbm":
            ach = gemm_bytes / kt / 1e9
            line["roofline"] = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "frac": ach / peaks["hbm_gbs"], "traffic": TRAFFIC_NCU.get(name), "kernel": "gemm_i8_decode_kernel",
                                "kernel_us": kt * 1e6, "algorithmic_bytes_per_launch": gemm_bytes,
                                "peak_source": "%s STREAM-copy GB/s" % peaks["source"],
                                "frac_of_8TBs_datasheet": ach / 8000.0}
        else:
            ach = 2.0 * wk.M * wk.Nw * wk.Kw / kt / 1e12
            peak = 2.0 * peaks["bf16_tflops"]
            line["roofline"] = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TOP/s",
                                "frac": ach / peak, "traffic": TRAFFIC_NCU.get(name), "kernel": "gemm_i8_tcgen05_pair_kernel",
                                "kernel_us": kt * 1e6,
                                "peak_source": "2 x %s cuBLAS bf16 burst TFLOP/s (int8 issues at twice the bf16 rate)" % peaks["source"],
                                "frac_of_4500_datasheet": ach / 4500.0}
    if want_cpu and rank == 0 and impl == "ours":
        line["cpu_baseline"] = cpu_baseline(name)
    if getattr(wk, "row_reduce", None) is not None:
        line["config"]["row_reduce"] = ("activations quantized shard by shard (row maxima exchanged in the kernel), int32 tiles pushed to the row owner over peer-mapped memory, fp16 rows fetched back"
                                        if wk.row_reduce == "p2p" else "NCCL int32 reduce-scatter + fp16 all-gather")
    if getattr(wk, "p2p", None) is not None:
        st = int(_max_over_ranks(float(wk.p2p.status()), world))  # same verdict on every rank
        torch.cuda.synchronize()
        import torch.distributed as dist
        dist.barrier()  # no rank unmaps its buffer while a peer may still read it
        wk.p2p.destroy()
        if st != 0:
            raise StatusWordSet("a bounded wait on a peer expired (status %d)" % st)
    if getattr(wk, "comm", None) is not None:
        torch.cuda.synchronize()
        pplb200.nccl_comm_destroy(wk.comm)
    return line


def aux_kernels(steps, warmup):
    """The memory-bound producers timed alone on c4's activation shape (M 8192 x K 8192, 134 MB in,
    67 MB out: larger than L2): the per-token quantizer and the fused skip + RMSNorm + quantize.
    Algorithmic bytes: quantizer 3 B per element + 2 B per row; fused producer 7 B per element
    (input, skip in; skip_out, int8 out) + 2 B per row + the 16 KB weight vector."""
    import torch
    import pplb200
    peaks = _peaks()
    M, K = 8192, 8192
    g = torch.Generator(device="cuda").manual_seed(0xB2000004)
    xs = [torch.randn((M, K), generator=g, device="cuda", dtype=torch.float16) for _ in range(2)]
    skip = torch.randn((M, K), generator=g, device="cuda", dtype=torch.float16)
    w = torch.ones((K,), device="cuda", dtype=torch.float16)
    q = torch.empty((M, K), dtype=torch.int8, device="cuda")
    sc = torch.empty((M,), dtype=torch.float16, device="cuda")
    out = {}
    cases = {
        "minmax_quantize_fp16": (lambda i: pplb200.minmax_quantize_fp16(xs[i % 2], out=q, scale=sc), 3 * M * K + 2 * M),
        "skip_rmsnorm_minmax_quantize_fp16": (lambda i: pplb200.skip_rmsnorm_minmax_quantize_fp16(xs[i % 2], w, skip), 7 * M * K + 2 * M + 2 * K),
    }
    for name, (fn, nbytes) in cases.items():
        ms = _time_steps(_Eager(fn), steps, warmup, 1)
        t = ms / steps * 1e-3
        out[name] = {"shape": [M, K], "us": t * 1e6, "gb_per_s": nbytes / t / 1e9,
                     "frac_of_measured_hbm": nbytes / t / 1e9 / peaks["hbm_gbs"], "algorithmic_bytes": nbytes}
    del xs, skip, q

    # c2's real successor: the fused gate+up projection (GEMM + dequantize + SwiGLU + re-quantize in one
    # pass) against the reference's structure (raw int32 linear, then the stand-alone SwiGLU kernel).
    M, K, D = 4096, 4096, 11008
    xq = torch.randint(-127, 128, (M, K), generator=g, device="cuda", dtype=torch.int8)
    ws_ = [torch.randint(-127, 128, (2 * D, K), generator=g, device="cuda", dtype=torch.int8) for _ in range(2)]
    sm = (torch.rand(M, device="cuda") + 0.5).half()
    sn = (torch.rand(2 * D, device="cuda") * 1e-2 + 1e-3).half()
    scratch = torch.empty((pplb200.lib.pplb200_i8i8_gate_up_swiglu_workspace_bytes(M, D, K),), dtype=torch.uint8, device="cuda")
    outs = (torch.empty((M, D), dtype=torch.float16, device="cuda"), torch.empty((M, D), dtype=torch.int8, device="cuda"),
            torch.empty((M,), dtype=torch.float16, device="cuda"))
    acc = torch.empty((M, 2 * D), dtype=torch.int32, device="cuda")

    def two_step(i):
        pplb200.column_parallel_linear(xq, ws_[i % 2], None, None, None, K, 2 * D, gather_output=False, out=acc)
        pplb200.minmax_requantize_swiglu_fp16(acc, sm, sn)

    for name, fn in (("gate_up_swiglu_requant (fused)", lambda i: pplb200.gate_up_swiglu_requant(xq, ws_[i % 2], sm, sn, ws=scratch, out=outs)),
                     ("raw linear + minmax_requantize_swiglu_fp16", two_step)):
        ms = _time_steps(_Eager(fn), steps, warmup, 1)
        t = ms / steps * 1e-3
        out[name] = {"shape": [M, K, 2 * D], "us": t * 1e6, "tops": 2.0 * M * 2 * D * K / t / 1e12}
    return out


def reference_on_cpu(args, name):
    """Fallback reference arm when oracle/_ref is absent: the host port of the path."""
    cb = cpu_baseline(name)
    return {"metric": "W8A8 linear TOPS (quant+GEMM+dequant)", "value": cb["value"], "unit": "TOPS", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 (int32 accumulate, fp16 in/out)",
            "data": "synthetic", "impl": "reference", "config": {"workload": name}, "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1")
    ap.add_argument("--extras", action="store_true", help="also run the other configurations (sharded where they shard)")
    ap.add_argument("--aux", action="store_true", help="also time the quantizer and the RMSNorm+quantize producer alone")
    ap.add_argument("--row-reduce", default="p2p", choices=["p2p", "nccl"],
                    help="reduction of the row-parallel linear: over peer-mapped memory (default) or NCCL collectives")
    ap.add_argument("--row-pieces", action="store_true",
                    help="row-parallel workload over peer memory: also time the sharded quantizer, the GEMM with its pushes and the whole linear")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graphs", action="store_true", help="launch eagerly instead of replaying CUDA graphs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    if args.impl == "reference":
        # the reference arm runs on rank 0 alone (no process group is needed); other ranks leave
        if int(os.environ.get("RANK", "0")) != 0:
            return
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        have_ref = os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libref_i8i8.so"))
        if not have_ref:
            print(json.dumps(reference_on_cpu(args, args.workload)))
            return
        line = run_config(args.workload, args, 0, 1, "reference", False, False)
        line["n_gpus"] = args.gpus
        print(json.dumps(line))
        return

    rank, world = _dist_setup(args.gpus)
    sharded = args.workload != "c1"
    line = run_config(args.workload, args, rank, world, "ours", sharded, not args.no_cpu and world == 1)
    # On more than one GPU the default line (c1 replicas) is accompanied by the two configurations
    # that really shard: c2 (column parallel, no communication) and c3 (row parallel, int32 reduction).
    extra_names = ("c0", "c1", "c2", "c3", "c4") if args.extras else (("c2", "c3") if world > 1 and not sharded else ())
    if extra_names:
        extras = {}
        for name in extra_names:
            if name == args.workload:
                continue
            try:
                ex = run_config(name, args, rank, world, "ours", True, False)
            except StatusWordSet as e:  # raised on every rank alike: the headline line survives
                extras[name] = {"error": str(e)}
                continue
            extras[name] = {k: ex[k] for k in ("value", "unit", "ms_per_step", "scaling", "config", "e2e") if k in ex}
            if "roofline" in ex:
                extras[name]["roofline"] = ex["roofline"]
        line["other_configs"] = extras
    if args.aux and rank == 0:
        line["aux_kernels"] = aux_kernels(args.steps, args.warmup)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
