#!/usr/bin/env python
"""W8A8 (i8i8) linear benchmark: quantize + int8 GEMM + dequant(+bias)(+re-quantize).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c0..c4]
                    [--only] [--aux]

One "step" = one pass of the whole path over one batch of synthetic input of the chosen
configuration.  Prints ONE JSON line on rank 0.  metric = TOPS = 2*M*N*K / t.

Headline workload: c4 (M 8192, K 8192, N 28672), the largest configuration that fits one GPU; on N > 1
GPUs its N dimension is split over the ranks (column parallel, no communication, "scaling": "strong").
The other configurations are measured in the same run and summarised under roofline.per_config
(c0 / c1 / c2 / c3 on one GPU; c2 column-parallel and c3 row-parallel on N > 1 GPUs), so that one line
carries all five.  --only skips them.

  value     device-resident: inputs already in HBM, CUDA-event time over K steps (max over ranks)
  e2e       same path with the step's activations copied from pinned host memory and the step's
            outputs copied back to pinned host memory inside the timed region (weights stay
            resident in HBM, as they do in the reference's deployment)
  roofline  dominant kernel (the tcgen05 GEMM with fused epilogue) timed alone with CUDA events;
            peak = the int8 tensor-core ceiling measured in this run by the library's issue-rate probe
            (prefill) or the measured copy bandwidth (decode)
  cpu_baseline  the scalar host oracle on the box's cores (a reported baseline, not a target)

--impl reference runs the reference's own kernels (compiled unmodified into oracle/_ref:
minmax_quantize_fp16 -> column_parallel_linear / row_parallel_linear with cuBLASLt int8 inside
[-> minmax_quantize_fp16]) for the same workloads on the same number of GPUs; it never loads this
repository's library.  If oracle/_ref is absent it times the host oracle port instead.
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
HEADLINE = "c4"
ALL_CONFIGS = ("c0", "c1", "c2", "c3", "c4")
METRIC = "W8A8 linear TOPS (quant+GEMM+dequant)"
DTYPE = "int8 (int32 accumulate, fp16 in/out)"
INT8_DATASHEET_TOPS = 4500.0
HBM_DATASHEET_GBS = 8000.0
# measured on this pool: SM stores of whole 128-byte lines into a peer's memory (GB/s per direction)
PEER_STORE_GBS = 680.0


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_sustained=1400.0, source="fallback")


def _ncu_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of each configuration's dominant kernel, from the
    ncu captures summarised under profiles/ (bytes)."""
    p = os.path.join(ROOT, "profiles", "ncu_dram_traffic.json")
    try:
        with open(p) as f:
            return json.load(f)["per_launch_bytes"]
    except (OSError, KeyError, ValueError):
        return {}


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


def _reduce_over_ranks(v, world, op="max"):
    import torch
    if world == 1:
        return v
    import torch.distributed as dist
    t = torch.tensor([v], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.MIN)
    return float(t.item())


def _max_over_ranks(ms, world):
    return _reduce_over_ranks(ms, world, "max")


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
    copies so that consecutive steps do not hit each other's data in L2.  Uses torch and numpy only
    (both arms of the benchmark build their inputs here)."""

    def __init__(self, name, rank, world, sharded, keep_full=False):
        import numpy as np
        import torch
        import w8a8_workloads as wl
        self.name, self.cfg = name, wl.CONFIGS[name]
        c = self.cfg
        self.M, self.K, self.N = c["M"], c["K"], c["N"]
        self.rank, self.world = rank, world
        self.shard = c["shard"] if (sharded and world > 1) else None
        x = wl.make_activations(name)
        w = wl.make_weights(name)
        sn = wl.make_column_scales(name)
        bias = wl.make_bias(name)
        # the unsharded operands, for the sharded-equals-unsharded check (a seeded sample of rows)
        self.full = None
        if keep_full and self.shard is not None:
            rows = np.unique(np.concatenate([np.arange(0, 128), np.arange(self.M - 128, self.M),
                                             np.random.default_rng(7).integers(0, self.M, 256)]))
            self.full = dict(rows=torch.from_numpy(rows).cuda(), x=torch.from_numpy(x[rows]).cuda(),
                             w=torch.from_numpy(w).cuda(), sn=torch.from_numpy(sn).cuda(),
                             bias=None if bias is None else torch.from_numpy(bias).cuda())
        self.Kw, self.Nw, self.n0 = self.K, self.N, 0
        if self.shard == "column":
            n0, n1 = wl.shard_rows(self.N, world, rank)
            w, sn = w[n0:n1], sn[n0:n1]
            bias = None if bias is None else bias[n0:n1]
            self.Nw, self.n0 = n1 - n0, n0
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

    def sharding_note(self):
        if self.shard is None:
            return "none"
        return "%s-parallel over %d GPUs" % (self.shard, self.world)


def _slices_leftover_tiles(M, N, K, pairs=74):
    """True when the large-batch GEMM of this shape cuts its leftover tiles into K slices, which adds one launch (the
    kernel that clears the slice scratch) to the step.  Mirrors the launcher's rule in csrc/gemm_i8_tcgen05.cu; only
    used for the launch count reported as `gpu_launches`."""
    if M <= 128:
        return False
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    if tiles < pairs:
        return False
    rest, nkb = tiles % pairs, (K + 127) // 128
    if rest == 0 or rest > 40:
        return False
    f = min(pairs // rest, 8, nkb // 4)
    return f >= 2 and 4 * (f - 1) * nkb >= f * (52 + 5 * rest)


def build_ours(wk):
    """Returns (step(i), e2e_step(i), kernel_only(i), launches_per_step, h2d, d2h, gemm_bytes, result(s))."""
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

        # end to end through the library's host-buffer entry point (pplb200_i8i8_linear_fp16_host): pinned host
        # activations in, pinned host results out, copies and compute of consecutive chunks (128, 128, 256, 512, then 1024 tokens) overlapped
        y_host = torch.empty((M, Nw), dtype=torch.float16).pin_memory()
        yq_host = torch.empty((M, Nw), dtype=torch.int8).pin_memory() if requant else None
        ys_host = torch.empty((M,), dtype=torch.float16).pin_memory() if requant else None
        hosts = [pplb200.W8A8LinearHost(wk.w[s], wk.sn, wk.bias, max_tokens=M, requant=requant) for s in range(min(wk.nsets, 2))]
        wk.e2e_eager = True  # the entry point drives three streams itself: launched eagerly, not from a captured graph

        def e2e(i):
            s = i % wk.nsets
            h = hosts[s % len(hosts)]
            h.w = wk.w[s]
            h(wk.x_host, y_host, yq_host, ys_host)

        h2d = wk.x_host.numel() * 2
        d2h = M * Nw * 2 + ((M * Nw + M * 2) if requant else 0)

        # dominant kernel alone: GEMM + fused epilogue on pre-quantized activations
        xq, sm = pplb200.minmax_quantize_fp16(wk.x[0])
        mode = pplb200.EPI_DEQUANT_F16
        ys = [l.y for l in lins]
        gws = torch.empty((max(pplb200.gemm_workspace_bytes(M, Nw, K, mode), 256),), dtype=torch.uint8, device=dev)

        def kernel_only(i):
            s = i % wk.nsets
            pplb200.gemm_i8i8(xq, wk.w[s], mode=mode, scale_m=sm, scale_n=wk.sn, bias=wk.bias, ws=gws, out=ys[s])

        gemm_bytes = M * K + Nw * K + 2 * Nw + (2 * Nw if wk.bias is not None else 0) + 2 * M + 2 * M * Nw
        launches = 2 + (1 if requant else 0) + (1 if _slices_leftover_tiles(M, Nw, K) else 0)
        return step, e2e, kernel_only, launches, h2d, d2h, gemm_bytes, (lambda s: lins[s].y)

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
        # the step's parts, timed one by one (phases = 1 runs the GEMM and its pushes only)
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

    gws = torch.empty((max(pplb200.gemm_workspace_bytes(M, N, Kw, pplb200.EPI_RAW_I32), 256),), dtype=torch.uint8, device=dev)

    def kernel_only(i):
        s = i % wk.nsets
        pplb200.gemm_i8i8(xq_full[:, wk.k0:wk.k1], wk.w[s], ws=gws, out=raw)

    gemm_bytes = M * Kw + N * Kw + 4 * M * N
    # quantizer, GEMM, 2 flag kernels, reduce + dequant, row fetch (+ the clearing of the K-slice scratch)
    launches = (6 if wk.row_reduce == "p2p" else 3) + (1 if _slices_leftover_tiles(M, N, Kw) else 0)
    return step, e2e, kernel_only, launches, h2d, M * N * 2, gemm_bytes, (lambda s: y)


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
        self.lib.ref_row_parallel_linear.argtypes = [vp, vp, vp, vp, vp, vp, f32, f32, i64, i64, i64, i32, i32, vp, vp, vp, i64, vp]
        self.lib.ref_nccl_get_unique_id.argtypes = [vp]
        self.lib.ref_nccl_comm_init.argtypes = [vp, i32, i32, ctypes.POINTER(vp)]
        self.lib.ref_nccl_comm_destroy.argtypes = [vp]


def build_reference(wk):
    """Reference arm, all the reference's own code: minmax_quantize_fp16 -> column_parallel_linear
    (gather_output = true on this rank's shard; cuBLASLt int8 inside) [-> minmax_quantize_fp16 of the
    output]; for the row-parallel workload every rank quantizes its own K shard and calls the reference's
    row_parallel_linear (dequantize, then fp16 all-reduce over NCCL)."""
    import torch
    ref = RefLib().lib
    M, K, N = wk.M, wk.Kw, wk.Nw
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
    row = wk.shard == "row"
    comm = ctypes.c_void_p()
    if row:
        import torch.distributed as dist
        buf = ctypes.create_string_buffer(128)
        if wk.rank == 0 and ref.ref_nccl_get_unique_id(buf):
            raise RuntimeError("ncclGetUniqueId failed")
        uid = [bytes(buf.raw) if wk.rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        if ref.ref_nccl_comm_init(ctypes.create_string_buffer(uid[0], 128), wk.rank, wk.world, ctypes.byref(comm)):
            raise RuntimeError("ncclCommInitRank failed")
        wk.ref_comm = (ref, comm)
        xs = [wk.x[s][:, wk.k0:wk.k1].contiguous() for s in range(wk.nsets)]
        xs_host = wk.x_host[:, wk.k0:wk.k1].contiguous().pin_memory()
    else:
        xs, xs_host = wk.x, wk.x_host

    def run(x, s):
        rc = ref.ref_minmax_quantize_fp16(S(), P(x), M, K, 4096.0, 0, P(xq), P(sm))
        if row:
            rc |= ref.ref_row_parallel_linear(S(), P(xq), P(wk.w[s]), P(wk.bias), P(sm), P(wk.sn), 1.0 / 4096, 1.0 / 8192,
                                              M, N, wk.K, wk.rank, wk.world, comm, P(acc), P(ws), ws.numel(), P(ys[s]))
        else:
            rc |= ref.ref_column_parallel_linear(S(), P(xq), P(wk.w[s]), P(wk.bias), P(sm), P(wk.sn), 1.0 / 4096, 1.0 / 8192,
                                                 M, N, K, 1, P(acc), P(ws), ws.numel(), P(ys[s]))
        if requant:
            rc |= ref.ref_minmax_quantize_fp16(S(), P(ys[s]), M, N, 4096.0, 0, P(yq), P(yqs))
        if rc:
            raise RuntimeError("reference call failed rc=%d" % rc)

    def step(i):
        s = i % wk.nsets
        run(xs[s], s)

    x_stage = torch.empty_like(xs[0])
    y_host = torch.empty((M, N), dtype=torch.float16).pin_memory()
    yq_host = torch.empty((M, N), dtype=torch.int8).pin_memory() if requant else None
    ys_host = torch.empty((M,), dtype=torch.float16).pin_memory() if requant else None

    def e2e(i):
        s = i % wk.nsets
        x_stage.copy_(xs_host, non_blocking=True)
        run(x_stage, s)
        y_host.copy_(ys[s], non_blocking=True)
        if requant:
            yq_host.copy_(yq, non_blocking=True)
            ys_host.copy_(yqs, non_blocking=True)

    # the reference's GEMM alone (cuBLASLt int8 through its gemm_i8i8i32 wrapper), on real operand values
    def kernel_only(i):
        s = i % wk.nsets
        if ref.ref_gemm_i8i8i32(S(), P(xq), P(wk.w[s]), M, N, K, P(ws), ws.numel(), P(acc)):
            raise RuntimeError("reference GEMM failed")

    h2d = xs_host.numel() * 2
    d2h = M * N * 2 + ((M * N + M * 2) if requant else 0)
    gemm_bytes = M * K + N * K + 4 * M * N
    return step, e2e, kernel_only, 3 + (1 if requant else 0), h2d, d2h, gemm_bytes, (lambda s: ys[s])


def cpu_baseline(name, budget_s=12.0):
    """Times the scalar host oracle (all host cores) on a bounded sample of the workload: the first
    `rows` token rows with the full N and K, repeated until about `budget_s` seconds of CPU work
    have been spent.  Returns the cpu_baseline object (TOPS from the fastest repetition)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as orc
    import w8a8_workloads as wl
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
            "sample": "%s: %d of %d token rows, full N=%d K=%d, %d repetitions, %.1f s of CPU work, best %.3f s"
                      % (name, rows, c["M"], c["N"], c["K"], reps, spent, best)}


def _sharded_equals_unsharded(wk, result_of):
    """Seeded sample of output rows of the sharded step against the unsharded fused linear run on this rank
    with the full operands: 1.0 when bit-identical on every rank, else 0.0 (minimum over ranks)."""
    import torch
    import pplb200
    f = wk.full
    lin = pplb200.W8A8Linear(f["w"], f["sn"], f["bias"], max_tokens=f["x"].shape[0], requant=False)
    y_full = lin(f["x"])
    y = result_of(0).index_select(0, f["rows"])
    if wk.shard == "column":
        y_full = y_full[:, wk.n0:wk.n0 + wk.Nw]
    torch.cuda.synchronize()
    same = 1.0 if torch.equal(y.view(torch.int16), y_full.contiguous().view(torch.int16)) else 0.0
    del lin, y_full
    return _reduce_over_ranks(same, wk.world, "min")


def run_config(name, args, rank, world, impl, sharded, sample_clocks=False, check_shard=False):
    """Measures one configuration; returns a dict of raw results (identical on every rank where it matters)."""
    import torch
    wk = Workload(name, rank, world, sharded, keep_full=check_shard and impl == "ours")
    wk.row_reduce_wanted = args.row_reduce
    build = build_ours if impl == "ours" else build_reference
    step, e2e, kernel_only, launches, h2d, d2h, gemm_bytes, result_of = build(wk)

    # Eager passes first (one-time set-up, the reference's autotuner), then one CUDA graph per
    # buffer set so that the host's launch cost does not bound microsecond-scale steps.
    # The row-parallel step exchanges data between ranks inside its kernels; it is launched eagerly.
    use_graphs = wk.shard != "row" and not args.no_graphs
    for s in range(wk.nsets):
        step(s)
        e2e(s)
        kernel_only(s)
    torch.cuda.synchronize()
    bit_exact = None
    if wk.full is not None:
        step(0)
        bit_exact = _sharded_equals_unsharded(wk, result_of) == 1.0
        wk.full = None
    wrap = (lambda f: _Captured(f, wk.nsets)) if use_graphs else _Eager
    step, e2e, kernel_only = wrap(step), (_Eager(e2e) if getattr(wk, "e2e_eager", False) else wrap(e2e)), wrap(kernel_only)
    sampler = ClockSampler(torch.cuda.current_device()) if (sample_clocks and rank == 0) else None
    if sampler:
        sampler.start()
    ms = _time_steps(step, args.steps, args.warmup, world)
    ms_e2e = _time_steps(e2e, args.steps, args.warmup, world)
    clocks = sampler.stop() if sampler else None
    ms_k = _time_steps(kernel_only, args.steps, args.warmup, 1)
    reps = max(5, min(20, args.steps // max(1, wk.nsets)))
    med_ms, min_ms = _round_stats(step, wk.nsets, reps, world)
    warm_ms = None
    if use_graphs and wk.nsets > 1 and wk.cfg["bound"] == "hbm":
        warm_ms = _time_steps(_SameSet(step), args.steps, args.warmup, world) / args.steps
    pieces = None
    if getattr(wk, "pieces", None):
        pieces = {k + "_us": _time_steps(_Eager(fn), args.steps, args.warmup, world) / args.steps * 1e3
                  for k, fn in wk.pieces.items()}
        wk.pieces = None

    status_error = None
    if impl == "ours":
        import pplb200
        st = int(_max_over_ranks(float(pplb200.gemm_status()), world))  # same verdict on every rank
        if st != 0:
            status_error = "GEMM kernel reported a timed-out wait (status %d)" % st
    row_reduce = getattr(wk, "row_reduce", None)
    if getattr(wk, "p2p", None) is not None:
        st = int(_max_over_ranks(float(wk.p2p.status()), world))
        torch.cuda.synchronize()
        import torch.distributed as dist
        dist.barrier()  # no rank unmaps its buffer while a peer may still read it
        wk.p2p.destroy()
        wk.p2p = None
        if st != 0:
            status_error = "a bounded wait on a peer expired (status %d)" % st
    if getattr(wk, "comm", None) is not None:
        import pplb200
        torch.cuda.synchronize()
        pplb200.nccl_comm_destroy(wk.comm)
        wk.comm = None
    if getattr(wk, "ref_comm", None) is not None:
        torch.cuda.synchronize()
        wk.ref_comm[0].ref_nccl_comm_destroy(wk.ref_comm[1])
        wk.ref_comm = None
    if status_error:
        raise StatusWordSet(status_error)

    # keep only plain numbers and strings: the device buffers are released when this function returns
    import w8a8_workloads as wl
    replicas = world if (wk.shard is None and world > 1) else 1
    return dict(name=name, desc=wk.cfg["desc"], bound=wk.cfg["bound"], M=wk.M, K=wk.K, N=wk.N, Kw=wk.Kw, Nw=wk.Nw,
                shard=wk.shard, world=world, replicas=replicas, ops=wk.ops, nsets=wk.nsets, l2_note=wk.l2_note,
                sharding=("replicas only (x%d)" % world) if replicas > 1 else wk.sharding_note(),
                alg_bytes=wl.algorithmic_bytes(name),
                ms=ms, ms_e2e=ms_e2e, ms_k=ms_k, med_ms=med_ms, min_ms=min_ms, warm_ms=warm_ms,
                launches=launches, h2d=h2d, d2h=d2h, gemm_bytes=gemm_bytes, clocks=clocks, use_graphs=use_graphs,
                pieces=pieces, row_reduce=row_reduce, bit_exact=bit_exact, reps=reps)


def static_config(res, others):
    """The part of the line that names the workload: no measured value, identical for both arms."""
    return {
        "workload": "%s: %s" % (res["name"], res["desc"]),
        "M": res["M"], "K": res["K"], "N": res["N"],
        "sharding": res["sharding"],
        "l2": res["l2_note"],
        "algorithmic_bytes_per_step": res["alg_bytes"],
        "inputs": "seeded synthetic tensors of the configuration's shapes and distributions (w8a8_workloads.py)",
        "also_measured": list(others),
    }


def kernel_roofline(res, args, peaks, tensor_peak, impl):
    """roofline-shaped object for the dominant kernel of one configuration."""
    kt = res["ms_k"] / args.steps * 1e-3
    traffic = _ncu_traffic().get(res["name"]) if (impl == "ours" and res["shard"] is None) else None
    ref_kernel = "cuBLASLt int8 via the reference's gemm_i8i8i32"
    if res["bound"] == "hbm":
        ach = res["gemm_bytes"] / kt / 1e9
        return {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                "traffic": traffic, "kernel": "gemm_i8_decode_kernel" if impl == "ours" else ref_kernel,
                "kernel_us": kt * 1e6, "algorithmic_bytes_per_launch": res["gemm_bytes"],
                "peak_source": "%s STREAM-copy GB/s" % peaks["source"], "frac_of_8TBs_datasheet": ach / HBM_DATASHEET_GBS}
    ach = 2.0 * res["M"] * res["Nw"] * res["Kw"] / kt / 1e12
    if tensor_peak is not None:
        peak, src = tensor_peak["tops"], "int8 tcgen05 issue-rate probe of this run (%s)" % tensor_peak["how"]
    else:
        peak, src = 2.0 * peaks["bf16_tflops"], "2 x %s cuBLAS bf16 burst TFLOP/s (no int8 probe in this arm)" % peaks["source"]
    return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TOP/s", "frac": ach / peak, "traffic": traffic,
            "kernel": "gemm_i8_tcgen05_pair_kernel" if impl == "ours" else ref_kernel,
            "kernel_us": kt * 1e6, "peak_source": src, "frac_of_4500_datasheet": ach / INT8_DATASHEET_TOPS,
            "frac_of_2x_bf16_burst": ach / (2.0 * peaks["bf16_tflops"])}


def compact(res, args, peaks, tensor_peak, impl):
    """Per-configuration summary (a few numbers) for roofline.per_config."""
    world = res["world"]
    per_step = res["ms"] / args.steps
    rf = kernel_roofline(res, args, peaks, tensor_peak, impl)
    out = {"sharding": res["sharding"], "ms_per_step": round(per_step, 6),
           "tops": round(res["ops"] * res["replicas"] / (per_step * 1e-3) / 1e12, 2),
           "e2e_tops": round(res["ops"] * res["replicas"] / (res["ms_e2e"] / args.steps * 1e-3) / 1e12, 2),
           "kernel_us": round(rf["kernel_us"], 2), "bound": rf["bound"], "frac": round(rf["frac"], 4)}
    if rf["bound"] == "tensor":
        out["frac_of_datasheet"] = round(rf["frac_of_4500_datasheet"], 4)
    else:
        out["frac_of_datasheet"] = round(rf["frac_of_8TBs_datasheet"], 4)
        out["step_gb_per_s"] = round(res["alg_bytes"] * res["replicas"] / (per_step * 1e-3) / 1e9, 1)
        if res["warm_ms"] is not None:
            out["l2_warm_ms_per_step"] = round(res["warm_ms"], 6)  # one buffer set replayed: NOT the headline
    if res["bit_exact"] is not None:
        out["sharded_bit_exact"] = bool(res["bit_exact"])
    if res["row_reduce"] is not None:
        out["row_reduce"] = res["row_reduce"]
    if res["pieces"]:
        out["pieces_us"] = {k: round(v, 1) for k, v in res["pieces"].items()}
        if res["shard"] == "row":
            wire = (world - 1) / world * res["M"] * res["N"] * 4 / (PEER_STORE_GBS * 1e9) * 1e6
            out["wire_bound_us"] = round(wire + res["pieces"].get("sharded_quantizer_us", 0.0), 1)
            out["wire_bound_note"] = ("int32 partials leaving each GPU / %.0f GB/s measured peer-store rate + sharded quantizer"
                                      % PEER_STORE_GBS)
    return out


def tensor_peak_probe():
    """The library's int8 tcgen05 issue-rate probe: every SM issues back-to-back kind::i8 MMAs on operands that
    stay in shared memory (no loads, no epilogue).  Returns {"tops", "how", ...} or None."""
    import pplb200
    if not hasattr(pplb200, "tensor_peak_probe"):
        return None
    try:
        return pplb200.tensor_peak_probe()
    except Exception as e:  # the probe is diagnostic: a failure must not cost the bench line
        sys.stderr.write("tensor peak probe failed: %s\n" % e)
        return None


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
    # single-launch read-only bulk-copy stream: what one launch of a weight matrix's size can reach
    out["tma_stream_read"] = pplb200.stream_read_probe()
    del xq, ws_, acc, outs, scratch
    torch.cuda.empty_cache()

    # where a small-batch GEMM launch spends its time (the kernel's own global-timer stamps), HBM-cold
    phases = {}
    for name, (M, K, N) in (("c0", (16, 4096, 4096)), ("c1", (128, 4096, 12288)), ("M16 N12288", (16, 4096, 12288)),
                            ("M64 N12288", (64, 4096, 12288))):
        nset = 10
        a = torch.randint(-127, 128, (M, K), generator=g, device="cuda", dtype=torch.int8)
        bs = [torch.randint(-127, 128, (N, K), generator=g, device="cuda", dtype=torch.int8) for _ in range(nset)]
        sm_ = (torch.rand(M, device="cuda") + 0.5).half()
        sn_ = (torch.rand(N, device="cuda") * 1e-2 + 1e-3).half()
        bias = torch.randn(N, device="cuda").half()
        y = torch.empty((M, N), dtype=torch.float16, device="cuda")
        fn = lambda i: pplb200.gemm_i8i8(a, bs[i % nset], mode=pplb200.EPI_DEQUANT_F16, scale_m=sm_, scale_n=sn_, bias=bias, out=y)
        for i in range(nset):
            fn(i)
        torch.cuda.synchronize()
        cap = _Captured(fn, nset)
        per_launch = _time_steps(cap, 4 * nset, nset, 1) / (4 * nset) * 1e3
        prof = pplb200.decode_phase_profile(lambda: fn(3))
        for _ in range(3):
            fn(0)
        warm = pplb200.decode_phase_profile(lambda: fn(0))
        phases[name] = dict(prof, us_per_launch_in_graph=round(per_launch, 2), l2_warm_main_loop_us=warm["main_loop_us"])
        del bs, cap
        torch.cuda.empty_cache()
    out["small_batch_gemm_phases"] = phases

    # wait counters of the CTA-pair GEMM's MMA / TMA / epilogue threads on c2's shape
    M, K, N = 4096, 4096, 22016
    a = torch.randint(-127, 128, (M, K), generator=g, device="cuda", dtype=torch.int8)
    b = torch.randint(-127, 128, (N, K), generator=g, device="cuda", dtype=torch.int8)
    sm_ = (torch.rand(M, device="cuda") + 0.5).half()
    sn_ = (torch.rand(N, device="cuda") * 1e-2 + 1e-3).half()
    y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    fn = lambda: pplb200.gemm_i8i8(a, b, mode=pplb200.EPI_DEQUANT_F16, scale_m=sm_, scale_n=sn_, out=y)
    for _ in range(3):
        fn()
    st = pplb200.gemm_stall_profile(fn)
    if st:
        tiles = -(-M // 256) * -(-N // 256)
        st["mma_thread_cycles_per_k_block"] = round(st["mma_thread_cycles"] / (tiles / 74.0 * (K // 128)), 1)
    out["pair_gemm_thread_waits_c2"] = st
    del a, b, y
    torch.cuda.empty_cache()

    # Leftover tiles: GEMM + fused dequant of shapes whose tile count is not a multiple of the 74 CTA pairs, with the K
    # slicing of the leftover tiles switched off and on (debug switch of the library); launches replayed from a CUDA
    # graph over enough operand sets to exceed L2.  The first two shapes are c4's and c2's shards on 8 GPUs.
    slices = {}
    for (M, N, K) in ((8192, 3584, 8192), (4096, 2752, 4096), (8192, 3328, 8192), (2048, 8192, 28672)):
        nset = max(2, int(200e6 // (N * K + M * K)) + 1)
        As = [torch.randint(-127, 128, (M, K), generator=g, device="cuda", dtype=torch.int8) for _ in range(nset)]
        Bs = [torch.randint(-127, 128, (N, K), generator=g, device="cuda", dtype=torch.int8) for _ in range(nset)]
        sm_ = (torch.rand(M, device="cuda") + 0.5).half()
        sn_ = (torch.rand(N, device="cuda") * 1e-2 + 1e-3).half()
        ys = [torch.empty((M, N), dtype=torch.float16, device="cuda") for _ in range(nset)]
        ws = torch.empty((pplb200.gemm_workspace_bytes(M, N, K, pplb200.EPI_DEQUANT_F16),), dtype=torch.uint8, device="cuda")
        graphs = {}
        try:
            for on in (False, True):
                pplb200.gemm_tail_split(on)
                run = lambda: [pplb200.gemm_i8i8(As[i], Bs[i], mode=pplb200.EPI_DEQUANT_F16, scale_m=sm_, scale_n=sn_, ws=ws, out=ys[i])
                               for i in range(nset)]
                run()
                torch.cuda.synchronize()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    run()
                graphs[on] = gr
        finally:
            pplb200.gemm_tail_split(True)
        times = {False: [], True: []}
        for it in range(12):
            for on in (False, True):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                graphs[on].replay()
                e1.record()
                torch.cuda.synchronize()
                if it >= 4:
                    times[on].append(e0.elapsed_time(e1) * 1e3 / nset)
        tiles = -(-M // 256) * -(-N // 256)
        med = lambda v: sorted(v)[len(v) // 2]
        slices["M%d N%d K%d" % (M, N, K)] = {"tiles": tiles, "waves": round(tiles / 74.0, 2), "leftover_tiles": tiles % 74,
                                              "sliced_by_default": _slices_leftover_tiles(M, N, K),
                                              "whole_tiles_us": round(med(times[False]), 1), "default_us": round(med(times[True]), 1)}
        del As, Bs, ys, ws, graphs
        torch.cuda.empty_cache()
    out["leftover_tile_slices"] = slices
    return out


def reference_on_cpu(args, name):
    """Fallback reference arm when oracle/_ref is absent: the host port of the path."""
    cb = cpu_baseline(name)
    return {"metric": METRIC, "value": cb["value"], "unit": "TOPS", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": DTYPE,
            "data": "synthetic", "impl": "reference", "config": {"workload": name}, "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def _free():
    import gc
    import torch
    gc.collect()
    torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=HEADLINE, choices=list(ALL_CONFIGS))
    ap.add_argument("--only", action="store_true", help="measure the chosen workload alone (no per_config summary of the others)")
    ap.add_argument("--aux", action="store_true", help="also time the quantizer, the RMSNorm+quantize producer and the probes alone")
    ap.add_argument("--row-reduce", default="p2p", choices=["p2p", "nccl"],
                    help="reduction of the row-parallel linear: over peer-mapped memory (default) or NCCL collectives")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-t1", action="store_true", help="N > 1: skip the unsharded runs that give the same-run 1-GPU times")
    ap.add_argument("--no-graphs", action="store_true", help="launch eagerly instead of replaying CUDA graphs")
    ap.add_argument("--no-probe", action="store_true", help="skip the tensor-peak probe (profiling runs); the fraction then uses 2 x bf16")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    impl = args.impl
    if impl == "reference" and not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libref_i8i8.so")):
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(reference_on_cpu(args, args.workload)))
        return

    rank, world = _dist_setup(args.gpus)
    peaks = _peaks()
    tensor_peak = tensor_peak_probe() if (impl == "ours" and not args.no_probe) else None
    import w8a8_workloads as wl
    head = args.workload
    if args.only:
        others = []
    elif world == 1:
        others = [c for c in ALL_CONFIGS if c != head]
    else:  # c0 / c1 are single-GPU configurations by definition
        others = [c for c in ALL_CONFIGS if c != head and wl.CONFIGS[c]["shard"] is not None]

    def summary_of(name):
        """One configuration, sharded where it shards; on N > 1 GPUs also unsharded for the same-run 1-GPU time."""
        r = run_config(name, args, rank, world, impl, True, sample_clocks=(name == head), check_shard=world > 1)
        _free()
        s = compact(r, args, peaks, tensor_peak, impl)
        if r["shard"] is not None and impl == "ours" and not args.no_t1:
            t1 = run_config(name, args, rank, world, impl, False)["ms"] / args.steps
            _free()
            s["ms_per_step_1gpu_same_run"] = round(t1, 6)
            s["scaling_vs_1gpu"] = round(t1 / s["ms_per_step"], 3)
        return r, s

    res, head_summary = summary_of(head)
    per_step = res["ms"] / args.steps
    ops_per_step = res["ops"] * res["replicas"]
    line = {
        "metric": METRIC,
        "value": ops_per_step / (per_step * 1e-3) / 1e12,
        "unit": "TOPS",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_step,
        "higher_is_better": True,
        "scaling": "weak" if res["replicas"] > 1 else "strong",
        "vs_baseline": None,
        "dtype": DTYPE,
        "data": "synthetic",
        "config": static_config(res, others),
        "e2e": {"value": ops_per_step / (res["ms_e2e"] / args.steps * 1e-3) / 1e12, "unit": "TOPS",
                "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"],
                "note": ("activations in / outputs out through pinned host memory each step; weights resident; "
                         + ("the library's host-buffer entry point (chunks of 1024 tokens after a ramp of 128, 128, 256, 512: copy in, compute and copy out overlap)"
                            if impl == "ours" and res["shard"] != "row" else "copy in, the operators, copy out, one after the other"))},
        "gpu_launches": res["launches"] * args.steps,
        "clocks": res["clocks"],
    }
    rf = kernel_roofline(res, args, peaks, tensor_peak, impl)
    if res["bit_exact"] is not None:
        rf["sharded_bit_exact"] = bool(res["bit_exact"])
    stats = {"launch": ("CUDA graph replay, %d step(s) per graph" % res["nsets"]) if res["use_graphs"] else "eager launches",
             "ms_per_step_median": res["med_ms"], "ms_per_step_min": res["min_ms"],
             "ms_per_step_stat": "over %d separately timed rounds of %d step(s)" % (res["reps"], res["nsets"])}
    if tensor_peak is not None:
        stats["tensor_peak_probe"] = tensor_peak
    per_config = {head: head_summary}
    for name in others:
        try:
            per_config[name] = summary_of(name)[1]
        except StatusWordSet as e:  # raised on every rank alike: the headline line survives
            per_config[name] = {"error": str(e)}
            _free()
    rf["per_config"] = per_config
    line["roofline"] = rf
    line["stats"] = stats
    if impl == "reference":
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "TOPS", "cores": 0, "kind": "reference",
                                "sample": "full workload; the reference path is CUDA-only, so its own kernels "
                                          "(compute_80 PTX JIT + cuBLASLt int8) run on the same GPUs, one rank per GPU"}
    elif world == 1 and rank == 0 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(head)
    if args.aux and rank == 0 and impl == "ours":
        line["aux_kernels"] = aux_kernels(args.steps, args.warmup)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
