#!/usr/bin/env python
"""Benchmark of the elementwise / reduction hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg3] [--no-side-configs]

Headline workload (one "step" = one pass of the hot path over one batch):
GpuReduction MAXANDARGMAX over the last axis of fp32 logits (16384, 32000) per
GPU, values N(0,1) rounded to 1/64 (ties occur), outputs fp32 max + 8-byte
first-occurrence index. With N GPUs every rank holds its own (16384, 32000)
slab of a (16384*N, 32000) array: rows shard with no communication (weak
scaling). Metric: effective HBM GB/s = algorithmic bytes / device time.
With N > 1 the line's `configs` also holds the STRONG-scaled configurations:
the same 16384 rows split over the ranks, and the fp64 (2048, 1024, 1024)
reductions whose reduced leading extent is split and finished by one
all-reduce, each with its time on one GPU measured in the same run.

The JSON line also carries: `e2e` (same call with HOST input: pinned
host->device copy of the slab and device->host read of the results inside the
timed region), `roofline` (dominant kernel against the measured copy peak),
`cpu_baseline` (the C oracle port on the host cores, bounded sample), `clocks`
(nvidia-smi samples during the timed region), `gpu_launches`, and `configs`
(the other single-GPU workloads of the suite, each timed on data that is not
resident in L2).

`--impl reference` times the reference arm: libgpuarray's CPU path is pygpu on
a CPU OpenCL device (pocl), which cannot run here (no OpenCL loader, no pocl,
no mako), so the arm is the C restatement of the reference kernel in
oracle/oracle_kernels.c with all host threads (OpenMP), on the same workload.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, COLS = 16384, 32000
NOMINAL_HBM_GBS = 8000.0


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def make_logits(rank, rows):
    """Seed 2; rank r draws from the r-th jumped copy of the stream."""
    bg = np.random.PCG64(2)
    rng = np.random.Generator(bg.jumped(rank) if rank else bg)
    x = rng.standard_normal((rows, COLS), dtype=np.float32)
    np.multiply(x, 64, out=x)
    np.round(x, out=x)
    np.multiply(x, np.float32(1.0 / 64), out=x)
    return x


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, dev):
        self.dev = dev
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.dev), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def device_timer(torch, stream):
    class T:
        def __init__(self):
            self.pairs = []

        def span(self):
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            self.pairs.append((a, b))
            return a, b

        def total_ms(self):
            return sum(a.elapsed_time(b) for a, b in self.pairs)
    return T()


# Both arms report the same metric on the same workload.
METRIC = "maxandargmax effective HBM GB/s"
WORKLOAD = ("cfg3 GpuReduction MAXANDARGMAX, last axis of fp32 (16384, 32000) logits per GPU "
            "(rows sharded, no communication)")

# --------------------------------------------------------------- reference arm

def host_threads():
    """Host cores this process may run on (the OpenMP team both CPU legs use)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def bench_config(rows):
    """`config` of the JSON line: identical in both arms (same workload, same
    rows, same bytes per step), so nothing measured goes in here."""
    return {"workload": WORKLOAD, "rows_per_gpu": rows,
            "bytes_per_step_per_gpu": rows * COLS * 4 + rows * 12,
            "l2": "2.1 GB input per step exceeds the 126 MB L2; no flush needed"}


def run_reference(args, rank):
    """CPU arm: the oracle's C port of the reference kernel over the WHOLE
    (rows, 32000) slab per step, with an OpenMP team of every host core this
    process may use - set explicitly, because launchers such as
    torch.distributed.run export OMP_NUM_THREADS=1."""
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    rows = args.rows
    threads = O.set_threads(host_threads())
    x = make_logits(0, rows)
    for _ in range(args.warmup):
        O.rowmaxarg_f32(x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.rowmaxarg_f32(x)
    dt = (time.perf_counter() - t0) / args.steps
    nbytes = x.nbytes + rows * 12
    val = nbytes / dt / 1e9
    emit({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": bench_config(rows),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port",
                         "host_cores": os.cpu_count(),
                         "omp_num_threads_env": os.environ.get("OMP_NUM_THREADS"),
                         "sample": "all %d rows per step in host memory, OpenMP team of %d set "
                                   "explicitly; pygpu-on-pocl (the reference's CPU path) is "
                                   "unavailable on this box" % (rows, threads)},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


# -------------------------------------------------------------------- our arm

def side_configs(api, ctx, torch, stream, once=False):
    """The other single-GPU workloads, each launch timed on data that is not in
    L2: either the working set of one launch exceeds the 126 MB L2 (cfg1, cfg4,
    cfg5) or successive launches rotate through distinct inputs totalling more
    than L2 (cfg2). A write-flush is deliberately not used: it leaves ~126 MB of
    dirty lines whose write-back would be billed to the next kernel."""
    out = {}
    R, W = api.GE_READ, api.GE_WRITE
    peak, _ = measured_peak()

    stall_buf = api.GpuArray.empty(ctx, (4096 if once else 2 << 30,), np.uint8)

    def timed(fn, nbytes, reps=20, launches=1):
        """fn(i) enqueues launch number i. The `reps` launches run back to back
        between two CUDA events on the library's stream; a ~1 ms memset is
        enqueued first so that the host is ahead of the device and launch
        latency of the short kernels is not billed to them."""
        if once:
            warm, reps = 0, 1
        else:
            warm = 3
        for i in range(warm):
            fn(i)
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        for _ in range(0 if once else 3):
            stall_buf.memset(0)
        a.record(stream)
        for i in range(reps):
            fn(i)
        b.record(stream)
        ctx.sync()
        us = a.elapsed_time(b) * 1e3 / reps
        gbs = nbytes / us / 1e3
        return {"us": round(us, 2), "GB/s": round(gbs, 1), "frac_nominal_8TBs": round(gbs / NOMINAL_HBM_GBS, 3),
                "frac_measured_peak": round(gbs / peak, 3), "bytes": nbytes, "launches": launches}

    g = torch.Generator(device="cuda").manual_seed(0)

    def dev_array(t):
        return api.GpuArray.from_pointer(ctx, t.data_ptr(), tuple(t.shape),
                                         {torch.float32: np.float32, torch.float16: np.float16,
                                          torch.float64: np.float64}[t.dtype])

    # cfg1: out = a*b + 0.5f, n = 2^24 fp32. One launch touches 192 MiB, only 1.6 x L2, so
    # successive launches rotate through NSET distinct (a, b, out) sets: a line is touched
    # again only after 3 x 192 MiB of other traffic.
    NSET = 1 if once else 3
    n = 1 << 24
    sets1 = []
    for _ in range(NSET):
        ta = torch.rand(n, device="cuda", generator=g) * 2 - 1
        tb = torch.rand(n, device="cuda", generator=g) * 2 - 1
        to = torch.empty(n, device="cuda")
        sets1.append((ta, tb, to, dev_array(ta), dev_array(tb), dev_array(to)))
    torch.cuda.synchronize()
    ge = api.GpuElemwise(ctx, "out = a * b + 0.5f", [("a", np.float32, R), ("b", np.float32, R),
                                                      ("out", np.float32, W)], nd=1)
    out["cfg1_elemwise_f32_contig"] = timed(
        lambda i: ge(*sets1[i % NSET][3:]), 3 * 4 * n)
    out["cfg1_elemwise_f32_contig"]["l2"] = "cold: %d buffer sets in rotation" % NSET
    del sets1

    # cfg2: SUM of fp32 4096x4096 over axis 1 and axis 0; cold = six distinct 64 MiB inputs in
    # rotation (384 MiB > 126 MB L2), warm = the same input every launch (it fits L2)
    nrot = 6
    txs = [torch.randn(4096, 4096, device="cuda", generator=g) for _ in range(nrot)]
    ts = torch.empty(4096, device="cuda")
    torch.cuda.synchronize()
    gxs, gs = [dev_array(t) for t in txs], dev_array(ts)
    gsum = api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float32)
    l0 = api.lib().gpuarray_b200_launch_count()
    gsum(gs, None, gxs[0], [1])
    l1 = api.lib().gpuarray_b200_launch_count()
    gsum(gs, None, gxs[0], [0])
    l2 = api.lib().gpuarray_b200_launch_count()
    for ax, nl in ((1, int(l1 - l0)), (0, int(l2 - l1))):
        cold = timed(lambda i: gsum(gs, None, gxs[i % nrot], [ax]),
                     4096 * 4096 * 4 + 4096 * 4, launches=nl)
        warm = timed(lambda i: gsum(gs, None, gxs[0], [ax]),
                     4096 * 4096 * 4 + 4096 * 4, launches=nl)
        cold["l2"] = "cold: %d inputs in rotation" % nrot
        cold["l2_warm_us"] = warm["us"]
        cold["l2_warm_GB/s"] = warm["GB/s"]
        out["cfg2_sum_axis%d" % ax] = cold
    del txs, gxs

    # cfg4: y = max(x + bias, 0), x an NHWC buffer viewed as NCHW, fp16; 196 MiB per launch,
    # rotated like cfg1
    sets4 = []
    tbias = (torch.rand(1, 256, 1, 1, device="cuda", generator=g) * 0.2 - 0.1).half()
    gbias = dev_array(tbias)
    for _ in range(NSET):
        tbuf = torch.randn(64, 56, 56, 256, device="cuda", generator=g).half()
        ty = torch.empty(64, 256, 56, 56, device="cuda", dtype=torch.float16)
        sets4.append((tbuf, ty, dev_array(tbuf).transpose((0, 3, 1, 2)), dev_array(ty)))
    torch.cuda.synchronize()
    ge4 = api.GpuElemwise(ctx, "y = fmaxf(x + bias, 0.0f)",
                          [("x", np.float16, R), ("bias", np.float16, R), ("y", np.float16, W)],
                          nd=4, convert_f16=True)
    out["cfg4_f16_bias_relu_nhwc_to_nchw"] = timed(
        lambda i: ge4(sets4[i % NSET][2], gbias, sets4[i % NSET][3], flags=api.GE_BROADCAST),
        2 * 64 * 56 * 56 * 256 * 2 + 512)
    out["cfg4_f16_bias_relu_nhwc_to_nchw"]["l2"] = "cold: %d buffer sets in rotation" % NSET
    del sets4

    # map + reduce in one pass: sum(a * b) over 2^26 fp32 (two 256 MiB inputs read once each;
    # elementwise-then-reduce would write and re-read a third 256 MiB array)
    nd = 1 << 26
    tda = torch.randn(nd, device="cuda", generator=g)
    tdb = torch.randn(nd, device="cuda", generator=g)
    tds = torch.empty((), device="cuda")
    torch.cuda.synchronize()
    gda, gdb, gds = dev_array(tda), dev_array(tdb), dev_array(tds)
    mr = api.GpuMapReduction(ctx, "a * b", "a + b", "0", np.float32,
                             [("a", np.float32, R), ("b", np.float32, R)])
    out["mapreduce_dot_f32_2^26"] = timed(lambda i: mr(gds, gda, gdb, axes=[0]), 2 * 4 * nd + 4,
                                           reps=10)
    ref = float((tda.double() * tdb.double()).sum())
    scale = float((tda.double() * tdb.double()).abs().sum())
    out["mapreduce_dot_f32_2^26"]["check"] = bool(abs(float(tds) - ref) <= 1e-6 * 26 * scale)
    del tda, tdb

    # cfg5: fp64 (2048, 1024, 1024) = 16 GiB: SUM over everything, MIN and MAX over (0, 2)
    try:
        planes = 128 if once else 2048
        t5 = torch.rand(planes, 1024, 1024, device="cuda", dtype=torch.float64, generator=g)
        t5.mul_(2).sub_(1)
        t1 = torch.empty((), device="cuda", dtype=torch.float64)
        tk = torch.empty(1024, device="cuda", dtype=torch.float64)
        torch.cuda.synchronize()
        g5, g1, gk = dev_array(t5), dev_array(t1), dev_array(tk)
        r_sum = api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float64)
        r_min = api.GpuReduction(ctx, api.GA_REDUCE_MIN, np.float64)
        r_max = api.GpuReduction(ctx, api.GA_REDUCE_MAX, np.float64)
        nb = t5.numel() * 8
        out["cfg5_f64_sum_all"] = timed(lambda i: r_sum(g1, None, g5, [0, 1, 2]), nb + 8, reps=5,
                                        launches=1)
        out["cfg5_f64_min_axes02"] = timed(lambda i: r_min(gk, None, g5, [0, 2]), nb + 8192, reps=5,
                                           launches=1)
        out["cfg5_f64_max_axes02"] = timed(lambda i: r_max(gk, None, g5, [0, 2]), nb + 8192, reps=5,
                                           launches=1)
        del t5
    except Exception as e:       # e.g. not enough free memory next to the headline buffers
        out["cfg5"] = {"skipped": str(e)[:200]}
    return out


def other_shapes(api, ctx, torch, stream, once=False, only=None):
    """`--other-shapes`: shapes outside the five named configurations that the
    same kernels meet in practice (short runs, kept axis in the middle,
    broadcasts, narrow element types), each 130-270 MB so that one launch
    exceeds L2, timed like the side configurations: 10 launches back to back
    behind a memset, CUDA events on the library's stream."""
    peak, _ = measured_peak()
    out = {}
    g = torch.Generator(device="cuda").manual_seed(7)
    stall_buf = api.GpuArray.empty(ctx, (4096 if once else 2 << 30,), np.uint8)
    npdt = {torch.float32: np.float32, torch.float16: np.float16, torch.float64: np.float64,
            torch.int8: np.int8, torch.uint8: np.uint8}

    def dev_array(t):
        return api.GpuArray.from_pointer(ctx, t.data_ptr(), tuple(t.shape), npdt[t.dtype])

    def timed(name, fn, nbytes, reps=10):
        if only and only not in name:
            return
        if once:                      # profiler captures: one launch per case
            reps = 1
        for _ in range(0 if once else 3):
            fn()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        for _ in range(0 if once else 3):
            stall_buf.memset(0)
        a.record(stream)
        for _ in range(reps):
            fn()
        b.record(stream)
        ctx.sync()
        us = a.elapsed_time(b) * 1e3 / reps
        out[name] = {"us": round(us, 2), "GB/s": round(nbytes / us / 1e3, 1),
                     "frac_measured_peak": round(nbytes / us / 1e3 / peak, 3), "bytes": nbytes}

    S, MX, AM, ANY = (api.GA_REDUCE_SUM, api.GA_REDUCE_MAX, api.GA_REDUCE_ARGMAX, api.GA_REDUCE_ANY)
    reductions = [
        ("sum f32 (64,256,56,56) over (0,2,3)", (64, 256, 56, 56), [0, 2, 3], torch.float32, S),
        ("sum f32 (64,56,56,256) over (0,1,2)", (64, 56, 56, 256), [0, 1, 2], torch.float32, S),
        ("sum f16 (64,256,56,56) over (0,2,3)", (64, 256, 56, 56), [0, 2, 3], torch.float16, S),
        ("sum f32 (512,512,256) over (0)", (512, 512, 256), [0], torch.float32, S),
        ("sum f32 (512,512,256) over (1)", (512, 512, 256), [1], torch.float32, S),
        ("sum f32 (512,512,256) over (2)", (512, 512, 256), [2], torch.float32, S),
        ("sum f32 (512,512,256) over (0,2)", (512, 512, 256), [0, 2], torch.float32, S),
        ("max f32 (8192,8192) over (1)", (8192, 8192), [1], torch.float32, MX),
        ("argmax f32 (8192,8192) over (0)", (8192, 8192), [0], torch.float32, AM),
        ("sum f32 (2^21,32) over (1)", (1 << 21, 32), [1], torch.float32, S),
        ("max f32 (2^22,16) over (1)", (1 << 22, 16), [1], torch.float32, MX),
        ("argmax f32 (2^17,512) over (1)", (1 << 17, 512), [1], torch.float32, AM),
        ("sum f32 (2^26) all", (1 << 26,), [0], torch.float32, S),
        ("sum f64 (4096,8192) over (0)", (4096, 8192), [0], torch.float64, S),
        ("sum i8->i64 (2^28) all", (1 << 28,), [0], torch.int8, S),
        ("any i8 (2^28) all", (1 << 28,), [0], torch.int8, ANY),
    ]
    for name, shape, axes, tdt, op in reductions:
        if only and only not in name:
            continue
        if tdt == torch.int8:
            t = torch.randint(-3, 4, shape, device="cuda", dtype=torch.int8, generator=g)
        else:
            t = torch.randn(*shape, device="cuda", generator=g).to(tdt)
        torch.cuda.synchronize()
        gx = dev_array(t)
        free = [s for i, s in enumerate(shape) if i not in axes]
        r = api.GpuReduction(ctx, op, npdt[tdt])
        if op == AM:
            di = api.GpuArray.empty(ctx, free, np.int64)
            fn = lambda: r(None, di, gx, axes)
        else:
            odt = np.bool_ if op == ANY else (np.int64 if tdt == torch.int8 else npdt[tdt])
            dv = api.GpuArray.empty(ctx, free, odt)
            fn = lambda: r(dv, None, gx, axes)
        timed(name, fn, t.numel() * t.element_size())
        del t, gx

    R, W = api.GE_READ, api.GE_WRITE
    M, N = 8192, 4096
    ta = torch.randn(M, N, device="cuda", generator=g)
    tb = torch.randn(1, N, device="cuda", generator=g)
    tc = torch.randn(M, 1, device="cuda", generator=g)
    to = torch.empty(M, N, device="cuda")
    torch.cuda.synchronize()
    ga, gb, gc, go = dev_array(ta), dev_array(tb), dev_array(tc), dev_array(to)
    add = api.GpuElemwise(ctx, "o = a + b", [("a", np.float32, R), ("b", np.float32, R),
                                             ("o", np.float32, W)], nd=2)
    scale = api.GpuElemwise(ctx, "o = a * 2.0f", [("a", np.float32, R), ("o", np.float32, W)], nd=2)
    timed("o = a + b, b a row (1,N) broadcast, f32 (8192,4096)", lambda: add(ga, gb, go, flags=api.GE_BROADCAST), 8 * M * N)
    timed("o = a + b, b a column (M,1) broadcast", lambda: add(ga, gc, go, flags=api.GE_BROADCAST), 8 * M * N)
    gt = ga.transpose((1, 0))
    got = dev_array(torch.empty(N, M, device="cuda"))
    timed("o = 2a, a the transposed view, f32", lambda: scale(gt, got), 8 * M * N)
    t3a = torch.randn(64, 1, 1024, device="cuda", generator=g)
    t3b = torch.randn(1, 512, 1, device="cuda", generator=g)
    t3o = torch.empty(64, 512, 1024, device="cuda")
    torch.cuda.synchronize()
    g3a, g3b, g3o = dev_array(t3a), dev_array(t3b), dev_array(t3o)
    timed("o = a + b, (64,1,1024) + (1,512,1) -> (64,512,1024) f32 (write only)",
          lambda: add(g3a, g3b, g3o, flags=api.GE_BROADCAST), 4 * 64 * 512 * 1024)
    tu = torch.randint(0, 255, (1 << 27,), device="cuda", dtype=torch.uint8, generator=g)
    tuo = torch.empty(1 << 27, device="cuda", dtype=torch.uint8)
    th = torch.randn(1 << 25, device="cuda", generator=g).half()
    tho = torch.empty(1 << 25, device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    gu, guo, gh, gho = dev_array(tu), dev_array(tuo), dev_array(th), dev_array(tho)
    inc8 = api.GpuElemwise(ctx, "o = a + 1", [("a", np.uint8, R), ("o", np.uint8, W)], nd=1)
    sc16 = api.GpuElemwise(ctx, "o = a * 2.0f", [("a", np.float16, R), ("o", np.float16, W)], nd=1,
                           convert_f16=True)
    timed("o = a + 1, uint8 2^27 contiguous", lambda: inc8(gu, guo), 2 * (1 << 27))
    timed("o = 2a, float16 2^25 contiguous", lambda: sc16(gh, gho), 4 * (1 << 25))
    return out


def sharded_configs(api, ctx, torch, dist, stream, rank, world, host_slab, t1_cfg3_us):
    """The configurations that SPLIT a fixed problem over the ranks (strong
    scaling), run whenever world > 1. Every time is the max over ranks of a
    CUDA-event span on the library's stream, launches back to back.

    cfg3_strong: the seed-2 (16384, 32000) logits, rank r owning rows
      [r*16384/world, (r+1)*16384/world); no communication.
    cfg5_*_sharded: fp64 (2048, 1024, 1024), rank r owning 2048/world leading
      planes, through GpuReduction_call_sharded: per-GPU partial of the final
      shape, then one exchange kernel over the communicator's peer windows
      (or one gpucomm all-reduce where those are unavailable). Reported: the
      whole call, the kernel alone, the same with an NCCL all-reduce instead,
      that all-reduce alone, and the same reduction over all 2048 planes on one
      GPU (x_vs_1gpu = that time / the sharded time).
    cfg5_f64_maxandargmax_axes02_sharded: (value, global first index) over the
      sharded extent through GpuReduction_call_sharded."""
    out = {}

    def span(fn, reps):
        for _ in range(3):
            fn()
        ctx.sync()
        dist.barrier()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            fn()
        b.record(stream)
        ctx.sync()
        t = torch.tensor([a.elapsed_time(b) / reps], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]) * 1e3

    # ---- cfg3, rows split
    rows = ROWS // world
    full = torch.empty((ROWS, COLS), dtype=torch.float32, device="cuda")
    if rank == 0:
        full.copy_(host_slab, non_blocking=False)
    dist.broadcast(full, 0)
    mine = full[rank * rows:(rank + 1) * rows]
    torch.cuda.synchronize()
    gx = api.GpuArray.from_pointer(ctx, mine.data_ptr(), (rows, COLS), np.float32)
    gmax = api.GpuArray.empty(ctx, (rows,), np.float32)
    garg = api.GpuArray.empty(ctx, (rows,), np.uint64)
    us = span(lambda: api.maxandargmax(gmax, garg, gx, [1]), 50)
    vm, am = gmax.to_numpy(), garg.to_numpy()
    ref = mine[:32].cpu().numpy()
    check = bool((vm[:32] == ref.max(1)).all() and (am[:32] == ref.argmax(1)).all())
    total = ROWS * COLS * 4 + ROWS * 12
    out["cfg3_strong"] = {
        "us": round(us, 2), "GB/s": round(total / us / 1e3, 1), "rows_per_gpu": rows,
        "x_vs_1gpu": round(t1_cfg3_us / us, 3), "t_1gpu_us": round(t1_cfg3_us, 2),
        "frac_nominal_8TBs_x_gpus": round(total / us / 1e3 / (NOMINAL_HBM_GBS * world), 3),
        "collective": "none", "scaling": "strong", "first_rows_check_rank0": check}
    del gx, mine, full

    # ---- cfg5, leading planes split
    planes = 2048 // world
    g = torch.Generator(device="cuda").manual_seed(4)
    t5 = torch.rand(2048, 1024, 1024, device="cuda", dtype=torch.float64, generator=g)
    t5.mul_(2).sub_(1)
    torch.cuda.synchronize()
    g_full = api.GpuArray.from_pointer(ctx, t5.data_ptr(), (2048, 1024, 1024), np.float64)
    shard = t5[rank * planes:(rank + 1) * planes]
    g5 = api.GpuArray.from_pointer(ctx, shard.data_ptr(), (planes, 1024, 1024), np.float64)
    cid = [api.GpuComm.gen_clique_id(ctx) if rank == 0 else None]
    dist.broadcast_object_list(cid, src=0)
    comm = api.GpuComm(ctx, cid[0], world, rank)
    p1 = api.GpuArray.empty(ctx, (), np.float64)
    o1 = api.GpuArray.empty(ctx, (), np.float64)
    pk = api.GpuArray.empty(ctx, (1024,), np.float64)
    ok = api.GpuArray.empty(ctx, (1024,), np.float64)
    ops = {"sum_all": (api.GA_REDUCE_SUM, [0, 1, 2], p1, o1, api.GA_SUM),
           "min_axes02": (api.GA_REDUCE_MIN, [0, 2], pk, ok, api.GA_MIN),
           "max_axes02": (api.GA_REDUCE_MAX, [0, 2], pk, ok, api.GA_MAX)}
    total_bytes = 2048 * 1024 * 1024 * 8
    for name, (rop, axes, part, res, cop) in ops.items():
        gr = api.GpuReduction(ctx, rop, np.float64)

        def both():
            api.reduction_call_sharded(gr, comm, res, None, g5, axes, rank * planes, 2048)

        def both_nccl():
            gr(part, None, g5, axes)
            comm.all_reduce(part, res, cop)
        us_both = span(both, 10)
        us_nccl = span(both_nccl, 10)
        us_kernel = span(lambda: gr(part, None, g5, axes), 10)
        us_comm = span(lambda: comm.all_reduce(part, res, cop), 20)
        both()
        got = res.to_numpy().copy()
        us_one = span(lambda: gr(res, None, g_full, axes), 4)
        want = res.to_numpy()
        check = bool(np.allclose(got, want, rtol=1e-12, atol=0) if name == "sum_all" else
                     got.tobytes() == want.tobytes())
        state = comm.peer_state()
        out["cfg5_f64_%s_sharded" % name] = {
            "us": round(us_both, 2), "GB/s": round(total_bytes / us_both / 1e3, 1),
            "kernel_only_us": round(us_kernel, 2), "all_reduce_only_us": round(us_comm, 2),
            "with_nccl_all_reduce_us": round(us_nccl, 2),
            "t_1gpu_us": round(us_one, 2), "x_vs_1gpu": round(us_one / us_both, 3),
            "frac_nominal_8TBs_x_gpus": round(total_bytes / us_both / 1e3 / (NOMINAL_HBM_GBS * world), 3),
            "planes_per_gpu": planes,
            "collective": ("GpuReduction_call_sharded: one exchange kernel over peer (NVLink) windows, %d B"
                           if state[0] == 1 else
                           "GpuReduction_call_sharded: gpucomm_all_reduce (NCCL), %d B") % res.nbytes,
            "peer_windows": state[0] == 1, "peer_windows_reason": state[1], "scaling": "strong",
            "matches_1gpu_result": check}
        gr.free()

    # ---- (value, first global index) with the reduced extent sharded
    if hasattr(api, "reduction_call_sharded"):
        gr = api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.float64)
        gv = api.GpuArray.empty(ctx, (1024,), np.float64)
        gi = api.GpuArray.empty(ctx, (1024,), np.uint64)
        us_both = span(lambda: api.reduction_call_sharded(gr, comm, gv, gi, g5, [0, 2],
                                                          rank * planes, 2048), 10)
        got = (gv.to_numpy().copy(), gi.to_numpy().copy())
        us_kernel = span(lambda: gr(gv, gi, g5, [0, 2]), 10)
        us_one = span(lambda: gr(gv, gi, g_full, [0, 2]), 4)
        check = bool(got[0].tobytes() == gv.to_numpy().tobytes() and (got[1] == gi.to_numpy()).all())
        out["cfg5_f64_maxandargmax_axes02_sharded"] = {
            "us": round(us_both, 2), "GB/s": round(total_bytes / us_both / 1e3, 1),
            "kernel_only_us": round(us_kernel, 2), "t_1gpu_us": round(us_one, 2),
            "x_vs_1gpu": round(us_one / us_both, 3),
            "frac_nominal_8TBs_x_gpus": round(total_bytes / us_both / 1e3 / (NOMINAL_HBM_GBS * world), 3),
            "planes_per_gpu": planes,
            "collective": ("one exchange kernel over peer (NVLink) windows: better value, then lower index"
                           if comm.peer_state()[0] == 1 else
                           "all-reduce of the value, candidate-index kernel, all-reduce MIN of the index"),
            "peer_windows": comm.peer_state()[0] == 1, "scaling": "strong", "matches_1gpu_result": check}
        gr.free()
    ctx.sync()
    comm.free()
    return out


def prefer_host_memory_near(ctx_ptr, api):
    """Host-side placement of the pinned input slab: asks the kernel to take this
    process's next pages from the NUMA node the GPU's PCIe root hangs off
    (set_mempolicy MPOL_PREFERRED), so that with several ranks per host each
    GPU's DMA reads cross no socket link. Returns (node, restore) - restore()
    puts the default policy back; node is None when the platform does not say
    (no sysfs entry, one node, not x86-64) and nothing was changed. Touches no
    GPU setting."""
    import ctypes
    import platform
    none = (None, lambda: None)
    try:
        buf = ctypes.create_string_buffer(16)
        if api.lib().gpucontext_property(ctx_ptr, 19, buf) != 0:      # GA_CTX_PROP_UNIQUE_ID: PCI bus id
            return none
        pci = buf.value.decode().strip().lower()
        with open("/sys/bus/pci/devices/%s/numa_node" % pci) as f:
            node = int(f.read().strip())
        if node < 0 or node > 62 or platform.machine() != "x86_64":
            return none
        libc = ctypes.CDLL(None, use_errno=True)
        mask = ctypes.c_ulong(1 << node)
        if libc.syscall(238, 1, ctypes.byref(mask), 65) != 0:          # set_mempolicy(MPOL_PREFERRED, ...)
            return none
        return node, lambda: libc.syscall(238, 0, None, 0)             # MPOL_DEFAULT
    except Exception:
        return none


def run_ours(args, rank, world, local_rank):
    global ROWS
    ROWS = args.rows
    import torch
    import torch.distributed as dist
    from libgpuarray_b200 import api

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = api.Context(local_rank, kernel_cache=os.path.join(ROOT, ".kernel_cache"))
    stream = torch.cuda.ExternalStream(ctx.stream, device=local_rank)
    peak, peak_kind = measured_peak()

    # ---- data: host slab in pinned memory, device copy for the resident run
    numa_node, restore_policy = prefer_host_memory_near(ctx.ptr, api) if not args.no_numa else (None, lambda: None)
    host = torch.empty((ROWS, COLS), dtype=torch.float32, pin_memory=True)
    host.numpy()[...] = make_logits(rank, ROWS)
    restore_policy()
    numa_nodes = [numa_node]
    if world > 1:
        numa_nodes = [None] * world
        dist.all_gather_object(numa_nodes, numa_node)
    gx = api.GpuArray.empty(ctx, (ROWS, COLS), np.float32)
    gx.write_raw(host.data_ptr(), host.numel() * 4)
    gmax = api.GpuArray.empty(ctx, (ROWS,), np.float32)
    garg = api.GpuArray.empty(ctx, (ROWS,), np.uint64)
    hmax = torch.empty(ROWS, dtype=torch.float32, pin_memory=True)
    harg = torch.empty(ROWS, dtype=torch.int64, pin_memory=True)
    ctx.sync()
    step_bytes = ROWS * COLS * 4 + ROWS * 12

    def step():
        api.maxandargmax(gmax, garg, gx, [1])

    def barrier():
        if world > 1:
            dist.barrier()
        ctx.sync()
        torch.cuda.synchronize()

    # ---- resident run. The clock sampler covers a window of about a second in
    # which this same step loops; the K timed steps are the first of them.
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sample = rank == 0 and not args.no_clocks
    if sample:
        sampler.start()
        time.sleep(0.25)
    launches0 = api.lib().gpuarray_b200_launch_count()
    timer = device_timer(torch, stream)
    barrier()
    a, b = timer.span()
    a.record(stream)
    for _ in range(args.steps):
        step()
    b.record(stream)
    barrier()
    ms = timer.total_ms()
    launches = api.lib().gpuarray_b200_launch_count() - launches0
    if sample:
        t_end = time.perf_counter() + 1.0
        while time.perf_counter() < t_end:
            for _ in range(20):
                step()
            ctx.sync()
    clocks = sampler.stop() if sample else None
    barrier()

    # quick self-check of the timed result on a few rows (host recomputation)
    vm, am = gmax.to_numpy(), garg.to_numpy()
    xs = host.numpy()[:64]
    assert (vm[:64] == xs.max(1)).all() and (am[:64] == xs.argmax(1)).all(), "result check failed"

    # ---- end-to-end run: host input, host output, every step
    def e2e_step():
        gx.write_raw(host.data_ptr(), host.numel() * 4)
        api.maxandargmax(gmax, garg, gx, [1])
        gmax.read_raw(hmax.data_ptr(), ROWS * 4)
        garg.read_raw(harg.data_ptr(), ROWS * 8)

    e2e_steps = max(2, min(args.steps, 10))
    e2e_ms = float("nan")
    if not args.no_e2e:
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3

    sharded = None
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    if world > 1 and not args.no_side_configs:
        del gx
        # no try/except here: a rank that carried on alone would leave its peers
        # waiting in a collective; an exception ends the whole launch instead
        sharded = sharded_configs(api, ctx, torch, dist, stream, rank, world, host,
                                  ms / args.steps * 1e3)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_per_step = ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    per_gpu = value / world
    e2e_value = world * step_bytes / (e2e_ms / e2e_steps * 1e-3) / 1e9

    # ---- CPU baseline (bounded sample, rank 0, N=1 only)
    cpu = None
    if world == 1 and not args.no_cpu:
        from oracle import oracle as O
        sample_rows = min(4096, ROWS)
        xs = host.numpy()[:sample_rows]
        threads = O.set_threads(host_threads())
        O.rowmaxarg_f32(xs)
        best = 1e9
        t_end = time.perf_counter() + 10.0
        reps = 0
        while time.perf_counter() < t_end and reps < 200:
            t0 = time.perf_counter()
            O.rowmaxarg_f32(xs)
            best = min(best, time.perf_counter() - t0)
            reps += 1
        t0 = time.perf_counter()
        xs.max(1)
        xs.argmax(1)
        t_np = time.perf_counter() - t0
        sb = xs.nbytes + sample_rows * 12
        cpu = {"value": sb / best / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
               "host_cores": os.cpu_count(),
               "sample": "first %d of %d rows, best of %d passes (~10 s), OpenMP team of %d"
                         % (sample_rows, ROWS, reps, threads),
               "numpy_1core_GBs": sb / t_np / 1e9}

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(ROWS),
        "frac_of_nominal_8TBs_per_gpu": per_gpu / NOMINAL_HBM_GBS,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": ROWS * COLS * 4,
                "d2h_bytes_per_step": ROWS * 12, "steps": e2e_steps,
                "host_slab_numa_node_per_rank": numa_nodes},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                     "frac": per_gpu / peak, "peak_kind": peak_kind, "kernel": "ga_rd_rows",
                     "traffic": TRAFFIC_BYTES_PER_LAUNCH if ROWS == 16384 else None},
        "clocks": clocks,
        "nvrtc": api.lib().gpuarray_b200_nvrtc_version() / 1000.0,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if sharded is not None:
        line["configs"] = sharded
    if world == 1 and not args.no_side_configs:
        del gx
        try:
            line["configs"] = side_configs(api, ctx, torch, stream, once=args.side_once)
        except Exception as e:
            line["configs"] = {"error": str(e)[:300]}
    if world == 1 and args.other_shapes:
        line["other_shapes"] = other_shapes(api, ctx, torch, stream, once=args.side_once, only=args.only)
    emit(line)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one 16384-row ga_rd_rows
# launch: 4 x the 4096-row ncu capture summarised in
# profiles/ga_rd_rows_cfg3_maxandargmax.md (traffic is proportional to rows).
TRAFFIC_BYTES_PER_LAUNCH = 2167131136


_REAL_STDOUT = None


def emit(obj):
    """The one JSON line goes to the real stdout; everything else that libraries
    print there (NCCL's version banner, for instance) was diverted to stderr."""
    data = (json.dumps(obj) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def main():
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3")
    ap.add_argument("--no-side-configs", action="store_true")
    ap.add_argument("--rows", type=int, default=ROWS,
                    help="rows per GPU (smaller values are for profiler captures only)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--side-once", action="store_true",
                    help="profiler captures: run every side config (and every --other-shapes case) "
                         "exactly once, cfg5 on 128 planes")
    ap.add_argument("--no-clocks", action="store_true",
                    help="skip the nvidia-smi sampling window (profiler captures)")
    ap.add_argument("--other-shapes", action="store_true",
                    help="also time reductions and elementwise calls on shapes outside the five "
                         "named configurations (adds an `other_shapes` object to the line)")
    ap.add_argument("--no-numa", action="store_true",
                    help="leave the placement of the pinned host slab to the default policy")
    ap.add_argument("--only", default=None,
                    help="with --other-shapes: run only the cases whose name contains this text "
                         "(profiler captures of one kernel)")
    ap.add_argument("--cfg5-sharded", action="store_true",
                    help="accepted for compatibility: with N > 1 the sharded configurations "
                         "(cfg3 rows split, cfg5 planes split + all-reduce) always run unless "
                         "--no-side-configs is given")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
