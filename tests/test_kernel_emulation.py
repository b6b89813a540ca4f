"""The reduction kernel TEMPLATES executed on the CPU.

For a handful of problems the library's planner picks the kernel variant and
fills the parameter block (gpuarray_b200_reduction_layout), the library's own
generator emits the variant's source (gpuarray_b200_reduction_source), and that
source - the very text NVRTC would get - is compiled with g++ against a small
SIMT emulator (tests/simt: the threads of a CTA as cooperative fibers, CTAs one
after the other) and run. Results are checked against the oracle exactly as
the GPU tests do. This exercises indexing, ragged ends, splits with arrival
tickets, part-of-a-warp groups, multi-run loads and the values-only scan
without a device; it says nothing about timing or data races."""
import ctypes
import hashlib
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SIMT = os.path.join(ROOT, "tests", "simt")
TEMPLATES = os.path.join(ROOT, "libgpuarray_b200", "csrc", "templates")
BUILD = os.path.join(ROOT, "libgpuarray_b200", "build", "simt")
KEYS = ["shape", "vec", "group", "flat", "mu", "onerun", "lazy", "fast8", "tpo", "idx64", "splits",
        "seg", "nseg", "units", "gx", "gy", "bx", "by", "nf", "nr"]
ENTRY = ["ga_rd_rows", "ga_rd_cols", "ga_rd_general"]

LAUNCHER = r'''
struct simt_args { const ga__rd_layout *L; const char *src; char *d0; char *d1;
                   GA_RD_ACC_T *pval; GA_RD_IDX_T *pidx; unsigned int *tickets; };
static void simt_body(void *p) {
  simt_args *a = (simt_args *)p;
  KERNEL_NAME(*a->L, a->src, a->d0, a->d1, a->pval, a->pidx, a->tickets);
}
extern "C" void simt_launch(const void *layout, const void *src, void *d0, void *d1, void *pval,
                            void *pidx, void *tickets, unsigned gx, unsigned gy, unsigned bx,
                            unsigned by) {
  simt_args a = {(const ga__rd_layout *)layout, (const char *)src, (char *)d0, (char *)d1,
                 (GA_RD_ACC_T *)pval, (GA_RD_IDX_T *)pidx, (unsigned int *)tickets};
  simt::run_grid(simt_body, &a, simt_dim3{gx, gy, 1}, simt_dim3{bx, by, 1});
}
'''


def plan_and_layout(api, op, x, axes, dst_dtype, sms):
    L = api.lib()
    fn = L.gpuarray_b200_reduction_layout
    fn.restype = ctypes.c_int
    nd = x.ndim
    out = (ctypes.c_ulonglong * 20)()
    layout = ctypes.create_string_buffer(4096)
    used = ctypes.c_size_t()
    err = fn(getattr(api, "GA_REDUCE_" + op), api.typecode(x.dtype), api.typecode(np.dtype(dst_dtype)),
             nd, (ctypes.c_size_t * nd)(*x.shape), (ctypes.c_ssize_t * nd)(*x.strides), len(axes),
             (ctypes.c_int * len(axes))(*axes), ctypes.c_ulonglong(x.ctypes.data), sms, out, layout,
             ctypes.c_size_t(4096), ctypes.byref(used))
    assert err == 0
    return dict(zip(KEYS, [int(v) for v in out])), layout


def build_variant(api, op, x, dst_dtype, p):
    L = api.lib()
    L.gpuarray_b200_reduction_source.restype = ctypes.c_void_p
    group = p["group"] | (p["mu"] << 16) | (p["onerun"] << 20) | (p["flat"] << 21)
    ptr = L.gpuarray_b200_reduction_source(getattr(api, "GA_REDUCE_" + op), api.typecode(x.dtype),
                                           api.typecode(np.dtype(dst_dtype)), p["shape"], p["vec"],
                                           p["idx64"], p["tpo"], group)
    text = ctypes.string_at(ptr).decode()
    text = text.replace("#define GA_RD_LAZY 0", "#define GA_RD_LAZY %d" % p["lazy"])
    text = text.replace("#define GA_RD_FAST8 0", "#define GA_RD_FAST8 %d" % p["fast8"])
    text += LAUNCHER.replace("KERNEL_NAME", ENTRY[p["shape"]])
    key = hashlib.sha1((text + open(os.path.join(TEMPLATES, "ga_reduce.cuh")).read() +
                        open(os.path.join(SIMT, "include", "simt_emul.h")).read()).encode()).hexdigest()[:16]
    os.makedirs(BUILD, exist_ok=True)
    so = os.path.join(BUILD, "v_%s.so" % key)
    if not os.path.exists(so):
        src = os.path.join(BUILD, "v_%s.cpp" % key)
        with open(src, "w") as f:
            f.write(text)
        subprocess.run(["g++", "-std=c++17", "-O1", "-shared", "-fPIC", "-w", "-I", os.path.join(SIMT, "include"),
                        "-I", TEMPLATES, src, os.path.join(SIMT, "simt_runtime.cpp"), "-o", so],
                       check=True, capture_output=True, text=True)
    return ctypes.CDLL(so)


def emulate(api, op, x, axes, dst_dtype=None, sms=2):
    """Runs the reduction on the emulator; returns (value array or None, index array or None, plan)."""
    dst_dtype = np.dtype(dst_dtype or x.dtype)
    p, layout = plan_and_layout(api, op, x, axes, dst_dtype, sms)
    lib = build_variant(api, op, x, dst_dtype, p)
    kept = tuple(d for i, d in enumerate(x.shape) if i not in axes)
    want_val = op not in ("ARGMAX", "ARGMIN")
    want_idx = op in ("ARGMAX", "ARGMIN", "MAXANDARGMAX", "MINANDARGMIN")
    d0 = None
    if want_val:                                     # pre-filled with a byte pattern
        d0 = np.frombuffer(bytearray(b"\x55" * (max(1, int(np.prod(kept))) * dst_dtype.itemsize)),
                           dtype=dst_dtype)[:max(1, int(np.prod(kept)))].reshape(kept)
    d1 = np.full(kept, -7, np.int64) if want_idx else None
    cells = max(1, p["splits"] * p["nf"])
    pval = np.zeros(cells * 8, np.uint8)
    pidx = np.zeros(cells * 8, np.uint8)
    tickets = np.zeros(max(p["nf"], p["units"], 1) + 8, np.uint32)

    def ptr(a):
        return ctypes.c_void_p(a.ctypes.data) if a is not None else ctypes.c_void_p(0)
    lib.simt_launch(layout, ptr(x), ptr(d0), ptr(d1), ptr(pval), ptr(pidx), ptr(tickets),
                    p["gx"], p["gy"], p["bx"], p["by"])
    assert (tickets == 0).all()                      # arrival counters are handed back at zero
    return d0, d1, p


def check(api, oracle, op, x, axes, dst_dtype=None, expect=None, sms=2):
    d0, d1, p = emulate(api, op, x, axes, dst_dtype, sms)
    if expect:
        for k, v in expect.items():
            assert p[k] == v, (k, p)
    if op in ("MAXANDARGMAX", "MINANDARGMIN", "ARGMAX", "ARGMIN", "MAX", "MIN"):
        wv, wi = oracle.minmaxarg(x, axes, is_min="MIN" in op)
        if d0 is not None:
            assert d0.tobytes() == wv.tobytes(), (op, axes, p)
        if d1 is not None:
            assert (d1 == wi).all(), (op, axes, p)
        return p
    out_dtype = np.dtype(dst_dtype or x.dtype)
    want = oracle.reduce_reference(op.lower(), x, axes, out_dtype)
    if out_dtype.kind != "f":
        assert (d0 == want.astype(out_dtype)).all(), (op, axes, p)
    else:
        n = max(2, int(np.prod([x.shape[a] for a in axes])))
        scale = np.abs(x.astype(np.float64)).sum(axis=tuple(axes))
        eps = 1e-6 if out_dtype == np.float32 else 1e-12
        assert (np.abs(d0.astype(np.float64) - want.astype(np.float64)) <=
                eps * np.log2(n) * np.maximum(scale, 1e-300)).all(), (op, axes, p)
    return p


def ties(rng, shape, dt=np.float32):
    return (np.round(rng.standard_normal(shape) * 2) / 2).astype(dt)


def test_rows_kernel_variants_on_the_emulator(api, oracle, rng):
    # a warp per long run with the values-only scan, ragged end (6001 = 1500 vectors + 1)
    x = ties(rng, (40, 6004))[:, :6001]
    check(api, oracle, "MAXANDARGMAX", x, [1],
          expect={"shape": 0, "group": 32, "vec": 4, "lazy": 1, "onerun": 0, "splits": 1})
    check(api, oracle, "MINANDARGMIN", x, [1])
    check(api, oracle, "SUM", x, [1], expect={"shape": 0, "lazy": 0})
    # NaN first, identity rows, signed zeros (the cases of the recovery step)
    y = ties(rng, (40, 5000))
    y[:3] = -np.inf
    y[1, :8] = np.nan
    y[2, 0] = np.nan
    y[3, :] = -1
    y[3, 130] = -0.0
    y[3, 131] = 0.0
    y[4, :] = 3
    y[4, [127, 128, 4000]] = 9
    y[5] = rng.standard_normal(5000)
    check(api, oracle, "MAXANDARGMAX", y, [1], expect={"lazy": 1})
    check(api, oracle, "MINANDARGMIN", -y, [1], expect={"lazy": 1})
    # few outputs, long rows: split over warps with arrival tickets
    z = ties(rng, (2, 40000))
    p = check(api, oracle, "MAXANDARGMAX", z, [1], sms=1)
    assert p["splits"] > 1
    check(api, oracle, "SUM", z, [1], sms=1)
    # whole-array reduction by CTA groups, split, ragged last segment
    w = ties(rng, (70001,))
    p = check(api, oracle, "SUM", w, [0], sms=1)
    assert p["group"] == 256 and p["splits"] > 1
    check(api, oracle, "ARGMIN", w, [0], sms=1)
    # scalar loads: a base that is not 16-byte aligned
    big = ties(rng, (3, 4100))
    u = big[:, 1:]
    check(api, oracle, "MAXANDARGMAX", u, [1], expect={"vec": 1})


def test_short_run_variants_on_the_emulator(api, oracle, rng):
    # one short run per output: 1, 2, 8 and 32 lanes per output, several outputs at once
    for cols, group in ((4, 1), (8, 2), (32, 2), (100, 8), (512, 32)):
        x = ties(rng, (301, cols))
        p = check(api, oracle, "SUM", x, [1], expect={"onerun": 1})
        assert p["group"] <= 32 and p["mu"] in (2, 4)
        check(api, oracle, "MAXANDARGMAX", x, [1], expect={"onerun": 1})
        check(api, oracle, "ARGMIN", x, [1])
    # rows that do not start on a 16-byte boundary (49 floats), fp64, int8 -> int64
    check(api, oracle, "SUM", ties(rng, (77, 49)), [1], expect={"onerun": 1, "vec": 1})
    check(api, oracle, "MAXANDARGMAX", ties(rng, (40, 64), np.float64), [1], expect={"onerun": 1, "vec": 2})
    i8 = rng.integers(-100, 100, (50, 96)).astype(np.int8)
    check(api, oracle, "SUM", i8, [1], dst_dtype=np.int64, expect={"onerun": 1, "fast8": 1})
    # several short runs per output: a warp on 2-4 runs at once; very short runs flattened
    y = ties(rng, (23, 4, 64))
    check(api, oracle, "MAXANDARGMAX", y, [0, 2], expect={"shape": 0, "onerun": 0, "mu": 4})
    check(api, oracle, "MAXANDARGMAX", y, [2, 0])            # index weights differ from memory order
    check(api, oracle, "SUM", ties(rng, (19, 3, 600)), [0, 2], expect={"mu": 2})
    check(api, oracle, "MINANDARGMIN", ties(rng, (37, 3, 20)), [0, 2], expect={"flat": 1})
    # 1-byte all / any with word tests
    b = (rng.random((9, 4096)) < 0.999)
    check(api, oracle, "ALL", b, [1], dst_dtype=np.bool_, expect={"fast8": 4})
    check(api, oracle, "ANY", ~b, [1], dst_dtype=np.bool_, expect={"fast8": 3})


def test_column_and_general_kernels_on_the_emulator(api, oracle, rng):
    x = ties(rng, (700, 130))
    p = check(api, oracle, "SUM", x, [0], expect={"shape": 1}, sms=4)
    assert p["splits"] > 1                                   # ticketed finish, [split][output] partials
    check(api, oracle, "MAXANDARGMAX", x, [0], expect={"shape": 1}, sms=4)
    check(api, oracle, "MAXANDARGMAX", ties(rng, (64, 2, 48)), [0, 1], expect={"shape": 1})
    check(api, oracle, "SUM", ties(rng, (500, 3, 40), np.float64), [0], expect={"shape": 1})
    g = ties(rng, (10, 11, 12))[:, :, ::2]                   # nothing contiguous: general kernel
    check(api, oracle, "MAXANDARGMAX", g, [1], expect={"shape": 2})
    check(api, oracle, "SUM", g, [0, 2], expect={"shape": 2})
