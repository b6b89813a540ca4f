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
        "seg", "nseg", "units", "gx", "gy", "bx", "by", "nf", "nr", "simple", "tiny"]
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
    out = (ctypes.c_ulonglong * 24)()
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
    group = p["group"] | (p["mu"] << 16) | (p["onerun"] << 20) | (p["flat"] << 21) | \
        (p.get("simple", 0) << 22) | (p.get("tiny", 0) << 23) | ((p["by"] if p["shape"] == 1 else 0) << 24)
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


def emulate(api, op, x, axes, dst_dtype=None, sms=2, force=None):
    """Runs the reduction on the emulator; returns (value array or None, index array or None, plan).
    `force` overrides fields of the plan that only select a build of the kernel (idx64)."""
    dst_dtype = np.dtype(dst_dtype or x.dtype)
    p, layout = plan_and_layout(api, op, x, axes, dst_dtype, sms)
    p.update(force or {})
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
    if p["splits"] > 1:
        # a second launch on the same scratch and counters (what back-to-back calls do)
        first = (None if d0 is None else d0.copy(), None if d1 is None else d1.copy())
        lib.simt_launch(layout, ptr(x), ptr(d0), ptr(d1), ptr(pval), ptr(pidx), ptr(tickets),
                        p["gx"], p["gy"], p["bx"], p["by"])
        assert (tickets == 0).all()
        assert d0 is None or d0.tobytes() == first[0].tobytes()
        assert d1 is None or (d1 == first[1]).all()
    return d0, d1, p


def check(api, oracle, op, x, axes, dst_dtype=None, expect=None, sms=2, force=None):
    d0, d1, p = emulate(api, op, x, axes, dst_dtype, sms, force)
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
    # a moderate number of long rows: two and four warps share a row (one barrier, fixed order)
    check(api, oracle, "MAXANDARGMAX", ties(rng, (30, 4100)), [1], sms=2, expect={"group": 64, "splits": 1})
    check(api, oracle, "SUM", ties(rng, (20, 4101)), [1], sms=2, expect={"group": 128})
    check(api, oracle, "MINANDARGMIN", ties(rng, (20, 16500)), [1], sms=2, expect={"group": 128, "lazy": 1})
    # scalar loads: a base that is not 16-byte aligned
    big = ties(rng, (3, 4100))
    u = big[:, 1:]
    check(api, oracle, "MAXANDARGMAX", u, [1], expect={"vec": 1})


def test_64_bit_index_builds_on_the_emulator(api, oracle, rng):
    """The builds with 64-bit flat indices (chosen by the planner beyond 2^32
    reduced elements) run here on small data; the GPU suite runs them at size."""
    f = {"idx64": 1}
    check(api, oracle, "MAXANDARGMAX", ties(rng, (40, 6000)), [1], force=f, expect={"lazy": 1})
    check(api, oracle, "MINANDARGMIN", ties(rng, (2, 40000)), [1], force=f, sms=1)
    check(api, oracle, "ARGMAX", ties(rng, (300, 24)), [1], force=f, expect={"onerun": 1})
    check(api, oracle, "MAXANDARGMAX", ties(rng, (23, 4, 64)), [2, 0], force=f)
    check(api, oracle, "MAXANDARGMAX", ties(rng, (700, 130)), [0], force=f, sms=4, expect={"shape": 1})
    check(api, oracle, "ARGMIN", ties(rng, (10, 11, 12))[:, :, ::2], [1], force=f, expect={"shape": 2})


def test_short_run_variants_on_the_emulator(api, oracle, rng):
    # one short run per output: 1, 2, 8 and 32 lanes per output, several outputs at once
    for cols, group in ((4, 1), (8, 2), (32, 2), (100, 8), (512, 32)):
        x = ties(rng, (301, cols + 4))[:, :cols]     # a pitch wider than the run: not the flat walk
        p = check(api, oracle, "SUM", x, [1], expect={"onerun": 1, "tiny": 0})
        assert p["group"] <= 32 and p["mu"] in (2, 4)
        check(api, oracle, "MAXANDARGMAX", x, [1], expect={"onerun": 1})
        check(api, oracle, "ARGMIN", x, [1])
    # one short run per output with the first element asked for up front: NaN first, NaNs later,
    # NaNs only, a run of the identity, signed zeros in both orders, ties; ragged groups
    for dtype, cols in ((np.float32, 100), (np.float32, 512), (np.float64, 200), (np.float16, 264), (np.int32, 60)):
        x = ties(rng, (57, cols + 8), dtype)[:, :cols]
        if np.dtype(dtype).kind == "f":
            x[0, 0] = np.nan
            x[1, cols - 1] = np.nan
            x[2, :] = -np.inf
            x[3, :] = -1
            x[3, cols // 2] = -0.0
            x[3, cols - 1] = 0.0
            x[4, :] = np.nan
            x[5, :] = 1
            x[5, 1] = 0.0
            x[5, cols - 2] = -0.0
            x[6, :] = np.inf
        for op in ("MAXANDARGMAX", "MINANDARGMIN", "ARGMAX", "MIN", "MAX"):
            check(api, oracle, op, x, [1], expect={"onerun": 1})
    check(api, oracle, "MAXANDARGMAX", ties(rng, (57, 104))[:, :101], [1], expect={"onerun": 1, "vec": 4})   # ragged end
    check(api, oracle, "MAXANDARGMAX", ties(rng, (57, 110))[:, :101], [1], expect={"onerun": 1, "vec": 1})   # scalar loads
    check(api, oracle, "SUM", ties(rng, (57, 108))[:, :100], [1], expect={"onerun": 1})
    # runs of 1, 2, 4, 8 full vectors lying back to back: the source walked as one flat array
    # of vectors, lanes-per-run = vectors per run; NaN first, NaNs later, signed zeros, ties,
    # a row of the identity; a count of vectors that leaves the last batch ragged
    for dtype, cols in ((np.float32, 4), (np.float32, 8), (np.float32, 16), (np.float32, 32),
                        (np.float64, 2), (np.float64, 16), (np.float16, 8), (np.float16, 64), (np.int32, 16)):
        x = ties(rng, (301, cols), dtype)
        if np.dtype(dtype).kind == "f":
            x[0, 0] = np.nan
            x[1, cols - 1] = np.nan
            x[2, :] = -np.inf
            x[3, :] = -1
            x[3, cols // 2] = -0.0
            x[3, cols - 1] = 0.0
            x[4, :] = np.nan
        want = {"tiny": 1, "onerun": 0, "group": cols * np.dtype(dtype).itemsize // 16}
        check(api, oracle, "MAXANDARGMAX", x, [1], expect=want)
        check(api, oracle, "MIN", x, [1], expect=want)
        check(api, oracle, "ARGMAX", x, [1], expect=want)
        if dtype == np.float64:                      # 8-byte sums stay on the short-run path (measured)
            check(api, oracle, "SUM", ties(rng, (301, cols), dtype), [1], expect={"tiny": 0, "onerun": 1})
        elif dtype != np.float16:
            check(api, oracle, "SUM", ties(rng, (301, cols), dtype), [1], expect=want)
    check(api, oracle, "SUM", ties(rng, (5000, 16)), [1], expect={"tiny": 1, "group": 4}, sms=1)
    # the vectors end inside a warp (100 and 400 of 256 threads' worth): whole warps keep iterating
    check(api, oracle, "MAXANDARGMAX", ties(rng, (100, 4)), [1], expect={"tiny": 1, "gx": 1})
    check(api, oracle, "MINANDARGMIN", ties(rng, (100, 16)), [1], expect={"tiny": 1, "gx": 1})
    check(api, oracle, "SUM", ties(rng, (1030, 4)), [1], expect={"tiny": 1})
    check(api, oracle, "SUM", ties(rng, (301, 12)), [1], expect={"tiny": 0})       # 3 vectors per run
    check(api, oracle, "SUM", ties(rng, (301, 64)), [1], expect={"tiny": 0, "onerun": 1})
    # (value, index) over one short run with several vectors per lane: values-only scan, then
    # the element, its bit pattern and its index from the winning vector; NaN first, NaNs
    # before the only candidate, signed zeros, ties, rows of the identity
    z = ties(rng, (40, 1024))
    z[0, :8] = np.nan
    z[1, 0] = np.nan
    z[2, :] = -np.inf
    z[2, 3:40] = np.nan
    z[3, :] = -1
    z[3, 130] = -0.0
    z[3, 131] = 0.0
    z[4, :] = 3
    z[4, [127, 128, 400]] = 9
    z[5, :] = np.nan
    for op in ("MAXANDARGMAX", "ARGMAX", "MAX"):
        check(api, oracle, op, z, [1], expect={"onerun": 1, "lazy": 1, "group": 32})
    check(api, oracle, "MINANDARGMIN", -z, [1], expect={"onerun": 1, "lazy": 1})
    check(api, oracle, "MINANDARGMIN", rng.integers(-5, 5, (100, 1024)).astype(np.int32), [1],
          expect={"onerun": 1, "lazy": 1})
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


# ------------------------------------------------------------- elementwise

class _Arg(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("typecode", ctypes.c_int), ("flags", ctypes.c_int)]


CTYPE = {np.dtype(np.float32): "float", np.dtype(np.float64): "double", np.dtype(np.float16): "ga_half",
         np.dtype(np.int32): "int", np.dtype(np.uint8): "unsigned char", np.dtype(np.int64): "long long",
         np.dtype(np.int16): "short"}
EW_KEYS = ["kind", "ept", "unroll", "nd", "idx", "modes", "tp", "tq", "pwi", "gx", "gy", "gz",
           "bx", "by", "bz", "n"]
EW_ENTRY = ["ga_ew_contig", "ga_ew_strided", "ga_ew_transpose"]


def emulate_elemwise(api, expr, spec, arrays, obj_flags=0, call_flags=0, sms=2, preamble=""):
    """spec: list of (name, dtype, GE flags); arrays: NumPy arrays (views allowed) or Python
    scalars, in the same order. Runs the call on the emulator, writing into the output arrays."""
    L = api.lib()
    n = len(spec)
    args = (_Arg * n)()
    nds = (ctypes.c_uint * n)()
    dimp = (ctypes.POINTER(ctypes.c_size_t) * n)()
    strp = (ctypes.POINTER(ctypes.c_ssize_t) * n)()
    addr = (ctypes.c_ulonglong * n)()
    keep = []
    for i, ((name, dt, fl), a) in enumerate(zip(spec, arrays)):
        args[i].name = name.encode()
        args[i].typecode = api.typecode(np.dtype(dt))
        args[i].flags = fl
        if not (fl & api.GE_SCALAR):
            nds[i] = a.ndim
            d = (ctypes.c_size_t * max(a.ndim, 1))(*a.shape)
            s = (ctypes.c_ssize_t * max(a.ndim, 1))(*a.strides)
            keep += [d, s]
            dimp[i] = ctypes.cast(d, ctypes.POINTER(ctypes.c_size_t))
            strp[i] = ctypes.cast(s, ctypes.POINTER(ctypes.c_ssize_t))
            addr[i] = a.ctypes.data
    out = (ctypes.c_ulonglong * 16)()
    blob = (ctypes.c_ulonglong * 1024)()
    words = ctypes.c_size_t()
    fn = L.gpuarray_b200_elemwise_plan
    fn.restype = ctypes.c_int
    err = fn(n, args, nds, dimp, strp, addr, obj_flags, call_flags, sms, out, blob, ctypes.c_size_t(1024),
             ctypes.byref(words))
    assert err == 0, err
    p = dict(zip(EW_KEYS, [int(v) for v in out]))
    if p["n"] == 0:
        return p
    src_fn = L.gpuarray_b200_elemwise_source
    src_fn.restype = ctypes.c_void_p
    src_fn.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint, ctypes.POINTER(_Arg), ctypes.c_int,
                       ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint, ctypes.c_int,
                       ctypes.c_ulonglong, ctypes.c_int, ctypes.c_int]
    ptr = src_fn(preamble.encode(), expr.encode(), n, args, obj_flags, p["kind"], p["ept"], p["unroll"],
                 p["nd"], p["idx"], p["modes"], p["tp"], p["tq"])
    text = ctypes.string_at(ptr).decode()
    if p["kind"] == 2:
        import re
        text = re.sub(r"#define GA_EW_PWI \d+", "#define GA_EW_PWI %d" % p["pwi"], text)
    # the launcher: layout block (strided / transposing kernels) or n, then pointers, then scalars
    arr_idx = [i for i, (nm, dt, fl) in enumerate(spec) if not (fl & api.GE_SCALAR)]
    sc_idx = [i for i, (nm, dt, fl) in enumerate(spec) if fl & api.GE_SCALAR]
    call = []
    for k, i in enumerate(arr_idx):
        ct = CTYPE[np.dtype(spec[i][1])]
        call.append("(%s *)a->ptr[%d]" % (ct if p["kind"] == 0 else "char", k))
    for k, i in enumerate(sc_idx):
        call.append("*(%s *)a->sc[%d]" % (CTYPE[np.dtype(spec[i][1])], k))
    first = "a->n" if p["kind"] == 0 else "*(const %s *)a->blob" % ("ga__ew_layout" if p["kind"] == 1
                                                                     else "ga__ewt_layout")
    text += '''
struct simt_ew_args { size_t n; const void *blob; void *ptr[32]; void *sc[32]; };
static void simt_body(void *q) {
  simt_ew_args *a = (simt_ew_args *)q;
  %s(%s);
}
extern "C" void simt_launch(size_t n, const void *blob, void **ptrs, void **scalars, unsigned np_,
                            unsigned ns_, unsigned gx, unsigned bx) {
  simt_ew_args a;
  a.n = n;
  a.blob = blob;
  for (unsigned i = 0; i < np_; i++) a.ptr[i] = ptrs[i];
  for (unsigned i = 0; i < ns_; i++) a.sc[i] = scalars[i];
  simt::run_grid(simt_body, &a, simt_dim3{gx, 1, 1}, simt_dim3{bx, 1, 1});
}
''' % (EW_ENTRY[p["kind"]], ", ".join([first] + call))
    tdeps = "".join(open(os.path.join(TEMPLATES, t)).read()
                    for t in ("ga_ew_common.cuh", "ga_ew_contig.cuh", "ga_ew_strided.cuh", "ga_ew_transpose.cuh"))
    key = hashlib.sha1((text + tdeps + open(os.path.join(SIMT, "include", "simt_emul.h")).read()).encode()
                       ).hexdigest()[:16]
    os.makedirs(BUILD, exist_ok=True)
    so = os.path.join(BUILD, "e_%s.so" % key)
    if not os.path.exists(so):
        src = os.path.join(BUILD, "e_%s.cpp" % key)
        with open(src, "w") as f:
            f.write(text)
        r = subprocess.run(["g++", "-std=c++17", "-O1", "-shared", "-fPIC", "-w", "-I",
                            os.path.join(SIMT, "include"), "-I", TEMPLATES, src,
                            os.path.join(SIMT, "simt_runtime.cpp"), "-o", so], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-3000:]
    lib = ctypes.CDLL(so)
    ptrs = (ctypes.c_void_p * 32)()
    scs = (ctypes.c_void_p * 32)()
    for k, i in enumerate(arr_idx):
        ptrs[k] = arrays[i].ctypes.data
    hold = []
    for k, i in enumerate(sc_idx):
        v = np.array(arrays[i], dtype=spec[i][1])
        hold.append(v)
        scs[k] = v.ctypes.data
    lib.simt_launch(ctypes.c_size_t(p["n"]), blob, ptrs, scs, len(arr_idx), len(sc_idx), p["gx"], p["bx"])
    return p


def test_elementwise_kernels_on_the_emulator(api, rng):
    R, W, S = api.GE_READ, api.GE_WRITE, api.GE_SCALAR
    # contiguous, ragged tail (4099 = 1024 vectors + 3), a scalar argument
    a = rng.standard_normal(4099).astype(np.float32)
    b = rng.standard_normal(4099).astype(np.float32)
    o = np.zeros(4099, np.float32)
    p = emulate_elemwise(api, "o = a * k + b", [("a", np.float32, R), ("k", np.float32, S), ("b", np.float32, R),
                                                ("o", np.float32, W)], [a, np.float32(3), b, o])
    assert p["kind"] == 0 and p["ept"] == 4
    assert np.allclose(o, a * np.float32(3) + b, rtol=1e-6, atol=1e-6)
    # uint8: 16 elements per chunk, wrap-around arithmetic
    u = rng.integers(0, 256, 5000).astype(np.uint8)
    uo = np.zeros(5000, np.uint8)
    p = emulate_elemwise(api, "o = a + 1", [("a", np.uint8, R), ("o", np.uint8, W)], [u, uo])
    assert p["ept"] == 16 and (uo == u + np.uint8(1)).all()
    # float16 storage, float32 arithmetic
    h = rng.standard_normal(3000).astype(np.float16)
    ho = np.zeros(3000, np.float16)
    p = emulate_elemwise(api, "o = a * 2.0f", [("a", np.float16, R), ("o", np.float16, W)], [h, ho],
                         obj_flags=api.GE_CONVERT_F16)
    assert p["ept"] == 8 and (ho == (h.astype(np.float32) * 2).astype(np.float16)).all()
    # strided kernel: row and column broadcasts, a reversed axis, a step-2 gather
    M, N = 37, 520
    A = rng.standard_normal((M, N)).astype(np.float32)
    row = rng.standard_normal((1, N)).astype(np.float32)
    col = rng.standard_normal((M, 1)).astype(np.float32)
    O = np.zeros((M, N), np.float32)
    spec3 = [("a", np.float32, R), ("b", np.float32, R), ("o", np.float32, W)]
    p = emulate_elemwise(api, "o = a + b", spec3, [A, row, O], call_flags=api.GE_BROADCAST)
    assert p["kind"] == 1 and (O == A + row).all()
    p = emulate_elemwise(api, "o = a + b", spec3, [A, col, O], call_flags=api.GE_BROADCAST)
    assert p["kind"] == 1 and (O == A + col).all()
    p = emulate_elemwise(api, "o = a + b", spec3, [A[::-1, ::-1], col, O], call_flags=api.GE_BROADCAST)
    assert (O == A[::-1, ::-1] + col).all()
    wide = rng.standard_normal((M, 2 * N)).astype(np.float32)
    p = emulate_elemwise(api, "o = a - b", spec3, [wide[:, ::2], A, O])
    assert p["kind"] == 1 and (O == wide[:, ::2] - A).all()
    # three dimensions that do not collapse, ragged innermost extent
    T = rng.standard_normal((5, 13, 2 * 31)).astype(np.float32)[:, ::2, ::2]
    TO = np.zeros((5, 7, 31), np.float32)
    p = emulate_elemwise(api, "o = a * a", [("a", np.float32, R), ("o", np.float32, W)], [T, TO])
    assert p["kind"] == 1 and p["nd"] == 3 and (TO == T * T).all()
    # tiled transpose: an fp32 transposed view, and the fp16 NHWC -> NCHW bias + ReLU of config 4 in small
    B = rng.standard_normal((100, 70)).astype(np.float32)
    BO = np.zeros((70, 100), np.float32)
    p = emulate_elemwise(api, "o = a * 2.0f", [("a", np.float32, R), ("o", np.float32, W)], [B.T, BO])
    assert p["kind"] == 2 and (BO == B.T * 2).all()
    nhwc = rng.standard_normal((2, 9, 7, 40)).astype(np.float16)
    x = nhwc.transpose(0, 3, 1, 2)
    bias = (0.2 * rng.random((1, 40, 1, 1)) - 0.1).astype(np.float16)
    y = np.zeros((2, 40, 9, 7), np.float16)
    p = emulate_elemwise(api, "y = fmaxf(x + bias, 0.0f)", [("x", np.float16, R), ("bias", np.float16, R),
                                                           ("y", np.float16, W)], [x, bias, y],
                         obj_flags=api.GE_CONVERT_F16, call_flags=api.GE_BROADCAST)
    assert p["kind"] == 2 and p["unroll"] == 2 and p["pwi"] == 1     # cp.async + ldmatrix build
    want = np.maximum(x.astype(np.float32) + bias.astype(np.float32), 0).astype(np.float16)
    assert (y == want).all()
    # the same with full tiles (64 channels, aligned rows: the 16-byte copy path) and a ragged Q edge
    nhwc = rng.standard_normal((2, 5, 9, 128)).astype(np.float16)
    x = nhwc.transpose(0, 3, 1, 2)
    bias = (0.2 * rng.random((1, 128, 1, 1)) - 0.1).astype(np.float16)
    y = np.zeros((2, 128, 5, 9), np.float16)
    p = emulate_elemwise(api, "y = fmaxf(x + bias, 0.0f)", [("x", np.float16, R), ("bias", np.float16, R),
                                                           ("y", np.float16, W)], [x, bias, y],
                         obj_flags=api.GE_CONVERT_F16, call_flags=api.GE_BROADCAST)
    assert p["kind"] == 2 and p["unroll"] == 2 and p["tp"] == 128
    want = np.maximum(x.astype(np.float32) + bias.astype(np.float32), 0).astype(np.float16)
    assert (y == want).all()
    # int16 through the same path, Q extent a multiple of 8 (vector stores)
    a16 = rng.integers(-300, 300, (64, 72)).astype(np.int16)
    o16 = np.zeros((72, 64), np.int16)
    p = emulate_elemwise(api, "o = a + 1", [("a", np.int16, R), ("o", np.int16, W)], [a16.T, o16])
    assert p["kind"] == 2 and p["unroll"] == 2 and (o16 == a16.T + 1).all()


def test_random_reductions_on_the_emulator(api, oracle):
    """A seeded sweep of shapes, axis lists, layouts, operators and element types
    through planner + generator + emulator against the oracle."""
    rng = np.random.default_rng(2024)
    ops = ["SUM", "MAXANDARGMAX", "MINANDARGMIN", "ARGMAX", "MAX", "PROD", "ANY"]
    dts = [np.float32, np.float64, np.float16, np.int32, np.int8, np.uint8]
    seen = set()
    for _ in range(90):
        nd = int(rng.integers(1, 5))
        shape = tuple(int(d) for d in rng.choice([1, 2, 3, 5, 8, 17, 40, 130, 600], size=nd))
        if np.prod(shape) > 400000 or np.prod(shape) == 0:
            shape = shape[:1] + (3,) * (nd - 1)
        dt = dts[int(rng.integers(0, len(dts)))]
        op = ops[int(rng.integers(0, len(ops)))]
        if np.dtype(dt).kind == "f":
            x = (np.round(rng.standard_normal(shape) * 2) / 2).astype(dt)
        else:
            lo = -4 if np.dtype(dt).kind == "i" else 0
            x = rng.integers(lo, 5, shape).astype(dt)
        r = rng.random()
        if r < 0.25 and nd > 1:
            x = np.asfortranarray(x)
        elif r < 0.5:
            big = np.zeros(tuple(2 * s + 1 for s in shape), dt)
            sl = tuple(slice(1, 1 + 2 * s, 2) for s in shape)
            big[sl] = x
            x = big[sl]
        k = int(rng.integers(1, nd + 1))
        axes = [int(a) for a in rng.permutation(nd)[:k]]
        dst = None
        if op == "ANY":
            dst = np.bool_
        elif op in ("SUM", "PROD") and np.dtype(dt).kind in "iu":
            dst = np.int64
        elif op in ("SUM", "PROD") and dt == np.float16:
            x = (x / 4).astype(dt) if op == "PROD" else x
            dst = np.float32                       # keeps the tolerance of the check simple
        if op == "PROD":
            x = np.sign(x).astype(dt) if np.dtype(dt).kind != "u" else (x % 2 + 1).astype(dt)
        p = check(api, oracle, op, x, axes, dst_dtype=dst, sms=int(rng.choice([1, 2, 4])))
        seen.add((p["shape"], p["onerun"], p["flat"], p["mu"] > 1, p["splits"] > 1))
    assert len(seen) >= 6                          # the sweep reached a spread of kernel variants
