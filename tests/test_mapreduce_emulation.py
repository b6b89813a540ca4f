"""The map-reduce kernel TEMPLATE (templates/ga_mapreduce.cuh) executed on the CPU.

As for the one-array reductions (test_kernel_emulation.py): the library's
planner picks the kernel shape, access modes, split and launch geometry for
NumPy arrays standing in for device arrays (gpuarray_b200_mapreduction_plan),
the library's generator emits the very source NVRTC would get
(gpuarray_b200_mapreduction_source), g++ compiles it against the SIMT emulator
and the result is compared with NumPy on the same inputs. Covers what the
reference's ReductionKernel offers (pygpu/reduction.py:137-291): a map
expression over several arguments, broadcasting, scalars, any reduce
expression with its neutral element."""
import ctypes
import hashlib
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SIMT = os.path.join(ROOT, "tests", "simt")
TEMPLATES = os.path.join(ROOT, "libgpuarray_b200", "csrc", "templates")
BUILD = os.path.join(ROOT, "libgpuarray_b200", "build", "simt")
KEYS = ["shape", "vec", "group", "tpo", "modes", "splits", "seg", "nseg", "units", "gx", "gy", "bx",
        "by", "nf"]
ENTRY = ["ga_mr_rows", "ga_mr_cols", "ga_mr_general"]
CT = {np.dtype(np.float32): "float", np.dtype(np.float64): "double", np.dtype(np.int32): "int",
      np.dtype(np.int16): "short", np.dtype(np.int64): "long long", np.dtype(np.uint8): "unsigned char",
      np.dtype(np.float16): "ga_half"}


def _descr(api, arrays, scalars):
    n = len(arrays) + len(scalars)
    args = (api._ElemwiseArg * n)()
    keep = []
    for i, (name, a) in enumerate(arrays):
        keep.append(name.encode())
        args[i].name, args[i].typecode, args[i].flags = keep[-1], api.typecode(a.dtype), api.GE_READ
    for j, (name, v) in enumerate(scalars):
        keep.append(name.encode())
        i = len(arrays) + j
        args[i].name, args[i].typecode, args[i].flags = keep[-1], api.typecode(v.dtype), api.GE_SCALAR
    return args, keep


def plan(api, out_dtype, arrays, scalars, axes, flags, sms):
    L = api.lib()
    fn = L.gpuarray_b200_mapreduction_plan
    fn.restype = ctypes.c_int
    args, keep = _descr(api, arrays, scalars)
    n = len(arrays) + len(scalars)
    nds = (ctypes.c_uint * n)()
    dims = (ctypes.POINTER(ctypes.c_size_t) * n)()
    strides = (ctypes.POINTER(ctypes.c_ssize_t) * n)()
    bases = (ctypes.c_ulonglong * n)()
    hold = []
    for i, (_, a) in enumerate(arrays):
        nds[i] = a.ndim
        d = (ctypes.c_size_t * max(a.ndim, 1))(*a.shape)
        s = (ctypes.c_ssize_t * max(a.ndim, 1))(*a.strides)
        hold += [d, s]
        dims[i] = ctypes.cast(d, ctypes.POINTER(ctypes.c_size_t))
        strides[i] = ctypes.cast(s, ctypes.POINTER(ctypes.c_ssize_t))
        bases[i] = a.ctypes.data
    out = (ctypes.c_ulonglong * 14)()
    layout = ctypes.create_string_buffer(8192)
    used = ctypes.c_size_t()
    err = fn(api.typecode(out_dtype), n, args, nds, dims, strides, bases, len(axes),
             (ctypes.c_int * max(len(axes), 1))(*axes), flags, sms, out, layout, ctypes.c_size_t(8192),
             ctypes.byref(used))
    return err, dict(zip(KEYS, [int(v) for v in out])), layout


def build_variant(api, map_expr, reduce_expr, neutral, out_dtype, arrays, scalars, p, obj_flags):
    L = api.lib()
    L.gpuarray_b200_mapreduction_source.restype = ctypes.c_void_p
    args, keep = _descr(api, arrays, scalars)
    ptr = L.gpuarray_b200_mapreduction_source(None, map_expr.encode(), reduce_expr.encode(),
                                              neutral.encode(), api.typecode(out_dtype),
                                              len(arrays) + len(scalars), args, obj_flags, p["shape"],
                                              p["vec"], p["group"], p["tpo"],
                                              ctypes.c_ulonglong(p["modes"]))
    text = ctypes.string_at(ptr).decode()
    call = ["*a->L", "a->dst", "(GA_MR_ACC_T *)a->pval", "a->tickets"]
    call += ["(const char *)a->arr[%d]" % i for i in range(len(arrays))]
    call += ["*(const %s *)a->sc[%d]" % (CT[v.dtype], j) for j, (_, v) in enumerate(scalars)]
    text += r'''
struct simt_args { const ga__mr_layout *L; char *dst; void *pval; unsigned int *tickets;
                   const void *const *arr; const void *const *sc; };
static void simt_body(void *p) {
  simt_args *a = (simt_args *)p;
  %s(%s);
}
extern "C" void simt_launch(const void *layout, void *dst, void *pval, void *tickets,
                            const void *const *arr, const void *const *sc, unsigned gx, unsigned gy,
                            unsigned bx, unsigned by) {
  simt_args a = {(const ga__mr_layout *)layout, (char *)dst, pval, (unsigned int *)tickets, arr, sc};
  simt::run_grid(simt_body, &a, simt_dim3{gx, gy, 1}, simt_dim3{bx, by, 1});
}
''' % (ENTRY[p["shape"]], ", ".join(call))
    deps = "".join(open(os.path.join(TEMPLATES, f)).read()
                   for f in ("ga_mapreduce.cuh", "ga_reduce.cuh", "ga_ew_common.cuh"))
    key = hashlib.sha1((text + deps + open(os.path.join(SIMT, "include", "simt_emul.h")).read())
                       .encode()).hexdigest()[:16]
    os.makedirs(BUILD, exist_ok=True)
    so = os.path.join(BUILD, "mr_%s.so" % key)
    if not os.path.exists(so):
        src = os.path.join(BUILD, "mr_%s.cpp" % key)
        with open(src, "w") as f:
            f.write(text)
        r = subprocess.run(["g++", "-std=c++17", "-O1", "-shared", "-fPIC", "-w", "-I",
                            os.path.join(SIMT, "include"), "-I", TEMPLATES, src,
                            os.path.join(SIMT, "simt_runtime.cpp"), "-o", so],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-3000:]
    return ctypes.CDLL(so)


def emulate(api, map_expr, reduce_expr, neutral, out_dtype, arrays, axes, scalars=(), flags=None,
            sms=2, obj_flags=0):
    out_dtype = np.dtype(out_dtype)
    flags = api.GE_BROADCAST | api.GE_PADSHAPE if flags is None else flags
    scalars = [(n, np.asarray(v)) for n, v in scalars]
    err, p, layout = plan(api, out_dtype, arrays, scalars, axes, flags, sms)
    assert err == 0, err
    shape = np.broadcast_shapes(*[a.shape for _, a in arrays])
    kept = tuple(d for i, d in enumerate(shape) if i not in axes)
    nout = max(1, int(np.prod(kept)))
    dst = np.frombuffer(bytearray(b"\x55" * (nout * out_dtype.itemsize)), dtype=out_dtype)[:nout]
    if p["nf"] == 0:
        return dst.reshape(kept), p
    lib = build_variant(api, map_expr, reduce_expr, neutral, out_dtype, arrays, scalars, p, obj_flags)
    pval = np.zeros(max(1, p["splits"] * p["nf"]) * 8, np.uint8)
    tickets = np.zeros(max(p["nf"], p["units"], 1) + 8, np.uint32)
    arr = (ctypes.c_void_p * max(len(arrays), 1))(*[a.ctypes.data for _, a in arrays])
    sc = (ctypes.c_void_p * max(len(scalars), 1))(*[v.ctypes.data for _, v in scalars])
    for _ in range(2 if p["splits"] > 1 else 1):     # twice on the same scratch and counters
        lib.simt_launch(layout, ctypes.c_void_p(dst.ctypes.data), ctypes.c_void_p(pval.ctypes.data),
                        ctypes.c_void_p(tickets.ctypes.data), arr, sc, p["gx"], p["gy"], p["bx"], p["by"])
        assert (tickets == 0).all()
    return dst.reshape(kept), p


def close(got, want, scale, n, dtype):
    if np.dtype(dtype).kind != "f":
        return (got == want).all()
    eps = 1e-6 if np.dtype(dtype) == np.float32 else 1e-12
    return (np.abs(got.astype(np.float64) - want) <= eps * np.log2(max(n, 2)) * np.maximum(scale, 1e-300)).all()


def dot_check(api, a, b, axes, out_dtype, expect=None, sms=2):
    got, p = emulate(api, "a * b", "a + b", "0", out_dtype, [("a", a), ("b", b)], axes, sms=sms)
    prod = a.astype(np.float64) * b.astype(np.float64)
    want = prod.sum(axis=tuple(axes))
    n = int(np.prod([prod.shape[i] for i in axes]))
    assert close(got, want, np.abs(prod).sum(axis=tuple(axes)), n, out_dtype), (p, got, want)
    for k, v in (expect or {}).items():
        assert p[k] == v, (k, p)
    return p


def test_the_reference_broadcast_case(api, rng):
    # pygpu/tests/test_reduction.py:57-84: (5,10,15) * (1,10,15), reduced over axis 1
    a = rng.standard_normal((5, 10, 15))
    b = rng.standard_normal((1, 10, 15))
    dot_check(api, a, b, [1], np.float64, expect={"shape": 2})


def test_rows_shapes(api, rng):
    f = np.float32
    a = rng.standard_normal((40, 6004)).astype(f)[:, :6001]
    b = rng.standard_normal((40, 6004)).astype(f)[:, :6001]
    # a warp per output, 128-bit loads, ragged end
    dot_check(api, a, b, [1], f, expect={"shape": 0, "group": 32, "vec": 4, "modes": 0b0101, "splits": 1}, sms=1)
    # one operand broadcast along the kept axis, the other along the reduced one
    dot_check(api, a, rng.standard_normal((1, 6001)).astype(f), [1], f, expect={"shape": 0, "modes": 0b0101}, sms=1)
    dot_check(api, a, rng.standard_normal((40, 1)).astype(f), [1], f, expect={"shape": 0, "modes": 0b1001}, sms=1)
    # mixed element sizes: fp32 x fp64 into fp64
    b64 = rng.standard_normal((40, 6004))[:, :6001]
    dot_check(api, a, b64, [1], np.float64, expect={"shape": 0, "vec": 4}, sms=1)
    # few outputs: the reduced extent is split, partials and tickets
    p = dot_check(api, rng.standard_normal((2, 40000)).astype(f),
                  rng.standard_normal((2, 40000)).astype(f), [1], f, sms=4)
    assert p["splits"] > 1
    # whole-array reduction by CTA groups over segments of one long run
    x = rng.standard_normal(70001).astype(f)
    y = rng.standard_normal(70001).astype(f)
    p = dot_check(api, x, y, [0], f, sms=1)
    assert p["group"] == 256 and p["splits"] > 1 and p["nseg"] > 1
    # a base that is not 16-byte aligned: scalar loads
    dot_check(api, a[:, 1:], b[:, 1:], [1], f, expect={"shape": 0, "vec": 1}, sms=1)
    # two reduced axes of a 3-D array that collapse into one run
    c = rng.standard_normal((6, 30, 64)).astype(f)
    d = rng.standard_normal((6, 30, 64)).astype(f)
    dot_check(api, c, d, [1, 2], f, expect={"shape": 0})
    # ... and that do not (reduced outer axis + contiguous run)
    dot_check(api, c, d, [0, 2], f, expect={"shape": 0})


def test_cols_shapes(api, rng):
    f = np.float32
    a = rng.standard_normal((700, 132)).astype(f)
    b = rng.standard_normal((700, 132)).astype(f)
    p = dot_check(api, a, b, [0], f, expect={"shape": 1, "vec": 4, "modes": 0b0101}, sms=4)
    assert p["splits"] > 1
    dot_check(api, a, rng.standard_normal((1, 132)).astype(f), [0], f, expect={"shape": 1}, sms=1)
    dot_check(api, a, rng.standard_normal((700, 1)).astype(f), [0], f, expect={"shape": 1, "modes": 0b1001}, sms=1)
    # kept axis in the middle
    c = rng.standard_normal((9, 20, 64)).astype(np.float64)
    d = rng.standard_normal((9, 20, 64)).astype(np.float64)
    dot_check(api, c, d, [0], np.float64, expect={"shape": 1, "vec": 2})
    # 130 columns: not a multiple of 4, two elements per thread
    dot_check(api, a[:, :130], b[:, :130], [0], f, expect={"shape": 1, "vec": 2})


def test_general_shapes_and_other_operators(api, rng):
    f = np.float32
    a = rng.standard_normal((30, 50)).astype(f)
    b = rng.standard_normal((30, 50)).astype(f)
    # every second column: neither dimension is contiguous
    dot_check(api, a[:, ::2], b[:, ::2], [1], f, expect={"shape": 2})
    dot_check(api, a[::-1, ::2], b[:, ::2], [0], f, expect={"shape": 2})
    # max |a - b| with a scalar scale
    got, p = emulate(api, "fabsf(a - b) * s", "fmaxf(a, b)", "0", f, [("a", a), ("b", b)], [0, 1],
                     scalars=[("s", np.float32(0.5))])
    assert got.reshape(()) == np.float32(np.abs(a - b).max() * np.float32(0.5))
    # integers are exact: int32 x int16 into int64
    i = rng.integers(-1000, 1000, (17, 300)).astype(np.int32)
    j = rng.integers(-1000, 1000, (17, 300)).astype(np.int16)
    got, p = emulate(api, "(ga_long)a * b", "a + b", "0", np.int64, [("a", i), ("b", j)], [1])
    assert (got == (i.astype(np.int64) * j).sum(1)).all()
    # three arguments, one of them a column
    c = rng.standard_normal((30, 1)).astype(f)
    got, p = emulate(api, "a * b + c", "a + b", "0", np.float64, [("a", a), ("b", b), ("c", c)], [1])
    want = (a.astype(np.float64) * b + c).sum(1)
    assert np.allclose(got, want, rtol=1e-5)
    # float16 arguments computed in float32
    h = rng.standard_normal((8, 256)).astype(np.float16)
    got, p = emulate(api, "a * a", "a + b", "0", f, [("a", h)], [1], obj_flags=api.GE_CONVERT_F16)
    assert np.allclose(got, (h.astype(np.float64) ** 2).sum(1), rtol=1e-5)
    # an empty reduced extent writes the neutral element
    e = np.zeros((4, 0), f)
    got, p = emulate(api, "a", "a * b", "1", f, [("a", e)], [1])
    assert (got == 1).all()


def test_shape_errors(api, rng):
    a = np.zeros((3, 4), np.float32)
    b = np.zeros((1, 4), np.float32)
    err, _, _ = plan(api, np.float32, [("a", a), ("b", b)], [], [0], 0, 2)
    assert err == api.GA_VALUE_ERROR                      # broadcasting was not asked for
    err, _, _ = plan(api, np.float32, [("a", a), ("b", np.zeros(4, np.float32))], [], [0],
                     api.GE_BROADCAST, 2)
    assert err == api.GA_VALUE_ERROR                      # differing rank without GE_PADSHAPE
    err, p, _ = plan(api, np.float32, [("a", a), ("b", np.zeros(4, np.float32))], [], [0],
                     api.GE_BROADCAST | api.GE_PADSHAPE, 2)
    assert err == 0 and p["nf"] == 4
    err, _, _ = plan(api, np.float32, [("a", a)], [], [2], 0, 2)
    assert err == api.GA_INVALID_ERROR                    # axis out of range
    err, _, _ = plan(api, np.float32, [("a", a)], [], [], 0, 2)
    assert err == api.GA_VALUE_ERROR                      # reduction along no axes
