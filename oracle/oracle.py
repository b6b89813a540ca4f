"""Python face of the CPU oracle. TEST INFRASTRUCTURE ONLY: imported by tests/,
by __graft_entry__.smoke() and by the cpu_baseline / reference legs of bench.py;
never by the product package.

  - minmaxarg / collapse / half conversion / fma: ctypes calls into
    oracle/liboracle.so (oracle_kernels.c, a C restatement of the reference
    kernels; see the citations there);
  - ElemwiseOracle: restates the reference's strided elementwise kernel
    generator (src/gpuarray_elemwise.c:123-250) as HOST C: per element the index
    is decoded with % and / over the dimensions, each READ argument is loaded
    (GA_HALF through half->float when GE_CONVERT_F16), the user expression is
    pasted once, each WRITE argument is stored. The text is compiled with gcc
    (-mfma -ffp-contract=fast, so a*b+c contracts to one fused multiply-add as
    NVRTC does by default) and run over NumPy buffers. Argument checking and
    broadcasting follow check_basic (:272-383);
  - reduce_reference: NumPy statement of SUM/PROD/PRODNZ/AND/OR/XOR/ALL/ANY
    (pygpu/reduction.py:83-132 and pygpu/_array.py:238-294 give the semantics of
    sum/prod/all/any; the other four have no implementation in the reference
    snapshot, so their parity is unpinned and NumPy is the stated choice).
"""
import ctypes
import hashlib
import os
import subprocess
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

GE_SCALAR, GE_READ, GE_WRITE = 1, 2, 4

_TC = {np.dtype(np.bool_): 0, np.dtype(np.int8): 1, np.dtype(np.uint8): 2, np.dtype(np.int16): 3,
       np.dtype(np.uint16): 4, np.dtype(np.int32): 5, np.dtype(np.uint32): 6,
       np.dtype(np.int64): 7, np.dtype(np.uint64): 8, np.dtype(np.float32): 11,
       np.dtype(np.float64): 12, np.dtype(np.float16): 23}

_CNAME = {0: "uint8_t", 1: "int8_t", 2: "uint8_t", 3: "int16_t", 4: "uint16_t", 5: "int32_t",
          6: "uint32_t", 7: "int64_t", 8: "uint64_t", 11: "float", 12: "double", 23: "ga_half"}
_GANAME = {0: "ga_bool", 1: "ga_byte", 2: "ga_ubyte", 3: "ga_short", 4: "ga_ushort", 5: "ga_int",
           6: "ga_uint", 7: "ga_long", 8: "ga_ulong", 11: "ga_float", 12: "ga_double",
           23: "ga_half"}


def reference_tree():
    """Root of the reference checkout used to build oracle/_ref, or None: the
    GPUARRAY_REFERENCE_TREE environment variable, else a directory named
    `reference` beside this repository."""
    cand = os.environ.get("GPUARRAY_REFERENCE_TREE") or os.path.join(
        os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src")) else None


def build():
    """Compiles liboracle.so (and oracle/_ref when a reference tree is found)."""
    cmd = ["make", "-C", _HERE]
    ref = reference_tree()
    if ref is not None:
        cmd.append("REF=" + ref)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stdout)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = ctypes.CDLL(path)
        L.oracle_half2float.restype = ctypes.c_float
        L.oracle_half2float.argtypes = [ctypes.c_uint16]
        L.oracle_float2half.restype = ctypes.c_uint16
        L.oracle_float2half.argtypes = [ctypes.c_float]
        L.oracle_fma_f32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                     ctypes.c_void_p, ctypes.c_size_t]
        L.oracle_collapse.argtypes = [ctypes.c_uint, ctypes.POINTER(ctypes.c_uint),
                                      ctypes.POINTER(ctypes.c_size_t),
                                      ctypes.POINTER(ctypes.POINTER(ctypes.c_ssize_t))]
        L.oracle_minmaxarg.restype = ctypes.c_int
        L.oracle_minmaxarg.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_uint,
                                       ctypes.POINTER(ctypes.c_size_t),
                                       ctypes.POINTER(ctypes.c_ssize_t), ctypes.c_uint,
                                       ctypes.POINTER(ctypes.c_uint), ctypes.c_void_p,
                                       ctypes.c_void_p]
        L.oracle_rowmaxarg_f32.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t,
                                           ctypes.c_void_p, ctypes.c_void_p]
        L.oracle_pcg_fill_f32.argtypes = [ctypes.c_uint64, ctypes.c_void_p, ctypes.c_size_t]
        L.oracle_set_threads.restype = ctypes.c_int
        L.oracle_set_threads.argtypes = [ctypes.c_int]
        L.oracle_threads_used.restype = ctypes.c_int
        _LIB = L
    return _LIB


def ref_lib():
    """The reference's own util code (oracle/_ref/libref_util.so) or None."""
    path = os.path.join(_HERE, "_ref", "libref_util.so")
    if not os.path.exists(path):
        return None
    L = ctypes.CDLL(path)
    L.ref_float2half.restype = ctypes.c_uint16
    L.ref_float2half.argtypes = [ctypes.c_float]
    L.gpuarray_elemwise_collapse.argtypes = [ctypes.c_uint, ctypes.POINTER(ctypes.c_uint),
                                             ctypes.POINTER(ctypes.c_size_t),
                                             ctypes.POINTER(ctypes.POINTER(ctypes.c_ssize_t))]
    L.gpuarray_get_elsize.restype = ctypes.c_size_t
    L.gpuarray_get_elsize.argtypes = [ctypes.c_int]
    L.gpuarray_error_str.restype = ctypes.c_char_p
    L.gpuarray_error_str.argtypes = [ctypes.c_int]
    return L


# ------------------------------------------------------------------ scalars

def float2half_bits(x):
    return lib().oracle_float2half(ctypes.c_float(x))


def fma_f32(a, b, c):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    out = np.empty_like(a)
    lib().oracle_fma_f32(a.ctypes.data, b.ctypes.data, ctypes.c_float(c), out.ctypes.data, a.size)
    return out


def pcg_fill_f32(seed, n):
    out = np.empty(n, dtype=np.float32)
    lib().oracle_pcg_fill_f32(seed, out.ctypes.data, n)
    return out


def collapse(dims, strides_list, fn=None):
    """Runs a collapse implementation (default: the oracle's) on Python lists.
    `fn` may be another C function with the same signature (the product's or
    the reference's). Returns (dims, strides_list)."""
    nd = ctypes.c_uint(len(dims))
    cd = (ctypes.c_size_t * len(dims))(*dims)
    rows = [(ctypes.c_ssize_t * len(dims))(*s) for s in strides_list]
    ptrs = (ctypes.POINTER(ctypes.c_ssize_t) * len(rows))(
        *[ctypes.cast(r, ctypes.POINTER(ctypes.c_ssize_t)) for r in rows])
    (fn or lib().oracle_collapse)(len(rows), ctypes.byref(nd), cd, ptrs)
    n = nd.value
    return list(cd[:n]), [list(r[:n]) for r in rows]


# --------------------------------------------------------------- reductions

def minmaxarg(x, axes, is_min=False):
    """(values, flat indices) over `axes` in the given order, reference rules."""
    x = np.asarray(x)
    axes = [int(a) for a in axes]
    free = [i for i in range(x.ndim) if i not in axes]
    oshape = tuple(x.shape[i] for i in free)
    vals = np.empty(oshape, dtype=x.dtype)
    idx = np.empty(oshape, dtype=np.int64)
    dims = (ctypes.c_size_t * x.ndim)(*x.shape)
    strs = (ctypes.c_ssize_t * x.ndim)(*x.strides)
    ax = (ctypes.c_uint * len(axes))(*axes)
    rc = lib().oracle_minmaxarg(_TC[x.dtype], 1 if is_min else 0, x.ctypes.data, x.ndim, dims, strs,
                                len(axes), ax, vals.ctypes.data, idx.ctypes.data)
    if rc != 0:
        raise ValueError("oracle_minmaxarg rejected the arguments")
    return vals, idx


def set_threads(n):
    """Fixes the OpenMP team of the timed loops to `n` threads, overriding
    OMP_NUM_THREADS; returns the team size a parallel region really gets."""
    lib().oracle_set_threads(int(n))
    return int(lib().oracle_threads_used())


def rowmaxarg_f32(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    vmax = np.empty(x.shape[0], dtype=np.float32)
    imax = np.empty(x.shape[0], dtype=np.int64)
    lib().oracle_rowmaxarg_f32(x.ctypes.data, x.shape[0], x.shape[1], vmax.ctypes.data,
                               imax.ctypes.data)
    return vmax, imax


def reduce_reference(op, x, axes, out_dtype):
    """High-precision value of an accumulate-type reduction, cast to out_dtype.
    op in {"sum","prod","prodnz","and","or","xor","all","any"}."""
    x = np.asarray(x)
    axes = tuple(int(a) for a in axes)
    out_dtype = np.dtype(out_dtype)
    if op in ("sum", "prod", "prodnz"):
        if out_dtype.kind == "f":
            wide = x.astype(np.longdouble if out_dtype == np.float64 else np.float64)
        else:
            wide = x.astype(out_dtype)       # integer arithmetic wraps in the output type
        if op == "sum":
            r = wide.sum(axis=axes)
        else:
            if op == "prodnz":
                wide = np.where(x != 0, wide, np.ones((), dtype=wide.dtype))
            r = wide.prod(axis=axes)
        return np.asarray(r)
    if op in ("and", "or", "xor"):
        fn = {"and": np.bitwise_and, "or": np.bitwise_or, "xor": np.bitwise_xor}[op]
        r = x.astype(out_dtype)
        for a in sorted(axes, reverse=True):
            r = fn.reduce(r, axis=a)
        return np.asarray(r)
    if op == "all":
        return np.asarray((x != 0).all(axis=axes)).astype(out_dtype)
    if op == "any":
        return np.asarray((x != 0).any(axis=axes)).astype(out_dtype)
    raise ValueError(op)


# -------------------------------------------------------------- elementwise

_HOST_CLUDA = r"""
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include <sys/types.h>
#define WITHIN_KERNEL static inline
#define KERNEL
#define GLOBAL_MEM
#define LOCAL_MEM
typedef uint8_t ga_bool; typedef int8_t ga_byte; typedef uint8_t ga_ubyte;
typedef int16_t ga_short; typedef uint16_t ga_ushort; typedef int32_t ga_int;
typedef uint32_t ga_uint; typedef long long ga_long; typedef unsigned long long ga_ulong;
typedef float ga_float; typedef double ga_double; typedef size_t ga_size; typedef ptrdiff_t ga_ssize;
typedef struct { uint16_t data; } ga_half;
float oracle_half2float(uint16_t h);
uint16_t oracle_float2half(float f);
static inline float ga_half2float(ga_half h) { return oracle_half2float(h.data); }
static inline ga_half ga_float2half(float f) { ga_half r; r.data = oracle_float2half(f); return r; }
"""


class ElemwiseOracle:
    """args: sequence of (name, numpy dtype, flags) exactly like GpuElemwise."""

    def __init__(self, expr, args, preamble="", convert_f16=False):
        self.args = [(n, np.dtype(dt), fl) for n, dt, fl in args]
        self.convert_f16 = convert_f16
        src = [_HOST_CLUDA, preamble or "", "\nvoid elem(size_t n, unsigned nd, const size_t *dims"]
        for name, dt, fl in self.args:
            tn = _GANAME[_TC[dt]]
            if fl & GE_SCALAR:
                src.append(", %s %s" % (tn, name))
            else:
                src.append(", char *%s_p, const ssize_t *%s_str" % (name, name))
        src.append(") {\n  size_t i;\n  for (i = 0; i < n; i++) {\n    size_t ii = i, pos; unsigned d;\n")
        arrays = [(n, dt, fl) for n, dt, fl in self.args if not fl & GE_SCALAR]
        for name, dt, fl in arrays:
            src.append("    char *%s_q = %s_p;\n" % (name, name))
        src.append("    for (d = nd; d > 1; d--) { pos = ii % dims[d-1]; ii /= dims[d-1];\n")
        for name, dt, fl in arrays:
            src.append("      %s_q += (ssize_t)pos * %s_str[d-1];\n" % (name, name))
        src.append("    }\n    if (nd > 0) {\n")
        for name, dt, fl in arrays:
            src.append("      %s_q += (ssize_t)ii * %s_str[0];\n" % (name, name))
        src.append("    }\n    {\n")
        for name, dt, fl in arrays:
            tn = _GANAME[_TC[dt]]
            half = dt == np.float16 and convert_f16
            src.append("    %s %s;\n" % ("ga_float" if half else tn, name))
            if fl & GE_READ:
                if half:
                    src.append("    %s = ga_half2float(*(ga_half *)%s_q);\n" % (name, name))
                else:
                    src.append("    %s = *(%s *)%s_q;\n" % (name, tn, name))
        src.append("    " + expr + ";\n")
        for name, dt, fl in arrays:
            tn = _GANAME[_TC[dt]]
            half = dt == np.float16 and convert_f16
            if fl & GE_WRITE:
                if half:
                    src.append("    *(ga_half *)%s_q = ga_float2half(%s);\n" % (name, name))
                else:
                    src.append("    *(%s *)%s_q = %s;\n" % (tn, name, name))
        src.append("    }\n  }\n}\n")
        self.source = "".join(src)
        self._fn = self._compile(self.source)

    @staticmethod
    def _compile(source):
        key = hashlib.sha1(source.encode()).hexdigest()[:20]
        cache = os.path.join(tempfile.gettempdir(), "ga_b200_oracle_ew")
        os.makedirs(cache, exist_ok=True)
        so = os.path.join(cache, key + ".so")
        if not os.path.exists(so):
            c = os.path.join(cache, key + ".c")
            with open(c, "w") as f:
                f.write(source)
            tmp = so + ".%d.tmp" % os.getpid()
            r = subprocess.run(["/usr/bin/gcc", "-O2", "-fPIC", "-shared", "-std=gnu11", "-mfma",
                                "-ffp-contract=fast", "-o", tmp, c,
                                os.path.join(_HERE, "liboracle.so"),
                                "-Wl,-rpath," + _HERE, "-lm"],
                               stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if r.returncode != 0:
                raise RuntimeError("oracle elementwise compile failed:\n%s\n%s" % (r.stdout, source))
            os.replace(tmp, so)
        lib()
        return ctypes.CDLL(so).elem

    def __call__(self, *values, broadcast=True, padshape=True):
        """values: NumPy arrays (outputs are written in place) and scalars."""
        arrays = [(i, v) for i, (v, a) in enumerate(zip(values, self.args)) if not a[2] & GE_SCALAR]
        out = next(v for (i, v) in arrays if self.args[i][2] & GE_WRITE)
        nd = max(v.ndim for _, v in arrays) if padshape else out.ndim
        for _, v in arrays:
            if v.ndim != nd and not padshape:
                raise ValueError("differing nd")
        if out.ndim != nd:
            raise ValueError("output cannot broadcast")
        dims = list(out.shape)
        strides = {}
        for i, v in arrays:
            pad = nd - v.ndim
            vd = [1] * pad + list(v.shape)
            vs = [0] * pad + list(v.strides)
            for j in range(nd):
                if vd[j] != dims[j]:
                    if not broadcast or (self.args[i][2] & GE_WRITE) or vd[j] != 1:
                        raise ValueError("Mismatched dimension %d for input %d" % (j, i))
                if vd[j] == 1:
                    vs[j] = 0
            strides[i] = vs
        n = int(np.prod(dims, dtype=np.int64)) if nd else 1
        if n == 0:
            return
        cargs = [ctypes.c_size_t(n), ctypes.c_uint(nd), (ctypes.c_size_t * max(nd, 1))(*dims)]
        keep = []
        for i, (v, a) in enumerate(zip(values, self.args)):
            if a[2] & GE_SCALAR:
                s = np.array(v, dtype=a[1])
                ct = {1: ctypes.c_uint8, 2: ctypes.c_uint16, 4: ctypes.c_uint32,
                      8: ctypes.c_uint64}[s.itemsize]
                if a[1].kind == "f" and a[1].itemsize == 4:
                    cargs.append(ctypes.c_float(float(s)))
                elif a[1].kind == "f" and a[1].itemsize == 8:
                    cargs.append(ctypes.c_double(float(s)))
                elif a[1].kind == "i":
                    cargs.append(ctypes.c_int64(int(s)))
                else:
                    cargs.append(ct(int(s.view(ct))))
            else:
                st = (ctypes.c_ssize_t * max(nd, 1))(*strides[i])
                keep.append(st)
                cargs.append(ctypes.c_void_p(v.ctypes.data))
                cargs.append(st)
        self._fn(*cargs)
