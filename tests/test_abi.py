"""CPU-only checks of the C ABI: the library loads without a driver, exports
every entry point the headers declare, its host-only functions behave, the
kernel templates compile for sm_100a with NVRTC, and anything that needs the
device fails loudly instead of falling back."""
import ctypes
import glob
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "gpuarray", "*.h")):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"GPUARRAY_PUBLIC\s+[^;(]*?\b(\w+)\s*\(", text):
            if not m.group(1).startswith("__"):
                names.add(m.group(1))
    return names


def test_every_declared_symbol_is_exported(api):
    L = api.lib()
    names = declared_symbols()
    assert len(names) > 100
    missing = [n for n in sorted(names) if not hasattr(L, n)]
    assert not missing, missing


def test_struct_layout_is_the_reference_abi(api):
    """GpuArray: data, dimensions, strides, offset (8 bytes each), nd, flags,
    typecode (4 bytes each) - reference src/gpuarray/array.h:21-101."""
    S = api._GpuArrayStruct
    assert [S.data.offset, S.dimensions.offset, S.strides.offset, S.offset.offset, S.nd.offset,
            S.flags.offset, S.typecode.offset] == [0, 8, 16, 24, 32, 36, 40]
    assert ctypes.sizeof(S) == 48
    assert ctypes.sizeof(api._ElemwiseArg) == 16


def test_constants(api):
    assert (api.GE_SCALAR, api.GE_READ, api.GE_WRITE) == (1, 2, 4)
    assert (api.GE_BROADCAST, api.GE_NOCOLLAPSE, api.GE_PADSHAPE) == (0x100, 0x200, 0x400)
    assert (api.GA_FLOAT, api.GA_DOUBLE, api.GA_HALF, api.GA_SIZE, api.GA_SSIZE) == (11, 12, 23, 24, 25)
    L = api.lib()
    sizes = {api.GA_BOOL: 1, api.GA_BYTE: 1, api.GA_UBYTE: 1, api.GA_SHORT: 2, api.GA_USHORT: 2,
             api.GA_INT: 4, api.GA_UINT: 4, api.GA_LONG: 8, api.GA_ULONG: 8, api.GA_FLOAT: 4,
             api.GA_DOUBLE: 8, api.GA_HALF: 2, api.GA_SIZE: 8, api.GA_SSIZE: 8, 14: 8, 15: 16,
             9: 16, 256: 2, 17: 0, 600: 0}
    for tc, sz in sizes.items():
        assert L.gpuarray_get_elsize(tc) == sz, tc
    assert L.gpuarray_error_str(0) == b"No error"
    assert L.gpuarray_error_str(2) == b"Value invalid or out of range"
    assert L.gpuarray_error_str(99) == b"Unknown GA error"


def test_type_flags(api):
    """Known answers of the reference's tests/check_util.c:24-39."""
    L = api.lib()
    f = L.gpuarray_type_flags
    f.restype = ctypes.c_int
    USE_SMALL, USE_DOUBLE, USE_COMPLEX, USE_HALF = 0x02, 0x04, 0x08, 0x10
    i = ctypes.c_int
    assert f(i(-1)) == 0
    assert f(i(api.GA_FLOAT), i(-1)) == 0
    assert f(i(api.GA_DOUBLE), i(-1)) == USE_DOUBLE
    assert f(i(14), i(-1)) == USE_COMPLEX
    assert f(i(15), i(-1)) == USE_DOUBLE | USE_COMPLEX
    assert f(i(api.GA_HALF), i(-1)) == USE_HALF | USE_SMALL
    assert f(i(api.GA_BYTE), i(-1)) == USE_SMALL
    assert f(i(api.GA_SHORT), i(api.GA_DOUBLE), i(-1)) == USE_SMALL | USE_DOUBLE


def test_no_device_means_loud_failure(api):
    """Without a CUDA driver a context cannot be made and the error says why;
    nothing falls back to the CPU."""
    try:
        import torch
        if torch.cuda.is_available():
            pytest.skip("a GPU is present")
    except ImportError:
        pass
    with pytest.raises(api.GpuArrayException) as ei:
        api.Context(0)
    assert ei.value.code in (api.GA_LOAD_ERROR, api.GA_NODEV_ERROR, api.GA_IMPL_ERROR)
    # refused backends
    L = api.lib()
    p = ctypes.c_void_p()
    assert L.gpucontext_init(ctypes.byref(p), b"opencl0:0", None) == api.GA_UNSUPPORTED_ERROR


def _compile(api, src):
    L = api.lib()
    sz = ctypes.c_size_t()
    log = ctypes.c_char_p()
    cache = os.path.join(ROOT, ".kernel_cache").encode()
    err = L.gpuarray_b200_compile_check(src, None, cache, ctypes.byref(sz), ctypes.byref(log))
    return err, sz.value, (log.value or b"").decode(errors="replace")


ELEMWISE_VARIANTS = [
    # expr, args, flags, kind, ept, unroll, nd, idx32, modes
    ("out = a * b + 0.5f", [("a", 11, 2), ("b", 11, 2), ("out", 11, 4)], 0, 0, 4, 4, 0, 1, 0),
    ("out = a * b + 0.5f", [("a", 11, 2), ("b", 11, 2), ("out", 11, 4)], 0, 0, 1, 4, 0, 0, 0),
    ("y = fmaxf(x + bias, 0.0f)", [("x", 23, 2), ("bias", 23, 2), ("y", 23, 4)], 2, 1, 8, 1, 3, 1, 0b010010),
    ("y = a * x + y", [("a", 11, 3), ("x", 2, 2), ("y", 12, 6)], 0, 1, 8, 1, 2, 0, 0),
    ("y = fmaxf(x + bias, 0.0f)", [("x", 23, 2), ("bias", 23, 2), ("y", 23, 4)], 2, 2, 8, 1, 3, 1, 0),
]


@pytest.mark.parametrize("case", ELEMWISE_VARIANTS)
def test_elementwise_templates_compile_for_sm100a(api, case):
    expr, args, flags, kind, ept, unroll, nd, idx32, modes = case
    L = api.lib()
    L.gpuarray_b200_elemwise_source.restype = ctypes.c_void_p
    A = (api._ElemwiseArg * len(args))(*[api._ElemwiseArg(n.encode(), t, f) for n, t, f in args])
    p = L.gpuarray_b200_elemwise_source(b"", expr.encode(), len(args), A, flags, kind, ept, unroll,
                                        nd, idx32, ctypes.c_ulonglong(modes), 64, 64)
    src = ctypes.string_at(p)
    assert src.startswith(b'#include "cluda.h"')
    err, size, log = _compile(api, src)
    assert err == 0 and size > 0, log


@pytest.mark.parametrize("op", range(14))
@pytest.mark.parametrize("shape", [0, 1, 2])
def test_reduction_templates_compile_for_sm100a(api, op, shape):
    L = api.lib()
    L.gpuarray_b200_reduction_source.restype = ctypes.c_void_p
    src_tc = api.GA_INT if op in (9, 10, 11) else api.GA_FLOAT
    dst_tc = api.GA_BOOL if op in (12, 13) else src_tc
    vec, tpo, group = {0: (4, 1, 32), 1: (4, 1, 0), 2: (1, 32, 0)}[shape]
    p = L.gpuarray_b200_reduction_source(op, src_tc, dst_tc, shape, vec, 0, tpo, group)
    err, size, log = _compile(api, ctypes.string_at(p))
    assert err == 0 and size > 0, log


ROWS_VARIANTS = [
    # (op, src typecode name, dst typecode name, vec, group | runs-at-once << 16 | one-run << 20 | flat << 21)
    ("SUM", "GA_FLOAT", "GA_FLOAT", 4, 8 | 4 << 16 | 1 << 20),        # 8 lanes per output, 4 outputs at once
    ("MAXANDARGMAX", "GA_FLOAT", "GA_FLOAT", 4, 1 | 4 << 16 | 1 << 20),  # one lane per output
    ("ARGMIN", "GA_HALF", "GA_HALF", 8, 32 | 2 << 16 | 1 << 20),
    ("SUM", "GA_DOUBLE", "GA_DOUBLE", 2, 32 | 4 << 16),                # a warp on 4 runs of its output at once
    ("MINANDARGMIN", "GA_INT", "GA_INT", 4, 32 | 2 << 16),
    ("SUM", "GA_FLOAT", "GA_FLOAT", 4, 32 | 1 << 21),                  # flattened (run, vector) space
    ("PROD", "GA_FLOAT", "GA_FLOAT", 4, 256),                          # a CTA per (output, split)
]


@pytest.mark.parametrize("op,src,dst,vec,group", ROWS_VARIANTS)
def test_row_reduction_variants_compile_for_sm100a(api, op, src, dst, vec, group):
    L = api.lib()
    L.gpuarray_b200_reduction_source.restype = ctypes.c_void_p
    p = L.gpuarray_b200_reduction_source(getattr(api, "GA_REDUCE_" + op), getattr(api, src),
                                         getattr(api, dst), 0, vec, 0, 1, group)
    text = ctypes.string_at(p)
    assert b"ga_reduce.cuh" in text
    err, size, log = _compile(api, text)
    assert err == 0 and size > 0, log


@pytest.mark.parametrize("fast8,op,src,dst", [(1, "SUM", "GA_BYTE", "GA_LONG"), (2, "SUM", "GA_UBYTE", "GA_UINT"),
                                              (3, "ANY", "GA_BOOL", "GA_BOOL"), (4, "ALL", "GA_UBYTE", "GA_BOOL")])
def test_byte_folding_variants_compile_for_sm100a(api, fast8, op, src, dst):
    """1-byte sums / all / any that fold whole 32-bit words: the host adds
    GA_RD_FAST8 to the variant; here it is put in front of the generated source."""
    L = api.lib()
    L.gpuarray_b200_reduction_source.restype = ctypes.c_void_p
    p = L.gpuarray_b200_reduction_source(getattr(api, "GA_REDUCE_" + op), getattr(api, src),
                                         getattr(api, dst), 0, 16, 0, 1, 32)
    text = ctypes.string_at(p).replace(b"#define GA_RD_FAST8 0", b"#define GA_RD_FAST8 %d" % fast8)
    assert (b"#define GA_RD_FAST8 %d" % fast8) in text
    err, size, log = _compile(api, text)
    assert err == 0 and size > 0, log


def test_bad_expression_reports_compiler_log(api):
    src = b'#include "cluda.h"\nKERNEL void k(GLOBAL_MEM ga_float *a) { a[0] = undefined_name; }\n'
    err, size, log = _compile(api, src)
    assert err == api.GA_IMPL_ERROR
    assert "undefined_name" in log and "0002\t" in log


def test_user_kernel_vocabulary_compiles(api):
    """A kernel in the style pygpu writes (CLUDA macros, atomics, ga_half)."""
    src = b"""#include "cluda.h"
WITHIN_KERNEL ga_float twice(ga_float x) { return 2 * x; }
KERNEL void k(GLOBAL_MEM ga_float *a, GLOBAL_MEM ga_half *h, GLOBAL_MEM ga_long *c, ga_size n) {
  LOCAL_MEM ga_float tmp[32];
  ga_size i = GID_0 * LDIM_0 + LID_0;
  if (i < n) {
    tmp[LID_0 % 32] = twice(a[i]) + ga_half2float(h[i]);
    local_barrier();
    a[i] = tmp[0] + (ga_float)M_PI + INFINITY;
    h[i] = ga_float2half(a[i]);
    atom_add_lg(c, 1);
    atom_add_fg(a, 1.0f);
    atom_add_eg(h, h[i]);
  }
}
"""
    err, size, log = _compile(api, src)
    assert err == 0, log
