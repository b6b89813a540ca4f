"""GpuArray entry points around the hot path (views, copies, gather): the
callers' side of the engine. Views are pure host bookkeeping; every typed or
strided copy below runs the elementwise engine ("dst = src"), as the
reference's ga_extcopy does (src/gpuarray_array.c:42-86)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_views_match_numpy(api, ctx, rng):
    x = rng.standard_normal((6, 7, 8)).astype(np.float32)
    g = api.GpuArray.from_numpy(ctx, x)
    assert (g[1:5, ::-2, 3].to_numpy() == x[1:5, ::-2, 3]).all()
    assert (g.transpose((2, 0, 1)).to_numpy() == x.transpose(2, 0, 1)).all()
    assert (g.transpose().to_numpy() == x.T).all()
    assert (g.reshape((42, 8)).to_numpy() == x.reshape(42, 8)).all()
    r = g.reshape((6, 56), nocopy=True)
    assert r.ga.data == g.ga.data                      # a view, not a copy
    t = g.transpose((1, 0, 2))
    with pytest.raises(api.GpuArrayException) as ei:
        t.reshape((42, 8), nocopy=True)
    assert ei.value.code == api.GA_COPY_ERROR
    assert (t.reshape((42, 8)).to_numpy() == x.transpose(1, 0, 2).reshape(42, 8)).all()
    f = api.GpuArray.from_numpy(ctx, x, order="F")
    assert f.flags & api.GA_F_CONTIGUOUS and not (f.flags & api.GA_C_CONTIGUOUS)
    assert (f.to_numpy() == x).all()
    assert (f.copy("C").to_numpy() == x).all()


def test_setarray_broadcasts(api, ctx, rng):
    a = api.GpuArray.from_numpy(ctx, np.zeros((4, 5, 6), np.float32))
    v = rng.standard_normal((5, 1)).astype(np.float32)
    gv = api.GpuArray.from_numpy(ctx, v)
    api._check(ctx.ptr, api.lib().GpuArray_setarray(ctypes.byref(a.ga), ctypes.byref(gv.ga)))
    assert (a.to_numpy() == np.broadcast_to(v, (4, 5, 6))).all()


def test_split_and_concatenate(api, ctx, rng):
    L = api.lib()
    x = rng.integers(0, 100, (7, 9)).astype(np.int32)
    g = api.GpuArray.from_numpy(ctx, x)
    parts = [api.GpuArray(ctx) for _ in range(3)]
    ptrs = (ctypes.POINTER(api._GpuArrayStruct) * 3)(*[ctypes.pointer(p.ga) for p in parts])
    cuts = (ctypes.c_size_t * 2)(2, 5)
    L.GpuArray_split.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                 ctypes.c_uint]
    api._check(ctx.ptr, L.GpuArray_split(ptrs, ctypes.byref(g.ga), 2, cuts, 1))
    for p in parts:
        p._live = True
    assert [p.shape for p in parts] == [(7, 2), (7, 3), (7, 4)]
    assert (parts[1].to_numpy() == x[:, 2:5]).all()
    out = api.GpuArray(ctx)
    L.GpuArray_concatenate.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                       ctypes.c_uint, ctypes.c_int]
    order = (ctypes.POINTER(api._GpuArrayStruct) * 3)(ctypes.pointer(parts[2].ga),
                                                      ctypes.pointer(parts[0].ga),
                                                      ctypes.pointer(parts[1].ga))
    api._check(ctx.ptr, L.GpuArray_concatenate(ctypes.byref(out.ga), order, 3, 1, api.GA_LONG))
    out._live = True
    want = np.concatenate([x[:, 5:], x[:, :2], x[:, 2:5]], axis=1).astype(np.int64)
    assert out.dtype == np.int64 and (out.to_numpy() == want).all()


def test_take1_gathers_rows(api, ctx, rng):
    L = api.lib()
    L.GpuArray_take1.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int]
    v = rng.standard_normal((11, 4, 5)).astype(np.float32)
    gv = api.GpuArray.from_numpy(ctx, v).transpose((0, 2, 1))      # strided source
    idx = np.array([3, -1, 0, 10, 3, -11], dtype=np.int64)
    gi = api.GpuArray.from_numpy(ctx, idx)
    out = api.GpuArray.empty(ctx, (6, 5, 4), np.float32)
    api._check(ctx.ptr, L.GpuArray_take1(ctypes.byref(out.ga), ctypes.byref(gv.ga),
                                         ctypes.byref(gi.ga), 1))
    assert (out.to_numpy() == v.transpose(0, 2, 1)[idx]).all()
    bad = api.GpuArray.from_numpy(ctx, np.array([0, 11, 1, 2, 3, 4], dtype=np.int64))
    err = L.GpuArray_take1(ctypes.byref(out.ga), ctypes.byref(gv.ga), ctypes.byref(bad.ga), 1)
    assert err == api.GA_VALUE_ERROR
    # the error word was handed back at zero: the next checked call succeeds
    api._check(ctx.ptr, L.GpuArray_take1(ctypes.byref(out.ga), ctypes.byref(gv.ga),
                                         ctypes.byref(gi.ga), 1))


def test_user_kernel_through_gpukernel(api, ctx, rng):
    """GpuKernel_init / _sched / _call with a caller-written kernel, as pygpu.GpuKernel does."""
    L = api.lib()

    class GpuKernel(ctypes.Structure):
        _fields_ = [("k", ctypes.c_void_p), ("args", ctypes.c_void_p)]
    src = (b'#include "cluda.h"\nKERNEL void axpy(GLOBAL_MEM ga_float *y, GLOBAL_MEM const ga_float *x, '
           b'ga_float a, ga_size n) {\n  for (ga_size i = GID_0 * LDIM_0 + LID_0; i < n; i += LDIM_0 * GDIM_0) '
           b'y[i] += a * x[i];\n}\n')
    k = GpuKernel()
    strs = (ctypes.c_char_p * 1)(src)
    types = (ctypes.c_int * 4)(api.GA_BUFFER, api.GA_BUFFER, api.GA_FLOAT, api.GA_SIZE)
    L.GpuKernel_init.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p,
                                 ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint, ctypes.c_void_p,
                                 ctypes.c_int, ctypes.c_void_p]
    api._check(ctx.ptr, L.GpuKernel_init(ctypes.byref(k), ctx.ptr, 1, strs, None, b"axpy", 4, types,
                                         0, None))
    n = 100003
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    gx, gy = api.GpuArray.from_numpy(ctx, x), api.GpuArray.from_numpy(ctx, y)
    a = ctypes.c_float(2.5)
    cn = ctypes.c_size_t(n)
    L.GpuKernel_setarg.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p]
    for i, p in enumerate((gy.ga.data, gx.ga.data, ctypes.addressof(a), ctypes.addressof(cn))):
        api._check(ctx.ptr, L.GpuKernel_setarg(ctypes.byref(k), i, p))
    gs, ls = ctypes.c_size_t(0), ctypes.c_size_t(0)
    L.GpuKernel_sched.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
    api._check(ctx.ptr, L.GpuKernel_sched(ctypes.byref(k), n, ctypes.byref(gs), ctypes.byref(ls)))
    assert ls.value % 32 == 0 and 0 < ls.value <= 512 and gs.value >= 1
    L.GpuKernel_call.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p,
                                 ctypes.c_size_t, ctypes.c_void_p]
    api._check(ctx.ptr, L.GpuKernel_call(ctypes.byref(k), 1, ctypes.byref(gs), ctypes.byref(ls), 0,
                                         None))
    # y += a*x is one fused multiply-add: round(y + 2.5*x) computed exactly in fp64
    want = (y.astype(np.float64) + 2.5 * x.astype(np.float64)).astype(np.float32)
    assert (gy.to_numpy() == want).all()
    L.GpuKernel_clear(ctypes.byref(k))


def test_arrays_that_reach_outside_their_buffer_are_refused_on_the_host(api, ctx):
    """A GpuArray whose extents and strides lead past its buffer (hand-built
    with GpuArray_fromdata, here through from_pointer with too small a size)
    is a host error, not a device access."""
    real = api.GpuArray.from_numpy(ctx, np.arange(4096, dtype=np.float32))
    out = api.GpuArray.empty(ctx, (4096,), np.float32)
    short = api.GpuArray.from_pointer(ctx, real.devptr, (4096,), np.float32, nbytes=4096 * 4 - 4)
    ge = api.GpuElemwise(ctx, "o = a + 1.0f", [("a", np.float32, api.GE_READ), ("o", np.float32, api.GE_WRITE)],
                         nd=1)
    with pytest.raises(api.GpuArrayException) as ei:
        ge(short, out)
    assert ei.value.code == api.GA_VALUE_ERROR and "outside its buffer" in str(ei.value)
    with pytest.raises(api.GpuArrayException) as ei:
        ge(real, short)                              # as the output
    assert ei.value.code == api.GA_VALUE_ERROR
    tot = api.GpuArray.empty(ctx, (), np.float32)
    rs = api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float32)
    with pytest.raises(api.GpuArrayException) as ei:
        rs(tot, None, short, [0])
    assert ei.value.code == api.GA_VALUE_ERROR and "outside its buffer" in str(ei.value)
    # a negative stride that starts at the buffer's first element walks below it
    back = api.GpuArray.from_pointer(ctx, real.devptr, (16,), np.float32, strides=[-4], nbytes=64)
    with pytest.raises(api.GpuArrayException):
        rs(tot, None, back, [0])
    # the same views with honest sizes work
    ok = api.GpuArray.from_pointer(ctx, real.devptr + 15 * 4, (16,), np.float32, strides=[-4])
    rs(tot, None, ok, [0])
    assert float(tot.to_numpy()) == float(np.arange(16, dtype=np.float32).sum())
    ge(real, out)
    assert (out.to_numpy() == np.arange(4096, dtype=np.float32) + 1).all()


def test_fresh_expression_compiles_into_an_empty_cache(api, tmp_path):
    """NVRTC JIT on the GPU box itself: a context whose cubin directory is empty builds a new
    expression (and a reduction variant), runs it, and leaves the cubins behind; a second
    context on the same directory loads them without compiling."""
    import os
    cache = tmp_path / "cubins"
    cache.mkdir()
    R, W = api.GE_READ, api.GE_WRITE
    x = np.arange(1000, dtype=np.float32)
    for attempt in range(2):
        c = api.Context(0, kernel_cache=str(cache))
        ge = api.GpuElemwise(c, "o = a * 3.25f + 41.0f", [("a", np.float32, R), ("o", np.float32, W)], nd=1)
        ga = api.GpuArray.from_numpy(c, x)
        go = api.GpuArray.empty(c, x.shape, np.float32)
        ge(ga, go)
        assert (go.to_numpy() == x * np.float32(3.25) + np.float32(41.0)).all()
        d = api.GpuArray.empty(c, (), np.float32)
        api.GpuReduction(c, api.GA_REDUCE_MAX, np.float32)(d, None, ga, [0])
        assert float(d.to_numpy()) == 999.0
        names = sorted(os.listdir(cache))
        assert len(names) >= 2 and all(n.endswith(".cubin") for n in names)
        if attempt == 0:
            first = names
        else:
            assert names == first                      # nothing new was compiled
        ge.free()
        c.close()


def test_operator_construction_on_a_module_cache_hit_is_cheap(api, ctx):
    """pygpu builds a new GpuElemwise for every Python operator it evaluates
    (pygpu/elemwise.py:35,76,94); after the first one the kernel is found in the context's
    module cache. Budget: 50 us per GpuElemwise_new + GpuElemwise_free pair (measured on the
    B200 box through a C caller: 4.1 us; through ctypes a little more)."""
    import ctypes
    import time
    L = api.lib()
    args = (api._ElemwiseArg * 3)()
    for i, (nm, fl) in enumerate(((b"a", api.GE_READ), (b"b", api.GE_READ), (b"o", api.GE_WRITE))):
        args[i].name, args[i].typecode, args[i].flags = nm, api.GA_FLOAT, fl
    p = L.GpuElemwise_new(ctx.ptr, b"", b"o = a * b + 7.5f", 3, args, 1, 0)
    assert p
    L.GpuElemwise_free(ctypes.c_void_p(p))
    best = 1e9
    for _ in range(5):
        t0 = time.perf_counter()
        for _ in range(200):
            q = L.GpuElemwise_new(ctx.ptr, b"", b"o = a * b + 7.5f", 3, args, 1, 0)
            L.GpuElemwise_free(ctypes.c_void_p(q))
        best = min(best, (time.perf_counter() - t0) / 200)
    assert best < 50e-6, best
