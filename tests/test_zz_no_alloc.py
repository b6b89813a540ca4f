"""The allocation-free float32 sum (gpuarray_b200_sum_f32_noalloc).

Some callers cannot allocate device memory at the point where they need a
reduction (they live inside another framework's memory pool, or must not block
on the driver's allocator). For them the library carries its scratch inside
its own image. This test calls that entry point through the C ABI twice in a
row - the scratch block is shared and keeps the previous call's contents - and
compares each result with the regular GpuReduction path on the same data,
within the float32 sum tolerance used everywhere else in this suite
(1e-6 * log2(n) relative to sum |x_i|). The file sorts last so that a failure
here cannot hide any other test of an -x run.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def regular_sum(api, ctx, g):
    d = api.GpuArray.empty(ctx, (), np.float32)
    api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float32)(d, None, g, [0])
    return float(d.to_numpy())


def noalloc_sum(api, ctx, g, out):
    err = api.lib().gpuarray_b200_sum_f32_noalloc(ctypes.c_void_p(g.devptr), g.size,
                                                  ctypes.c_void_p(out.devptr),
                                                  ctypes.c_void_p(ctx.stream))
    assert err == 0, api.lib().gpucontext_error(None, err)
    return float(out.to_numpy())


def test_noalloc_sum_matches_regular_path_twice(api, ctx, rng):
    out = api.GpuArray.empty(ctx, (), np.float32)
    for n in (3_000_001, 1 << 22):                   # two calls in a row, shared scratch
        x = rng.standard_normal(n).astype(np.float32)
        g = api.GpuArray.from_numpy(ctx, x)
        out.memset(0xFF)
        got = noalloc_sum(api, ctx, g, out)
        ref = regular_sum(api, ctx, g)
        scale = float(np.abs(x.astype(np.float64)).sum())
        tol = 1e-6 * np.log2(n) * scale
        assert abs(got - ref) <= tol, (n, got, ref)
        assert abs(got - float(x.astype(np.float64).sum())) <= tol
    # small inputs and the empty sum
    x = np.arange(1, 11, dtype=np.float32)
    g = api.GpuArray.from_numpy(ctx, x)
    assert noalloc_sum(api, ctx, g, out) == 55.0
    err = api.lib().gpuarray_b200_sum_f32_noalloc(None, 0, ctypes.c_void_p(out.devptr),
                                                  ctypes.c_void_p(ctx.stream))
    assert err == 0 and float(out.to_numpy()) == 0.0


def test_noalloc_sum_rejects_what_it_cannot_do(api, ctx):
    out = api.GpuArray.empty(ctx, (), np.float32)
    g = api.GpuArray.from_numpy(ctx, np.zeros(64, np.float32))
    L = api.lib()
    too_many = (1 << 32) + 1
    err = L.gpuarray_b200_sum_f32_noalloc(ctypes.c_void_p(g.devptr), too_many,
                                          ctypes.c_void_p(out.devptr), ctypes.c_void_p(ctx.stream))
    assert err == api.GA_XLARGE_ERROR
    assert b"exceed the maximum" in L.gpucontext_error(None, err)
    err = L.gpuarray_b200_sum_f32_noalloc(ctypes.c_void_p(g.devptr + 4), 8,
                                          ctypes.c_void_p(out.devptr), ctypes.c_void_p(ctx.stream))
    assert err == api.GA_UNALIGNED_ERROR
    # a host pointer (or memory of another device) is refused before anything is queued
    host = np.zeros(72, np.float32)
    addr = (host.ctypes.data + 15) & ~15
    err = L.gpuarray_b200_sum_f32_noalloc(ctypes.c_void_p(addr), 8, ctypes.c_void_p(out.devptr),
                                          ctypes.c_void_p(ctx.stream))
    assert err == api.GA_VALUE_ERROR and b"device memory" in L.gpucontext_error(None, err)
