"""Extents beyond 32-bit indexing (the 64-bit index builds of the kernels):
a reduction over more than 2^32 elements and an elementwise call over more
than 2^31 elements, on 1-byte types so that a few GiB suffice. Device memory
is filled on the device; only a few bytes cross the bus."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def put(arr, pos, values):
    """Write `values` at arr[pos:pos+len] through a slice view."""
    v = np.asarray(values, dtype=arr.dtype)
    arr[pos:pos + v.size].write(v)


def test_reduction_over_more_than_2_32_elements(api, ctx):
    n = (1 << 32) + 4096 + 40                       # ragged past the last full vector
    x = api.GpuArray.empty(ctx, (n,), np.int8)
    x.memset(0)
    first = (1 << 32) + 77                          # beyond 32 bits
    put(x, first, [5])
    put(x, first + 1000, [5])                       # a later tie must lose
    put(x, 123456789, [-3])
    put(x, n - 1, [4])
    idx = api.GpuArray.empty(ctx, (), np.int64)
    val = api.GpuArray.empty(ctx, (), np.int8)
    api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.int8)(val, idx, x, [0])
    assert int(val.to_numpy()) == 5 and int(idx.to_numpy()) == first
    api.GpuReduction(ctx, api.GA_REDUCE_ARGMIN, np.int8)(None, idx, x, [0])
    assert int(idx.to_numpy()) == 123456789
    tot = api.GpuArray.empty(ctx, (), np.int64)
    api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.int8)(tot, None, x, [0])
    assert int(tot.to_numpy()) == 5 + 5 - 3 + 4
    anyv = api.GpuArray.empty(ctx, (), np.bool_)
    api.GpuReduction(ctx, api.GA_REDUCE_ANY, np.int8)(anyv, None, x, [0])
    assert bool(anyv.to_numpy())
    # two rows of 2^31 + 20: outputs whose reduced extent alone needs no 64 bits, the array does
    m = (1 << 31) + 20
    y = x[:2 * m].reshape((2, m))
    put(x, m + 9, [7])                              # row 1, column 9
    put(x, m - 1, [6])                              # row 0, last column
    v2 = api.GpuArray.empty(ctx, (2,), np.int8)
    i2 = api.GpuArray.empty(ctx, (2,), np.int64)
    api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.int8)(v2, i2, y, [1])
    assert v2.to_numpy().tolist() == [6, 7] and i2.to_numpy().tolist() == [m - 1, 9]


def test_elementwise_over_more_than_2_31_elements(api, ctx):
    n = (1 << 31) + 4096 + 13
    a = api.GpuArray.empty(ctx, (n,), np.uint8)
    o = api.GpuArray.empty(ctx, (n,), np.uint8)
    a.memset(3)
    o.memset(0)
    put(a, n - 5, [10, 20, 30, 40, 50])
    put(a, (1 << 31) + 1, [100])
    ge = api.GpuElemwise(ctx, "o = a + 1", [("a", np.uint8, api.GE_READ), ("o", np.uint8, api.GE_WRITE)], nd=1)
    ge(a, o)
    assert o[n - 5:].to_numpy().tolist() == [11, 21, 31, 41, 51]
    assert o[(1 << 31) - 2:(1 << 31) + 4].to_numpy().tolist() == [4, 4, 4, 101, 4, 4]
    assert o[:8].to_numpy().tolist() == [4] * 8
    # the strided kernel with 64-bit indices: every other element of the same buffers
    a2, o2 = a[::2], o[::2]
    o.memset(0)
    ge(a2, o2)
    tail = o[n - 5:].to_numpy().tolist()
    want = [11, 21, 31, 41, 51]
    first_even = (n - 5) % 2
    assert tail == [w if (i % 2) == first_even else 0 for i, w in enumerate(want)]
