"""GPU parity tests of GpuMapReduction_* through the C ABI: reductions of a
mapped expression over several broadcastable arguments, what the reference
offers as pygpu's ReductionKernel (pygpu/reduction.py:137-291, tested there
by pygpu/tests/test_reduction.py:57-84 against NumPy with allclose).

Oracle: NumPy on the same inputs with the map evaluated in float64; sums
within |got - ref| <= eps * log2(n) * sum|map_i| (eps 1e-6 fp32, 1e-12 fp64),
integer and max/min results exact."""
import itertools

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def device_view(api, ctx, a):
    """A device array with the layout of NumPy array `a` (any strides): the
    underlying buffer is copied whole, the view is rebuilt on top of it."""
    base = a
    while base.base is not None and isinstance(base.base, np.ndarray):
        base = base.base
    if base is a or not (base.flags.c_contiguous or base.flags.f_contiguous):
        return api.GpuArray.from_numpy(ctx, a), None
    g = api.GpuArray.from_numpy(ctx, base)
    off = a.__array_interface__["data"][0] - base.__array_interface__["data"][0]
    v = api.GpuArray.from_pointer(ctx, g.devptr + off, a.shape, a.dtype, strides=a.strides)
    return v, g


def run(api, ctx, map_expr, reduce_expr, neutral, out_dtype, named, axes, scalars=(), broadcast=True,
        out=None, convert_f16=False):
    spec = [(n, a.dtype, api.GE_READ) for n, a in named] + \
           [(n, np.asarray(v).dtype, api.GE_SCALAR) for n, v in scalars]
    mr = api.GpuMapReduction(ctx, map_expr, reduce_expr, neutral, out_dtype, spec,
                             convert_f16=convert_f16)
    dev = [device_view(api, ctx, a) for _, a in named]
    shape = np.broadcast_shapes(*[a.shape for _, a in named])
    kept = tuple(d for i, d in enumerate(shape) if i not in axes)
    if out is None:
        out = api.GpuArray.empty(ctx, kept, out_dtype)
        out.memset(0x55)
    mr(out, *([d[0] for d in dev] + [v for _, v in scalars]), axes=axes, broadcast=broadcast)
    res = out.to_numpy()
    mr.free()
    return res


def close_sum(got, terms, axes, dtype):
    want = terms.sum(axis=tuple(axes))
    n = max(2, int(np.prod([terms.shape[i] for i in axes])))
    eps = 1e-6 if np.dtype(dtype) == np.float32 else 1e-12
    scale = np.abs(terms).sum(axis=tuple(axes))
    return (np.abs(got.astype(np.float64) - want) <= eps * np.log2(n) * np.maximum(scale, 1e-300)).all()


def test_reference_broadcast_case(api, ctx, rng):
    # pygpu/tests/test_reduction.py:57-84
    a = rng.standard_normal((5, 10, 15))
    b = rng.standard_normal((1, 10, 15))
    got = run(api, ctx, "a * b", "a + b", "0", np.float64, [("a", a), ("b", b)], [1])
    assert got.shape == (5, 15) and np.allclose(got, (a * b).sum(1))
    assert close_sum(got, a * b, [1], np.float64)


LAYOUTS = ["C", "F", "strided", "reversed", "row", "col"]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("la,lb", [("C", "C"), ("C", "F"), ("F", "F"), ("C", "strided"),
                                   ("reversed", "C"), ("C", "row"), ("C", "col"), ("col", "row"),
                                   ("strided", "strided")])
def test_dot_like_sums_over_layouts(api, ctx, rng, dtype, la, lb):
    shape = (96, 70, 40)

    def make(layout):
        if layout == "C":
            return rng.standard_normal(shape).astype(dtype)
        if layout == "F":
            return np.asfortranarray(rng.standard_normal(shape).astype(dtype))
        if layout == "strided":
            return rng.standard_normal((96, 70, 80)).astype(dtype)[:, :, ::2]
        if layout == "reversed":
            return rng.standard_normal(shape).astype(dtype)[::-1]
        if layout == "row":
            return rng.standard_normal((1, 70, 40)).astype(dtype)
        return rng.standard_normal((96, 1, 40)).astype(dtype)
    a, b = make(la), make(lb)
    terms = a.astype(np.float64) * b.astype(np.float64)
    for axes in ([0], [1], [2], [0, 1], [1, 2], [0, 2], [0, 1, 2], [2, 0]):
        got = run(api, ctx, "a * b", "a + b", "0", dtype, [("a", a), ("b", b)], axes)
        assert close_sum(got, np.broadcast_to(terms, np.broadcast_shapes(a.shape, b.shape)),
                         axes, dtype), (la, lb, axes)


def test_max_abs_difference_and_scalars(api, ctx, rng):
    a = rng.standard_normal((300, 257)).astype(np.float32)
    b = rng.standard_normal((300, 257)).astype(np.float32)
    for axes in ([0], [1], [0, 1]):
        got = run(api, ctx, "fabsf(a - b)", "fmaxf(a, b)", "0", np.float32, [("a", a), ("b", b)], axes)
        assert (got == np.abs(a - b).max(axis=tuple(axes))).all()
    got = run(api, ctx, "a * s + b", "a + b", "0", np.float64, [("a", a), ("b", b)], [1],
              scalars=[("s", np.float32(0.25))])
    want = (a * np.float32(0.25) + b).astype(np.float64)      # the map is evaluated in float32
    assert np.allclose(got, want.sum(1), rtol=1e-6, atol=1e-5)
    # min with a large neutral element
    got = run(api, ctx, "a + b", "fminf(a, b)", "INFINITY", np.float32, [("a", a), ("b", b)], [0])
    assert (got == (a + b).min(0)).all()


def test_integer_results_are_exact(api, ctx, rng):
    i = rng.integers(-1000, 1000, (64, 3000)).astype(np.int32)
    j = rng.integers(-100, 100, (64, 3000)).astype(np.int16)
    got = run(api, ctx, "(ga_long)a * b", "a + b", "0", np.int64, [("a", i), ("b", j)], [1])
    assert (got == (i.astype(np.int64) * j).sum(1)).all()
    got = run(api, ctx, "(ga_long)a * b", "a + b", "0", np.int64, [("a", i), ("b", j)], [0])
    assert (got == (i.astype(np.int64) * j).sum(0)).all()
    # count of matches: a boolean map summed into uint32
    got = run(api, ctx, "a == b", "a + b", "0", np.uint32,
              [("a", (i % 7).astype(np.int32)), ("b", (j % 7).astype(np.int16))], [0, 1])
    assert int(got) == int(((i % 7) == (j % 7)).sum())


def test_large_contiguous_dot_and_repeatability(api, ctx, rng):
    n = 1 << 24
    a = rng.standard_normal(n).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    spec = [("a", np.float32, api.GE_READ), ("b", np.float32, api.GE_READ)]
    mr = api.GpuMapReduction(ctx, "a * b", "a + b", "0", np.float32, spec)
    ga, gb = api.GpuArray.from_numpy(ctx, a), api.GpuArray.from_numpy(ctx, b)
    out = api.GpuArray.empty(ctx, (), np.float32)
    results = []
    for _ in range(3):
        mr(out, ga, gb, axes=[0])
        results.append(out.to_numpy().tobytes())
    assert results[0] == results[1] == results[2]          # fixed combination order
    terms = a.astype(np.float64) * b
    got = np.frombuffer(results[0], np.float32)[0]
    assert abs(got - terms.sum()) <= 1e-6 * np.log2(n) * np.abs(terms).sum()
    # (4096, 4096): both axes
    x = a.reshape(4096, 4096)
    y = b.reshape(4096, 4096)
    gx, gy = api.GpuArray.from_numpy(ctx, x), api.GpuArray.from_numpy(ctx, y)
    for ax in (0, 1):
        o = api.GpuArray.empty(ctx, (4096,), np.float32)
        mr(o, gx, gy, axes=[ax])
        assert close_sum(o.to_numpy(), terms.reshape(4096, 4096), [ax], np.float32)
    mr.free()


def test_float16_arguments_and_destination_strides(api, ctx, rng):
    h = rng.standard_normal((50, 1000)).astype(np.float16)
    got = run(api, ctx, "a * a", "a + b", "0", np.float32, [("a", h)], [1], convert_f16=True)
    assert np.allclose(got, (h.astype(np.float64) ** 2).sum(1), rtol=1e-5)
    # every second cell of a wider destination; the cells in between stay as they were
    a = rng.standard_normal((40, 300)).astype(np.float32)
    b = rng.standard_normal((40, 300)).astype(np.float32)
    wide = api.GpuArray.from_numpy(ctx, np.full(80, -7, np.float32))
    view = wide[::2]
    run(api, ctx, "a * b", "a + b", "0", np.float32, [("a", a), ("b", b)], [1], out=view)
    w = wide.to_numpy()
    assert (w[1::2] == -7).all() and close_sum(w[::2], a.astype(np.float64) * b, [1], np.float32)


def test_errors(api, ctx, rng):
    spec = [("a", np.float32, api.GE_READ), ("b", np.float32, api.GE_READ)]
    with pytest.raises(api.GpuArrayException) as e:
        api.GpuMapReduction(ctx, "a * undefined_name", "a + b", "0", np.float32, spec)
    assert e.value.code == api.GA_IMPL_ERROR and "undefined_name" in str(e.value)
    mr = api.GpuMapReduction(ctx, "a * b", "a + b", "0", np.float32, spec)
    a = api.GpuArray.from_numpy(ctx, np.ones((3, 4), np.float32))
    b = api.GpuArray.from_numpy(ctx, np.ones((1, 4), np.float32))
    out = api.GpuArray.empty(ctx, (4,), np.float32)
    with pytest.raises(api.GpuArrayException) as e:
        mr(out, a, b, axes=[0], broadcast=False)
    assert e.value.code == api.GA_VALUE_ERROR
    with pytest.raises(api.GpuArrayException) as e:
        mr(api.GpuArray.empty(ctx, (3,), np.float32), a, b, axes=[0])      # wrong destination shape
    assert e.value.code == api.GA_VALUE_ERROR
    with pytest.raises(api.GpuArrayException) as e:
        mr(api.GpuArray.empty(ctx, (4,), np.float64), a, b, axes=[0])      # wrong destination type
    assert e.value.code == api.GA_VALUE_ERROR
    with pytest.raises(api.GpuArrayException) as e:
        mr(out, a, b, axes=[])
    assert e.value.code == api.GA_VALUE_ERROR
    mr(out, a, b, axes=[0])
    assert (out.to_numpy() == 3).all()
    # empty reduced extent: the neutral element
    z = api.GpuArray.empty(ctx, (4, 0), np.float32)
    o4 = api.GpuArray.empty(ctx, (4,), np.float32)
    mr(o4, z, z, axes=[1])
    assert (o4.to_numpy() == 0).all()
    mr.free()
