"""GPU parity tests of the reduction engine through the C ABI.

Part 1 restates the reference's tests/check_reduction.c (:70-431): PCG(seed 1)
data, GpuArray_maxandargmax, destinations pre-filled with 0xFF, exact equality
on value and index. Part 2 sweeps operators x dtypes x axis sets x layouts
against the CPU oracle: bit-exact for integer / bool / index / min / max
results, and for floating sums and products within
    |got - ref| <= eps * log2(n) * sum|x_i|     (eps = 1e-6 fp32, 1e-12 fp64)
with ref computed in higher precision; fp16 results within 2 ulp of the
correctly rounded value after fp32 accumulation.
"""
import itertools

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PAIR_OPS = {"minandargmin", "maxandargmax", "argmin", "argmax", "min", "max"}


def opcode(api, name):
    return getattr(api, "GA_REDUCE_" + name.upper())


def run_maxandargmax(api, ctx, x, axes):
    g = api.GpuArray.from_numpy(ctx, x)
    free = [x.shape[i] for i in range(x.ndim) if i not in axes]
    gmax = api.GpuArray.empty(ctx, free, x.dtype)
    garg = api.GpuArray.empty(ctx, free, np.uint64)
    gmax.memset(0xFF)
    garg.memset(0xFF)
    api.maxandargmax(gmax, garg, g, axes)
    return gmax.to_numpy(), garg.to_numpy()


# ------------------------------------------------- part 1: check_reduction.c

def test_reduction(api, ctx, oracle):
    dims = (32, 50, 79)
    x = oracle.pcg_fill_f32(1, int(np.prod(dims))).reshape(dims)
    vmax, amax = run_maxandargmax(api, ctx, x, [0, 2])
    for j in range(dims[1]):
        plane = x[:, j, :]
        k = int(plane.reshape(-1).argmax())          # i*dims[2] + k, first occurrence
        assert vmax[j] == plane.reshape(-1)[k] and amax[j] == k


def test_idxtranspose(api, ctx, oracle):
    dims = (32, 50, 79)
    x = oracle.pcg_fill_f32(1, int(np.prod(dims))).reshape(dims)
    vmax, amax = run_maxandargmax(api, ctx, x, [2, 0])
    for j in range(dims[1]):
        plane = x[:, j, :].T                          # k major, i minor: index k*dims[0] + i
        k = int(plane.reshape(-1).argmax())
        assert vmax[j] == plane.reshape(-1)[k] and amax[j] == k


def test_veryhighrank(api, ctx, oracle):
    dims = (1171, 373, 2, 1, 2, 1, 2, 1)
    x = oracle.pcg_fill_f32(1, int(np.prod(dims))).reshape(dims)
    vmax, amax = run_maxandargmax(api, ctx, x, [2, 4, 7, 5])
    assert vmax.shape == (1171, 373, 1, 2)
    want_v, want_i = oracle.minmaxarg(x, [2, 4, 7, 5])
    assert (vmax == want_v).all() and (amax.astype(np.int64) == want_i).all()
    # and an independent NumPy statement: reduced axes in list order, last fastest
    xt = x.transpose(0, 1, 3, 6, 2, 4, 7, 5).reshape(1171, 373, 1, 2, -1)
    assert (vmax == xt.max(-1)).all() and (amax == xt.argmax(-1)).all()


def test_alldimsreduced(api, ctx, oracle):
    dims = (32, 50, 79)
    x = oracle.pcg_fill_f32(1, int(np.prod(dims))).reshape(dims)
    vmax, amax = run_maxandargmax(api, ctx, x, [0, 1, 2])
    assert vmax.shape == () and amax.shape == ()
    assert vmax == x.max() and amax == x.reshape(-1).argmax()


def test_maxandargmax_argument_errors(api, ctx):
    x = api.GpuArray.from_numpy(ctx, np.zeros((4, 5), np.float32))
    v = api.GpuArray.empty(ctx, (4,), np.float32)
    i = api.GpuArray.empty(ctx, (4,), np.uint64)
    for axes in ([], [2], [1, 1], [0, 1, 0]):
        with pytest.raises(api.GpuArrayException) as ei:
            api.maxandargmax(v, i, x, axes)
        assert ei.value.code == api.GA_INVALID_ERROR
    bad = api.GpuArray.empty(ctx, (5,), np.float32)
    with pytest.raises(api.GpuArrayException) as ei:
        api.maxandargmax(bad, i, x, [1])
    assert ei.value.code == api.GA_VALUE_ERROR


# --------------------------------------------------- part 2: operator sweeps

def make_data(rng, dt, shape, ties=True):
    dt = np.dtype(dt)
    if dt.kind == "f":
        x = rng.standard_normal(shape)
        if ties:
            x = np.round(x * 4) / 4
        return x.astype(dt)
    if dt.kind == "b":
        return rng.random(shape) < 0.7
    hi = 5 if ties else 100
    lo = -hi if dt.kind == "i" else 0
    return rng.integers(lo, hi, shape).astype(dt)


def check_reduce(api, ctx, oracle, name, x, axes, out_dtype=None, layout="C"):
    """Runs one reduction on the device and checks it against the oracle."""
    op = opcode(api, name)
    if layout == "C":
        g = api.GpuArray.from_numpy(ctx, x)
    elif layout == "F":
        g = api.GpuArray.from_numpy(ctx, x, order="F")
    else:                                   # a strided window of a larger buffer
        big = np.zeros(tuple(2 * s + 1 for s in x.shape), x.dtype)
        sl = tuple(slice(1, 1 + 2 * s, 2) for s in x.shape)
        big[sl] = x
        g = api.GpuArray.from_numpy(ctx, big)[sl]
    free = [x.shape[i] for i in range(x.ndim) if i not in axes]
    gr = api.GpuReduction(ctx, op, x.dtype)
    n = max(1, int(np.prod([x.shape[a] for a in axes])))
    if name in PAIR_OPS:
        is_min = "min" in name
        want_v, want_i = oracle.minmaxarg(x, axes, is_min=is_min)
        d0 = api.GpuArray.empty(ctx, free, x.dtype) if name not in ("argmin", "argmax") else None
        d1 = api.GpuArray.empty(ctx, free, np.int64) if name not in ("min", "max") else None
        gr(d0, d1, g, axes)
        if d0 is not None:
            got = d0.to_numpy()
            assert got.tobytes() == want_v.tobytes(), (name, axes, layout)
        if d1 is not None:
            assert (d1.to_numpy() == want_i).all(), (name, axes, layout)
        return
    out_dtype = np.dtype(out_dtype or x.dtype)
    d0 = api.GpuArray.empty(ctx, free, out_dtype)
    gr(d0, None, g, axes)
    got = d0.to_numpy()
    want = oracle.reduce_reference(name, x, axes, out_dtype)
    if out_dtype.kind != "f":
        assert (got == want.astype(out_dtype)).all(), (name, axes, layout)
        return
    if name == "sum":
        scale = np.abs(x.astype(np.float64)).sum(axis=tuple(axes))
    else:
        scale = np.abs(want.astype(np.float64))
    if out_dtype == np.float16:
        # fp32 accumulation, then one rounding: within 2 half ulps of the exact value
        ref16 = want.astype(np.float64)
        ulp = np.maximum(np.abs(ref16), 2.0 ** -14) * 2.0 ** -10
        slack = 1e-6 * np.log2(max(n, 2)) * scale
        assert (np.abs(got.astype(np.float64) - ref16) <= 2 * ulp + slack).all(), (name, axes)
        return
    eps = 1e-6 if out_dtype == np.float32 else 1e-12
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bound = eps * np.log2(max(n, 2)) * np.maximum(scale, np.finfo(np.float64).tiny)
    assert (err <= bound).all(), (name, axes, layout, float(err.max()), float(bound.min()))


AXES_3D = [(0,), (1,), (2,), (0, 1), (0, 2), (1, 2), (2, 0), (0, 1, 2), (2, 1, 0)]


@pytest.mark.parametrize("axes", AXES_3D)
@pytest.mark.parametrize("name", ["sum", "maxandargmax", "minandargmin"])
@pytest.mark.parametrize("layout", ["C", "F", "window"])
def test_small_3d_all_axis_sets(api, ctx, oracle, rng, axes, name, layout):
    x = make_data(rng, np.float32, (5, 4, 7))
    check_reduce(api, ctx, oracle, name, x, list(axes), layout=layout)


@pytest.mark.parametrize("dt", [np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64,
                                np.uint64, np.float32, np.float64, np.float16, np.bool_])
@pytest.mark.parametrize("name", ["max", "min", "argmax", "argmin", "maxandargmax", "minandargmin"])
def test_minmax_family_every_dtype(api, ctx, oracle, rng, dt, name):
    x = make_data(rng, dt, (6, 300))
    check_reduce(api, ctx, oracle, name, x, [1])
    check_reduce(api, ctx, oracle, name, x, [0])


@pytest.mark.parametrize("dt,odt", [(np.float32, np.float32), (np.float64, np.float64),
                                    (np.float16, np.float16), (np.float16, np.float32),
                                    (np.int8, np.int64), (np.uint8, np.uint64), (np.int32, np.int32),
                                    (np.int64, np.int64), (np.float32, np.float64)])
@pytest.mark.parametrize("name", ["sum", "prod", "prodnz"])
def test_sum_prod_dtypes(api, ctx, oracle, rng, dt, odt, name):
    x = make_data(rng, dt, (7, 40), ties=True)
    if name != "sum" and np.dtype(dt).kind == "f":
        x = (1 + x / 64).astype(dt)             # keep products in range
    if name != "sum" and np.dtype(dt).kind != "f":
        x = (x % 3).astype(dt)                  # zeros, ones and twos
    for axes in ([1], [0], [0, 1]):
        check_reduce(api, ctx, oracle, name, x, axes, out_dtype=odt)


@pytest.mark.parametrize("dt", [np.int8, np.uint16, np.int32, np.uint64, np.bool_])
@pytest.mark.parametrize("name", ["and", "or", "xor"])
def test_bitwise(api, ctx, oracle, rng, dt, name):
    x = rng.integers(0, 2 if dt is np.bool_ else 127, (9, 33)).astype(dt)
    for axes in ([1], [0], [0, 1]):
        check_reduce(api, ctx, oracle, name, x, axes)


@pytest.mark.parametrize("dt", [np.float32, np.float16, np.int32, np.uint8, np.bool_, np.float64])
@pytest.mark.parametrize("name", ["all", "any"])
def test_all_any(api, ctx, oracle, rng, dt, name):
    x = make_data(rng, dt, (11, 70))
    x[3] = 0
    x[5] = 1
    for axes in ([1], [0], [0, 1]):
        check_reduce(api, ctx, oracle, name, x, axes, out_dtype=np.bool_)


@pytest.mark.parametrize("shape,axes", [((5, 70000), [1]), ((300017,), [0]), ((1000, 64), [1]),
                                        ((40, 3, 4096), [0, 2]), ((64, 48), [1]), ((2, 1 << 20), [1])])
def test_one_byte_elements_fold_by_words(api, ctx, oracle, rng, shape, axes):
    """Contiguous runs of 1-byte elements are summed / tested a 32-bit word at a
    time; every byte position and the byte values that stress the word tricks
    (0x00, 0x01, 0x7f, 0x80, 0xff) must give the per-element answers."""
    special = np.array([0, 1, 0x7f, 0x80, 0xff], np.uint8)
    u = special[rng.integers(0, 5, shape)]
    check_reduce(api, ctx, oracle, "sum", u, axes, out_dtype=np.uint64)
    check_reduce(api, ctx, oracle, "sum", u, axes, out_dtype=np.int32)
    check_reduce(api, ctx, oracle, "sum", u.view(np.int8), axes, out_dtype=np.int64)
    b = rng.random(shape) < 0.5
    check_reduce(api, ctx, oracle, "sum", b, axes, out_dtype=np.int64)
    # all / any: mostly-nonzero and mostly-zero data with single exceptions at
    # every byte position of a word
    for base, exc in ((0x80, 0), (0xff, 0), (1, 0), (0, 1), (0, 0x80)):
        x = np.full(shape, base, np.uint8)
        flat = x.reshape(-1)
        for pos in range(0, min(flat.size, 4096), 4):
            if (pos // 4) % 9 == 0:
                flat[pos + (pos // 36) % 4] = exc
        flat[-1 - (flat.size // 3) % 4] = exc
        for name in ("all", "any"):
            check_reduce(api, ctx, oracle, name, x, axes, out_dtype=np.bool_)
            check_reduce(api, ctx, oracle, name, x.view(np.int8), axes, out_dtype=np.bool_)
    for name in ("all", "any"):
        check_reduce(api, ctx, oracle, name, b, axes, out_dtype=np.bool_)
        check_reduce(api, ctx, oracle, name, np.ones(shape, np.bool_), axes, out_dtype=np.bool_)
        check_reduce(api, ctx, oracle, name, np.zeros(shape, np.bool_), axes, out_dtype=np.bool_)


def test_high_rank_windows_that_do_not_collapse(api, ctx, oracle, rng):
    """Seven dimensions, step-2 windows on every axis: up to 5 kept and 4
    reduced dimensions survive collapsing."""
    shape = (3, 2, 4, 2, 3, 2, 5)
    x = make_data(rng, np.float32, shape)
    for axes in ([1, 3, 5], [0, 2, 4, 6], [6], [0], [5, 1], [2, 3, 4, 5, 6]):
        for name in ("sum", "maxandargmax"):
            check_reduce(api, ctx, oracle, name, x, axes, layout="window")
            check_reduce(api, ctx, oracle, name, x, axes, layout="F")


def test_bitwise_on_floats_is_refused(api, ctx):
    with pytest.raises(api.GpuArrayException) as ei:
        api.GpuReduction(ctx, api.GA_REDUCE_XOR, np.float32)
    assert ei.value.code == api.GA_UNSUPPORTED_ERROR


SHAPES_KERNEL_PATHS = [
    # rows kernel: long contiguous reduced run, with and without vector alignment
    ((3, 5000), [1]), ((3, 4099), [1]), ((2, 3, 2048), [2]), ((4, 2, 1500), [1, 2]),
    # rows kernel split over several CTAs per output (few outputs, long rows)
    ((1, 200000), [1]), ((2, 40, 3000), [1, 2]), ((300000,), [0]),
    # cols kernel: contiguous kept run, two passes
    ((3000, 64), [0]), ((500, 3, 40), [0]), ((700, 130), [0]), ((64, 2, 48), [0, 1]),
    # kept axis in the middle: reduce (0, 2)
    ((40, 6, 1024), [0, 2]), ((9, 5, 70), [0, 2]), ((9, 5, 70), [2, 0]),
    # general kernel
    ((10, 11, 12), [1]), ((3, 4, 5, 6), [1, 3]), ((3, 4, 5, 6), [3, 1]), ((2, 2, 2, 2, 2, 3), [0, 2, 4]),
]


@pytest.mark.parametrize("shape,axes", SHAPES_KERNEL_PATHS)
@pytest.mark.parametrize("name", ["sum", "maxandargmax", "minandargmin", "any"])
def test_kernel_paths(api, ctx, oracle, rng, shape, axes, name):
    dt = np.float32
    x = make_data(rng, dt, shape)
    check_reduce(api, ctx, oracle, name, x, axes,
                 out_dtype=np.bool_ if name == "any" else None)


SHAPES_SHORT_RUNS = [
    # one short contiguous run per output: part of a warp per output, several outputs at once
    ((1000, 2), [1]), ((999, 3), [1]), ((777, 4), [1]), ((1500, 8), [1]), ((700, 16), [1]),
    ((1201, 32), [1]), ((33, 49), [1]), ((260, 64), [1]), ((300, 100), [1]), ((130, 256), [1]),
    ((67, 511), [1]), ((70, 512), [1]), ((35, 1000), [1]), ((40, 1024), [1]), ((5, 7, 48), [2]),
    ((6, 5, 7, 7), [2, 3]), ((1, 20), [1]), ((9000, 12), [1]),
    # several short runs per output: a warp loads from a few runs at once
    ((50, 6, 256), [0, 2]), ((41, 5, 100), [0, 2]), ((23, 4, 64), [2, 0]), ((37, 3, 20), [0, 2]),
    ((64, 9, 7, 7), [0, 2, 3]), ((19, 2, 600), [0, 2]), ((300, 2, 8), [0, 2]),
]


# float32 on every shape; the other element sizes (2, 8 and 1 bytes: other vector
# widths and group sizes) on every third shape, which keeps the number of kernels
# the suite has to compile in check
SHORT_RUN_CASES = [(sh, ax, np.float32) for sh, ax in SHAPES_SHORT_RUNS] + \
                  [(sh, ax, dt) for i, (sh, ax) in enumerate(SHAPES_SHORT_RUNS)
                   for dt in (np.float16, np.float64, np.int8) if i % 3 == 0]


@pytest.mark.parametrize("shape,axes,dt", SHORT_RUN_CASES)
def test_short_contiguous_runs(api, ctx, oracle, rng, shape, axes, dt):
    x = make_data(rng, dt, shape)
    sum_out = np.int64 if dt == np.int8 else None
    check_reduce(api, ctx, oracle, "sum", x, axes, out_dtype=sum_out)
    check_reduce(api, ctx, oracle, "maxandargmax", x, axes)
    check_reduce(api, ctx, oracle, "argmin", x, axes)
    if len(shape) == 2:
        # rows that do not start on a 16-byte boundary, and a padded row pitch
        check_reduce(api, ctx, oracle, "sum", x, axes, out_dtype=sum_out, layout="window")
        check_reduce(api, ctx, oracle, "maxandargmax", x, axes, layout="window")
        wide = np.zeros((shape[0], shape[1] + 8), np.dtype(dt))
        wide[:, :shape[1]] = x
        g = api.GpuArray.from_numpy(ctx, wide)[:, :shape[1]]
        d0 = api.GpuArray.empty(ctx, (shape[0],), np.dtype(dt))
        d1 = api.GpuArray.empty(ctx, (shape[0],), np.int64)
        api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.dtype(dt))(d0, d1, g, [1])
        want_v, want_i = oracle.minmaxarg(x, [1])
        assert d0.to_numpy().tobytes() == want_v.tobytes() and (d1.to_numpy() == want_i).all()


def test_short_runs_nan_first_and_ties(api, ctx, oracle):
    x = np.full((500, 24), 1.5, np.float32)
    x[7, 0] = np.nan          # NaN as first element is kept, elsewhere it never wins
    x[8, 5] = np.nan
    x[9, 23] = 3.0
    x[10, :] = -0.0
    x[10, 3] = 0.0
    for name in ("maxandargmax", "minandargmin"):
        check_reduce(api, ctx, oracle, name, x, [1])


@pytest.mark.parametrize("dt,cols", [(np.float32, 4), (np.float32, 8), (np.float32, 16), (np.float32, 32),
                                     (np.float64, 2), (np.float64, 8), (np.float16, 8), (np.float16, 64),
                                     (np.int32, 16), (np.int16, 32)])
def test_tiny_runs_walked_as_one_array_of_vectors(api, ctx, oracle, rng, dt, cols):
    """Rows of 1, 2, 4 or 8 full vectors lying back to back (GA_RD_TINY): every operator kind,
    row counts whose vectors end inside a warp, the NaN-first rule from the writing lane's own
    vector, the first zero's sign in the values-only MIN / MAX, strided destinations, and a
    shard (global indices, no NaN-first rule)."""
    for rows in (100, 1030, 7, 4097):
        x = (np.round(rng.standard_normal((rows, cols)) * 2) / 2).astype(dt)
        if np.dtype(dt).kind == "f":
            x[0, 0] = np.nan
            x[1, cols - 1] = np.nan
            x[2, :] = -np.inf
            x[3, :] = -1
            x[3, cols // 2] = -0.0
            x[3, cols - 1] = 0.0
            x[4, :] = 1
            x[4, 0] = 0.0
            x[4, cols - 1] = -0.0
            x[5, :] = np.nan
        g = api.GpuArray.from_numpy(ctx, x)
        for name in ("max", "min", "argmax", "argmin", "maxandargmax", "minandargmin"):
            want_v, want_i = oracle.minmaxarg(x, [1], is_min="min" in name)
            d0 = api.GpuArray.empty(ctx, (rows,), x.dtype) if name not in ("argmin", "argmax") else None
            d1 = api.GpuArray.empty(ctx, (rows,), np.int64) if name not in ("min", "max") else None
            api.GpuReduction(ctx, opcode(api, name), x.dtype)(d0, d1, g, [1])
            if d0 is not None:
                got = d0.to_numpy()
                nan = np.isnan(want_v) if x.dtype.kind == "f" else np.zeros(rows, bool)
                # a float16 NaN comes back as a NaN, not necessarily with the same payload
                assert (np.isnan(got) == nan).all() if x.dtype.kind == "f" else True
                assert got[~nan].tobytes() == want_v[~nan].tobytes(), (name, rows)
                if x.dtype != np.float16:
                    assert got.tobytes() == want_v.tobytes(), (name, rows)
            if d1 is not None:
                assert (d1.to_numpy() == want_i).all(), (name, rows)
        clean = (np.round(rng.standard_normal((rows, cols)) * 2) / 2).astype(dt)
        check_reduce(api, ctx, oracle, "sum", clean, [1])
    # destinations with strides, and the same rows as the second shard of a longer axis
    rows = 333
    x = (np.round(rng.standard_normal((rows, cols)) * 2) / 2).astype(dt)
    if np.dtype(dt).kind == "f":
        x[0, 0] = np.nan                                   # not the first element of the WHOLE extent
    g = api.GpuArray.from_numpy(ctx, x)
    wide_v = api.GpuArray.from_numpy(ctx, np.full((rows, 3), 9, np.dtype(dt)))
    wide_i = api.GpuArray.from_numpy(ctx, np.full((rows, 2), -9, np.int64))
    gr = api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.dtype(dt))
    gr(wide_v[:, 1], wide_i[:, 0], g, [1])
    wv, wi = oracle.minmaxarg(x, [1])
    got_v, got_i = wide_v.to_numpy(), wide_i.to_numpy()
    keep = ~np.isnan(wv) if np.dtype(dt).kind == "f" else np.ones(rows, bool)
    assert got_v[keep, 1].tobytes() == wv[keep].tobytes() and (got_i[:, 0] == wi).all()
    assert np.dtype(dt).kind != "f" or np.isnan(got_v[~keep, 1]).all()
    assert (got_v[:, 0] == 9).all() and (got_v[:, 2] == 9).all() and (got_i[:, 1] == -9).all()
    full = np.concatenate([np.ones((rows, cols), np.dtype(dt)) * 0 - 5, x], axis=1)      # the shard is the tail
    dv = api.GpuArray.empty(ctx, (rows,), np.dtype(dt))
    di = api.GpuArray.empty(ctx, (rows,), np.int64)
    api.reduction_call_sharded(gr, None, dv, di, g, [1], cols, 2 * cols)
    sv, si = oracle.minmaxarg(full[:, cols:], [1])
    nan_rows = np.isnan(x[:, 0]) if np.dtype(dt).kind == "f" else np.zeros(rows, bool)
    ok = ~nan_rows                                         # a leading NaN of a later shard never wins
    assert (di.to_numpy()[ok] == si[ok] + cols).all() and dv.to_numpy()[ok].tobytes() == sv[ok].tobytes()


@pytest.mark.parametrize("shape,axes", [((5, 4100), [1]), ((2100, 36), [0]), ((30, 7, 600), [0, 2])])
def test_kernel_paths_fp64_and_fp16(api, ctx, oracle, rng, shape, axes):
    for dt in (np.float64, np.float16):
        x = make_data(rng, dt, shape)
        for name in ("sum", "maxandargmax", "min"):
            check_reduce(api, ctx, oracle, name, x, axes)


def test_ties_take_first_occurrence_across_ctas(api, ctx, oracle, rng):
    """Every element equal: the first index must win whatever thread, warp or
    CTA saw the other copies."""
    for shape, axes in (((2, 300000), [1]), ((5000, 8), [0]), ((60, 3, 2000), [0, 2]),
                        ((60, 3, 2000), [2, 0])):
        x = np.full(shape, 2.5, np.float32)
        check_reduce(api, ctx, oracle, "maxandargmax", x, axes)
        check_reduce(api, ctx, oracle, "minandargmin", x, axes)
        x[..., -1] = 7
        check_reduce(api, ctx, oracle, "maxandargmax", x, axes)


def test_nan_and_signed_zero_rules(api, ctx, oracle):
    nan = np.float32("nan")
    rows = np.array([[1, nan, 3, nan] + [0] * 996,
                     [nan, 5, 7, 1] + [0] * 996,
                     [-0.0, 0.0, -0.0, 0.0] + [-1] * 996,
                     [0.0, -0.0, 0.0, -0.0] + [-1] * 996,
                     [-np.inf] * 1000,
                     [nan] * 1000], dtype=np.float32)
    for axes, x in (([1], rows), ([0], np.ascontiguousarray(rows.T))):
        check_reduce(api, ctx, oracle, "maxandargmax", x, axes)
        check_reduce(api, ctx, oracle, "minandargmin", -x, axes)
        check_reduce(api, ctx, oracle, "max", x, axes)
    g = api.GpuArray.from_numpy(ctx, rows)
    v = api.GpuArray.empty(ctx, (6,), np.float32)
    i = api.GpuArray.empty(ctx, (6,), np.int64)
    api.maxandargmax(v, i, g, [1])
    got_v, got_i = v.to_numpy(), i.to_numpy()
    assert got_v[0] == 3 and got_i[0] == 2
    assert np.isnan(got_v[1]) and got_i[1] == 0
    assert got_i[2] == 0 and np.signbit(got_v[2])
    assert got_i[3] == 0 and not np.signbit(got_v[3])
    assert got_i[4] == 0 and got_v[4] == -np.inf
    assert np.isnan(got_v[5]) and got_i[5] == 0


def test_long_runs_scan_values_then_recover_the_index(api, ctx, oracle, rng):
    """Over long contiguous runs the arg-reductions scan values only and find the
    element afterwards; the corner cases of that recovery, per row of 6000:"""
    n = 6000
    nan, inf = np.float32("nan"), np.float32("inf")
    rows = []
    r = np.full(n, -inf, np.float32); rows.append(r)                       # identity everywhere
    r = np.full(n, -inf, np.float32); r[:8] = nan; rows.append(r)          # NaNs first, identity after
    r = np.full(n, nan, np.float32); r[4097] = -inf; rows.append(r)        # one identity among NaNs
    r = np.full(n, nan, np.float32); r[0] = -inf; r[5] = 2; rows.append(r)
    r = np.full(n, nan, np.float32); rows.append(r)                        # NaN first: kept
    r = np.full(n, -1, np.float32); r[130] = -0.0; r[131] = 0.0; r[4000] = 0.0; rows.append(r)
    r = np.full(n, -1, np.float32); r[131] = 0.0; r[132] = -0.0; r[77] = -0.0; rows.append(r)
    r = np.full(n, 3, np.float32); rows.append(r)                          # all equal
    r = np.full(n, 3, np.float32); r[-1] = 4; rows.append(r)               # winner in the ragged end
    r = np.full(n, 3, np.float32); r[127] = 9; r[128] = 9; r[5000] = 9; rows.append(r)  # ties across lanes
    r = rng.standard_normal(n).astype(np.float32); r[3001] = inf; r[3000] = nan; rows.append(r)
    x = np.stack(rows)
    for name, data in (("maxandargmax", x), ("minandargmin", -x), ("argmax", x), ("max", x), ("min", -x)):
        check_reduce(api, ctx, oracle, name, data, [1])
        check_reduce(api, ctx, oracle, name, data, [1], layout="window")   # scalar loads
    check_reduce(api, ctx, oracle, "maxandargmax", x.astype(np.float64), [1])
    # float16 goes through float32 and back, which does not keep a NaN's payload bits:
    # rows without NaN only
    check_reduce(api, ctx, oracle, "minandargmin", (-x[[0, 5, 6, 7, 8, 9]]).astype(np.float16), [1])
    # whole-array reductions: runs cut into segments, CTA groups, tickets
    big = np.full(3_000_000, -inf, np.float32)
    check_reduce(api, ctx, oracle, "maxandargmax", big, [0])
    big[2_000_001] = nan
    big[1_999_999] = 5
    big[2_500_000] = 5
    check_reduce(api, ctx, oracle, "maxandargmax", big, [0])
    check_reduce(api, ctx, oracle, "minandargmin", -big, [0])
    for dt in (np.int32, np.int8, np.uint16, np.int64):
        info = np.iinfo(dt)
        xi = np.full((7, n), info.min, dt)
        xi[1, 4321] = info.min + 1
        xi[2, :] = info.max
        xi[3, 17] = info.max
        xi[3, 5017] = info.max
        xi[4] = rng.integers(info.min, info.max, n, dtype=dt)
        xi[5, -3:] = info.max
        xi[6, 0] = info.max
        check_reduce(api, ctx, oracle, "maxandargmax", xi, [1])
        check_reduce(api, ctx, oracle, "minandargmin", xi, [1])
    # several long runs per output, listed in an order that differs from memory order
    y = np.round(rng.standard_normal((12, 3, 2048)) * 2).astype(np.float32)
    check_reduce(api, ctx, oracle, "maxandargmax", y, [0, 2])
    check_reduce(api, ctx, oracle, "maxandargmax", y, [2, 0])
    check_reduce(api, ctx, oracle, "minandargmin", y, [2, 0])


@pytest.mark.parametrize("shape,axes", [((50, 2000), [1]),        # a warp per long run
                                        ((50, 24), [1]),          # part of a warp per short run
                                        ((50, 300), [1]),
                                        ((6, 50, 40), [0, 2]),    # several short runs per output
                                        ((900, 50), [0])])        # column kernel
def test_destination_strides_and_offsets_are_honoured(api, ctx, oracle, rng, shape, axes):
    x = make_data(rng, np.float32, shape)
    g = api.GpuArray.from_numpy(ctx, x)
    vbuf = api.GpuArray.from_numpy(ctx, np.full(200, -7, np.float32))
    ibuf = api.GpuArray.from_numpy(ctx, np.full(200, -7, np.int64))
    v, i = vbuf[150:0:-3], ibuf[3:103:2]        # 50 elements each, odd strides
    assert v.shape == (50,) and i.shape == (50,)
    api.maxandargmax(v, i, g, axes)
    want_v, want_i = oracle.minmaxarg(x, axes)
    hv, hi = vbuf.to_numpy(), ibuf.to_numpy()
    assert (hv[150:0:-3] == want_v).all() and (hi[3:103:2] == want_i).all()
    mask = np.ones(200, bool)
    mask[150:0:-3] = False
    assert (hv[mask] == -7).all()                # nothing else was written


def test_empty_reductions(api, ctx):
    g = api.GpuArray.empty(ctx, (4, 0), np.float32)
    d = api.GpuArray.empty(ctx, (4,), np.float32)
    d.memset(0xFF)
    api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float32)(d, None, g, [1])
    assert (d.to_numpy() == 0).all()
    api.GpuReduction(ctx, api.GA_REDUCE_PROD, np.float32)(d, None, g, [1])
    assert (d.to_numpy() == 1).all()
    with pytest.raises(api.GpuArrayException) as ei:
        api.GpuReduction(ctx, api.GA_REDUCE_MAX, np.float32)(d, None, g, [1])
    assert ei.value.code == api.GA_VALUE_ERROR
    d0 = api.GpuArray.empty(ctx, (0,), np.float32)
    api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float32)(d0, None, g, [0])   # no outputs: no-op


def test_wrong_destination_is_rejected(api, ctx):
    g = api.GpuArray.from_numpy(ctx, np.zeros((4, 5), np.float32))
    gr = api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.float32)
    v = api.GpuArray.empty(ctx, (4,), np.float32)
    for bad_i in (api.GpuArray.empty(ctx, (4,), np.int32), api.GpuArray.empty(ctx, (5,), np.int64)):
        with pytest.raises(api.GpuArrayException) as ei:
            gr(v, bad_i, g, [1])
        assert ei.value.code == api.GA_VALUE_ERROR
    i = api.GpuArray.empty(ctx, (4,), np.int64)
    with pytest.raises(api.GpuArrayException):
        gr(api.GpuArray.empty(ctx, (4,), np.float64), i, g, [1])   # value type must match


def test_run_to_run_determinism(api, ctx, rng):
    """Two-pass reductions combine partials in a fixed order: bitwise repeatable."""
    x = rng.standard_normal((3, 700000)).astype(np.float32)
    g = api.GpuArray.from_numpy(ctx, x)
    gr = api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float32)
    outs = []
    for _ in range(3):
        d = api.GpuArray.empty(ctx, (3,), np.float32)
        gr(d, None, g, [1])
        outs.append(d.to_numpy().tobytes())
    assert outs[0] == outs[1] == outs[2]
