"""GpuReduction_call_sharded on ONE GPU (comm = NULL: the whole device path but
the two all-reduces): a source that is a slab of a larger array along a
reduced axis. Checked against the CPU oracle on the whole array: the indices
written are flat indices of the WHOLE reduced extent, ties go to the lowest
global index, the NaN-first rule applies only to the slab holding element 0
(src/gpuarray_reduction.c:557-606 for the rule; the reference's collectives,
src/gpuarray_collectives_cuda_nccl.c:158-185, have no pair operator, which is why the
combination is built from max/min all-reduces). The two-rank run of the same
entry point over NCCL is in test_multigpu.py; the protocol itself also runs
over gloo on CPU (test_sharding_cpu.py)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def combine(parts, is_min):
    """Host stand-in for the two all-reduces: better value, then lower index."""
    v = parts[0][0].copy()
    i = parts[0][1].copy()
    for pv, pi in parts[1:]:
        better = (pv < v) if is_min else (pv > v)
        better |= (pv == v) & (pi < i)
        better &= ~np.isnan(v)                       # a NaN only comes from the first slab and stays
        v = np.where(better, pv, v)
        i = np.where(better, pi, i)
    return v, i


@pytest.mark.parametrize("dtype", [np.float64, np.float32, np.int32])
@pytest.mark.parametrize("axes,shard_axis", [([0, 2], 0), ([2, 0], 0), ([0], 0), ([1, 0], 1)])
def test_slabs_give_global_indices_and_first_occurrence(api, ctx, oracle, rng, dtype, axes, shard_axis):
    x = np.round(rng.standard_normal((64, 48, 256)) * 4) / 4
    if np.dtype(dtype).kind == "f":
        x[0, 5, 0] = np.nan                          # first reduced element of output 5 (axes 0,2)
        x[32, 7, 0] = np.nan                         # first element of the second slab only
        x[:, 9, :] = -1.0
        x[40, 9, 3] = -0.0
        x[41, 9, 0] = 0.0
    x = x.astype(dtype)
    n = x.shape[shard_axis]
    for name, is_min in (("MAXANDARGMAX", False), ("MINANDARGMIN", True)):
        gr = api.GpuReduction(ctx, getattr(api, "GA_REDUCE_" + name), dtype)
        kept = [d for k, d in enumerate(x.shape) if k not in axes]
        parts = []
        for lo, hi in ((0, n // 2), (n // 2, n)):
            sl = [slice(None)] * 3
            sl[shard_axis] = slice(lo, hi)
            g = api.GpuArray.from_numpy(ctx, np.ascontiguousarray(x[tuple(sl)]))
            gv = api.GpuArray.empty(ctx, kept, dtype)
            gi = api.GpuArray.empty(ctx, kept, np.int64)
            api.reduction_call_sharded(gr, None, gv, gi, g, axes, lo, n, shard_axis=shard_axis)
            parts.append((gv.to_numpy(), gi.to_numpy()))
        v, i = combine(parts, is_min)
        wv, wi = oracle.minmaxarg(x, axes, is_min=is_min)
        assert (i == wi).all(), (name, axes)
        nan = np.isnan(wv) if np.dtype(dtype).kind == "f" else np.zeros(wv.shape, bool)
        assert (np.isnan(v) == nan).all() if nan.any() else True
        assert v[~nan].tobytes() == wv[~nan].tobytes(), (name, axes)
        # the whole array as one shard is the plain call, bit for bit
        g = api.GpuArray.from_numpy(ctx, x)
        gv = api.GpuArray.empty(ctx, kept, dtype)
        gi = api.GpuArray.empty(ctx, kept, np.int64)
        api.reduction_call_sharded(gr, None, gv, gi, g, axes, 0, n, shard_axis=shard_axis)
        pv = api.GpuArray.empty(ctx, kept, dtype)
        pi = api.GpuArray.empty(ctx, kept, np.int64)
        gr(pv, pi, g, axes)
        assert (gi.to_numpy() == pi.to_numpy()).all()
        a, b = gv.to_numpy(), pv.to_numpy()
        same_nan = np.isnan(a) == np.isnan(b) if np.dtype(dtype).kind == "f" else True
        ok = ~np.isnan(b) if np.dtype(dtype).kind == "f" else np.ones(b.shape, bool)
        assert np.all(same_nan) and a[ok].tobytes() == b[ok].tobytes()
        gr.free()


def test_value_only_and_index_only_operators(api, ctx, oracle, rng):
    x = (np.round(rng.standard_normal((40, 300)) * 2) / 2).astype(np.float32)
    g = api.GpuArray.from_numpy(ctx, np.ascontiguousarray(x[20:]))
    wv, wi = oracle.minmaxarg(x[20:], [0])
    gr = api.GpuReduction(ctx, api.GA_REDUCE_MAX, np.float32)
    gv = api.GpuArray.empty(ctx, (300,), np.float32)
    api.reduction_call_sharded(gr, None, gv, None, g, [0], 20, 40)
    assert gv.to_numpy().tobytes() == wv.tobytes()
    gr = api.GpuReduction(ctx, api.GA_REDUCE_ARGMAX, np.float32)
    wide = api.GpuArray.from_numpy(ctx, np.full(600, -5, np.int64))
    api.reduction_call_sharded(gr, None, None, wide[::2], g, [0], 20, 40)      # strided index destination
    w = wide.to_numpy()
    assert (w[::2] == wi + 20).all() and (w[1::2] == -5).all()


def test_indices_beyond_32_bits_come_from_the_shard_offset(api, ctx, rng):
    x = rng.integers(0, 100, (64, 50)).astype(np.int32)
    x[17, :] = 1000                                   # unique maximum in local row 17
    g = api.GpuArray.from_numpy(ctx, x)
    gr = api.GpuReduction(ctx, api.GA_REDUCE_ARGMAX, np.int32)
    gi = api.GpuArray.empty(ctx, (50,), np.uint64)
    lo, glob = (1 << 33) - 64, 1 << 33
    api.reduction_call_sharded(gr, None, None, gi, g, [0], lo, glob)
    assert (gi.to_numpy() == lo + 17).all()
    # last listed axis fastest: with axes (1, 0) the sharded axis 0 is the fast one
    y = rng.integers(0, 100, (64, 50, 3)).astype(np.int32)
    y[5, 7, :] = 1000
    gy = api.GpuArray.from_numpy(ctx, y)
    gj = api.GpuArray.empty(ctx, (3,), np.uint64)
    api.reduction_call_sharded(gr, None, None, gj, gy, [1, 0], lo, glob, shard_axis=0)
    assert (gj.to_numpy() == 7 * glob + lo + 5).all()


def test_accumulating_operators_and_errors(api, ctx, rng):
    x = rng.standard_normal((30, 20, 10))
    g = api.GpuArray.from_numpy(ctx, x)
    gr = api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float64)
    wide = api.GpuArray.from_numpy(ctx, np.zeros((20, 20)))
    api.reduction_call_sharded(gr, None, wide[:, ::2], None, g, [0], 0, 60)     # strided destination
    assert np.allclose(wide.to_numpy()[:, ::2], x.sum(0)) and (wide.to_numpy()[:, 1::2] == 0).all()
    out = api.GpuArray.empty(ctx, (20, 10), np.float64)
    with pytest.raises(api.GpuArrayException) as e:
        api.reduction_call_sharded(gr, None, out, None, g, [0], 0, 60, shard_axis=1)   # axis 1 is kept
    assert e.value.code == api.GA_VALUE_ERROR
    with pytest.raises(api.GpuArrayException) as e:
        api.reduction_call_sharded(gr, None, out, None, g, [0], 40, 60)             # slab sticks out
    assert e.value.code == api.GA_VALUE_ERROR
    b = api.GpuArray.from_numpy(ctx, rng.integers(0, 255, (30, 20)).astype(np.uint8))
    gx = api.GpuReduction(ctx, api.GA_REDUCE_XOR, np.uint8)
    with pytest.raises(api.GpuArrayException) as e:
        api.reduction_call_sharded(gx, None, api.GpuArray.empty(ctx, (20,), np.uint8), None, b, [0], 0, 60)
    assert e.value.code == api.GA_UNSUPPORTED_ERROR
    ga = api.GpuReduction(ctx, api.GA_REDUCE_ANY, np.uint8)
    o = api.GpuArray.empty(ctx, (20,), np.bool_)
    api.reduction_call_sharded(ga, None, o, None, b, [0], 30, 60)
    assert (o.to_numpy() == b.to_numpy().any(0)).all()
