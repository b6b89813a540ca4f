"""The five benchmark configurations at their FULL sizes, through the C ABI.

Configs 1-4 are checked element for element against the CPU oracle on the
seeded synthetic inputs (np.random.Generator(PCG64(seed)), draws in the order
listed in the docstrings). Config 5 (16 GiB of fp64) is checked through exact,
size-independent properties: the array is built on the device as
a[i] + b[j] + c[k] from three small vectors of dyadic rationals, so every sum,
minimum and maximum has a closed form that is exact in binary floating point.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
R, W = 2, 4


def test_config1_elemwise_fp32_contiguous(api, ctx, oracle):
    """out = a*b + 0.5f, n = 2^24, a, b ~ U[-1,1) from seed 0. Bit-exact against
    the fused multiply-add the reference's NVRTC build produces."""
    rng = np.random.Generator(np.random.PCG64(0))
    n = 1 << 24
    a = 2 * rng.random(n, dtype=np.float32) - 1
    b = 2 * rng.random(n, dtype=np.float32) - 1
    ga, gb = api.GpuArray.from_numpy(ctx, a), api.GpuArray.from_numpy(ctx, b)
    go = api.GpuArray.empty(ctx, (n,), np.float32)
    ge = api.GpuElemwise(ctx, "out = a * b + 0.5f", [("a", np.float32, R), ("b", np.float32, R),
                                                      ("out", np.float32, W)], nd=1)
    ge(ga, gb, go)
    got = go.to_numpy()
    want = oracle.fma_f32(a, b, 0.5)
    assert (got.view(np.uint32) == want.view(np.uint32)).all()
    # against NumPy's unfused expression: error relative to |a*b| + 0.5
    unfused = a * b + np.float32(0.5)
    rel = np.abs(got.astype(np.float64) - unfused) / (np.abs(a.astype(np.float64) * b) + 0.5)
    assert rel.max() <= 1e-6 * np.log2(2)


def test_config2_sum_fp32_4096x4096(api, ctx):
    """SUM over axis 1 and axis 0 of N(0,1) from seed 1; fp32 outputs within
    1e-6 * log2(4096) of the fp64 sum, relative to sum |x_i|."""
    rng = np.random.Generator(np.random.PCG64(1))
    x = rng.standard_normal((4096, 4096), dtype=np.float32)
    g = api.GpuArray.from_numpy(ctx, x)
    gr = api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float32)
    x64 = x.astype(np.float64)
    for axis in (1, 0):
        d = api.GpuArray.empty(ctx, (4096,), np.float32)
        gr(d, None, g, [axis])
        got = d.to_numpy().astype(np.float64)
        err = np.abs(got - x64.sum(axis=axis)) / np.abs(x64).sum(axis=axis)
        assert err.max() <= 1e-6 * np.log2(4096), (axis, err.max())


def test_config3_maxandargmax_logits(api, ctx, oracle):
    """MAXANDARGMAX over the last axis of (16384, 32000) fp32, N(0,1) rounded to
    1/64 from seed 2 (ties in every row); max fp32 + first-occurrence uint64
    index, bit-exact."""
    rng = np.random.Generator(np.random.PCG64(2))
    x = rng.standard_normal((16384, 32000), dtype=np.float32)
    np.multiply(x, 64, out=x)
    np.round(x, out=x)
    np.multiply(x, np.float32(1 / 64), out=x)
    g = api.GpuArray.from_numpy(ctx, x)
    vmax = api.GpuArray.empty(ctx, (16384,), np.float32)
    amax = api.GpuArray.empty(ctx, (16384,), np.uint64)
    api.maxandargmax(vmax, amax, g, [1])
    want_v, want_i = oracle.rowmaxarg_f32(x)
    got_v, got_i = vmax.to_numpy(), amax.to_numpy()
    assert (got_v == want_v).all()
    assert (got_i.astype(np.int64) == want_i).all()
    # ties really occur: the maximum appears more than once in many rows
    ties = (x[:256] == want_v[:256, None]).sum(axis=1)
    assert (ties > 1).any()
    assert (got_i[:256].astype(np.int64) == x[:256].argmax(1)).all()


def test_config4_fp16_bias_relu_nhwc_view(api, ctx):
    """y = max(x + bias, 0): x is the (0,3,1,2) view of an NHWC fp16 buffer
    (64,56,56,256) ~ N(0,1), bias fp16 (1,256,1,1) ~ U[-0.1,0.1), seed 3; fp32
    compute, fp16 NCHW output. One fp32 add and one rounding: bit-exact."""
    rng = np.random.Generator(np.random.PCG64(3))
    buf = rng.standard_normal((64, 56, 56, 256), dtype=np.float32).astype(np.float16)
    bias = (0.2 * rng.random((1, 256, 1, 1), dtype=np.float32) - 0.1).astype(np.float16)
    gbuf = api.GpuArray.from_numpy(ctx, buf)
    gx = gbuf.transpose((0, 3, 1, 2))
    assert gx.shape == (64, 256, 56, 56) and gx.strides == (1605632, 2, 28672, 512)
    gbias = api.GpuArray.from_numpy(ctx, bias)
    gy = api.GpuArray.empty(ctx, (64, 256, 56, 56), np.float16)
    ge = api.GpuElemwise(ctx, "y = fmaxf(x + bias, 0.0f)",
                         [("x", np.float16, R), ("bias", np.float16, R), ("y", np.float16, W)],
                         nd=4, convert_f16=True)
    ge(gx, gbias, gy, flags=api.GE_BROADCAST)
    got = gy.to_numpy()
    want = np.maximum(buf.transpose(0, 3, 1, 2).astype(np.float32) + bias.astype(np.float32),
                      0).astype(np.float16)
    assert (got.view(np.uint16) == want.view(np.uint16)).all()


def test_config5_fp64_16gib_properties(api, ctx):
    """SUM over all axes and MIN / MAX / MAXANDARGMAX over axes (0, 2) of a
    (2048, 1024, 1024) fp64 array (16 GiB, 2^31 elements: 64-bit indexing)."""
    free = ctx.prop_size(10)
    if free < 20 * (1 << 30):
        pytest.skip("needs 20 GiB of free device memory")
    rng = np.random.Generator(np.random.PCG64(4))
    # dyadic rationals with few bits: every partial sum below is exact in fp64
    a = rng.integers(-512, 512, (2048, 1, 1)).astype(np.float64) / 1024
    b = rng.integers(-512, 512, (1, 1024, 1)).astype(np.float64) / 1024
    c = rng.integers(-512, 512, (1, 1, 1024)).astype(np.float64) / 1024
    ga, gb, gc = (api.GpuArray.from_numpy(ctx, v) for v in (a, b, c))
    gx = api.GpuArray.empty(ctx, (2048, 1024, 1024), np.float64)
    build = api.GpuElemwise(ctx, "x = a + b + c", [("a", np.float64, R), ("b", np.float64, R),
                                                    ("c", np.float64, R), ("x", np.float64, W)], nd=3)
    build(ga, gb, gc, gx, flags=api.GE_BROADCAST)

    d = api.GpuArray.empty(ctx, (), np.float64)
    api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float64)(d, None, gx, [0, 1, 2])
    want = 1024.0 * 1024 * a.sum() + 2048.0 * 1024 * b.sum() + 2048.0 * 1024 * c.sum()
    assert float(d.to_numpy()) == want          # all terms are multiples of 2^-10 below 2^53

    dk = api.GpuArray.empty(ctx, (1024,), np.float64)
    api.GpuReduction(ctx, api.GA_REDUCE_MIN, np.float64)(dk, None, gx, [0, 2])
    assert (dk.to_numpy() == a.min() + b.reshape(-1) + c.min()).all()
    api.GpuReduction(ctx, api.GA_REDUCE_MAX, np.float64)(dk, None, gx, [0, 2])
    assert (dk.to_numpy() == a.max() + b.reshape(-1) + c.max()).all()

    di = api.GpuArray.empty(ctx, (1024,), np.int64)
    api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.float64)(dk, di, gx, [0, 2])
    i0 = int(a.reshape(-1).argmax())            # first occurrence along axis 0
    k0 = int(c.reshape(-1).argmax())            # first occurrence along axis 2
    assert (di.to_numpy() == i0 * 1024 + k0).all()
    # leading-axis shards: partials of the final shape combine to the same result
    parts = []
    for lo, hi in ((0, 1024), (1024, 2048)):
        api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float64)(d, None, gx[lo:hi], [0, 1, 2])
        parts.append(float(d.to_numpy()))
    assert parts[0] + parts[1] == want


def test_config5_named_input_full_size(api, ctx):
    """Configuration 5 on its NAMED input: seed 4, x = 2 * U[0, 1) - 1 in fp64, shape
    (2048, 1024, 1024), generated on the host in axis-0 chunks (one PCG64 stream, so the
    chunks are consecutive pieces of the one array) and uploaded chunk by chunk.
    SUM over all axes against a chunked long-double sum with the stated bound
    |err| <= 1e-12 * log2(n) * sum|x|; MIN and MAX over axes (0, 2) bit-exact against
    NumPy; MAXANDARGMAX over (0, 2): the value is MAX's and the element at the returned
    flat index is that value."""
    free = ctx.prop_size(10)
    if free < 20 * (1 << 30):
        pytest.skip("needs 20 GiB of free device memory")
    rng = np.random.Generator(np.random.PCG64(4))
    gx = api.GpuArray.empty(ctx, (2048, 1024, 1024), np.float64)
    planes = 64
    total = np.longdouble(0)
    total_abs = np.longdouble(0)
    mn = np.full(1024, np.inf)
    mx = np.full(1024, -np.inf)
    first_plane_of_max = np.zeros(1024, np.int64)
    for lo in range(0, 2048, planes):
        chunk = rng.random((planes, 1024, 1024))
        chunk *= 2
        chunk -= 1
        gx[lo:lo + planes].write(chunk)
        total += chunk.sum(dtype=np.longdouble)
        total_abs += np.abs(chunk).sum(dtype=np.longdouble)
        mn = np.minimum(mn, chunk.min(axis=(0, 2)))
        cmx = chunk.max(axis=(0, 2))
        mx = np.where(cmx > mx, cmx, mx)
    n = 2048 * 1024 * 1024
    d = api.GpuArray.empty(ctx, (), np.float64)
    api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float64)(d, None, gx, [0, 1, 2])
    got = np.longdouble(float(d.to_numpy()))
    assert abs(got - total) <= np.longdouble(1e-12) * np.log2(n) * total_abs, (got, total)
    dk = api.GpuArray.empty(ctx, (1024,), np.float64)
    api.GpuReduction(ctx, api.GA_REDUCE_MIN, np.float64)(dk, None, gx, [0, 2])
    assert dk.to_numpy().tobytes() == mn.tobytes()
    api.GpuReduction(ctx, api.GA_REDUCE_MAX, np.float64)(dk, None, gx, [0, 2])
    assert dk.to_numpy().tobytes() == mx.tobytes()
    di = api.GpuArray.empty(ctx, (1024,), np.int64)
    api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.float64)(dk, di, gx, [0, 2])
    idx = di.to_numpy()
    assert dk.to_numpy().tobytes() == mx.tobytes() and (idx >= 0).all() and (idx < 2048 * 1024).all()
    # the element the index points at: (i, j, k) with flat = i * 1024 + k
    for j in (0, 1, 511, 1023):
        i, k = divmod(int(idx[j]), 1024)
        assert float(gx[i:i + 1, j:j + 1, k:k + 1].to_numpy().reshape(())) == mx[j]
