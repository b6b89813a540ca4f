"""GPU parity tests of the elementwise engine through the C ABI.

Part 1 restates the reference's device tests tests/check_elemwise.c (:39-880)
case by case with their literal vectors. Part 2 follows the spirit of
pygpu/tests/test_elemwise.py: dtype x operator sweeps, broadcasting, in-place
and scalar arguments, strided / offset / negative-stride views, each checked
bit for bit against the CPU oracle (oracle.ElemwiseOracle), which restates the
reference's kernel generator.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

R, W, S = 2, 4, 1
F16 = np.array([0x0000, 0x3c00, 0x4000, 0x4200, 0x4400, 0x4500, 0x4600, 0x4700, 0x4800, 0x4880],
               dtype=np.uint16)   # 0.0 .. 9.0 as in the reference test


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[a.dtype.itemsize])


def abc(api, ctx, dt=np.uint32, flags=0, expr="c = a + b", nd=1):
    return api.GpuElemwise(ctx, expr, [("a", dt, R), ("b", dt, R), ("c", dt, W)], nd=nd, flags=flags)


# --------------------------------------------------- part 1: check_elemwise.c

def test_contig_simple(api, ctx):
    a = api.GpuArray.from_numpy(ctx, np.array([1, 2, 3], np.uint32))
    b = api.GpuArray.from_numpy(ctx, np.array([4, 5, 6], np.uint32))
    c = api.GpuArray.empty(ctx, (3,), np.uint32)
    abc(api, ctx)(a, b, c, flags=api.GE_NOCOLLAPSE)
    assert c.to_numpy().tolist() == [5, 7, 9]


def test_contig_f16(api, ctx):
    a = api.GpuArray.from_numpy(ctx, F16[[1, 2, 3]].view(np.float16))
    b = api.GpuArray.from_numpy(ctx, F16[[4, 5, 6]].view(np.float16))
    c = api.GpuArray.empty(ctx, (3,), np.float16)
    abc(api, ctx, np.float16, api.GE_CONVERT_F16)(a, b, c, flags=api.GE_NOCOLLAPSE)
    assert bits(c.to_numpy()).tolist() == F16[[5, 7, 9]].tolist()


def test_contig_0(api, ctx):
    a = api.GpuArray.empty(ctx, (0,), np.uint32)
    b = api.GpuArray.empty(ctx, (0,), np.uint32)
    c = api.GpuArray.empty(ctx, (0,), np.uint32)
    abc(api, ctx)(a, b, c, flags=api.GE_NOCOLLAPSE)      # succeeds without a launch


def test_basic_simple_mixed_order(api, ctx):
    a = api.GpuArray.from_numpy(ctx, np.array([[1, 2, 3]], np.uint32), order="C")
    b = api.GpuArray.from_numpy(ctx, np.array([[4, 5, 6]], np.uint32), order="F")
    c = api.GpuArray.empty(ctx, (1, 3), np.uint32)
    abc(api, ctx, nd=2)(a, b, c, flags=api.GE_NOCOLLAPSE)
    assert c.to_numpy().tolist() == [[5, 7, 9]]


def test_basic_f16_mixed_order(api, ctx):
    a = api.GpuArray.from_numpy(ctx, F16[[1, 2, 3]].view(np.float16).reshape(1, 3), order="C")
    b = api.GpuArray.from_numpy(ctx, F16[[4, 5, 6]].view(np.float16).reshape(1, 3), order="F")
    c = api.GpuArray.empty(ctx, (1, 3), np.float16)
    abc(api, ctx, np.float16, api.GE_CONVERT_F16, nd=2)(a, b, c, flags=api.GE_NOCOLLAPSE)
    assert bits(c.to_numpy()).reshape(-1).tolist() == F16[[5, 7, 9]].tolist()


def test_basic_offset(api, ctx):
    """`a` is a (1,3) window at byte offset 12 of a (1,6) buffer."""
    big = api.GpuArray.from_numpy(ctx, np.array([[9, 9, 9, 1, 2, 3]], np.uint32))
    a = big[:, 3:6]
    assert a.ga.offset == 12
    b = api.GpuArray.from_numpy(ctx, np.array([[4, 5, 6]], np.uint32), order="F")
    c = api.GpuArray.empty(ctx, (1, 3), np.uint32)
    abc(api, ctx, nd=2)(a, b, c, flags=api.GE_NOCOLLAPSE)
    assert c.to_numpy().tolist() == [[5, 7, 9]]


def test_basic_scalar_and_broadcast(api, ctx):
    a = api.GpuArray.from_numpy(ctx, np.array([[1, 2, 3]], np.uint32))
    b = api.GpuArray.from_numpy(ctx, np.array([[4], [5]], np.uint32), order="F")
    c = api.GpuArray.empty(ctx, (2, 3), np.uint32)
    ge = api.GpuElemwise(ctx, "c = a + x * b", [("a", np.uint32, R), ("x", np.uint32, S | R),
                                               ("b", np.uint32, R), ("c", np.uint32, W)], nd=2)
    ge(a, 2, b, c, flags=api.GE_BROADCAST)
    assert c.to_numpy().tolist() == [[9, 10, 11], [11, 12, 13]]


def test_basic_scalar_dtype(api, ctx):
    """y = a*x + y with a float scalar, int x (C order) and float y (F order), in place."""
    x = api.GpuArray.from_numpy(ctx, np.array([[0, 1], [2, 3]], np.int32), order="C")
    y = api.GpuArray.from_numpy(ctx, np.full((2, 2), 2.0, np.float32), order="F")
    ge = api.GpuElemwise(ctx, "y = a * x + y", [("a", np.float32, S), ("x", np.int32, R),
                                               ("y", np.float32, R | W)], nd=2)
    ge(np.float32(1.1), x, y, flags=0)
    got = y.to_numpy()
    want = np.float32(1.1) * np.array([[0, 1], [2, 3]], np.float32) + np.float32(2.0)
    assert np.allclose(got, want, rtol=1e-6)
    # the memory order the reference test reads back: 2.0, 4.2, 3.1, 5.3
    assert np.allclose(got.reshape(-1, order="F"), [2.0, 4.2, 3.1, 5.3], rtol=1e-6)


def test_basic_remove1(api, ctx):
    """4-d arrays with size-1 axes, operator built with nd=0."""
    data = np.arange(1, 7, dtype=np.uint32)
    a = api.GpuArray.from_numpy(ctx, data.reshape(1, 3, 2, 1), order="C")
    b = api.GpuArray.from_numpy(ctx, (data + 6).reshape(1, 3, 2, 1), order="F")
    c = api.GpuArray.empty(ctx, (1, 3, 2, 1), np.uint32)
    abc(api, ctx, nd=0)(a, b, c, flags=0)
    assert (c.to_numpy() == (2 * data + 6).reshape(1, 3, 2, 1)).all()


def test_basic_broadcast_needs_flag(api, ctx):
    a = api.GpuArray.from_numpy(ctx, np.array([[1, 2, 3]], np.uint32))
    b = api.GpuArray.from_numpy(ctx, np.array([[4], [5]], np.uint32), order="F")
    c = api.GpuArray.empty(ctx, (2, 3), np.uint32)
    ge = abc(api, ctx, nd=2)
    with pytest.raises(api.GpuArrayException) as ei:
        ge(a, b, c, flags=api.GE_NOCOLLAPSE)
    assert ei.value.code == api.GA_VALUE_ERROR
    ge(a, b, c, flags=api.GE_NOCOLLAPSE | api.GE_BROADCAST)
    assert c.to_numpy().tolist() == [[5, 6, 7], [6, 7, 8]]


def test_basic_padshape(api, ctx):
    a = api.GpuArray.from_numpy(ctx, np.array([1, 2, 3], np.uint32))
    b = api.GpuArray.from_numpy(ctx, np.array([[4], [5]], np.uint32), order="F")
    c = api.GpuArray.empty(ctx, (2, 3), np.uint32)
    ge = abc(api, ctx, nd=2)
    with pytest.raises(api.GpuArrayException) as ei:
        ge(a, b, c, flags=api.GE_NOCOLLAPSE)
    assert ei.value.code == api.GA_VALUE_ERROR
    ge(a, b, c, flags=api.GE_NOCOLLAPSE | api.GE_BROADCAST | api.GE_PADSHAPE)
    assert c.to_numpy().tolist() == [[5, 6, 7], [6, 7, 8]]


def test_basic_collapse(api, ctx):
    a = api.GpuArray.from_numpy(ctx, np.arange(1, 7, dtype=np.uint32).reshape(2, 3))
    b = api.GpuArray.from_numpy(ctx, np.arange(7, 13, dtype=np.uint32).reshape(2, 3))
    c = api.GpuArray.empty(ctx, (2, 3), np.uint32)
    abc(api, ctx, nd=2)(a, b, c, flags=0)
    assert c.to_numpy().tolist() == [[8, 10, 12], [14, 16, 18]]


def test_basic_neg_strides(api, ctx):
    a = api.GpuArray.from_numpy(ctx, np.arange(1, 7, dtype=np.uint32))
    bfull = api.GpuArray.from_numpy(ctx, np.arange(7, 13, dtype=np.uint32))
    b = bfull[::-1]
    assert b.strides == (-4,)
    c = api.GpuArray.empty(ctx, (6,), np.uint32)
    abc(api, ctx)(a, b, c, flags=0)
    assert c.to_numpy().tolist() == [13, 13, 13, 13, 13, 13]


def test_basic_0(api, ctx):
    a = api.GpuArray.empty(ctx, (0, 3), np.uint32, order="C")
    b = api.GpuArray.empty(ctx, (0, 3), np.uint32, order="F")
    c = api.GpuArray.empty(ctx, (0, 3), np.uint32)
    abc(api, ctx, nd=2)(a, b, c, flags=0)


# ------------------------------------------- part 2: sweeps against the oracle

def run_both(api, ctx, oracle, expr, spec, values, convert_f16=False, preamble="", **callkw):
    """spec: [(name, dtype, flags)]; values: numpy arrays / scalars. Arrays may be
    views; the same view geometry is rebuilt on the device. Returns nothing;
    asserts bit equality of every written array."""
    O = oracle.ElemwiseOracle(expr, spec, preamble=preamble, convert_f16=convert_f16)
    G = api.GpuElemwise(ctx, expr, spec, preamble=preamble, convert_f16=convert_f16)
    host, dev, bases = [], [], []
    for v, (name, dt, fl) in zip(values, spec):
        if fl & S:
            host.append(v)
            dev.append(v)
            continue
        # find the owning buffer of the view and mirror it on the device
        base = v
        while base.base is not None:
            base = base.base
        gbase = api.GpuArray.from_numpy(ctx, np.ascontiguousarray(base.ravel(order="K")))
        off = v.__array_interface__["data"][0] - base.__array_interface__["data"][0]
        g = api.GpuArray(ctx)
        dims = (ctypes.c_size_t * max(v.ndim, 1))(*v.shape)
        strs = (ctypes.c_ssize_t * max(v.ndim, 1))(*v.strides)
        err = api.lib().GpuArray_fromdata(ctypes.byref(g.ga), gbase.ga.data, off, api.typecode(dt),
                                          v.ndim, dims, strs, 1)
        assert err == 0
        g._live = True
        host.append(v)
        dev.append(g)
        bases.append((base, gbase, fl))
    O(*host, **callkw)
    flags = (api.GE_BROADCAST if callkw.get("broadcast", True) else 0) | \
            (api.GE_PADSHAPE if callkw.get("padshape", True) else 0)
    G(*dev, flags=flags)
    for base, gbase, fl in bases:
        if fl & W:
            got = gbase.to_numpy()
            want = np.ascontiguousarray(base.ravel(order="K"))
            assert (bits(got) == bits(want)).all(), (expr, got[:8], want[:8])


DTYPES = [np.float32, np.int8, np.uint64, np.float64, np.int32, np.uint16]
BINOPS = ["+", "-", "*"]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("op", BINOPS)
def test_binary_ops_contiguous(api, ctx, oracle, rng, dt, op):
    n = 1000 + 3           # not a multiple of the vector width: exercises the tail
    if np.dtype(dt).kind == "f":
        a = rng.standard_normal(n).astype(dt)
        b = rng.standard_normal(n).astype(dt)
    else:
        a = rng.integers(0, 100, n).astype(dt)
        b = rng.integers(1, 100, n).astype(dt)
    c = np.zeros(n, dt)
    run_both(api, ctx, oracle, "c = a %s b" % op, [("a", dt, R), ("b", dt, R), ("c", dt, W)],
             [a, b, c])


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 7, 8, 15, 16, 17, 255, 256, 257, 1023, 1025, 4099])
def test_contiguous_sizes_and_tails(api, ctx, oracle, rng, n):
    a = rng.standard_normal(n).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    c = np.zeros(n, np.float32)
    run_both(api, ctx, oracle, "c = a * b + 0.5f", [("a", np.float32, R), ("b", np.float32, R),
                                                    ("c", np.float32, W)], [a, b, c])


def test_unaligned_base_takes_scalar_path(api, ctx, oracle, rng):
    """Views starting 4 bytes into a buffer are not 16-byte aligned."""
    abuf = rng.standard_normal(1001).astype(np.float32)
    bbuf = rng.standard_normal(1001).astype(np.float32)
    cbuf = np.zeros(1001, np.float32)
    run_both(api, ctx, oracle, "c = a * b + 0.5f", [("a", np.float32, R), ("b", np.float32, R),
                                                    ("c", np.float32, W)],
             [abuf[1:], bbuf[1:], cbuf[1:]])


def test_mixed_dtypes_and_widths(api, ctx, oracle, rng):
    x = rng.integers(0, 255, 4099).astype(np.uint8)
    y = rng.standard_normal(4099)
    run_both(api, ctx, oracle, "y = a * x + y", [("a", np.float32, S), ("x", np.uint8, R),
                                                ("y", np.float64, R | W)], [np.float32(1.5), x, y])


def test_f16_convert(api, ctx, oracle, rng):
    a = rng.standard_normal(3001).astype(np.float16)
    b = rng.standard_normal(3001).astype(np.float16)
    c = np.zeros(3001, np.float16)
    run_both(api, ctx, oracle, "c = a * b + a", [("a", np.float16, R), ("b", np.float16, R),
                                                ("c", np.float16, W)], [a, b, c], convert_f16=True)


def test_inplace_and_aliasing(api, ctx, oracle, rng):
    a = rng.standard_normal(2049).astype(np.float32)
    b = rng.standard_normal(2049).astype(np.float32)
    run_both(api, ctx, oracle, "a = a + b", [("a", np.float32, R | W), ("b", np.float32, R)], [a, b])


def test_multiple_outputs_divmod_style(api, ctx, oracle, rng):
    """Two outputs from one expression with a comma, as pygpu's divmod builds."""
    a = rng.integers(1, 1000, 1500).astype(np.int32)
    b = rng.integers(1, 37, 1500).astype(np.int32)
    d = np.zeros(1500, np.int32)
    m = np.zeros(1500, np.int32)
    run_both(api, ctx, oracle, "d = a / b, m = a % b",
             [("a", np.int32, R), ("b", np.int32, R), ("d", np.int32, W), ("m", np.int32, W)],
             [a, b, d, m])


def test_preamble_function(api, ctx, oracle, rng):
    """User preamble with the kernel vocabulary (pygpu/tests/test_elemwise.py:310-346)."""
    pre = "WITHIN_KERNEL ga_float clip01(ga_float x) { return x < 0 ? 0 : (x > 1 ? 1 : x); }\n"
    a = rng.standard_normal(777).astype(np.float32)
    c = np.zeros(777, np.float32)
    run_both(api, ctx, oracle, "c = clip01(a)", [("a", np.float32, R), ("c", np.float32, W)], [a, c],
             preamble=pre)


BROADCAST_SHAPES = [((3, 4), (1, 4)), ((3, 4), (3, 1)), ((5, 1, 7), (5, 6, 7)), ((2, 3, 4), (4,)),
                    ((1,), (6, 5)), ((), (4, 3)), ((7, 1, 1, 3), (1, 5, 2, 3))]


@pytest.mark.parametrize("sa,sb", BROADCAST_SHAPES)
def test_broadcast_shapes(api, ctx, oracle, rng, sa, sb):
    a = rng.standard_normal(sa).astype(np.float32)
    b = rng.standard_normal(sb).astype(np.float32)
    c = np.zeros(np.broadcast_shapes(sa, sb), np.float32)
    run_both(api, ctx, oracle, "c = a - b", [("a", np.float32, R), ("b", np.float32, R),
                                             ("c", np.float32, W)], [a, b, c])


def test_output_never_broadcasts(api, ctx):
    a = api.GpuArray.from_numpy(ctx, np.ones((3, 4), np.float32))
    c = api.GpuArray.empty(ctx, (1, 4), np.float32)
    ge = api.GpuElemwise(ctx, "c = a", [("a", np.float32, R), ("c", np.float32, W)])
    with pytest.raises(api.GpuArrayException) as ei:
        ge(a, c)
    assert ei.value.code == api.GA_VALUE_ERROR


def strided_views(rng, dt, shape):
    """A few views of the same logical shape with different memory layouts."""
    shape = tuple(shape)
    full = tuple(2 * s + 1 for s in shape)

    def data(sh):
        if np.dtype(dt).kind == "f":
            return rng.standard_normal(sh).astype(dt)
        return rng.integers(0, 50, sh).astype(dt)
    out = [data(shape)]                                              # C contiguous
    out.append(np.asfortranarray(data(shape)))                       # F contiguous
    out.append(data(full)[tuple(slice(1, 1 + 2 * s, 2) for s in shape)])   # step-2 window
    out.append(data(shape)[tuple(slice(None, None, -1) for _ in shape)])   # all axes reversed
    if len(shape) >= 2:
        out.append(data(shape[::-1]).transpose())                    # transposed
    return out


@pytest.mark.parametrize("shape", [(37,), (5, 8), (3, 4, 5), (2, 3, 4, 5), (1, 6, 1, 5)])
@pytest.mark.parametrize("dt", [np.float32, np.float16, np.int64])
def test_strided_layouts(api, ctx, oracle, rng, shape, dt):
    va = strided_views(rng, dt, shape)
    vb = strided_views(rng, dt, shape)
    f16 = np.dtype(dt) == np.float16
    for i, a in enumerate(va):
        b = vb[(i + 1) % len(vb)]
        c = strided_views(rng, dt, shape)[(i + 2) % len(va)]
        run_both(api, ctx, oracle, "c = a + b", [("a", dt, R), ("b", dt, R), ("c", dt, W)],
                 [a, b, c], convert_f16=f16)


def test_high_rank_layouts_that_do_not_collapse(api, ctx, oracle, rng):
    """The rank given to GpuElemwise_new is only a hint (the reference's
    tests/check_elemwise.c:552 passes 0 and calls with 4-D arrays): 6 and 9
    dimensions, step-2 windows on every axis so that nothing collapses."""
    for shape in ((2, 3, 2, 3, 2, 5), (2, 2, 2, 3, 2, 2, 2, 2, 3)):
        va = strided_views(rng, np.float32, shape)
        vb = strided_views(rng, np.float32, shape)
        for i in (2, 3):                                             # window, reversed
            run_both(api, ctx, oracle, "c = a * b", [("a", np.float32, R), ("b", np.float32, R),
                                                      ("c", np.float32, W)],
                     [va[i], vb[2], strided_views(rng, np.float32, shape)[2]])


@pytest.mark.parametrize("shape", [(2, 5, 7, 24), (3, 8, 8, 64), (1, 3, 5, 130), (2, 17, 9, 16)])
def test_nhwc_view_to_nchw_bias_relu(api, ctx, oracle, rng, shape):
    """The broadcast + transposing case: NHWC buffer viewed as NCHW, bias (1,C,1,1)."""
    N, H, Wd, C = shape
    buf = rng.standard_normal(shape).astype(np.float16)
    x = buf.transpose(0, 3, 1, 2)
    bias = (0.2 * rng.random((1, C, 1, 1), dtype=np.float32) - 0.1).astype(np.float16)
    y = np.zeros((N, C, H, Wd), np.float16)
    run_both(api, ctx, oracle, "y = fmaxf(x + bias, 0.0f)",
             [("x", np.float16, R), ("bias", np.float16, R), ("y", np.float16, W)], [x, bias, y],
             convert_f16=True)
    want = np.maximum(x.astype(np.float32) + bias.astype(np.float32), 0).astype(np.float16)
    assert (bits(y) == bits(want)).all()


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.uint8])
def test_transposed_inputs_other_widths(api, ctx, oracle, rng, dt):
    a = (rng.standard_normal((70, 130)) * 10).astype(dt).transpose()     # (130, 70) column major
    b = (rng.standard_normal((130, 70)) * 10).astype(dt)
    c = np.zeros((130, 70), dt)
    run_both(api, ctx, oracle, "c = a + b", [("a", dt, R), ("b", dt, R), ("c", dt, W)], [a, b, c])


def test_bad_expression_fails_in_constructor(api, ctx):
    with pytest.raises(api.GpuArrayException) as ei:
        api.GpuElemwise(ctx, "c = a + no_such_symbol", [("a", np.float32, R), ("c", np.float32, W)])
    assert ei.value.code == api.GA_IMPL_ERROR
    assert "no_such_symbol" in str(ei.value)


def test_half_without_convert_flag_does_not_compile(api, ctx):
    """Without GE_CONVERT_F16 a half argument is a storage-only struct."""
    with pytest.raises(api.GpuArrayException):
        api.GpuElemwise(ctx, "c = a + a", [("a", np.float16, R), ("c", np.float16, W)])


def test_complex_types_are_refused(api, ctx):
    with pytest.raises(api.GpuArrayException) as ei:
        api.GpuElemwise(ctx, "c = a", [("a", api.GA_CFLOAT, R), ("c", api.GA_CFLOAT, W)])
    assert ei.value.code == api.GA_UNSUPPORTED_ERROR


def test_typed_and_strided_copies_use_the_engine(api, ctx, rng):
    """GpuArray_copy / GpuArray_move of non-contiguous or re-typed data run
    "dst = src" through the elementwise engine (reference ga_extcopy)."""
    x = rng.standard_normal((33, 65)).astype(np.float32)
    g = api.GpuArray.from_numpy(ctx, x)
    assert (g.transpose().copy("C").to_numpy() == x.T).all()
    assert (g[::2, ::-3].to_numpy() == x[::2, ::-3]).all()
    d = api.GpuArray.empty(ctx, x.shape, np.float64)
    api._check(ctx.ptr, api.lib().GpuArray_move(ctypes.byref(d.ga), ctypes.byref(g.ga)))
    assert (d.to_numpy() == x.astype(np.float64)).all()
    h = api.GpuArray.empty(ctx, x.shape, np.float16)
    api._check(ctx.ptr, api.lib().GpuArray_move(ctypes.byref(h.ga), ctypes.byref(g.ga)))
    assert (bits(h.to_numpy()) == bits(x.astype(np.float16))).all()


def test_guard_bands_untouched(api, ctx, rng):
    """Writes stay inside the output view: sentinel bytes around it survive."""
    buf = np.full(3000, 0x7B, np.uint8)
    g = api.GpuArray.from_numpy(ctx, buf)
    a = api.GpuArray.from_numpy(ctx, rng.integers(0, 9, 999).astype(np.uint8))
    out = g[1000:1999]
    ge = api.GpuElemwise(ctx, "c = a + 1", [("a", np.uint8, R), ("c", np.uint8, W)])
    ge(a, out)
    back = g.to_numpy()
    assert (back[:1000] == 0x7B).all() and (back[1999:] == 0x7B).all()
    assert (back[1000:1999] == a.to_numpy() + 1).all()


def test_back_to_back_producer_consumer_chains(api, ctx, rng):
    """Kernels are launched with stream serialization relaxed (programmatic
    dependent launch): each may become resident while its predecessor drains
    and waits for it before touching memory. A chain in which every kernel
    consumes what the previous one produced must still see complete inputs."""
    n = (1 << 22) + 77
    a = rng.integers(-1000, 1000, n).astype(np.int32)
    bufs = [api.GpuArray.from_numpy(ctx, a), api.GpuArray.empty(ctx, (n,), np.int32)]
    inc = api.GpuElemwise(ctx, "o = a + k", [("a", np.int32, api.GE_READ), ("k", np.int32, api.GE_SCALAR),
                                              ("o", np.int32, api.GE_WRITE)], nd=1)
    tot = api.GpuArray.empty(ctx, (), np.int64)
    rsum = api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.int32)
    sums = []
    steps = 40
    for i in range(steps):
        inc(bufs[i % 2], np.int32(i + 1), bufs[(i + 1) % 2])
        if i % 8 == 7:                       # a split reduction in the middle of the chain
            rsum(tot, None, bufs[(i + 1) % 2], [0])
            sums.append((i, tot.to_numpy().copy()))
    final = bufs[steps % 2].to_numpy()
    assert (final == a + sum(range(1, steps + 1))).all()
    for i, got in sums:
        assert int(got) == int(a.astype(np.int64).sum()) + n * sum(range(1, i + 2))
    # the same split reduction back to back on different inputs: the arrival
    # counters are handed from one launch to the next
    xs = [rng.integers(-5, 6, (3, 300000)).astype(np.int32) for _ in range(6)]
    gx = [api.GpuArray.from_numpy(ctx, x) for x in xs]
    outs = [api.GpuArray.empty(ctx, (3,), np.int64) for _ in xs]
    for _ in range(3):
        for g, o in zip(gx, outs):
            rsum(o, None, g, [1])
    for x, o in zip(xs, outs):
        assert (o.to_numpy() == x.sum(axis=1, dtype=np.int64)).all()
