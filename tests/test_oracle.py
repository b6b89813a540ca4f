"""Pins the CPU oracle against the reference's own known answers (CPU only).

Sources of truth used here:
  - tests/check_util.c:41-119 of the reference: the four hand cases of
    gpuarray_elemwise_collapse;
  - tests/check_util.c:121-148: seven float -> half known answers;
  - when oracle/_ref/libref_util.so exists (built from the reference's own
    sources), the reference's compiled collapse / type sizes / half routine on
    randomised inputs;
  - NumPy for first-occurrence argmax on NaN-free data and for IEEE half
    rounding.
"""
import ctypes
import itertools

import numpy as np
import pytest

# the four cases of the reference's test_elemwise_collapse: (dims, strides[2]) -> expected
COLLAPSE_CASES = [
    ([50, 1, 20], [[80, 80, 4], [80, 80, 4]], [1000], [[4], [4]]),
    ([50, 1, 20], [[168, 80, 4], [80, 80, 4]], [50, 20], [[168, 4], [80, 4]]),
    ([20, 1, 50], [[4, 80, 168], [4, 80, 80]], [20, 50], [[4, 168], [4, 80]]),
    ([1, 1], [[4, 4]], [1], [[4]]),
]

FLOAT2HALF_CASES = [(2.9831426e-08, 0x0001), (2e-25, 0x0000), (2e-26, 0x0000),
                    (1.0005035, 0x3c01), (1.0002441, 0x3c00), (65519.0, 0x7bff),
                    (65520.0, 0x7c00)]


@pytest.mark.parametrize("dims,strs,edims,estrs", COLLAPSE_CASES)
def test_collapse_known_answers(oracle, api, dims, strs, edims, estrs):
    assert oracle.collapse(dims, strs) == (edims, estrs)
    # the product's exported collapse obeys the same cases
    assert oracle.collapse(dims, strs, fn=api.lib().gpuarray_elemwise_collapse) == (edims, estrs)


def test_collapse_against_reference_build(oracle, api, rng):
    ref = oracle.ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    for _ in range(300):
        nd = int(rng.integers(1, 6))
        dims = [int(d) for d in rng.choice([1, 2, 3, 4, 5], size=nd)]
        strs = []
        for _k in range(int(rng.integers(1, 4))):
            # start from a contiguous layout, then perturb some strides
            s, step = [], 4
            for d in reversed(dims):
                s.insert(0, step)
                step *= d
            for j in range(nd):
                r = rng.random()
                if r < 0.15:
                    s[j] = 0
                elif r < 0.3:
                    s[j] = -s[j]
                elif r < 0.4:
                    s[j] *= 2
            strs.append(s)
        want = oracle.collapse(dims, strs, fn=ref.gpuarray_elemwise_collapse)
        assert oracle.collapse(dims, strs) == want
        assert oracle.collapse(dims, strs, fn=api.lib().gpuarray_elemwise_collapse) == want


@pytest.mark.parametrize("value,bits", FLOAT2HALF_CASES)
def test_float2half_known_answers(oracle, value, bits):
    assert oracle.float2half_bits(value) == bits


def test_float2half_is_ieee_rne(oracle, rng):
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * 100,
                         (rng.standard_normal(2000) * 1e-6).astype(np.float32),
                         np.array([0.0, -0.0, 65504, 1 + 2.0 ** -11, 1 + 3 * 2.0 ** -11],
                                  dtype=np.float32)])
    want = xs.astype(np.float16).view(np.uint16)
    got = np.array([oracle.float2half_bits(float(x)) for x in xs], dtype=np.uint16)
    assert (got == want).all()
    # and the round trip half -> float is exact for every finite half
    L = oracle.lib()
    hs = np.arange(0, 0x7c00, 7, dtype=np.uint16)
    back = np.array([L.oracle_half2float(int(h)) for h in hs], dtype=np.float32)
    assert (back == hs.view(np.float16).astype(np.float32)).all()


def test_reference_host_half_routine_differs_only_on_ties(oracle, rng):
    """The reference's host ga_float2half rounds exact ties away from zero
    (src/gpuarray/util.h:103-183); the device instruction rounds to even. The
    oracle models the device."""
    ref = oracle.ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref not built")
    xs = rng.standard_normal(5000).astype(np.float32)
    for x in xs:
        a = oracle.float2half_bits(float(x))
        b = ref.ref_float2half(ctypes.c_float(float(x)))
        if a != b:
            lost = np.float32(x).view(np.uint32) & 0x1fff
            assert lost == 0x1000
    assert ref.ref_float2half(ctypes.c_float(1 + 2.0 ** -11)) == 0x3c01   # tie, away from zero
    assert oracle.float2half_bits(1 + 2.0 ** -11) == 0x3c00               # tie, to even


def test_type_table_matches_reference_build(oracle, api):
    ref = oracle.ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref not built")
    L = api.lib()
    for tc in list(range(-1, 27)) + list(range(256, 310)) + [511, 512, 1000]:
        assert L.gpuarray_get_elsize(tc) == ref.gpuarray_get_elsize(tc), tc
    for code in range(-1, 21):
        if code == 6:      # GA_SYS_ERROR prints errno
            continue
        assert L.gpuarray_error_str(code) == ref.gpuarray_error_str(code), code


def test_minmaxarg_first_occurrence(oracle, rng):
    x = np.round(rng.standard_normal((6, 5, 7)) * 4).astype(np.float32) / 4   # many ties
    for axes in [(0,), (1,), (2,), (0, 2), (2, 0), (1, 2), (0, 1, 2), (2, 1, 0)]:
        free = [i for i in range(3) if i not in axes]
        xt = x.transpose(free + list(axes)).reshape([x.shape[i] for i in free] + [-1])
        v, i = oracle.minmaxarg(x, axes)
        assert (v == xt.max(-1)).all() and (i == xt.argmax(-1)).all(), axes
        v, i = oracle.minmaxarg(x, axes, is_min=True)
        assert (v == xt.min(-1)).all() and (i == xt.argmin(-1)).all(), axes


def test_minmaxarg_nan_and_signed_zero_rules(oracle):
    """Strict comparison from the first element (src/gpuarray_reduction.c:557-586):
    a NaN wins only in first position; equal zeros keep the earlier bit pattern."""
    nan = np.float32("nan")
    v, i = oracle.minmaxarg(np.array([[1, nan, 3, nan]], dtype=np.float32), [1])
    assert v[0] == 3 and i[0] == 2
    v, i = oracle.minmaxarg(np.array([[nan, 5, 7]], dtype=np.float32), [1])
    assert np.isnan(v[0]) and i[0] == 0
    v, i = oracle.minmaxarg(np.array([[-0.0, 0.0, -0.0]], dtype=np.float32), [1])
    assert i[0] == 0 and np.signbit(v[0])
    v, i = oracle.minmaxarg(np.array([[0.0, -0.0]], dtype=np.float32), [1])
    assert i[0] == 0 and not np.signbit(v[0])
    v, i = oracle.minmaxarg(np.array([[-np.inf, -np.inf]], dtype=np.float32), [1])
    assert i[0] == 0


def test_reference_reduction_test_shapes(oracle):
    """The reference's check_reduction.c fills PCG(seed 1) data and recomputes
    the answer with host loops; here the same data goes through the oracle and
    through an independent NumPy statement of those loops."""
    dims = (32, 50, 79)
    x = oracle.pcg_fill_f32(1, int(np.prod(dims))).reshape(dims)
    assert 0.0 <= x.min() and x.max() < 1.0
    v, i = oracle.minmaxarg(x, [0, 2])
    xt = x.transpose(1, 0, 2).reshape(50, -1)
    assert (v == xt.max(1)).all() and (i == xt.argmax(1)).all()
    v, i = oracle.minmaxarg(x, [2, 0])                       # test_idxtranspose
    xt = x.transpose(1, 2, 0).reshape(50, -1)
    assert (i == xt.argmax(1)).all()
    v, i = oracle.minmaxarg(x, [0, 1, 2])                    # test_alldimsreduced
    assert v.shape == () and i == x.reshape(-1).argmax()


def test_elementwise_oracle_fma_contraction(oracle, rng):
    """a*b+0.5f is one fused multiply-add, as NVRTC compiles it by default."""
    a = (2 * rng.random(4096, dtype=np.float32) - 1)
    b = (2 * rng.random(4096, dtype=np.float32) - 1)
    out = np.zeros_like(a)
    E = oracle.ElemwiseOracle("out = a * b + 0.5f", [("a", np.float32, 2), ("b", np.float32, 2),
                                                     ("out", np.float32, 4)])
    E(a, b, out)
    exact = (a.astype(np.float64) * b.astype(np.float64) + 0.5).astype(np.float32)
    assert (out == exact).all()
    assert (out == oracle.fma_f32(a, b, 0.5)).all()


def test_elementwise_oracle_reference_vectors(oracle):
    """Literal vectors of the reference's tests/check_elemwise.c."""
    u32 = np.uint32
    a, b, c = np.array([1, 2, 3], u32), np.array([4, 5, 6], u32), np.zeros(3, u32)
    oracle.ElemwiseOracle("c = a + b", [("a", u32, 2), ("b", u32, 2), ("c", u32, 4)])(a, b, c)
    assert c.tolist() == [5, 7, 9]
    f16 = np.array([0x0000, 0x3c00, 0x4000, 0x4200, 0x4400, 0x4500, 0x4600, 0x4700, 0x4800, 0x4880],
                   dtype=np.uint16)
    a = f16[[1, 2, 3]].view(np.float16)
    b = f16[[4, 5, 6]].view(np.float16)
    c = np.zeros(3, np.float16)
    oracle.ElemwiseOracle("c = a + b", [("a", np.float16, 2), ("b", np.float16, 2),
                                        ("c", np.float16, 4)], convert_f16=True)(a, b, c)
    assert c.view(np.uint16).tolist() == f16[[5, 7, 9]].tolist()
    # broadcast 2x3 with a (1,3) row (test_basic_broadcast)
    a = np.arange(1, 7, dtype=u32).reshape(2, 3)
    b = np.array([[7, 8, 9]], dtype=u32)
    c = np.zeros((2, 3), u32)
    E = oracle.ElemwiseOracle("c = a + b", [("a", u32, 2), ("b", u32, 2), ("c", u32, 4)])
    with pytest.raises(ValueError):
        E(a, b, c, broadcast=False)
    E(a, b, c)
    assert c.tolist() == [[8, 10, 12], [11, 13, 15]]
