"""Host-side planning of reductions (kernel variant, splits, launch geometry),
exercised without a device through gpuarray_b200_reduction_plan: invariants
that must hold for ANY shape, including extents no memory could hold."""
import ctypes
import itertools

import numpy as np
import pytest

SHAPE_ROWS, SHAPE_COLS, SHAPE_GENERAL = 0, 1, 2
KEYS = ["shape", "vec", "group", "flat", "mu", "onerun", "lazy", "fast8", "tpo", "idx64", "splits",
        "seg", "nseg", "units", "gx", "gy", "bx", "by", "nf", "nr", "simple", "tiny"]


def plan(api, op, dt, dims, strides, axes, base=0x7f0000000000, sms=148, dst=None):
    L = api.lib()
    fn = L.gpuarray_b200_reduction_plan
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint,
                   ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_ssize_t), ctypes.c_uint,
                   ctypes.POINTER(ctypes.c_int), ctypes.c_ulonglong, ctypes.c_uint,
                   ctypes.POINTER(ctypes.c_ulonglong)]
    nd = len(dims)
    out = (ctypes.c_ulonglong * 24)()
    tc = api.typecode(np.dtype(dt))
    dtc = api.typecode(np.dtype(dst)) if dst is not None else tc
    err = fn(getattr(api, "GA_REDUCE_" + op), tc, dtc, nd, (ctypes.c_size_t * nd)(*dims),
             (ctypes.c_ssize_t * nd)(*strides), len(axes), (ctypes.c_int * len(axes))(*axes), base, sms, out)
    return err, dict(zip(KEYS, [int(v) for v in out]))


def c_strides(dims, itemsize):
    s, step = [], itemsize
    for d in reversed(dims):
        s.insert(0, step)
        step *= d
    return s


def check_invariants(p, itemsize, kind_pair):
    assert 1 <= p["gx"] <= 0x7fffffff and 1 <= p["gy"] <= 65535
    threads = p["bx"] * p["by"]
    assert threads % 32 == 0 and 32 <= threads <= 1024
    assert p["splits"] >= 1
    assert p["vec"] in (1, 2, 4, 8, 16) and p["vec"] * itemsize <= 16
    if p["shape"] == SHAPE_ROWS:
        assert p["group"] in (1, 2, 4, 8, 16, 32, 64, 128, 256)
        assert p["seg"] >= 1 and p["nseg"] >= 1 and p["seg"] < 2 ** 31
        assert p["splits"] <= max(p["units"], 1)
        if p["onerun"]:
            assert p["units"] == 1 and p["splits"] == 1 and p["mu"] in (2, 4) and p["group"] <= 32
        elif p["tiny"]:
            assert p["units"] == 1 and p["splits"] == 1 and p["group"] in (1, 2, 4, 8) and p["mu"] == 1
            assert p["vec"] * itemsize == 16 and p["nf"] * p["group"] < 2 ** 31
            assert p["nr"] == p["group"] * p["vec"] and p["gx"] <= 148 * 8
        else:
            assert p["group"] in (32, 64, 128, 256)
        if p["group"] > 32:
            assert p["flat"] == 0 and p["mu"] == 1
        if p["lazy"]:                                 # values-only scan: long runs, or one short run
            assert kind_pair and not p["flat"] and (p["onerun"] or p["mu"] == 1) and p["vec"] > 1 or \
                (kind_pair and not p["onerun"] and not p["flat"] and p["mu"] == 1)
        if p["fast8"]:
            assert itemsize == 1 and p["vec"] % 4 == 0
    elif p["shape"] == SHAPE_COLS:
        assert p["bx"] == 32 and p["splits"] == p["gy"] and p["vec"] <= 4
    else:
        assert p["tpo"] in (1, 32, 256)


def test_named_configurations_get_the_intended_kernels(api):
    # cfg3: a warp per 128 KB row, no split, values-only scan
    err, p = plan(api, "MAXANDARGMAX", np.float32, [16384, 32000], c_strides([16384, 32000], 4), [1])
    assert err == 0 and p["shape"] == SHAPE_ROWS and p["group"] == 32 and p["splits"] == 1
    assert p["vec"] == 4 and p["lazy"] == 1 and p["gx"] == 2048
    # the headline's 8-GPU shard: 2048 rows, two warps per row (27 warps per SM), values-only scan
    err, p = plan(api, "MAXANDARGMAX", np.float32, [2048, 32000], c_strides([2048, 32000], 4), [1])
    assert err == 0 and p["group"] == 64 and p["lazy"] == 1 and p["splits"] == 1 and p["gx"] == 512
    err, p = plan(api, "MAXANDARGMAX", np.float32, [1024, 32000], c_strides([1024, 32000], 4), [1])
    assert err == 0 and p["group"] == 128 and p["gx"] == 512
    # cfg2: rows and columns
    err, p = plan(api, "SUM", np.float32, [4096, 4096], c_strides([4096, 4096], 4), [1])
    assert err == 0 and p["shape"] == SHAPE_ROWS and p["splits"] == 1 and p["gx"] == 512
    assert p["simple"] == 1                      # one run per output, a warp each: the lean loop
    err, p = plan(api, "SUM", np.float32, [4096, 4096], c_strides([4096, 4096], 4), [0])
    # 16 row lanes x 16 splits: every thread walks 16 rows, the grid is resident at once
    assert err == 0 and p["shape"] == SHAPE_COLS and p["gx"] == 32 and p["splits"] == 16 and p["by"] == 16
    # cfg5: full sum by CTA groups, 4 per SM; MIN over (0, 2) by warps with shares >= 24 KiB
    dims = [2048, 1024, 1024]
    err, p = plan(api, "SUM", np.float64, dims, c_strides(dims, 8), [0, 1, 2])
    assert err == 0 and p["group"] == 256 and p["splits"] == 148 * 4 and p["gx"] == 148 * 4
    err, p = plan(api, "MIN", np.float64, dims, c_strides(dims, 8), [0, 2])
    assert err == 0 and p["group"] == 32 and p["nf"] == 1024 and p["splits"] == 37
    assert p["nr"] * 8 // p["splits"] >= 24 * 1024
    # short runs: part of a warp per output, several outputs at once, 3 CTAs per SM
    err, p = plan(api, "SUM", np.float32, [1 << 21, 40], [160, 4], [1])
    assert err == 0 and p["onerun"] == 1 and p["group"] == 4 and p["mu"] == 2 and p["gx"] == 148 * 3
    err, p = plan(api, "SUM", np.float32, [1 << 21, 32], [160, 4], [1])          # a pitch wider than the run
    assert err == 0 and p["onerun"] == 1 and p["group"] == 2 and p["tiny"] == 0
    # runs of 1, 2, 4, 8 vectors back to back: one flat walk over the vectors, lanes per run =
    # vectors per run, 8 CTAs per SM at most; MIN / MAX / ARG* of rows of 16: the same
    err, p = plan(api, "SUM", np.float32, [1 << 21, 32], c_strides([1 << 21, 32], 4), [1])
    assert err == 0 and p["tiny"] == 1 and p["onerun"] == 0 and p["group"] == 8 and p["gx"] == 148 * 8
    err, p = plan(api, "MAX", np.float32, [1 << 22, 16], c_strides([1 << 22, 16], 4), [1])
    assert err == 0 and p["tiny"] == 1 and p["group"] == 4 and p["vec"] == 4
    err, p = plan(api, "MAX", np.float32, [100, 16], c_strides([100, 16], 4), [1])
    assert err == 0 and p["tiny"] == 1 and p["gx"] == 1
    err, p = plan(api, "MAX", np.float32, [1 << 22, 12], c_strides([1 << 22, 12], 4), [1])   # 3 vectors
    assert err == 0 and p["tiny"] == 0 and p["onerun"] == 1
    # ARGMAX over 1024-element rows: one run per output, 32 lanes x 8 vectors, values-only scan;
    # 512-element rows (4 vectors per lane) compare pairs element by element
    err, p = plan(api, "ARGMAX", np.float32, [1 << 16, 1024], c_strides([1 << 16, 1024], 4), [1])
    assert err == 0 and p["onerun"] == 1 and p["group"] == 32 and p["lazy"] == 1
    err, p = plan(api, "ARGMAX", np.float32, [1 << 17, 512], c_strides([1 << 17, 512], 4), [1])
    assert err == 0 and p["onerun"] == 1 and p["group"] == 32 and p["lazy"] == 0
    # an unaligned base drops to scalar loads
    err, p = plan(api, "SUM", np.float32, [4096, 4096], c_strides([4096, 4096], 4), [1], base=0x7f0000000004)
    assert err == 0 and p["vec"] == 1
    # 1-byte sums fold words
    err, p = plan(api, "SUM", np.int8, [1 << 28], [1], [0], dst=np.int64)
    assert err == 0 and p["fast8"] == 1 and p["vec"] == 16


def test_plan_invariants_over_random_and_extreme_shapes(api, rng):
    ops = ["SUM", "MAXANDARGMAX", "ARGMIN", "ANY", "PROD"]
    extents = [1, 2, 3, 7, 16, 31, 64, 100, 257, 1024, 4099, 65536, 1 << 20, (1 << 31) + 5, 1 << 33]
    n = 0
    for _ in range(4000):
        nd = int(rng.integers(1, 6))
        dims = [int(rng.choice(extents)) for _ in range(nd)]
        total = 1
        for d in dims:
            total *= d
        if total >= 1 << 62:
            continue
        dt = [np.float32, np.float64, np.float16, np.int8, np.int32][int(rng.integers(0, 5))]
        isz = np.dtype(dt).itemsize
        strides = c_strides(dims, isz)
        r = rng.random()
        if r < 0.25:                                  # a permuted view
            perm = rng.permutation(nd)
            dims = [dims[i] for i in perm]
            strides = [strides[i] for i in perm]
        elif r < 0.4:                                 # every other element of the last axis
            strides[-1] *= 2
        elif r < 0.5:                                 # reversed last axis
            strides[-1] = -strides[-1]
        k = int(rng.integers(1, nd + 1))
        axes = [int(a) for a in rng.permutation(nd)[:k]]
        op = ops[int(rng.integers(0, len(ops)))]
        dst = np.bool_ if op == "ANY" else (np.int64 if dt in (np.int8, np.int32) and op == "SUM" else None)
        sms = int(rng.choice([1, 8, 132, 148]))
        base = 0x7f0000000000 + int(rng.choice([0, 0, 0, 2, 4, 8])) * (isz if isz < 8 else 1)
        err, p = plan(api, op, dt, dims, strides, axes, base=base, sms=sms, dst=dst)
        if err != 0:
            assert err in (api.GA_XLARGE_ERROR, api.GA_UNSUPPORTED_ERROR), (err, dims, axes)
            continue
        want_nr = 1
        for a in axes:
            want_nr *= dims[a]
        assert p["nr"] == want_nr and p["nf"] * want_nr == total
        check_invariants(p, isz, op in ("MAXANDARGMAX", "ARGMIN"))
        n += 1
    assert n > 3000


@pytest.mark.parametrize("bad", [dict(axes=[2]), dict(axes=[0, 0]), dict(axes=[])])
def test_plan_rejects_bad_axes(api, bad):
    err, _ = plan(api, "SUM", np.float32, [4, 5], [20, 4], bad["axes"])
    assert err == api.GA_INVALID_ERROR


def test_split_counts_are_trimmed_to_whole_waves(api):
    """rd_fit_waves (ga_reduction.c): grids a little over a whole number of waves of resident
    CTAs lose their last, mostly idle, wave; grids within one wave and grids already ending on
    a full or >= 70 % full wave stay; the count only ever goes down, by a third at most."""
    f = api.lib().gpuarray_b200_reduction_fit_waves
    f.restype = ctypes.c_ulonglong
    f.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_ulonglong,
                  ctypes.POINTER(ctypes.c_uint)]

    def fit(outputs, splits, group=32, slots=592):
        ctas = ctypes.c_uint()
        s = int(f(outputs, splits, group, slots, ctypes.byref(ctas)))
        return s, int(ctas.value)

    assert fit(64, 170) == (148, 1184)          # (256, 64, 4096) over (0, 2): 2.3 waves -> 2.0
    assert fit(512, 21) == (18, 1152)           # (512, 512, 256) over (1, 2): 2.27 -> 1.95 waves
    assert fit(512, 21, slots=444) == (20, 1280)  # three CTAs per SM: 3.03 -> 2.88 waves
    assert fit(256, 32) == (32, 1024)           # 1.73 waves: the last one is 73 % full, stays
    assert fit(256, 16) == (16, 512)            # within one wave: untouched
    assert fit(1024, 37) == (37, 4736)          # exactly 8 waves
    assert fit(100, 3) == (3, 38)
    s, c = fit(7, 1000)
    assert 667 <= s <= 1000 and (c % 592 == 0 or c % 592 >= 415)
    assert fit(64, 170, slots=0) == (170, 1360)  # occupancy unknown: nothing changes
    # two warps per work item
    assert fit(2048, 3, group=64) == (2, 1024)  # 2.59 waves -> 1.73
    assert fit(2048, 7, group=64) == (7, 3584)  # 6.05 waves; 6 and 5 splits end on 19 % / 32 % full waves: left alone

