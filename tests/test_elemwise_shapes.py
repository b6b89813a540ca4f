"""Host-side shape logic of GpuElemwise_call (reference check_contig /
check_basic, src/gpuarray_elemwise.c:272-383,547-576), exercised without a
device through gpuarray_b200_elemwise_shapes: contiguous fast path, rank
padding on the left, broadcast of inputs only, output-defines-shape, and
dimension collapsing (checked against the oracle's collapse and NumPy)."""
import ctypes

import numpy as np
import pytest


class Arg(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("typecode", ctypes.c_int), ("flags", ctypes.c_int)]


def shapes(api, specs, flags):
    """specs: list of (dtype, GE flags, shape or None, byte strides or None)."""
    L = api.lib()
    fn = L.gpuarray_b200_elemwise_shapes
    fn.restype = ctypes.c_int
    n = len(specs)
    args = (Arg * n)()
    nds = (ctypes.c_uint * n)()
    dimp = (ctypes.POINTER(ctypes.c_size_t) * n)()
    strp = (ctypes.POINTER(ctypes.c_ssize_t) * n)()
    keep = []
    for i, (dt, fl, shape, strides) in enumerate(specs):
        args[i].name = b"a%d" % i
        args[i].typecode = api.typecode(np.dtype(dt))
        args[i].flags = fl
        if shape is not None:
            nds[i] = len(shape)
            d = (ctypes.c_size_t * max(len(shape), 1))(*shape)
            s = (ctypes.c_ssize_t * max(len(shape), 1))(*strides)
            keep += [d, s]
            dimp[i] = ctypes.cast(d, ctypes.POINTER(ctypes.c_size_t))
            strp[i] = ctypes.cast(s, ctypes.POINTER(ctypes.c_ssize_t))
    out = (ctypes.c_longlong * (3 + 8 + 8 * n))()
    err = fn(n, args, nds, dimp, strp, flags, out)
    if err != 0:
        return err, None
    nd = out[2]
    res = {"path": out[0], "n": out[1], "dims": list(out[3:3 + nd])}
    narr = sum(1 for sp in specs if sp[2] is not None)
    if out[0] == 1:
        res["strides"] = [list(out[3 + nd + k * nd:3 + nd + (k + 1) * nd]) for k in range(narr)]
    return 0, res


def cs(shape, isz):
    s, step = [], isz
    for d in reversed(shape):
        s.insert(0, step)
        step *= d
    return s


def fs(shape, isz):
    s, step = [], isz
    for d in shape:
        s.append(step)
        step *= d
    return s


def test_contiguous_fast_path(api):
    R, W = api.GE_READ, api.GE_WRITE
    sh = (7, 5, 3)
    err, r = shapes(api, [(np.float32, R, sh, cs(sh, 4)), (np.float64, R, sh, cs(sh, 8)),
                          (np.float32, W, sh, cs(sh, 4))], 0)
    assert err == 0 and r["path"] == 0 and r["n"] == 105          # dtype mix does not matter
    err, r = shapes(api, [(np.float32, R, sh, fs(sh, 4)), (np.float32, W, sh, fs(sh, 4))], 0)
    assert err == 0 and r["path"] == 0                            # all F-contiguous
    err, r = shapes(api, [(np.float32, R, sh, fs(sh, 4)), (np.float32, W, sh, cs(sh, 4))], 0)
    assert err == 0 and r["path"] == 1 and r["n"] == 105          # C and F mixed: strided kernels
    err, r = shapes(api, [(np.float32, R, (), []), (np.float32, W, (), [])], 0)
    assert err == 0 and r["path"] == 0 and r["n"] == 1            # 0-d arrays
    err, r = shapes(api, [(np.float32, R, (4, 0), cs((4, 0), 4)), (np.float32, W, (4, 0), cs((4, 0), 4))], 0)
    assert err == 0 and r["n"] == 0                               # zero-size: success, nothing to do
    # a scalar argument takes no part in the shape
    err, r = shapes(api, [(np.float32, R, sh, cs(sh, 4)), (np.float32, api.GE_SCALAR, None, None),
                          (np.float32, W, sh, cs(sh, 4))], 0)
    assert err == 0 and r["path"] == 0


def test_broadcast_padshape_and_output_rules(api):
    R, W = api.GE_READ, api.GE_WRITE
    B, P = api.GE_BROADCAST, api.GE_PADSHAPE
    a = (np.float32, R, (2, 1), cs((2, 1), 4))
    b = (np.float32, R, (1, 3), cs((1, 3), 4))
    out = (np.float32, W, (2, 3), cs((2, 3), 4))
    assert shapes(api, [a, b, out], 0)[0] == api.GA_VALUE_ERROR    # broadcast needs the flag
    err, r = shapes(api, [a, b, out], B)
    assert err == 0 and r["path"] == 1 and r["dims"] == [2, 3]
    assert r["strides"] == [[4, 0], [0, 4], [12, 4]]               # size-1 dims get stride 0
    # the first output defines the shape and never broadcasts, flag or not
    small_out = (np.float32, W, (1, 3), cs((1, 3), 4))
    big_in = (np.float32, R, (2, 3), cs((2, 3), 4))
    assert shapes(api, [big_in, small_out], B)[0] == api.GA_VALUE_ERROR
    # ranks must agree unless GE_PADSHAPE, which pads on the left
    v = (np.float32, R, (3,), [4])
    assert shapes(api, [v, out], B)[0] == api.GA_VALUE_ERROR
    err, r = shapes(api, [v, out], B | P)
    assert err == 0 and r["dims"] == [2, 3] and r["strides"][0] == [0, 4]
    # ... but an output of lower rank is refused
    low_out = (np.float32, W, (3,), [4])
    assert shapes(api, [big_in, low_out], B | P)[0] == api.GA_VALUE_ERROR
    # no output at all
    assert shapes(api, [a, b], B)[0] == api.GA_VALUE_ERROR


def test_config4_collapses_to_three_dimensions(api):
    """fp16 NHWC buffer viewed as NCHW + per-channel bias -> NCHW output."""
    R, W = api.GE_READ, api.GE_WRITE
    x = (np.float16, R, (64, 256, 56, 56), [1605632, 2, 28672, 512])
    bias = (np.float16, R, (1, 256, 1, 1), [512, 2, 2, 2])
    y = (np.float16, W, (64, 256, 56, 56), cs((64, 256, 56, 56), 2))
    err, r = shapes(api, [x, bias, y], api.GE_BROADCAST)
    assert err == 0 and r["path"] == 1 and r["n"] == 51380224
    assert r["dims"] == [64, 256, 3136]
    assert r["strides"] == [[1605632, 2, 512], [0, 2, 0], [1605632, 6272, 2]]


def test_random_broadcasts_match_numpy_and_the_oracle_collapse(api, oracle, rng):
    R, W, B = api.GE_READ, api.GE_WRITE, api.GE_BROADCAST
    done = 0
    for _ in range(600):
        nd = int(rng.integers(1, 6))
        shape = tuple(int(d) for d in rng.choice([1, 2, 3, 4, 5], size=nd))
        specs, views = [], []
        for k in range(int(rng.integers(1, 4))):
            ish = tuple(1 if rng.random() < 0.3 else d for d in shape)
            base = np.zeros(tuple(2 * d for d in ish), np.float32)
            v = base[tuple(slice(0, d) for d in ish)]                  # a window: non-trivial strides
            if rng.random() < 0.4 and nd > 1:
                perm = rng.permutation(nd)
                v = np.zeros(tuple(ish[i] for i in perm), np.float32).transpose(np.argsort(perm))
            assert v.shape == ish
            specs.append((np.float32, R, ish, list(v.strides)))
            views.append(v)
        o = np.zeros(shape, np.float32)
        specs.append((np.float32, W, shape, list(o.strides)))
        views.append(o)
        err, r = shapes(api, specs, B)
        assert err == 0
        if r["path"] == 0:
            assert all(s[2] == shape for s in specs)
            continue
        # expectation: NumPy's broadcast strides (0 on size-1 dims), then the oracle's collapse
        bstr = [[0 if v.shape[j] == 1 else v.strides[j] for j in range(nd)] for v in views]
        edims, estr = oracle.collapse(list(shape), bstr)
        assert r["dims"] == edims and r["strides"] == estr
        assert r["n"] == int(np.prod(shape))
        done += 1
    assert done > 300


# ---------------------------------------------------------------- call plans

def plan(api, specs, obj_flags=0, call_flags=0, sms=148, bases=None):
    """specs as for shapes(); returns the decisions GpuElemwise_call would take."""
    L = api.lib()
    fn = L.gpuarray_b200_elemwise_plan
    fn.restype = ctypes.c_int
    n = len(specs)
    args = (Arg * n)()
    nds = (ctypes.c_uint * n)()
    dimp = (ctypes.POINTER(ctypes.c_size_t) * n)()
    strp = (ctypes.POINTER(ctypes.c_ssize_t) * n)()
    addr = (ctypes.c_ulonglong * n)()
    keep = []
    for i, (dt, fl, shape, strides) in enumerate(specs):
        args[i].name = b"a%d" % i
        args[i].typecode = api.typecode(np.dtype(dt))
        args[i].flags = fl
        addr[i] = (bases[i] if bases else 0x7f0000000000 + (i << 32))
        if shape is not None:
            nds[i] = len(shape)
            d = (ctypes.c_size_t * max(len(shape), 1))(*shape)
            s = (ctypes.c_ssize_t * max(len(shape), 1))(*strides)
            keep += [d, s]
            dimp[i] = ctypes.cast(d, ctypes.POINTER(ctypes.c_size_t))
            strp[i] = ctypes.cast(s, ctypes.POINTER(ctypes.c_ssize_t))
    out = (ctypes.c_ulonglong * 16)()
    err = fn(n, args, nds, dimp, strp, addr, obj_flags, call_flags, sms, out, None, ctypes.c_size_t(0), None)
    keys = ["kind", "ept", "unroll", "nd", "idx", "modes", "tp", "tq", "pwi", "gx", "gy", "gz",
            "bx", "by", "bz", "n"]
    return err, dict(zip(keys, [int(v) for v in out]))


def modes(p, narr):
    return [(p["modes"] >> (2 * k)) & 3 for k in range(narr)]


def test_plans_of_the_named_elementwise_configurations(api):
    R, W = api.GE_READ, api.GE_WRITE
    n = 1 << 24
    # config 1: contiguous fp32, 4 elements per chunk, 4 chunks in flight, 4096 CTAs of 256
    err, p = plan(api, [(np.float32, R, (n,), [4]), (np.float32, R, (n,), [4]), (np.float32, W, (n,), [4])])
    assert err == 0 and (p["kind"], p["ept"], p["unroll"], p["idx"] & 1) == (0, 4, 4, 1)
    assert p["gx"] == n // (4 * 4 * 256) and p["bx"] == 256
    # an unaligned base: one element at a time
    err, p = plan(api, [(np.float32, R, (n,), [4]), (np.float32, W, (n,), [4])],
                  bases=[0x7f0000000004, 0x7f1000000000])
    assert err == 0 and p["kind"] == 0 and p["ept"] == 1
    # narrow types: 16 / 8 elements per chunk, 2 chunks in flight
    err, p = plan(api, [(np.uint8, R, (n,), [1]), (np.uint8, W, (n,), [1])])
    assert err == 0 and (p["ept"], p["unroll"]) == (16, 2)
    err, p = plan(api, [(np.float16, R, (n,), [2]), (np.float16, W, (n,), [2])], obj_flags=api.GE_CONVERT_F16)
    assert err == 0 and (p["ept"], p["unroll"]) == (8, 2)
    # more than 2^31 elements: 64-bit indices
    big = (1 << 31) + 64
    err, p = plan(api, [(np.uint8, R, (big,), [1]), (np.uint8, W, (big,), [1])])
    assert err == 0 and p["idx"] & 1 == 0
    # config 4: fp16 NHWC view -> NCHW: tiled transpose through cp.async + ldmatrix (unroll == 2
    # marks that build), 256 x 32 tile, one P position x 8 Q positions per thread
    x = (np.float16, R, (64, 256, 56, 56), [1605632, 2, 28672, 512])
    bias = (np.float16, R, (1, 256, 1, 1), [512, 2, 2, 2])
    y = (np.float16, W, (64, 256, 56, 56), cs((64, 256, 56, 56), 2))
    err, p = plan(api, [x, bias, y], obj_flags=api.GE_CONVERT_F16, call_flags=api.GE_BROADCAST)
    assert err == 0 and p["kind"] == 2 and (p["tp"], p["tq"], p["pwi"], p["nd"]) == (256, 32, 1, 3)
    assert p["unroll"] == 2
    assert modes(p, 3)[0] == 3 and p["gx"] == 64 * 1 * 98                  # 64 images x (256/256) x (3136/32)
    # an fp32 transposed view: 128 x 32 tiles
    M, N = 8192, 4096
    a_t = (np.float32, R, (N, M), [4, 4 * N])
    o = (np.float32, W, (N, M), cs((N, M), 4))
    err, p = plan(api, [a_t, o])
    assert err == 0 and p["kind"] == 2 and (p["tp"], p["tq"], p["pwi"]) == (128, 32, 1)
    # row / column broadcasts: strided kernel, vector + broadcast modes, 32-bit offsets, capped grid
    a = (np.float32, R, (M, N), cs((M, N), 4))
    row = (np.float32, R, (1, N), cs((1, N), 4))
    col = (np.float32, R, (M, 1), cs((M, 1), 4))
    out = (np.float32, W, (M, N), cs((M, N), 4))
    err, p = plan(api, [a, row, out], call_flags=api.GE_BROADCAST)
    assert err == 0 and p["kind"] == 1 and modes(p, 3) == [1, 1, 1] and p["idx"] == 3
    assert p["gx"] == 148 * 32
    err, p = plan(api, [a, col, out], call_flags=api.GE_BROADCAST)
    assert err == 0 and p["kind"] == 1 and modes(p, 3) == [1, 2, 1]
    # a step-2 slice is gathered element by element
    half = (np.float32, R, (M, N // 2), [4 * N, 8])
    oh = (np.float32, W, (M, N // 2), cs((M, N // 2), 4))
    err, p = plan(api, [half, oh])
    assert err == 0 and p["kind"] == 1 and modes(p, 2) == [0, 1]
    # arrays spanning more than 2 GiB keep 64-bit row offsets
    wide = (np.float32, R, (1 << 15, 1 << 13), [1 << 17, 8])                # 4 GiB span, step 2
    ow = (np.float32, W, (1 << 15, 1 << 13), cs((1 << 15, 1 << 13), 4))
    err, p = plan(api, [wide, ow])
    assert err == 0 and p["kind"] == 1 and p["idx"] == 1


def test_plan_invariants_over_random_layouts(api, rng):
    R, W, B = api.GE_READ, api.GE_WRITE, api.GE_BROADCAST
    done = 0
    for _ in range(1500):
        nd = int(rng.integers(1, 5))
        shape = tuple(int(d) for d in rng.choice([1, 2, 3, 8, 17, 64, 300, 4096], size=nd))
        dt = [np.float32, np.float16, np.float64, np.uint8][int(rng.integers(0, 4))]
        isz = np.dtype(dt).itemsize
        specs = []
        for k in range(int(rng.integers(1, 4))):
            ish = tuple(1 if rng.random() < 0.25 else d for d in shape)
            st = cs(ish, isz)
            r = rng.random()
            if r < 0.3 and nd > 1:
                perm = [int(q) for q in rng.permutation(nd)]
                st2 = cs(tuple(ish[i] for i in perm), isz)
                st = [st2[perm.index(j)] for j in range(nd)]
            elif r < 0.45:
                st = [2 * v for v in st]
            elif r < 0.55:
                st[-1] = -st[-1]
            specs.append((dt, R, ish, st))
        specs.append((dt, W, shape, cs(shape, isz)))
        sms = int(rng.choice([1, 16, 148]))
        err, p = plan(api, specs, obj_flags=api.GE_CONVERT_F16 if dt == np.float16 else 0, call_flags=B,
                      sms=sms)
        assert err == 0
        total = int(np.prod(shape))
        assert p["n"] == total
        assert p["kind"] in (0, 1, 2) and p["bx"] * p["by"] * p["bz"] == 256
        assert 1 <= p["gx"] <= 0x7fffffff and p["gy"] == 1 and p["gz"] == 1
        assert p["ept"] in (1, 2, 4, 8, 16) and p["ept"] * isz <= 16
        if p["kind"] == 1:
            assert p["gx"] <= sms * 32 and p["unroll"] == 1 and 1 <= p["nd"] <= nd
        if p["kind"] == 2:
            assert p["tp"] in (32, 64, 128, 256) and p["tq"] in (32, 64) and p["tq"] % p["ept"] == 0
            assert 3 in modes(p, len(specs))
        done += 1
    assert done == 1500
