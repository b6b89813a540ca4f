"""Host-only view arithmetic of GpuArray (reference src/gpuarray_array.c:
fromdata, view, index, reshape without copy, transpose, contiguity flags,
src/gpuarray/array.h:21-101,265-421), checked against NumPy's own view
arithmetic without a device: the buffer is a stand-in that only carries a
reference count, which is all these calls touch on their success paths."""
import ctypes

import numpy as np
import pytest

GA_C_CONTIGUOUS, GA_F_CONTIGUOUS = 0x0001, 0x0002


class FakeBuffer(ctypes.Structure):
    """Same leading fields as the library's gpudata: device pointer, context,
    two sizes, reference count."""
    _fields_ = [("ptr", ctypes.c_uint64), ("ctx", ctypes.c_void_p), ("sz", ctypes.c_size_t),
                ("asz", ctypes.c_size_t), ("refcnt", ctypes.c_uint), ("flags", ctypes.c_int),
                ("host", ctypes.c_void_p)]


@pytest.fixture()
def env(api):
    L = api.lib()
    # a stand-in context: its first field is the pointer to the error record the calls write to
    errrec = ctypes.create_string_buffer(16384)
    fakectx = ctypes.create_string_buffer(4096)
    ctypes.cast(fakectx, ctypes.POINTER(ctypes.c_void_p))[0] = ctypes.addressof(errrec)
    buf = FakeBuffer(ptr=0x7f0000000000, ctx=ctypes.addressof(fakectx), sz=1 << 30, asz=1 << 30,
                     refcnt=1 << 20)
    buf._keep = (errrec, fakectx)
    return api, L, buf


def from_numpy_view(api, L, buf, base, view):
    """GpuArray describing `view`, a view of the NumPy array `base` (base plays the buffer)."""
    a = api._GpuArrayStruct()
    nd = view.ndim
    off = view.__array_interface__["data"][0] - base.__array_interface__["data"][0]
    # GpuArray_fromdata wants a non-negative offset to element [0, ..., 0]
    dims = (ctypes.c_size_t * max(nd, 1))(*view.shape)
    strs = (ctypes.c_ssize_t * max(nd, 1))(*view.strides)
    err = L.GpuArray_fromdata(ctypes.byref(a), ctypes.byref(buf), off, api.typecode(view.dtype), nd,
                              dims, strs, 1)
    assert err == 0
    return a


def describe(a):
    nd = a.nd
    return (tuple(a.dimensions[i] for i in range(nd)), tuple(a.strides[i] for i in range(nd)),
            a.offset, bool(a.flags & GA_C_CONTIGUOUS), bool(a.flags & GA_F_CONTIGUOUS))


def expect(base, view):
    off = view.__array_interface__["data"][0] - base.__array_interface__["data"][0]
    return (view.shape, view.strides, off, view.flags.c_contiguous, view.flags.f_contiguous)


def same(a, base, view):
    got, want = describe(a), expect(base, view)
    assert got[0] == want[0]
    if 0 in want[0]:
        return                      # nothing addressable: offset and strides are free
    assert got[2] == want[2]
    # strides of size-1 dimensions are free (NumPy and the library may differ there)
    for d, gs, ws in zip(want[0], got[1], want[1]):
        if d != 1:
            assert gs == ws
    assert got[3] == want[3] and got[4] == want[4]


def test_index_matches_numpy_slicing(env, rng):
    api, L, buf = env
    base = np.zeros((9, 8, 7), np.float32)
    for _ in range(300):
        key = []
        for d in base.shape:
            r = rng.random()
            if r < 0.2:
                key.append(int(rng.integers(0, d)))
            else:
                step = int(rng.choice([1, 1, 2, 3, -1, -2]))
                lo, hi = sorted(int(v) for v in rng.integers(0, d + 1, size=2))
                key.append(slice(hi - 1 if step < 0 else lo, (lo - 1 if lo > 0 else None) if step < 0 else hi,
                                 step))
        view = base[tuple(key) + (Ellipsis,)]        # the Ellipsis keeps a 0-d result a view
        a = from_numpy_view(api, L, buf, base, base)
        starts = (ctypes.c_ssize_t * 3)()
        stops = (ctypes.c_ssize_t * 3)()
        steps = (ctypes.c_ssize_t * 3)()
        for i, (k, d) in enumerate(zip(key, base.shape)):
            if isinstance(k, slice):
                s0, s1, st = k.indices(d)
                if st < 0 and s1 < 0:
                    s1 = -1
                starts[i], stops[i], steps[i] = s0, s1, st
            else:
                starts[i], stops[i], steps[i] = k, k + 1, 0
        r = api._GpuArrayStruct()
        assert L.GpuArray_index(ctypes.byref(r), ctypes.byref(a), starts, stops, steps) == 0
        same(r, base, view)
        L.GpuArray_clear(ctypes.byref(r))
        L.GpuArray_clear(ctypes.byref(a))


def test_transpose_and_reshape_without_copy_match_numpy(env, rng):
    api, L, buf = env
    base = np.zeros((4, 6, 5, 2), np.float64)
    for _ in range(100):
        perm = [int(p) for p in rng.permutation(4)]
        a = from_numpy_view(api, L, buf, base, base)
        r = api._GpuArrayStruct()
        ax = (ctypes.c_uint * 4)(*perm)
        assert L.GpuArray_transpose(ctypes.byref(r), ctypes.byref(a), ax) == 0
        same(r, base, base.transpose(perm))
        L.GpuArray_clear(ctypes.byref(r))
        L.GpuArray_clear(ctypes.byref(a))
    a = from_numpy_view(api, L, buf, base, base)
    r = api._GpuArrayStruct()
    assert L.GpuArray_transpose(ctypes.byref(r), ctypes.byref(a), None) == 0     # NULL reverses the axes
    same(r, base, base.T)
    L.GpuArray_clear(ctypes.byref(r))
    for newshape in [(24, 10), (4, 30, 2), (240,), (2, 2, 6, 5, 2), (4, 6, 10)]:
        r = api._GpuArrayStruct()
        dims = (ctypes.c_size_t * len(newshape))(*newshape)
        assert L.GpuArray_reshape(ctypes.byref(r), ctypes.byref(a), len(newshape), dims, 0, 1) == 0
        same(r, base, base.reshape(newshape))
        L.GpuArray_clear(ctypes.byref(r))
    # a view whose merge is impossible cannot be reshaped without a copy
    view = base[:, ::2]
    v = from_numpy_view(api, L, buf, base, view)
    r = api._GpuArrayStruct()
    dims = (ctypes.c_size_t * 1)(view.size)
    assert L.GpuArray_reshape(ctypes.byref(r), ctypes.byref(v), 1, dims, 0, 1) != 0
    # but splitting one of its axes is fine
    dims = (ctypes.c_size_t * 5)(2, 2, 3, 5, 2)
    assert L.GpuArray_reshape(ctypes.byref(r), ctypes.byref(v), 5, dims, 0, 1) == 0
    same(r, base, view.reshape(2, 2, 3, 5, 2))
    L.GpuArray_clear(ctypes.byref(r))
    L.GpuArray_clear(ctypes.byref(v))
    L.GpuArray_clear(ctypes.byref(a))
    assert buf.refcnt == 1 << 20                                   # every view gave its reference back
