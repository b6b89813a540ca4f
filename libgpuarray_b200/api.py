"""ctypes bindings over the C ABI of libgpuarray.so.

This is the Python stand-in for the reference's Cython layer (pygpu/gpuarray.pyx,
pygpu/_elemwise.pyx): thin objects that own the C structs and call the exported
entry points declared in include/gpuarray/*.h. There is no computation here and
no fallback: if the shared library or the CUDA driver is missing, the calls
raise.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgpuarray.so")

# ---- constants (include/gpuarray/types.h, elemwise.h, array.h, reduction.h) ----
GA_BUFFER = -1
GA_BOOL, GA_BYTE, GA_UBYTE, GA_SHORT, GA_USHORT, GA_INT, GA_UINT, GA_LONG, GA_ULONG = range(9)
GA_FLOAT, GA_DOUBLE, GA_HALF, GA_SIZE, GA_SSIZE = 11, 12, 23, 24, 25
GA_CFLOAT, GA_CDOUBLE = 14, 15

GE_SCALAR, GE_READ, GE_WRITE = 0x1, 0x2, 0x4
GE_NOADDR64, GE_CONVERT_F16 = 0x1, 0x2
GE_BROADCAST, GE_NOCOLLAPSE, GE_PADSHAPE = 0x100, 0x200, 0x400

GA_C_CONTIGUOUS, GA_F_CONTIGUOUS, GA_ALIGNED, GA_WRITEABLE = 0x1, 0x2, 0x100, 0x400
GA_ANY_ORDER, GA_C_ORDER, GA_F_ORDER = -1, 0, 1

(GA_NO_ERROR, GA_MEMORY_ERROR, GA_VALUE_ERROR, GA_IMPL_ERROR, GA_INVALID_ERROR,
 GA_UNSUPPORTED_ERROR, GA_SYS_ERROR, GA_RUN_ERROR, GA_DEVSUP_ERROR, GA_READONLY_ERROR,
 GA_WRITEONLY_ERROR, GA_BLAS_ERROR, GA_UNALIGNED_ERROR, GA_COPY_ERROR, GA_NODEV_ERROR,
 GA_MISC_ERROR, GA_COMM_ERROR, GA_XLARGE_ERROR, GA_LOAD_ERROR) = range(19)

(GA_REDUCE_SUM, GA_REDUCE_PROD, GA_REDUCE_PRODNZ, GA_REDUCE_MIN, GA_REDUCE_MAX,
 GA_REDUCE_ARGMIN, GA_REDUCE_ARGMAX, GA_REDUCE_MINANDARGMIN, GA_REDUCE_MAXANDARGMAX,
 GA_REDUCE_AND, GA_REDUCE_OR, GA_REDUCE_XOR, GA_REDUCE_ALL, GA_REDUCE_ANY) = range(14)

GA_SUM, GA_PROD, GA_MAX, GA_MIN = range(4)
GA_COMM_ID_BYTES = 128

_NP2GA = {
    np.dtype(np.bool_): GA_BOOL, np.dtype(np.int8): GA_BYTE, np.dtype(np.uint8): GA_UBYTE,
    np.dtype(np.int16): GA_SHORT, np.dtype(np.uint16): GA_USHORT, np.dtype(np.int32): GA_INT,
    np.dtype(np.uint32): GA_UINT, np.dtype(np.int64): GA_LONG, np.dtype(np.uint64): GA_ULONG,
    np.dtype(np.float16): GA_HALF, np.dtype(np.float32): GA_FLOAT, np.dtype(np.float64): GA_DOUBLE,
}
_GA2NP = {v: k for k, v in _NP2GA.items()}


def typecode(dtype):
    """NumPy dtype -> GA_* typecode."""
    return _NP2GA[np.dtype(dtype)]


def np_dtype(tc):
    return _GA2NP[tc]


class GpuArrayException(Exception):
    def __init__(self, msg, code):
        super().__init__("%s (GA error %d)" % (msg, code))
        self.code = code


class _GpuArrayStruct(ctypes.Structure):
    """struct _GpuArray of include/gpuarray/array.h."""
    _fields_ = [("data", ctypes.c_void_p), ("dimensions", ctypes.POINTER(ctypes.c_size_t)),
                ("strides", ctypes.POINTER(ctypes.c_ssize_t)), ("offset", ctypes.c_size_t),
                ("nd", ctypes.c_uint), ("flags", ctypes.c_int), ("typecode", ctypes.c_int)]


class _ElemwiseArg(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("typecode", ctypes.c_int), ("flags", ctypes.c_int)]


class _CliqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_ubyte * GA_COMM_ID_BYTES)]


_lib = None


def _already_loaded():
    """Path of a libgpuarray this process has mapped already (say through pygpu's
    extension modules), so that both users share one copy of the library's state."""
    try:
        with open("/proc/self/maps") as f:
            for line in f:
                path = line.rstrip("\n").split(" ")[-1]
                if os.path.basename(path).startswith("libgpuarray.so"):
                    return path
    except OSError:
        pass
    return None


def lib():
    """The loaded shared library with argument types declared. Raises OSError
    when it has not been built (python -m libgpuarray_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    L = ctypes.CDLL(_already_loaded() or LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    vp, ci, cu, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_size_t
    A = ctypes.POINTER(_GpuArrayStruct)
    psz, pss = ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_ssize_t)

    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)

    sig("gpuarray_error_str", ctypes.c_char_p, ci)
    sig("gpucontext_props_new", ci, ctypes.POINTER(vp))
    sig("gpucontext_props_cuda_dev", ci, vp, ci)
    sig("gpucontext_props_kernel_cache", ci, vp, ctypes.c_char_p)
    sig("gpucontext_props_alloc_cache", ci, vp, sz, sz)
    sig("gpucontext_props_del", None, vp)
    sig("gpucontext_init", ci, ctypes.POINTER(vp), ctypes.c_char_p, vp)
    sig("gpucontext_deref", None, vp)
    sig("gpucontext_property", ci, vp, ci, vp)
    sig("gpucontext_error", ctypes.c_char_p, vp, ci)
    sig("gpu_get_device_count", ci, ctypes.c_char_p, cu, ctypes.POINTER(cu))
    sig("gpudata_alloc", vp, vp, sz, vp, ci, ctypes.POINTER(ci))
    sig("gpudata_release", None, vp)
    sig("gpudata_retain", None, vp)
    sig("gpudata_read", ci, vp, vp, sz, sz)
    sig("gpudata_write", ci, vp, sz, vp, sz)
    sig("gpudata_memset", ci, vp, sz, ci)
    sig("gpudata_sync", ci, vp)
    sig("gpudata_property", ci, vp, ci, vp)
    sig("gpuarray_get_elsize", sz, ci)
    sig("gpuarray_get_extension", vp, ctypes.c_char_p)
    sig("gpuarray_elemwise_collapse", None, cu, ctypes.POINTER(cu), psz, ctypes.POINTER(pss))
    sig("gpuarray_type_flagsa", ci, cu, ctypes.POINTER(_ElemwiseArg))
    sig("GpuArray_empty", ci, A, vp, ci, cu, psz, ci)
    sig("GpuArray_zeros", ci, A, vp, ci, cu, psz, ci)
    sig("GpuArray_fromdata", ci, A, vp, sz, ci, cu, psz, pss, ci)
    sig("GpuArray_view", ci, A, A)
    sig("GpuArray_sync", ci, A)
    sig("GpuArray_index", ci, A, A, pss, pss, pss)
    sig("GpuArray_reshape", ci, A, A, cu, psz, ci, ci)
    sig("GpuArray_transpose", ci, A, A, ctypes.POINTER(cu))
    sig("GpuArray_clear", None, A)
    sig("GpuArray_move", ci, A, A)
    sig("GpuArray_setarray", ci, A, A)
    sig("GpuArray_write", ci, A, vp, sz)
    sig("GpuArray_read", ci, vp, sz, A)
    sig("GpuArray_memset", ci, A, ci)
    sig("GpuArray_copy", ci, A, A, ci)
    sig("GpuArray_fix_flags", None, A)
    sig("GpuArray_maxandargmax", ci, A, A, A, cu, ctypes.POINTER(cu))
    sig("GpuElemwise_new", vp, vp, ctypes.c_char_p, ctypes.c_char_p, cu,
        ctypes.POINTER(_ElemwiseArg), cu, ci)
    sig("GpuElemwise_free", None, vp)
    sig("GpuElemwise_call", ci, vp, ctypes.POINTER(vp), ci)
    sig("GpuReduction_new", ci, ctypes.POINTER(vp), vp, ci, cu, cu, ci, ci)
    sig("GpuReduction_free", None, vp)
    sig("GpuReduction_call", ci, vp, A, A, A, cu, ctypes.POINTER(ci), ci)
    sig("GpuReduction_call_sharded", ci, vp, vp, A, A, A, cu, ctypes.POINTER(ci), ci, sz, sz, ci)
    sig("GpuMapReduction_new", vp, vp, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p,
        ctypes.c_char_p, ci, cu, ctypes.POINTER(_ElemwiseArg), ci)
    sig("GpuMapReduction_free", None, vp)
    sig("GpuMapReduction_call", ci, vp, A, ctypes.POINTER(vp), cu, ctypes.POINTER(ci), ci)
    for name in ("gpucomm_new", "gpucomm_free", "gpucomm_gen_clique_id", "gpucomm_all_reduce",
                 "gpucomm_get_count", "gpucomm_get_rank"):
        if not hasattr(L, name):
            break
    else:
        sig("gpucomm_new", ci, ctypes.POINTER(vp), vp, _CliqueId, ci, ci)
        sig("gpucomm_free", None, vp)
        sig("gpucomm_gen_clique_id", ci, vp, ctypes.POINTER(_CliqueId))
        sig("gpucomm_get_count", ci, vp, ctypes.POINTER(ci))
        sig("gpucomm_get_rank", ci, vp, ctypes.POINTER(ci))
        sig("gpucomm_all_reduce", ci, vp, sz, vp, sz, sz, ci, ci, vp)
        sig("GpuArray_all_reduce", ci, A, A, ci, vp)
        sig("GpuArray_reduce", ci, A, A, ci, ci, vp)
        sig("GpuArray_reduce_from", ci, A, ci, ci, vp)
        sig("GpuArray_reduce_scatter", ci, A, A, ci, vp)
        sig("GpuArray_broadcast", ci, A, ci, vp)
        sig("GpuArray_all_gather", ci, A, A, vp)
    sig("gpuarray_b200_error_code", ci, vp)
    sig("gpuarray_b200_sum_f32_noalloc", ci, vp, sz, vp, vp)
    sig("gpuarray_b200_launch_count", ctypes.c_ulonglong)
    sig("gpuarray_b200_compile_check", ci, ctypes.c_char_p, vp, ctypes.c_char_p,
        ctypes.POINTER(sz), ctypes.POINTER(ctypes.c_char_p))
    _lib = L
    return L


def _check(ctx_ptr, err):
    if err != GA_NO_ERROR:
        msg = lib().gpucontext_error(ctx_ptr, err)
        raise GpuArrayException(msg.decode(errors="replace") if msg else "?", err)


class Context:
    """A gpucontext on one B200 (reference: pygpu.gpuarray.GpuContext / init())."""

    def __init__(self, dev=0, kernel_cache=None, alloc_cache_max=None):
        L = lib()
        props = ctypes.c_void_p()
        _check(None, L.gpucontext_props_new(ctypes.byref(props)))
        L.gpucontext_props_cuda_dev(props, dev)
        if kernel_cache is not None:
            L.gpucontext_props_kernel_cache(props, kernel_cache.encode())
        if alloc_cache_max is not None:
            L.gpucontext_props_alloc_cache(props, 0, alloc_cache_max)
        p = ctypes.c_void_p()
        _check(None, L.gpucontext_init(ctypes.byref(p), b"cuda", props))
        self.ptr = p
        self.dev = dev

    @classmethod
    def borrow(cls, pointer):
        """Wraps a gpucontext* owned by someone else (e.g. pygpu's GpuContext.ptr)."""
        self = cls.__new__(cls)
        self.ptr = ctypes.c_void_p(pointer)
        self.dev = None
        self._borrowed = True
        return self

    def close(self):
        if self.ptr is not None:
            if not getattr(self, "_borrowed", False):
                lib().gpucontext_deref(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def stream(self):
        """CUstream handle (int) of the context's stream, for event timing."""
        fn = lib().gpuarray_get_extension(b"cuda_get_stream")
        proto = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p)
        return proto(fn)(self.ptr) or 0

    def wrap_device_pointer(self, devptr, nbytes):
        """gpudata* over memory owned elsewhere (e.g. a torch tensor)."""
        fn = lib().gpuarray_get_extension(b"cuda_make_buf")
        proto = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_size_t)
        return proto(fn)(self.ptr, devptr, nbytes)

    def prop_uint(self, prop_id):
        v = ctypes.c_uint()
        _check(self.ptr, lib().gpucontext_property(self.ptr, prop_id, ctypes.byref(v)))
        return v.value

    def prop_size(self, prop_id):
        v = ctypes.c_size_t()
        _check(self.ptr, lib().gpucontext_property(self.ptr, prop_id, ctypes.byref(v)))
        return v.value

    def devname(self):
        buf = ctypes.create_string_buffer(256)
        _check(self.ptr, lib().gpucontext_property(self.ptr, 1, buf))
        return buf.value.decode()

    def sync(self):
        errbuf = ctypes.c_void_p()
        _check(self.ptr, lib().gpucontext_property(self.ptr, 8, ctypes.byref(errbuf)))
        _check(self.ptr, lib().gpudata_sync(errbuf))


class GpuArray:
    """Owns one C GpuArray struct (reference: pygpu.gpuarray.GpuArray)."""

    def __init__(self, ctx):
        self.ctx = ctx
        self.ga = _GpuArrayStruct()
        self._live = False

    # ---- construction ----
    @classmethod
    def empty(cls, ctx, shape, dtype, order="C"):
        self = cls(ctx)
        shape = tuple(int(s) for s in shape)
        dims = (ctypes.c_size_t * max(len(shape), 1))(*shape)
        _check(ctx.ptr, lib().GpuArray_empty(ctypes.byref(self.ga), ctx.ptr, typecode(dtype),
                                             len(shape), dims,
                                             GA_F_ORDER if order == "F" else GA_C_ORDER))
        self._live = True
        return self

    @classmethod
    def from_numpy(cls, ctx, arr, order=None):
        """Copies a NumPy array to the device, keeping C or F order."""
        arr = np.asarray(arr)
        if order is None:
            order = "F" if (arr.flags.f_contiguous and not arr.flags.c_contiguous) else "C"
        host = np.asfortranarray(arr) if order == "F" else np.ascontiguousarray(arr)
        self = cls.empty(ctx, arr.shape, arr.dtype, order)
        self.write(host)
        return self

    @classmethod
    def from_pointer(cls, ctx, devptr, shape, dtype, strides=None, nbytes=None, writeable=True):
        """View over external device memory (borrowed; caller keeps it alive).
        `devptr` is the address of element [0, ..., 0]; with `strides` (bytes,
        may be negative) the wrapped buffer is the span the view reaches, or
        `nbytes` starting at `devptr` when that is given."""
        dtype = np.dtype(dtype)
        shape = tuple(int(s) for s in shape)
        if strides is None:
            strides, step = [], dtype.itemsize
            for s in reversed(shape):
                strides.insert(0, step)
                step *= s
        lo = hi = 0
        if 0 not in shape:
            for d, st in zip(shape, strides):
                span = (d - 1) * int(st)
                if span < 0:
                    lo += span
                else:
                    hi += span
        hi += dtype.itemsize
        if nbytes is None:
            base, offset, nbytes = devptr + lo, -lo, hi - lo
        else:
            base, offset = devptr, 0
        buf = ctx.wrap_device_pointer(base, nbytes)
        if not buf:
            raise GpuArrayException("cuda_make_buf failed", GA_MEMORY_ERROR)
        self = cls(ctx)
        dims = (ctypes.c_size_t * max(len(shape), 1))(*shape)
        strs = (ctypes.c_ssize_t * max(len(shape), 1))(*strides)
        err = lib().GpuArray_fromdata(ctypes.byref(self.ga), buf, offset, typecode(dtype), len(shape),
                                      dims, strs, 1 if writeable else 0)
        lib().gpudata_release(buf)
        _check(ctx.ptr, err)
        self._live = True
        return self

    def _derived(self):
        out = GpuArray(self.ctx)
        return out

    # ---- views ----
    def transpose(self, axes=None):
        out = self._derived()
        ax = None if axes is None else (ctypes.c_uint * len(axes))(*axes)
        _check(self.ctx.ptr, lib().GpuArray_transpose(ctypes.byref(out.ga), ctypes.byref(self.ga), ax))
        out._live = True
        return out

    def reshape(self, shape, order="C", nocopy=False):
        out = self._derived()
        dims = (ctypes.c_size_t * max(len(shape), 1))(*shape)
        _check(self.ctx.ptr, lib().GpuArray_reshape(
            ctypes.byref(out.ga), ctypes.byref(self.ga), len(shape), dims,
            {"C": GA_C_ORDER, "F": GA_F_ORDER, "A": GA_ANY_ORDER}[order], 1 if nocopy else 0))
        out._live = True
        return out

    def __getitem__(self, key):
        """Basic slicing and integer indexing, as pygpu implements over GpuArray_index."""
        if not isinstance(key, tuple):
            key = (key,)
        nd = self.ga.nd
        key = key + (slice(None),) * (nd - len(key))
        starts = (ctypes.c_ssize_t * max(nd, 1))()
        stops = (ctypes.c_ssize_t * max(nd, 1))()
        steps = (ctypes.c_ssize_t * max(nd, 1))()
        for i, k in enumerate(key):
            dim = self.ga.dimensions[i]
            if isinstance(k, slice):
                a, b, c = k.indices(dim)
                if c < 0 and b < 0:
                    b = -1
                starts[i], stops[i], steps[i] = a, b, c
            else:
                k = int(k)
                if k < 0:
                    k += dim
                starts[i], stops[i], steps[i] = k, k + 1, 0
        out = self._derived()
        _check(self.ctx.ptr, lib().GpuArray_index(ctypes.byref(out.ga), ctypes.byref(self.ga),
                                                  starts, stops, steps))
        out._live = True
        return out

    def copy(self, order="C"):
        out = self._derived()
        _check(self.ctx.ptr, lib().GpuArray_copy(ctypes.byref(out.ga), ctypes.byref(self.ga),
                                                 GA_F_ORDER if order == "F" else GA_C_ORDER))
        out._live = True
        return out

    # ---- properties ----
    @property
    def shape(self):
        return tuple(self.ga.dimensions[i] for i in range(self.ga.nd))

    @property
    def strides(self):
        return tuple(self.ga.strides[i] for i in range(self.ga.nd))

    @property
    def dtype(self):
        return np_dtype(self.ga.typecode)

    @property
    def size(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self):
        return self.size * self.dtype.itemsize

    @property
    def flags(self):
        return self.ga.flags

    @property
    def devptr(self):
        """Device address of element [0,...,0]."""
        return ctypes.cast(self.ga.data, ctypes.POINTER(ctypes.c_uint64))[0] + self.ga.offset

    # ---- data ----
    def write(self, host):
        host = np.asarray(host)
        assert host.nbytes == self.nbytes, (host.nbytes, self.nbytes)
        _check(self.ctx.ptr, lib().GpuArray_write(ctypes.byref(self.ga),
                                                  host.ctypes.data_as(ctypes.c_void_p), host.nbytes))
        self.ctx.sync()

    def write_raw(self, pointer, nbytes):
        """Enqueue a host->device copy from a raw (ideally pinned) host pointer; no sync."""
        _check(self.ctx.ptr, lib().GpuArray_write(ctypes.byref(self.ga), pointer, nbytes))

    def read_raw(self, pointer, nbytes):
        _check(self.ctx.ptr, lib().GpuArray_read(pointer, nbytes, ctypes.byref(self.ga)))

    def memset(self, byte):
        _check(self.ctx.ptr, lib().GpuArray_memset(ctypes.byref(self.ga), byte))

    def to_numpy(self):
        """Device -> host; strided views go through a contiguous device copy."""
        fl = self.ga.flags
        if not (fl & (GA_C_CONTIGUOUS | GA_F_CONTIGUOUS)):
            return self.copy("C").to_numpy()
        order = "C" if (fl & GA_C_CONTIGUOUS) else "F"
        out = np.empty(self.shape, dtype=self.dtype, order=order)
        if out.nbytes:
            _check(self.ctx.ptr, lib().GpuArray_read(out.ctypes.data_as(ctypes.c_void_p),
                                                     out.nbytes, ctypes.byref(self.ga)))
        return out

    def clear(self):
        if self._live:
            lib().GpuArray_clear(ctypes.byref(self.ga))
            self._live = False

    def __del__(self):
        try:
            if self.ctx.ptr is not None:
                self.clear()
        except Exception:
            pass


class GpuElemwise:
    """GpuElemwise_new/_call/_free (reference: pygpu/_elemwise.pyx:104-221).

    args: sequence of (name, dtype-or-typecode, flags)."""

    def __init__(self, ctx, expr, args, preamble="", nd=0, convert_f16=False, flags=0):
        self.ctx = ctx
        self.ptr = None
        n = len(args)
        self._names = [a[0].encode() for a in args]
        arr = (_ElemwiseArg * max(n, 1))()
        self.argspec = []
        for i, (name, tc, fl) in enumerate(args):
            if not isinstance(tc, int):
                tc = typecode(tc)
            arr[i].name = self._names[i]
            arr[i].typecode = tc
            arr[i].flags = fl
            self.argspec.append((tc, fl))
        if convert_f16:
            flags |= GE_CONVERT_F16
        p = lib().GpuElemwise_new(ctx.ptr, preamble.encode() if preamble is not None else None,
                                  expr.encode(), n, arr, nd, flags)
        if not p:
            msg = lib().gpucontext_error(ctx.ptr, -1)
            # the code is stored in the context; recover it from the message table
            raise GpuArrayException(msg.decode(errors="replace"), _last_code(ctx))
        self.ptr = ctypes.c_void_p(p)

    def __call__(self, *args, broadcast=True, padshape=True, flags=None):
        if flags is None:
            flags = (GE_BROADCAST if broadcast else 0) | (GE_PADSHAPE if padshape else 0)
        n = len(self.argspec)
        assert len(args) == n
        ptrs = (ctypes.c_void_p * max(n, 1))()
        keep = []
        for i, (a, (tc, fl)) in enumerate(zip(args, self.argspec)):
            if fl & GE_SCALAR:
                v = np.array(a, dtype=np_dtype(tc))
                keep.append(v)
                ptrs[i] = v.ctypes.data
            else:
                ptrs[i] = ctypes.addressof(a.ga)
        _check(self.ctx.ptr, lib().GpuElemwise_call(self.ptr, ptrs, flags))

    def free(self):
        if self.ptr is not None:
            lib().GpuElemwise_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            if self.ctx.ptr is not None:
                self.free()
        except Exception:
            pass


def _last_code(ctx):
    """Error code of the last failure recorded on the context."""
    return lib().gpuarray_b200_error_code(ctx.ptr if ctx is not None else None)


class GpuReduction:
    """GpuReduction_new/_call/_free (include/gpuarray/reduction.h)."""

    def __init__(self, ctx, op, src_dtype, ndf=0, ndr=0):
        self.ctx = ctx
        self.op = op
        self.ptr = None
        p = ctypes.c_void_p()
        tc = src_dtype if isinstance(src_dtype, int) else typecode(src_dtype)
        _check(ctx.ptr, lib().GpuReduction_new(ctypes.byref(p), ctx.ptr, op, ndf, ndr, tc, 0))
        self.ptr = p

    def __call__(self, d0, d1, src, axes):
        ax = (ctypes.c_int * max(len(axes), 1))(*axes)
        _check(self.ctx.ptr, lib().GpuReduction_call(
            self.ptr, ctypes.byref(d0.ga) if d0 is not None else None,
            ctypes.byref(d1.ga) if d1 is not None else None, ctypes.byref(src.ga), len(axes), ax, 0))

    def free(self):
        if self.ptr is not None:
            lib().GpuReduction_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            if self.ctx.ptr is not None:
                self.free()
        except Exception:
            pass


def reduction_call_sharded(gr, comm, d0, d1, src, axes, shard_lo, shard_global, shard_axis=None):
    """GpuReduction_call_sharded (include/gpuarray/reduction.h): `src` is this
    rank's slab [shard_lo, shard_lo + extent) of an axis of extent shard_global;
    `shard_axis` defaults to the first listed axis. comm=None: no collective."""
    ax = (ctypes.c_int * max(len(axes), 1))(*axes)
    _check(gr.ctx.ptr, lib().GpuReduction_call_sharded(
        gr.ptr, comm.ptr if comm is not None else None,
        ctypes.byref(d0.ga) if d0 is not None else None,
        ctypes.byref(d1.ga) if d1 is not None else None, ctypes.byref(src.ga), len(axes), ax,
        axes[0] if shard_axis is None else shard_axis, shard_lo, shard_global, 0))


class GpuMapReduction:
    """GpuMapReduction_new/_call/_free (include/gpuarray/reduction.h): the
    reduction of a mapped expression over several broadcastable arguments, the
    C form of pygpu's ReductionKernel (pygpu/reduction.py:137-291).

    args: sequence of (name, dtype-or-typecode, flags) as for GpuElemwise;
    arrays are GE_READ, scalars GE_SCALAR."""

    def __init__(self, ctx, map_expr, reduce_expr, neutral, out_dtype, args, preamble="",
                 convert_f16=False):
        self.ctx = ctx
        self.ptr = None
        n = len(args)
        self._names = [a[0].encode() for a in args]
        arr = (_ElemwiseArg * max(n, 1))()
        self.argspec = []
        for i, (name, tc, fl) in enumerate(args):
            if not isinstance(tc, int):
                tc = typecode(tc)
            arr[i].name = self._names[i]
            arr[i].typecode = tc
            arr[i].flags = fl
            self.argspec.append((tc, fl))
        self.out_tc = out_dtype if isinstance(out_dtype, int) else typecode(out_dtype)
        p = lib().GpuMapReduction_new(ctx.ptr, preamble.encode() if preamble else None,
                                      map_expr.encode(), reduce_expr.encode(), str(neutral).encode(),
                                      self.out_tc, n, arr, GE_CONVERT_F16 if convert_f16 else 0)
        if not p:
            msg = lib().gpucontext_error(ctx.ptr, -1)
            raise GpuArrayException(msg.decode(errors="replace"), _last_code(ctx))
        self.ptr = ctypes.c_void_p(p)

    def __call__(self, out, *args, axes, broadcast=True, padshape=True):
        flags = (GE_BROADCAST if broadcast else 0) | (GE_PADSHAPE if padshape else 0)
        n = len(self.argspec)
        assert len(args) == n
        ptrs = (ctypes.c_void_p * max(n, 1))()
        keep = []
        for i, (a, (tc, fl)) in enumerate(zip(args, self.argspec)):
            if fl & GE_SCALAR:
                v = np.array(a, dtype=np_dtype(tc))
                keep.append(v)
                ptrs[i] = v.ctypes.data
            else:
                ptrs[i] = ctypes.addressof(a.ga)
        ax = (ctypes.c_int * max(len(axes), 1))(*axes)
        _check(self.ctx.ptr, lib().GpuMapReduction_call(self.ptr, ctypes.byref(out.ga), ptrs,
                                                        len(axes), ax, flags))

    def free(self):
        if self.ptr is not None:
            lib().GpuMapReduction_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            if self.ctx.ptr is not None:
                self.free()
        except Exception:
            pass


def maxandargmax(dst_max, dst_argmax, src, axes):
    """GpuArray_maxandargmax (include/gpuarray/array.h)."""
    ax = (ctypes.c_uint * max(len(axes), 1))(*axes)
    _check(src.ctx.ptr, lib().GpuArray_maxandargmax(ctypes.byref(dst_max.ga),
                                                    ctypes.byref(dst_argmax.ga),
                                                    ctypes.byref(src.ga), len(axes), ax))


class GpuComm:
    """gpucomm_* (include/gpuarray/buffer_collectives.h); one per rank."""

    @staticmethod
    def gen_clique_id(ctx):
        cid = _CliqueId()
        _check(ctx.ptr, lib().gpucomm_gen_clique_id(ctx.ptr, ctypes.byref(cid)))
        return ctypes.string_at(ctypes.addressof(cid), GA_COMM_ID_BYTES)

    def __init__(self, ctx, clique_id, ndev, rank):
        self.ctx = ctx
        cid = _CliqueId()
        assert len(clique_id) == GA_COMM_ID_BYTES
        ctypes.memmove(ctypes.addressof(cid), clique_id, GA_COMM_ID_BYTES)
        p = ctypes.c_void_p()
        _check(ctx.ptr, lib().gpucomm_new(ctypes.byref(p), ctx.ptr, cid, ndev, rank))
        self.ptr = p

    def all_reduce(self, src, dst, opcode):
        _check(self.ctx.ptr, lib().GpuArray_all_reduce(ctypes.byref(src.ga), ctypes.byref(dst.ga),
                                                       opcode, self.ptr))

    def reduce(self, src, dst, opcode, root):
        """dst is the root's result array; the other ranks pass None."""
        if dst is None:
            _check(self.ctx.ptr, lib().GpuArray_reduce_from(ctypes.byref(src.ga), opcode, root, self.ptr))
        else:
            _check(self.ctx.ptr, lib().GpuArray_reduce(ctypes.byref(src.ga), ctypes.byref(dst.ga),
                                                       opcode, root, self.ptr))

    def reduce_scatter(self, src, dst, opcode):
        _check(self.ctx.ptr, lib().GpuArray_reduce_scatter(ctypes.byref(src.ga), ctypes.byref(dst.ga),
                                                           opcode, self.ptr))

    def broadcast(self, arr, root):
        _check(self.ctx.ptr, lib().GpuArray_broadcast(ctypes.byref(arr.ga), root, self.ptr))

    def all_gather(self, src, dst):
        _check(self.ctx.ptr, lib().GpuArray_all_gather(ctypes.byref(src.ga), ctypes.byref(dst.ga),
                                                       self.ptr))

    def peer_state(self):
        """(state, reason, timed_out) of the communicator's peer-memory windows: state 0 before
        the first sharded reduction, 1 in use, -1 unavailable (reason says why; NCCL all-reduces
        are used instead); timed_out != 0 once a kernel gave up waiting for a rank."""
        f = lib().gpuarray_b200_comm_peer_state
        f.restype = ctypes.c_int
        f.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_uint)]
        reason, timed = ctypes.c_char_p(), ctypes.c_uint()
        st = f(self.ptr, ctypes.byref(reason), ctypes.byref(timed))
        return st, (reason.value or b"").decode(errors="replace"), int(timed.value)

    def free(self):
        if self.ptr is not None:
            lib().gpucomm_free(self.ptr)
            self.ptr = None
