"""Child process of tests/test_reference_kernels_gpu.py: runs the REFERENCE's own
generated kernels (`elem` from src/gpuarray_elemwise.c:123-250 and :444-545,
`maxandargmax` from src/gpuarray_reduction.c:520-607) on the GPU, through the
reference's library compiled in place by oracle/Makefile
(oracle/_ref/libgpuarray_ref.so), on inputs read from .npy files; writes the
outputs as .npy files. Only the reference library is loaded here, by plain
ctypes over its C API (the struct layouts are the shared ABI)."""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from libgpuarray_b200.api import (_GpuArrayStruct, _ElemwiseArg, typecode, GE_READ, GE_WRITE,  # noqa: E402
                                  GE_CONVERT_F16, GE_BROADCAST, GA_C_ORDER)


def main(workdir):
    L = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libgpuarray_ref.so"), mode=ctypes.RTLD_LOCAL)
    vp, ci, cu, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_size_t
    A = ctypes.POINTER(_GpuArrayStruct)
    L.gpucontext_props_new.argtypes = [ctypes.POINTER(vp)]
    L.gpucontext_props_cuda_dev.argtypes = [vp, ci]
    L.gpucontext_init.argtypes = [ctypes.POINTER(vp), ctypes.c_char_p, vp]
    L.gpucontext_error.restype = ctypes.c_char_p
    L.gpucontext_error.argtypes = [vp, ci]
    L.GpuArray_empty.argtypes = [A, vp, ci, cu, ctypes.POINTER(sz), ci]
    L.GpuArray_write.argtypes = [A, vp, sz]
    L.GpuArray_read.argtypes = [vp, sz, A]
    L.GpuArray_transpose.argtypes = [A, A, ctypes.POINTER(cu)]
    L.GpuArray_maxandargmax.argtypes = [A, A, A, cu, ctypes.POINTER(cu)]
    L.GpuElemwise_new.restype = vp
    L.GpuElemwise_new.argtypes = [vp, ctypes.c_char_p, ctypes.c_char_p, cu, ctypes.POINTER(_ElemwiseArg), cu, ci]
    L.GpuElemwise_call.argtypes = [vp, ctypes.POINTER(vp), ci]

    props, ctx = vp(), vp()
    assert L.gpucontext_props_new(ctypes.byref(props)) == 0
    L.gpucontext_props_cuda_dev(props, 0)
    err = L.gpucontext_init(ctypes.byref(ctx), b"cuda", props)
    if err != 0:
        msg = L.gpucontext_error(None, err)
        print("REFERENCE_INIT_FAILED: %s" % (msg.decode(errors="replace") if msg else err))
        return 3

    def check(code, what):
        if code != 0:
            msg = L.gpucontext_error(ctx, code)
            raise RuntimeError("%s: %s" % (what, msg.decode(errors="replace") if msg else code))

    def upload(a):
        g = _GpuArrayStruct()
        dims = (sz * max(a.ndim, 1))(*a.shape)
        check(L.GpuArray_empty(ctypes.byref(g), ctx, typecode(a.dtype), a.ndim, dims, GA_C_ORDER), "empty")
        a = np.ascontiguousarray(a)
        check(L.GpuArray_write(ctypes.byref(g), a.ctypes.data_as(vp), a.nbytes), "write")
        return g

    def empty(shape, dtype):
        g = _GpuArrayStruct()
        dims = (sz * max(len(shape), 1))(*shape)
        check(L.GpuArray_empty(ctypes.byref(g), ctx, typecode(dtype), len(shape), dims, GA_C_ORDER), "empty")
        return g

    def download(g, shape, dtype):
        out = np.empty(shape, dtype)
        check(L.GpuArray_read(out.ctypes.data_as(vp), out.nbytes, ctypes.byref(g)), "read")
        return out

    def elemwise(expr, spec, arrays, flags=0, call_flags=0):
        args = (_ElemwiseArg * len(spec))()
        names = [s[0].encode() for s in spec]
        for i, (nm, dt, fl) in enumerate(spec):
            args[i].name, args[i].typecode, args[i].flags = names[i], typecode(dt), fl
        ge = L.GpuElemwise_new(ctx, b"", expr.encode(), len(spec), args, 0, flags)
        if not ge:
            raise RuntimeError("GpuElemwise_new: %s" % L.gpucontext_error(ctx, 0).decode(errors="replace"))
        ptrs = (vp * len(spec))(*[ctypes.addressof(a) for a in arrays])
        check(L.GpuElemwise_call(ge, ptrs, call_flags), "GpuElemwise_call")

    # 1. contiguous `elem`: out = a * b + 0.5f
    a = np.load(os.path.join(workdir, "c1_a.npy"))
    b = np.load(os.path.join(workdir, "c1_b.npy"))
    ga, gb, go = upload(a), upload(b), empty(a.shape, np.float32)
    elemwise("out = a * b + 0.5f", [("a", np.float32, GE_READ), ("b", np.float32, GE_READ),
                                    ("out", np.float32, GE_WRITE)], [ga, gb, go])
    np.save(os.path.join(workdir, "c1_out.npy"), download(go, a.shape, np.float32))

    # 2. strided + broadcast `elem`: y = max(x + bias, 0) on an NHWC buffer viewed as NCHW, fp16
    buf = np.load(os.path.join(workdir, "c4_buf.npy"))
    bias = np.load(os.path.join(workdir, "c4_bias.npy"))
    gbuf, gbias = upload(buf), upload(bias)
    gx = _GpuArrayStruct()
    check(L.GpuArray_transpose(ctypes.byref(gx), ctypes.byref(gbuf), (cu * 4)(0, 3, 1, 2)), "transpose")
    n, h, w, c = buf.shape
    gy = empty((n, c, h, w), np.float16)
    elemwise("y = fmaxf(x + bias, 0.0f)", [("x", np.float16, GE_READ), ("bias", np.float16, GE_READ),
                                           ("y", np.float16, GE_WRITE)], [gx, gbias, gy],
             flags=GE_CONVERT_F16, call_flags=GE_BROADCAST)
    np.save(os.path.join(workdir, "c4_out.npy"), download(gy, (n, c, h, w), np.float16))

    # 3. maxandargmax over the last axis, and over four axes of an 8-d array
    for tag, axes in (("c3", [1]), ("hr", [2, 4, 7, 5])):
        x = np.load(os.path.join(workdir, tag + "_x.npy"))
        g = upload(x)
        kept = [d for i, d in enumerate(x.shape) if i not in axes]
        gv, gi = empty(kept, np.float32), empty(kept, np.uint64)
        check(L.GpuArray_maxandargmax(ctypes.byref(gv), ctypes.byref(gi), ctypes.byref(g), len(axes),
                                      (cu * len(axes))(*axes)), "GpuArray_maxandargmax")
        np.save(os.path.join(workdir, tag + "_v.npy"), download(gv, kept, np.float32))
        np.save(os.path.join(workdir, tag + "_i.npy"), download(gi, kept, np.uint64))
    print("REFERENCE_DONE")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1]))
