"""Bit-for-bit comparison with the REFERENCE's own kernels on the GPU.

oracle/Makefile compiles the reference library (CUDA backend) from its sources
where they lie into oracle/_ref/libgpuarray_ref.so, with the one-character
buffer fix its detect_arch needs for compute capability 10.0
(src/gpuarray_buffer_cuda.c:1088-1102). A child process (reference_kernels_driver.py)
loads only that library and runs the kernels the reference generates itself:
`elem` contiguous (src/gpuarray_elemwise.c:444-545) and strided with broadcast
and float16 conversion (:123-250), and `maxandargmax`
(src/gpuarray_reduction.c:520-607). This process runs the same calls through
this repository's library and compares every output element by bit pattern.
Shapes are small because the reference's reduction gives one thread a whole
row. Skipped when the reference build is absent or cannot start on this
machine (the reason is printed)."""
import ctypes
import ctypes.util
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libgpuarray_ref.so")


def _mapped_path(soname):
    """Path of a shared object this process can load (the reference dlopens the
    unversioned names libcuda.so / libnvrtc.so, which only development installs have)."""
    try:
        ctypes.CDLL(soname)
    except OSError:
        return None
    with open("/proc/self/maps") as f:
        for line in f:
            path = line.rstrip("\n").split(" ")[-1]
            if os.path.basename(path).startswith(soname.split(".so")[0] + ".so"):
                return path
    return None


@pytest.fixture(scope="module")
def reference_outputs(tmp_path_factory, oracle):
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libgpuarray_ref.so has not been built (needs the reference tree)")
    work = tmp_path_factory.mktemp("refkernels")
    rng = np.random.Generator(np.random.PCG64(0))
    n = 1 << 20
    a = (2 * rng.random(n, dtype=np.float32) - 1)
    b = (2 * rng.random(n, dtype=np.float32) - 1)
    rng3 = np.random.Generator(np.random.PCG64(3))
    buf = rng3.standard_normal((4, 14, 14, 64), dtype=np.float32).astype(np.float16)
    bias = (0.2 * rng3.random((1, 64, 1, 1), dtype=np.float32) - 0.1).astype(np.float16)
    rng2 = np.random.Generator(np.random.PCG64(2))
    x3 = (np.round(rng2.standard_normal((256, 32000), dtype=np.float32) * 64) / 64).astype(np.float32)
    dims = (117, 37, 2, 1, 2, 1, 2, 1)
    xhr = oracle.pcg_fill_f32(1, int(np.prod(dims))).reshape(dims)
    data = {"c1_a": a, "c1_b": b, "c4_buf": buf, "c4_bias": bias, "c3_x": x3, "hr_x": xhr}
    for k, v in data.items():
        np.save(os.path.join(work, k + ".npy"), v)
    # the unversioned library names the reference asks the loader for
    links = os.path.join(work, "libs")
    os.makedirs(links)
    for soname, plain in (("libcuda.so.1", "libcuda.so"), ("libnvrtc.so.12", "libnvrtc.so")):
        path = _mapped_path(soname)
        if path is None and soname.startswith("libnvrtc"):
            cand = "/usr/local/cuda/lib64/libnvrtc.so.12"
            path = cand if os.path.exists(cand) else None
        if path is None:
            pytest.skip("%s is not loadable here" % soname)
        os.symlink(path, os.path.join(links, plain))
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = links + os.pathsep + os.path.dirname(os.path.realpath(
        os.path.join(links, "libnvrtc.so"))) + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "reference_kernels_driver.py"), str(work)],
                       env=env, capture_output=True, text=True, timeout=900)
    if "REFERENCE_INIT_FAILED" in r.stdout:
        pytest.skip("the reference library cannot create a context here: " + r.stdout.strip()[-300:])
    assert r.returncode == 0 and "REFERENCE_DONE" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])
    out = {k: np.load(os.path.join(work, k + ".npy"))
           for k in ("c1_out", "c4_out", "c3_v", "c3_i", "hr_v", "hr_i")}
    out.update(data)
    return out


def test_contiguous_elemwise_matches_the_reference_kernel(api, ctx, reference_outputs):
    d = reference_outputs
    R, W = api.GE_READ, api.GE_WRITE
    ga, gb = api.GpuArray.from_numpy(ctx, d["c1_a"]), api.GpuArray.from_numpy(ctx, d["c1_b"])
    go = api.GpuArray.empty(ctx, d["c1_a"].shape, np.float32)
    ge = api.GpuElemwise(ctx, "out = a * b + 0.5f", [("a", np.float32, R), ("b", np.float32, R),
                                                      ("out", np.float32, W)], nd=1)
    ge(ga, gb, go)
    assert go.to_numpy().view(np.uint32).tobytes() == d["c1_out"].view(np.uint32).tobytes()


def test_strided_broadcast_f16_elemwise_matches_the_reference_kernel(api, ctx, reference_outputs):
    d = reference_outputs
    R, W = api.GE_READ, api.GE_WRITE
    gbuf = api.GpuArray.from_numpy(ctx, d["c4_buf"])
    gx = gbuf.transpose((0, 3, 1, 2))
    gbias = api.GpuArray.from_numpy(ctx, d["c4_bias"])
    n, h, w, c = d["c4_buf"].shape
    gy = api.GpuArray.empty(ctx, (n, c, h, w), np.float16)
    ge = api.GpuElemwise(ctx, "y = fmaxf(x + bias, 0.0f)", [("x", np.float16, R), ("bias", np.float16, R),
                                                            ("y", np.float16, W)], nd=4, convert_f16=True)
    ge(gx, gbias, gy, flags=api.GE_BROADCAST)
    assert gy.to_numpy().view(np.uint16).tobytes() == d["c4_out"].view(np.uint16).tobytes()


@pytest.mark.parametrize("tag,axes", [("c3", [1]), ("hr", [2, 4, 7, 5])])
def test_maxandargmax_matches_the_reference_kernel(api, ctx, reference_outputs, tag, axes):
    d = reference_outputs
    x = d[tag + "_x"]
    g = api.GpuArray.from_numpy(ctx, x)
    kept = [s for i, s in enumerate(x.shape) if i not in axes]
    gv, gi = api.GpuArray.empty(ctx, kept, np.float32), api.GpuArray.empty(ctx, kept, np.uint64)
    api.maxandargmax(gv, gi, g, axes)
    assert gv.to_numpy().view(np.uint32).tobytes() == d[tag + "_v"].view(np.uint32).tobytes()
    assert (gi.to_numpy() == d[tag + "_i"]).all()
