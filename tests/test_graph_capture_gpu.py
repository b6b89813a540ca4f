"""Repeated identical calls captured in a CUDA graph.

The library enqueues everything on one stream that a host framework can get
with the `cuda_get_stream` extension (reference: src/gpuarray/ext_cuda.h:20-44).
Once an operator has run once (kernels compiled, scratch of split reductions
allocated) a call allocates nothing and synchronises nothing, so a sequence of
calls can be captured from that stream and replayed. The capture itself is done
with torch's CUDA-graph wrapper, which is only plumbing here.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_elemwise_and_reductions_replay_from_a_graph(api, ctx, rng):
    torch = pytest.importorskip("torch")
    stream = torch.cuda.ExternalStream(ctx.stream, device=0)
    rows, cols = 2048, 3000
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    gx = api.GpuArray.from_numpy(ctx, x)
    gy = api.GpuArray.empty(ctx, (rows, cols), np.float32)
    gmax = api.GpuArray.empty(ctx, (rows,), np.float32)
    garg = api.GpuArray.empty(ctx, (rows,), np.int64)
    gsum = api.GpuArray.empty(ctx, (), np.float32)
    ge = api.GpuElemwise(ctx, "y = x * s + 1.0f", [("x", np.float32, api.GE_READ),
                                                   ("s", np.float32, api.GE_SCALAR),
                                                   ("y", np.float32, api.GE_WRITE)], nd=2)
    rmax = api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.float32)
    rsum = api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float32)

    def sequence():
        ge(gx, np.float32(0.5), gy)
        rmax(gmax, garg, gy, [1])
        rsum(gsum, None, gy, [0, 1])          # a split reduction: scratch + arrival counters

    sequence()                                # warm: compile, allocate scratch
    ctx.sync()
    launches0 = api.lib().gpuarray_b200_launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
        sequence()
    captured = api.lib().gpuarray_b200_launch_count() - launches0
    assert captured == 3

    for trial in range(3):                    # new input contents, same buffers
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        gx.write_raw(x.ctypes.data, x.nbytes)
        gy.memset(0)
        ctx.sync()
        graph.replay()
        torch.cuda.synchronize()
        want = (x * np.float32(0.5) + np.float32(1.0)).astype(np.float32)
        got = gy.to_numpy()
        assert np.abs(got - want).max() <= 1e-6       # FMA contraction vs two roundings
        assert (gmax.to_numpy() == got.max(axis=1)).all()
        assert (garg.to_numpy() == got.argmax(axis=1)).all()
        ref = got.astype(np.float64).sum()
        assert abs(float(gsum.to_numpy()) - ref) <= 1e-6 * np.log2(got.size) * np.abs(got).sum()
