"""Two ranks on two GPUs: sharded reductions finished with gpucomm_all_reduce
(NCCL over NVLink). Skipped when fewer than two GPUs are visible. NVLS is
switched off for these short-lived child processes."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _ngpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _worker(rank, world, q_id, q_err):
    try:
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        from libgpuarray_b200 import api, sharding
        from oracle import oracle as O
        ctx = api.Context(rank, kernel_cache=os.path.join(ROOT, ".kernel_cache"))
        if rank == 0:
            cid = api.GpuComm.gen_clique_id(ctx)
            for _ in range(world - 1):
                q_id.put(cid)
        else:
            cid = q_id.get(timeout=120)
        comm = api.GpuComm(ctx, cid, world, rank)

        def allreduce(arr, op):
            src = api.GpuArray.from_numpy(ctx, arr)
            dst = api.GpuArray.empty(ctx, arr.shape, arr.dtype)
            comm.all_reduce(src, dst, {"sum": api.GA_SUM, "prod": api.GA_PROD,
                                       "max": api.GA_MAX, "min": api.GA_MIN}[op])
            return dst.to_numpy()

        rng = np.random.default_rng(11)
        x = (2 * rng.random((64, 48, 256)) - 1)                  # fp64, same on both ranks
        lo, hi = sharding.shard_bounds(x.shape[0], world, rank)
        g = api.GpuArray.from_numpy(ctx, x[lo:hi])

        # SUM over everything: per-GPU partial + one all-reduce
        d = api.GpuArray.empty(ctx, (), np.float64)
        api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float64)(d, None, g, [0, 1, 2])
        tot = sharding.finish_accumulate(allreduce, d.to_numpy().reshape(1), "sum")[0]
        ref = float(np.sum(x.astype(np.longdouble)))
        assert abs(tot - ref) <= 1e-12 * np.log2(x.size) * np.abs(x).sum()

        # MIN / MAX over axes (0, 2)
        for name, op, red in (("min", api.GA_REDUCE_MIN, "min"), ("max", api.GA_REDUCE_MAX, "max")):
            dk = api.GpuArray.empty(ctx, (48,), np.float64)
            api.GpuReduction(ctx, op, np.float64)(dk, None, g, [0, 2])
            out = sharding.finish_accumulate(allreduce, dk.to_numpy(), red)
            want = x.min(axis=(0, 2)) if name == "min" else x.max(axis=(0, 2))
            assert (out == want).all()

        # MAXANDARGMAX over (0, 2) with ties: lowest global index wins
        xt = np.round(x * 8) / 8
        gt = api.GpuArray.from_numpy(ctx, xt[lo:hi])
        v = api.GpuArray.empty(ctx, (48,), np.float64)
        i = api.GpuArray.empty(ctx, (48,), np.int64)
        api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.float64)(v, i, gt, [0, 2])
        gi = sharding.global_flat_index(i.to_numpy(), lo, hi - lo, 0, [64, 256])
        bv, bi = sharding.finish_minmaxarg(allreduce, v.to_numpy(), gi)
        wv, wi = O.minmaxarg(xt, [0, 2])
        assert (bv == wv).all() and (bi == wi).all()
        # the other collectives of the reference's interface
        # (src/gpuarray/collectives.h): reduce to a root, reduce-scatter,
        # broadcast, all-gather
        a = np.arange(6 * world, dtype=np.float32).reshape(world, 6) + 100 * rank
        ga = api.GpuArray.from_numpy(ctx, a)
        if rank == 1:
            res = api.GpuArray.empty(ctx, a.shape, np.float32)
            comm.reduce(ga, res, api.GA_SUM, 1)
            want = sum(np.arange(6 * world, dtype=np.float32).reshape(world, 6) + 100 * r
                       for r in range(world))
            assert (res.to_numpy() == want).all()
        else:
            comm.reduce(ga, None, api.GA_SUM, 1)
        part = api.GpuArray.empty(ctx, (6,), np.float32)
        comm.reduce_scatter(ga, part, api.GA_MAX)
        assert (part.to_numpy() == a[rank] - 100 * rank + 100 * (world - 1)).all()
        b = api.GpuArray.from_numpy(ctx, np.full(5, rank + 7, np.int32))
        comm.broadcast(b, 0)
        assert (b.to_numpy() == 7).all()
        mine = api.GpuArray.from_numpy(ctx, np.full(3, rank, np.int64))
        everyone = api.GpuArray.empty(ctx, (world, 3), np.int64)
        comm.all_gather(mine, everyone)
        assert (everyone.to_numpy() == np.arange(world)[:, None]).all()
        ctx.sync()
        comm.free()
        ctx.close()
    except Exception as e:
        import traceback
        q_err.put("rank %d: %s\n%s" % (rank, e, traceback.format_exc()))


@pytest.mark.skipif(_ngpus() < 2, reason="needs two GPUs")
def test_sharded_reduction_with_gpucomm():
    import torch.multiprocessing as mp
    m = mp.get_context("spawn")
    q_id, q_err = m.Queue(), m.Queue()
    world = 2
    procs = [m.Process(target=_worker, args=(r, world, q_id, q_err)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
    msgs = []
    while not q_err.empty():
        msgs.append(q_err.get())
    assert not hung, "rank hung"
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs)
