"""Two ranks on two GPUs: reductions whose reduced extent is sharded, combined
on the device - once through the communicator's peer-memory windows (one
exchange kernel per GPU over NVLink, templates/ga_exchange.cuh) and once
through gpucomm_all_reduce (NCCL), the path taken where the windows cannot be
set up. Skipped when fewer than two GPUs are visible. NVLS is switched off for
these short-lived child processes."""
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


def _worker(rank, world, q_id, q_err, peer):
    """Every collective is enqueued BEFORE anything is checked: a rank that
    failed an assertion between two collectives would leave its peer's kernel
    waiting on the GPU for a rank that has already left."""
    try:
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        os.environ["GPUARRAY_B200_PEER_TIMEOUT_MS"] = "4000"
        if not peer:
            os.environ["GPUARRAY_B200_NO_PEER_WINDOW"] = "1"
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
        got = {}

        rng = np.random.default_rng(11)
        x = (2 * rng.random((64, 48, 256)) - 1)                  # fp64, same on both ranks
        lo, hi = sharding.shard_bounds(x.shape[0], world, rank)
        g = api.GpuArray.from_numpy(ctx, x[lo:hi])

        # SUM over everything, MIN / MAX over axes (0, 2): per-GPU partial + one all-reduce,
        # through the sharded entry point of the C API
        d = api.GpuArray.empty(ctx, (), np.float64)
        api.reduction_call_sharded(api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float64), comm, d, None,
                                   g, [0, 1, 2], lo, 64)
        got["sum"] = d
        for name, op in (("min", api.GA_REDUCE_MIN), ("max", api.GA_REDUCE_MAX)):
            dk = api.GpuArray.empty(ctx, (48,), np.float64)
            api.reduction_call_sharded(api.GpuReduction(ctx, op, np.float64), comm, dk, None, g, [0, 2],
                                       lo, 64)
            got[name] = dk

        # (value, first global index) over (0, 2) and (2, 0) with ties, a NaN as the first
        # element of the whole extent, a NaN at the start of the second slab, signed zeros
        xt = np.round(x * 8) / 8
        xt[0, 3, 0] = np.nan
        xt[32, 4, 0] = np.nan
        xt[:, 6, :] = -1.0
        xt[40, 6, 3] = -0.0
        xt[10, 6, 200] = 0.0
        gt = api.GpuArray.from_numpy(ctx, xt[lo:hi])
        for tag, opname, axes in (("maxarg02", "MAXANDARGMAX", [0, 2]), ("minarg20", "MINANDARGMIN", [2, 0])):
            v = api.GpuArray.empty(ctx, (48,), np.float64)
            i = api.GpuArray.empty(ctx, (48,), np.int64)
            api.reduction_call_sharded(api.GpuReduction(ctx, getattr(api, "GA_REDUCE_" + opname), np.float64),
                                       comm, v, i, gt, axes, lo, 64, shard_axis=0)
            got[tag] = (v, i)

        # value-only extremes of the array with signed zeros and NaNs: sharded axis slowest
        # (the keyed exchange) and fastest (falls back to the pair exchange)
        for tag, opname, axes in (("max02", "MAX", [0, 2]), ("max20", "MAX", [2, 0]), ("min02", "MIN", [0, 2])):
            v = api.GpuArray.empty(ctx, (48,), np.float64)
            api.reduction_call_sharded(api.GpuReduction(ctx, getattr(api, "GA_REDUCE_" + opname), np.float64),
                                       comm, v, None, gt, axes, lo, 64, shard_axis=0)
            got[tag] = v

        # destinations that are not dense, an index-only operator, other types, and many
        # exchanges in a row (the two halves of the windows alternate)
        wide_v = api.GpuArray.from_numpy(ctx, np.full((48, 2), 7.0))
        wide_i = api.GpuArray.from_numpy(ctx, np.full((48, 2), -7, np.int64))
        api.reduction_call_sharded(api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.float64), comm,
                                   wide_v[:, 0], wide_i[:, 1], gt, [0, 2], lo, 64, shard_axis=0)
        only_i = api.GpuArray.empty(ctx, (48,), np.uint64)
        api.reduction_call_sharded(api.GpuReduction(ctx, api.GA_REDUCE_ARGMIN, np.float64), comm, None,
                                   only_i, gt, [0, 2], lo, 64, shard_axis=0)
        xh = (np.round(rng.standard_normal((64, 300)) * 4) / 4).astype(np.float16)
        gh = api.GpuArray.from_numpy(ctx, xh[lo:hi])
        sum_h = api.GpuArray.empty(ctx, (300,), np.float16)
        api.reduction_call_sharded(api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float16), comm, sum_h, None,
                                   gh, [0], lo, 64)
        max_h = (api.GpuArray.empty(ctx, (300,), np.float16), api.GpuArray.empty(ctx, (300,), np.int64))
        api.reduction_call_sharded(api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.float16), comm,
                                   max_h[0], max_h[1], gh, [0], lo, 64)
        xb = (rng.random((64, 5000)) < 0.01).astype(np.uint8)
        gb = api.GpuArray.from_numpy(ctx, xb[lo:hi])
        any_b = api.GpuArray.empty(ctx, (5000,), np.bool_)
        api.reduction_call_sharded(api.GpuReduction(ctx, api.GA_REDUCE_ANY, np.uint8), comm, any_b, None,
                                   gb, [0], lo, 64)
        x8 = rng.integers(0, 256, (64, 5000)).astype(np.uint8)
        g8 = api.GpuArray.from_numpy(ctx, x8[lo:hi])
        xor_d = api.GpuArray.empty(ctx, (5000,), np.uint8)
        try:            # bitwise folds exist in the exchange kernel only; both ranks agree on which path runs
            api.reduction_call_sharded(api.GpuReduction(ctx, api.GA_REDUCE_XOR, np.uint8), comm, xor_d, None,
                                       g8, [0], lo, 64)
            xor_code = 0
        except api.GpuArrayException as e:
            xor_code = e.code
        xi = rng.integers(-1000, 1000, (64, 70000)).astype(np.int32)     # 70000 outputs: 64 CTAs, ragged chunks
        gi32 = api.GpuArray.from_numpy(ctx, xi[lo:hi])
        min_i = (api.GpuArray.empty(ctx, (70000,), np.int32), api.GpuArray.empty(ctx, (70000,), np.int64))
        api.reduction_call_sharded(api.GpuReduction(ctx, api.GA_REDUCE_MINANDARGMIN, np.int32), comm,
                                   min_i[0], min_i[1], gi32, [0], lo, 64)
        many = []
        gr_sum = api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float64)
        gr_max = api.GpuReduction(ctx, api.GA_REDUCE_MAXANDARGMAX, np.float64)
        for rep in range(24):
            dv = api.GpuArray.empty(ctx, (48,), np.float64)
            if rep % 2:
                api.reduction_call_sharded(gr_sum, comm, dv, None, g, [0, 2], lo, 64)
                many.append((dv, None))
            else:
                di = api.GpuArray.empty(ctx, (48,), np.int64)
                api.reduction_call_sharded(gr_max, comm, dv, di, gt, [0, 2], lo, 64, shard_axis=0)
                many.append((dv, di))
        state = comm.peer_state()

        # the other collectives of the reference's interface (src/gpuarray/collectives.h):
        # reduce to a root, reduce-scatter, broadcast, all-gather
        a = np.arange(6 * world, dtype=np.float32).reshape(world, 6) + 100 * rank
        ga = api.GpuArray.from_numpy(ctx, a)
        res = api.GpuArray.empty(ctx, a.shape, np.float32)
        comm.reduce(ga, res if rank == 1 else None, api.GA_SUM, 1)
        part = api.GpuArray.empty(ctx, (6,), np.float32)
        comm.reduce_scatter(ga, part, api.GA_MAX)
        b = api.GpuArray.from_numpy(ctx, np.full(5, rank + 7, np.int32))
        comm.broadcast(b, 0)
        mine = api.GpuArray.from_numpy(ctx, np.full(3, rank, np.int64))
        everyone = api.GpuArray.empty(ctx, (world, 3), np.int64)
        comm.all_gather(mine, everyone)
        ctx.sync()

        # ---- nothing below enqueues a collective
        tot = float(got["sum"].to_numpy())
        ref = float(np.sum(x.astype(np.longdouble)))
        assert abs(tot - ref) <= 1e-12 * np.log2(x.size) * np.abs(x).sum()
        assert (got["min"].to_numpy() == x.min(axis=(0, 2))).all()
        assert (got["max"].to_numpy() == x.max(axis=(0, 2))).all()
        for tag, is_min, axes in (("maxarg02", False, [0, 2]), ("minarg20", True, [2, 0])):
            bv, bi = got[tag][0].to_numpy(), got[tag][1].to_numpy()
            wv, wi = O.minmaxarg(xt, axes, is_min=is_min)
            assert (bi == wi).all(), (tag, bi, wi)
            nan = np.isnan(wv)
            assert (np.isnan(bv) == nan).all() and bv[~nan].tobytes() == wv[~nan].tobytes(), tag
        assert state[0] == (1 if peer else -1) and state[2] == 0, state
        assert comm.peer_state()[2] == 0
        for tag, is_min, axes in (("max02", False, [0, 2]), ("max20", False, [2, 0]), ("min02", True, [0, 2])):
            bv = got[tag].to_numpy()
            wv = O.minmaxarg(xt, axes, is_min=is_min)[0]
            nan = np.isnan(wv)
            assert (np.isnan(bv) == nan).all() and bv[~nan].tobytes() == wv[~nan].tobytes(), tag
        assert np.signbit(got["max20"].to_numpy()[6]) and not np.signbit(got["max02"].to_numpy()[6])
        wv, wi = O.minmaxarg(xt, [0, 2])
        ok = ~np.isnan(wv)
        hv, hi_ = wide_v.to_numpy(), wide_i.to_numpy()
        assert (hi_[:, 1] == wi).all() and (hi_[:, 0] == -7).all() and (hv[:, 1] == 7.0).all()
        assert (np.isnan(hv[:, 0]) == ~ok).all() and hv[ok, 0].tobytes() == wv[ok].tobytes()
        assert (only_i.to_numpy().astype(np.int64) == O.minmaxarg(xt, [0, 2], is_min=True)[1]).all()
        assert (sum_h.to_numpy() == xh.astype(np.float64).sum(0).astype(np.float16)).all()   # quarter steps: exact
        wv, wi = O.minmaxarg(xh, [0])
        assert max_h[0].to_numpy().tobytes() == wv.tobytes() and (max_h[1].to_numpy() == wi).all()
        assert (any_b.to_numpy() == xb.any(0)).all()
        if peer:
            assert xor_code == 0 and (xor_d.to_numpy() == np.bitwise_xor.reduce(x8, axis=0)).all()
        else:
            assert xor_code == api.GA_UNSUPPORTED_ERROR
        wv, wi = O.minmaxarg(xi, [0], is_min=True)
        assert (min_i[0].to_numpy() == wv).all() and (min_i[1].to_numpy() == wi).all()
        wv, wi = O.minmaxarg(xt, [0, 2])
        first_sum = None
        for rep, (dv, di) in enumerate(many):
            if di is None:
                first_sum = dv.to_numpy() if first_sum is None else first_sum
                assert dv.to_numpy().tobytes() == first_sum.tobytes()               # same bits every time
                assert np.allclose(first_sum, x.sum(axis=(0, 2)), rtol=1e-12, atol=1e-9)
            else:
                assert (di.to_numpy() == wi).all() and dv.to_numpy()[ok].tobytes() == wv[ok].tobytes()
        if rank == 1:
            want = sum(np.arange(6 * world, dtype=np.float32).reshape(world, 6) + 100 * r
                       for r in range(world))
            assert (res.to_numpy() == want).all()
        assert (part.to_numpy() == a[rank] - 100 * rank + 100 * (world - 1)).all()
        assert (b.to_numpy() == 7).all()
        assert (everyone.to_numpy() == np.arange(world)[:, None]).all()
        comm.free()
        ctx.close()
    except Exception as e:
        import traceback
        q_err.put("rank %d: %s\n%s" % (rank, e, traceback.format_exc()))


def _transfer_worker(q_err):
    """One process, two contexts: a cross-GPU transfer followed at once by an
    overwrite and a release of the source. The copy is ordered on both streams
    with events (ga_context.c, gpudata_transfer), so it must carry the old
    contents."""
    try:
        import ctypes
        from libgpuarray_b200 import api
        c0 = api.Context(0, kernel_cache=os.path.join(ROOT, ".kernel_cache"))
        c1 = api.Context(1, kernel_cache=os.path.join(ROOT, ".kernel_cache"))
        L = api.lib()
        L.GpuArray_transfer.restype = ctypes.c_int
        L.GpuArray_transfer.argtypes = [ctypes.POINTER(api._GpuArrayStruct), ctypes.POINTER(api._GpuArrayStruct)]
        n = 1 << 26                                              # 256 MiB: the copy takes a while
        for rep in range(3):
            src = api.GpuArray.from_numpy(c0, np.full(n, rep + 1, np.float32))
            dst = api.GpuArray.empty(c1, (n,), np.float32)
            assert L.GpuArray_transfer(ctypes.byref(dst.ga), ctypes.byref(src.ga)) == 0
            src.memset(0)                                        # overwrite ...
            src.clear()                                          # ... and release the source at once
            again = api.GpuArray.empty(c0, (n,), np.float32)     # the freed block is handed out again
            again.memset(0xFF)
            out = dst.to_numpy()
            assert (out == rep + 1).all(), (rep, out[:4], out[-4:])
        c0.close()
        c1.close()
    except Exception as e:
        import traceback
        q_err.put("transfer: %s\n%s" % (e, traceback.format_exc()))


def _absent_rank_worker(rank, world, q_id, q_err, ready, done):
    """Failure detection without a fault: after one complete exchange, rank 1 simply makes no
    further call (it sits idle on the host, nothing of it in flight) while rank 0 makes one
    more. Rank 0's exchange kernel waits for a flag that nothing sets, gives up after the
    300 ms limit and returns; the host then finds the status word set and refuses further
    sharded calls on that communicator."""
    try:
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        os.environ["GPUARRAY_B200_PEER_TIMEOUT_MS"] = "300"
        from libgpuarray_b200 import api
        ctx = api.Context(rank, kernel_cache=os.path.join(ROOT, ".kernel_cache"))
        if rank == 0:
            cid = api.GpuComm.gen_clique_id(ctx)
            q_id.put(cid)
        else:
            cid = q_id.get(timeout=120)
        comm = api.GpuComm(ctx, cid, world, rank)
        x = np.arange(64 * 100, dtype=np.float64).reshape(64, 100)
        g = api.GpuArray.from_numpy(ctx, x[rank * 32:(rank + 1) * 32])
        gr = api.GpuReduction(ctx, api.GA_REDUCE_SUM, np.float64)
        d = api.GpuArray.empty(ctx, (100,), np.float64)
        api.reduction_call_sharded(gr, comm, d, None, g, [0], rank * 32, 64)        # both ranks: complete
        ctx.sync()
        first = d.to_numpy()
        state = comm.peer_state()
        ready.wait(timeout=60) if rank == 0 else ready.set()                        # rank 1 is idle from here on
        if rank == 0:
            import time
            t0 = time.perf_counter()
            api.reduction_call_sharded(gr, comm, d, None, g, [0], 0, 64)            # nobody answers
            ctx.sync()
            waited = time.perf_counter() - t0
            after = comm.peer_state()
            code = 0
            try:
                api.reduction_call_sharded(gr, comm, d, None, g, [0], 0, 64)
            except api.GpuArrayException as e:
                code = e.code
            done.set()
            assert state[0] == 1 and state[2] == 0 and (first == x.sum(0)).all()
            assert after[2] != 0, after
            assert 0.25 <= waited < 5.0, waited
            assert code == api.GA_COMM_ERROR, code
        else:
            done.wait(timeout=60)
            assert state[0] == 1 and (first == x.sum(0)).all()
        comm.free()
        ctx.close()
    except Exception as e:
        import traceback
        q_err.put("rank %d: %s\n%s" % (rank, e, traceback.format_exc()))


@pytest.mark.skipif(_ngpus() < 2, reason="needs two GPUs")
def test_a_rank_that_stays_away_is_reported_after_a_bounded_wait():
    import torch.multiprocessing as mp
    m = mp.get_context("spawn")
    q_id, q_err, ready, done = m.Queue(), m.Queue(), m.Event(), m.Event()
    procs = [m.Process(target=_absent_rank_worker, args=(r, 2, q_id, q_err, ready, done)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
    msgs = []
    while not q_err.empty():
        msgs.append(q_err.get())
    assert not hung, "rank hung"
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs)


@pytest.mark.skipif(_ngpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("peer", [True, False], ids=["peer_windows", "nccl_all_reduce"])
def test_sharded_reduction_with_gpucomm(peer):
    import torch.multiprocessing as mp
    m = mp.get_context("spawn")
    q_id, q_err = m.Queue(), m.Queue()
    world = 2
    procs = [m.Process(target=_worker, args=(r, world, q_id, q_err, peer)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
    msgs = []
    while not q_err.empty():
        msgs.append(q_err.get())
    assert not hung, "rank hung"
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs)


@pytest.mark.skipif(_ngpus() < 2, reason="needs two GPUs")
def test_cross_gpu_transfer_is_ordered_on_both_streams():
    import torch.multiprocessing as mp
    m = mp.get_context("spawn")
    q_err = m.Queue()
    p = m.Process(target=_transfer_worker, args=(q_err,))
    p.start()
    p.join(timeout=180)
    if p.is_alive():
        p.kill()
        pytest.fail("transfer worker hung")
    msgs = []
    while not q_err.empty():
        msgs.append(q_err.get())
    assert not msgs, "\n".join(msgs)
    assert p.exitcode == 0
