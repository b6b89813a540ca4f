"""Host logic of the multi-GPU paths, run as real ranks over gloo on CPU
(world_size 2 and 3): slab bounds, leading-axis partial + all-reduce, and the
two-all-reduce combination of (value, global index) pairs with
lowest-index-wins ties. The per-rank "kernel" is the CPU oracle."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _allreduce(arr, op):
    arr = np.ascontiguousarray(arr)
    if arr.dtype == np.uint64:
        # gloo has no unsigned 64-bit type: flipping the top bit maps uint64 order onto int64 order
        flip = np.uint64(1 << 63)
        return _allreduce((arr ^ flip).view(np.int64), op).view(np.uint64) ^ flip
    t = torch.from_numpy(arr.copy())
    dist.all_reduce(t, op={"sum": dist.ReduceOp.SUM, "prod": dist.ReduceOp.PRODUCT,
                           "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX}[op])
    return t.numpy()


def _worker(rank, world, port, errors):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from libgpuarray_b200 import sharding
        from oracle import oracle as O

        rng = np.random.default_rng(7)               # same data on every rank
        x = np.round(rng.standard_normal((11, 5, 13)) * 2).astype(np.float32) / 2
        x[0, 2, 0] = np.nan                          # NaN as the first reduced element of column 2
        x[4, 1, 3] = np.nan                          # NaN elsewhere: ignored
        x[:, 3, :] = 1.5                             # all ties in column 3
        lo, hi = sharding.shard_bounds(x.shape[0], world, rank)
        slab = x[lo:hi]

        # kept leading axis: results are slabs, no communication
        v, i = O.minmaxarg(slab, [2])
        gv, gi = O.minmaxarg(x, [2])
        assert v.tobytes() == gv[lo:hi].tobytes() and (i == gi[lo:hi]).all()

        # reduced leading axis, accumulate op: partial + one all-reduce
        part = slab.astype(np.float64).sum(axis=(0, 2)) if hi > lo else np.zeros(5)
        y = np.nan_to_num(x)
        part = np.nan_to_num(slab).astype(np.float64).sum(axis=(0, 2))
        tot = sharding.finish_accumulate(_allreduce, part, "sum")
        assert np.allclose(tot, y.astype(np.float64).sum(axis=(0, 2)))

        # reduced leading axis, arg op in both axis orders
        for axes, pos in (([0, 2], 0), ([2, 0], 1)):
            for is_min in (False, True):
                if hi > lo:
                    lv, li = O.minmaxarg(slab, axes, is_min=is_min)
                    redux = [x.shape[a] for a in axes]
                    lgi = sharding.global_flat_index(li, lo, hi - lo, pos, redux)
                else:
                    lv = np.full(5, np.inf if is_min else -np.inf, np.float32)
                    lgi = np.full(5, sharding.INDEX_NONE, np.int64)
                bv, bi = sharding.finish_minmaxarg(_allreduce, lv, lgi, is_min=is_min)
                wv, wi = O.minmaxarg(x, axes, is_min=is_min)
                assert (bi == wi).all(), (axes, is_min, bi, wi)
                assert bv.tobytes() == wv.tobytes() or \
                    (np.isnan(bv) == np.isnan(wv)).all() and \
                    (bv[~np.isnan(bv)] == wv[~np.isnan(wv)]).all()

        # the two-collective protocol of GpuReduction_call_sharded (payload bits in the
        # candidate index). Local results as the device kernel gives them: global flat
        # indices, the NaN-first rule only on the shard that holds element 0, all-ones for
        # "no element".
        z = x.copy()
        z[:, 4, :] = -1.0
        z[7, 4, 2] = -0.0                            # first zero is negative ...
        z[9, 4, 5] = 0.0                             # ... a positive one follows (another rank at world 3)
        z[6, 0, 0] = np.nan                          # NaN at the start of a later slab: not a result
        none = np.uint64(0xFFFFFFFFFFFFFFFF)
        for axes, pos in (([0, 2], 0), ([2, 0], 1)):
            for is_min in (False, True):
                zz = -z if is_min else z
                sl = zz[lo:hi]
                if hi > lo:
                    ident = np.float32(np.inf if is_min else -np.inf)
                    loc = sl if lo == 0 else np.where(np.isnan(sl), ident, sl)
                    lv, li = O.minmaxarg(loc, axes, is_min=is_min)
                    redux = [zz.shape[a] for a in axes]
                    lgi = sharding.global_flat_index(li, lo, hi - lo, pos, redux).astype(np.uint64)
                    if lo != 0:                      # a shard of NaNs only has no element to offer
                        allnan = np.isnan(sl).all(axis=(0, 2))
                        lgi = np.where(allnan, none, lgi)
                else:
                    lv = np.full(5, np.inf if is_min else -np.inf, np.float32)
                    lgi = np.full(5, none, np.uint64)
                bv, bi = sharding.finish_minmaxarg_packed(_allreduce, lv, lgi, is_min=is_min)
                wv, wi = O.minmaxarg(zz, axes, is_min=is_min)
                assert (bi == wi).all(), (axes, is_min, bi, wi)
                nanmask = np.isnan(wv)
                assert (np.isnan(bv) == nanmask).all()
                assert bv[~nanmask].tobytes() == wv[~nanmask].tobytes(), (axes, is_min, bv, wv)
        dist.destroy_process_group()
    except Exception as e:                           # surfaces in the parent
        import traceback
        errors.put("rank %d: %s\n%s" % (rank, e, traceback.format_exc()))


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_reductions_over_gloo(world):
    ctxm = mp.get_context("spawn")
    errors = ctxm.Queue()
    port = _free_port()
    procs = [ctxm.Process(target=_worker, args=(r, world, port, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("rank hung")
    msgs = []
    while not errors.empty():
        msgs.append(errors.get())
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs)


def test_shard_bounds_cover_everything():
    from libgpuarray_b200 import sharding
    for n in (0, 1, 7, 16384, 2048):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
