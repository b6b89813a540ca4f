"""Child process of tests/test_pygpu_dropin.py: drives the engine through the
reference's UNMODIFIED pygpu package (built into oracle/_ref/pygpu_site by
oracle/build_pygpu.py). Part 1: this file's own checks of the Python operator
layer against NumPy. Part 2: the reference's pygpu/tests/test_elemwise.py, run
by a minimal nose-style runner (plain functions and generator tests)."""
import inspect
import os
import sys
import traceback
import unittest

import numpy as np


def part1():
    import pygpu
    from pygpu import gpuarray, ndgpuarray
    from pygpu._elemwise import GpuElemwise, arg
    ctx = pygpu.init(os.environ.get("DEVICE", "cuda0"))
    print("device:", ctx.devname)
    rng = np.random.default_rng(5)
    a = rng.standard_normal((33, 47)).astype(np.float32)
    b = rng.standard_normal((33, 47)).astype(np.float32)
    ga = pygpu.array(a, context=ctx, cls=ndgpuarray)
    gb = pygpu.array(b, context=ctx, cls=ndgpuarray)
    assert np.allclose(np.asarray(ga + gb), a + b)
    assert np.allclose(np.asarray(ga * gb - ga), a * b - a, rtol=1e-5, atol=1e-6)
    assert np.allclose(np.asarray(ga / (gb * gb + 1)), a / (b * b + 1), rtol=1e-5)
    assert (np.asarray(ga < gb) == (a < b)).all()
    assert np.allclose(np.asarray(ga + 2.5), a + np.float32(2.5))
    assert np.allclose(np.asarray(-ga), -a) and np.allclose(np.asarray(abs(ga)), abs(a))
    gc = ga.copy()
    gc += gb
    assert np.allclose(np.asarray(gc), a + b)
    row = rng.standard_normal((1, 47)).astype(np.float32)            # broadcasting
    assert np.allclose(np.asarray(ga + pygpu.array(row, context=ctx, cls=ndgpuarray)), a + row)
    assert np.allclose(np.asarray(ga.T + gb.T), (a + b).T)             # strided views
    assert np.allclose(np.asarray(ga[::2, 3:40:3] * 2), a[::2, 3:40:3] * 2)
    i64 = rng.integers(-50, 50, (20, 30)).astype(np.int64)
    gi = pygpu.array(i64, context=ctx, cls=ndgpuarray)
    assert (np.asarray(gi + gi) == i64 + i64).all()
    assert np.allclose(np.asarray(gi.astype("float32")), i64.astype(np.float32))
    h = rng.standard_normal((64, 64)).astype(np.float16)
    gh = pygpu.array(h, context=ctx, cls=ndgpuarray)
    assert (np.asarray(gh + gh).view(np.uint16) == (h + h).view(np.uint16)).all()
    # the class pygpu's operators are built on, used directly
    out = pygpu.empty((33, 47), dtype="float32", context=ctx)
    ge = GpuElemwise(ctx, "res = a * b + 0.5f", [arg("a", "float32", read=True),
                                                 arg("b", "float32", read=True),
                                                 arg("res", "float32", write=True)])
    ge(ga, gb, out)
    want = (a.astype(np.float64) * b + 0.5).astype(np.float32)      # one fused multiply-add
    assert (np.asarray(out) == want).all()
    # array bookkeeping that pygpu forwards to the library
    assert np.allclose(np.asarray(ga.reshape((47, 33))), a.reshape(47, 33))
    assert np.allclose(np.asarray(ga.transpose(1, 0).copy()), a.T)
    idx = np.array([5, 0, 32, 7], dtype=np.int64)
    assert np.allclose(np.asarray(ga.take1(pygpu.array(idx, context=ctx))), a[idx])
    parts = pygpu.split(ga, [10, 20], axis=1)
    assert [p.shape for p in parts] == [(33, 10), (33, 10), (33, 27)]
    assert np.allclose(np.asarray(pygpu.concatenate(parts[::-1], axis=1)),
                       np.concatenate([a[:, 20:], a[:, 10:20], a[:, :10]], axis=1))
    print("part1 ok")


def run_callable(f, args, stats, name):
    try:
        f(*args)
        stats["pass"] += 1
    except unittest.SkipTest as e:
        stats["skip"] += 1
    except Exception:
        stats["fail"] += 1
        # the innermost function of the reference's test file names the case
        frames = [fr.name for fr in traceback.extract_tb(sys.exc_info()[2])
                  if "pygpu/tests/test_" in fr.filename]
        key = frames[-1] if frames else name
        stats["failed_names"][key] = stats["failed_names"].get(key, 0) + 1
        stats["failures"].append("%s%r\n%s" % (name, args if len(repr(args)) < 200 else "(...)",
                                               traceback.format_exc(limit=6)))


def part2(modname):
    import importlib
    mod = importlib.import_module(modname)
    stats = {"pass": 0, "fail": 0, "skip": 0, "failures": [], "failed_names": {}}
    for name, obj in sorted(vars(mod).items()):
        if not name.startswith("test"):
            continue
        if inspect.isgeneratorfunction(obj):
            try:
                for item in obj():
                    run_callable(item[0], item[1:], stats, name)
            except unittest.SkipTest:
                stats["skip"] += 1
            except Exception:
                stats["fail"] += 1
                stats["failures"].append("%s (generator)\n%s" % (name, traceback.format_exc(limit=6)))
        elif inspect.isfunction(obj):
            run_callable(obj, (), stats, name)
        elif inspect.isclass(obj) and issubclass(obj, unittest.TestCase):
            res = unittest.TextTestRunner(verbosity=0).run(
                unittest.defaultTestLoader.loadTestsFromTestCase(obj))
            stats["pass"] += res.testsRun - len(res.failures) - len(res.errors)
            stats["fail"] += len(res.failures) + len(res.errors)
            stats["failures"] += [t[1] for t in res.failures + res.errors]
    print("%s: pass=%d fail=%d skip=%d" % (modname, stats["pass"], stats["fail"], stats["skip"]))
    print("FAILED_NAMES", sorted(stats["failed_names"].items()))
    for f in stats["failures"][:6]:
        print("FAILURE:", f)
    return stats


def part3():
    """ndgpuarray.sum/prod/all/any through GpuReduction_* (pygpu_compat.install)."""
    import pygpu
    from pygpu import ndgpuarray
    from libgpuarray_b200 import pygpu_compat
    pygpu_compat.install()
    ctx = pygpu.init(os.environ.get("DEVICE", "cuda0"))
    rng = np.random.default_rng(9)
    x = rng.standard_normal((37, 500, 6)).astype(np.float32)
    g = pygpu.array(x, context=ctx, cls=ndgpuarray)
    for axis in (None, 0, 1, 2, (0, 2), (1, 2)):
        want = x.astype(np.float64).sum(axis=axis)
        got = np.asarray(g.sum(axis=axis)).astype(np.float64)
        scale = np.abs(x.astype(np.float64)).sum(axis=axis)
        assert (np.abs(got - want) <= 1e-6 * np.log2(x.size) * scale).all(), axis
    assert np.asarray(g.T.sum(axis=0)).shape == (500, 37)            # strided view
    h = pygpu.array(x.astype(np.float16), context=ctx, cls=ndgpuarray)  # float16 works here
    assert np.allclose(np.asarray(h.sum(axis=1)).astype(np.float32),
                       x.astype(np.float16).astype(np.float32).sum(axis=1), rtol=2e-2, atol=0.5)
    i8 = rng.integers(-3, 4, (20, 30)).astype(np.int8)
    gi = pygpu.array(i8, context=ctx, cls=ndgpuarray)
    r = gi.sum(axis=1)
    assert r.dtype == np.dtype("int") and (np.asarray(r) == i8.sum(axis=1, dtype="int")).all()
    assert (np.asarray(gi.prod(axis=0)) == i8.prod(axis=0, dtype="int")).all()
    b = rng.random((50, 60)) < 0.97
    gb = pygpu.array(b, context=ctx, cls=ndgpuarray)
    assert (np.asarray(gb.all(axis=1)) == b.all(axis=1)).all()
    assert (np.asarray(gb.any(axis=0)) == b.any(axis=0)).all()
    assert bool(np.asarray(gb.any())) == bool(b.any())
    # max / min / argmax / argmin, added to ndgpuarray by install()
    y = np.round(x * 4) / 4                                           # ties
    gy = pygpu.array(y, context=ctx, cls=ndgpuarray)
    for axis in (None, 0, 1, 2, -1):
        assert (np.asarray(gy.max(axis=axis)) == y.max(axis=axis)).all(), axis
        assert (np.asarray(gy.min(axis=axis)) == y.min(axis=axis)).all(), axis
        assert (np.asarray(gy.argmax(axis=axis)) == y.argmax(axis=axis)).all(), axis
        assert (np.asarray(gy.argmin(axis=axis)) == y.argmin(axis=axis)).all(), axis
    v, i = pygpu_compat.maxandargmax(gy, axis=(0, 2))
    flat = y.transpose(1, 0, 2).reshape(500, -1)
    assert (np.asarray(v) == flat.max(1)).all() and (np.asarray(i) == flat.argmax(1)).all()
    print("part3 ok")


if __name__ == "__main__":
    mods = [m for m in sys.argv[1:] if not m.startswith("--")]
    part1()
    if "--reductions" in sys.argv:
        part3()
        import pygpu.tests.test_reduction as tr
        from libgpuarray_b200 import pygpu_compat
        tr.ReductionKernel = pygpu_compat.ReductionKernel
    for m in mods:
        part2(m)
    sys.exit(0)
