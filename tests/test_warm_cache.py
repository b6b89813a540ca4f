"""The cubin cache can be filled on a machine without a GPU from recorded kernel
sources (libgpuarray_b200/warm_cache.py): NVRTC needs no device and the cache
key depends only on the source text, the built-in templates and the compiler."""
import ctypes
import gzip
import json
import os

from libgpuarray_b200 import api, warm_cache


def _reduction_sources():
    """Source texts of a few reduction variants, from the library's generator."""
    L = api.lib()
    fn = L.gpuarray_b200_reduction_source
    fn.restype = ctypes.c_void_p
    fn.argtypes = [ctypes.c_int] * 8
    libc = ctypes.CDLL(None)
    libc.free.argtypes = [ctypes.c_void_p]
    texts = []
    for op, tc, shape, vec, group in ((api.GA_REDUCE_SUM, api.GA_FLOAT, 0, 4, 32),
                                      (api.GA_REDUCE_MAXANDARGMAX, api.GA_FLOAT, 0, 4, 256),
                                      (api.GA_REDUCE_SUM, api.GA_DOUBLE, 1, 2, 0),
                                      (api.GA_REDUCE_ANY, api.GA_BYTE, 2, 1, 0)):
        dst = api.GA_BOOL if op == api.GA_REDUCE_ANY else tc
        p = fn(op, tc, dst, shape, vec, 0, 32 if shape == 2 else 1, group)
        assert p
        texts.append(ctypes.string_at(p).decode())
        libc.free(p)
    return texts


def test_recorded_variants_compile_into_a_cache_directory(built, tmp_path):
    texts = _reduction_sources()
    src_dir = tmp_path / "ksrc"
    src_dir.mkdir()
    for i, t in enumerate(texts):
        (src_dir / ("%03d.src" % i)).write_text(t)
    sample = tmp_path / "sample.json.gz"
    assert warm_cache.pack(str(src_dir), str(sample)) == len(texts)
    with gzip.open(sample, "rt") as f:
        assert json.load(f) == texts
    cache = tmp_path / "cache"
    done, bad = warm_cache.warm(str(sample), str(cache), jobs=1)
    assert (done, bad) == (len(texts), 0)
    names = sorted(os.listdir(cache))
    assert len(names) == len(texts) and all(n.endswith(".cubin") for n in names)
    # a second pass finds everything in place (same keys)
    done, bad = warm_cache.warm(str(sample), str(cache), jobs=1)
    assert (done, bad) == (len(texts), 0) and sorted(os.listdir(cache)) == names
