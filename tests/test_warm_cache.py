"""The cubin cache can be filled on a machine without a GPU from recorded kernel
sources (libgpuarray_b200/warm_cache.py): NVRTC needs no device and the cache
key depends only on the source text and the built-in templates."""
import gzip
import json
import os

from libgpuarray_b200 import warm_cache


def test_recorded_variants_compile_into_a_cache_directory(built, tmp_path):
    with gzip.open(warm_cache.DEFAULT_SOURCES, "rt") as f:
        texts = json.load(f)
    assert len(texts) > 1000
    good = [t for t in texts if "undefined_name" not in t and "ga_ew_" in t][:3] + \
           [t for t in texts if "ga_reduce.cuh" in t][:3]
    sample = tmp_path / "sample.json.gz"
    with gzip.open(sample, "wt") as f:
        json.dump(good, f)
    cache = tmp_path / "cache"
    done, bad = warm_cache.warm(str(sample), str(cache), jobs=1)
    assert (done, bad) == (6, 0)
    names = sorted(os.listdir(cache))
    assert len(names) == 6 and all(n.endswith(".cubin") for n in names)
    # a second pass finds everything in place (same keys)
    done, bad = warm_cache.warm(str(sample), str(cache), jobs=1)
    assert (done, bad) == (6, 0) and sorted(os.listdir(cache)) == names
