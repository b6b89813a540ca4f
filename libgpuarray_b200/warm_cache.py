"""Builds the cubin cache on a machine WITHOUT a GPU.

NVRTC compiles for sm_100a without a device, and the cache key of a kernel is
a hash of its source text and of the kernel templates built into the library
(csrc/ga_compile.c). So, given the source texts of the kernel variants a
workload uses, the cache can be filled ahead of time - after the templates
changed, or before a deployment that must not compile at start-up:

    # 1. on a GPU machine, once: record the variants the workload builds
    GPUARRAY_B200_SOURCE_LOG=/tmp/ksrc python my_workload.py
    python -m libgpuarray_b200.warm_cache --pack /tmp/ksrc sources.json.gz
    # 2. anywhere: compile them into a cache directory
    python -m libgpuarray_b200.warm_cache sources.json.gz .kernel_cache -j 8
"""
import ctypes
import gzip
import json
import multiprocessing
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def pack(src_dir, out_path):
    texts = []
    for name in sorted(os.listdir(src_dir)):
        if name.endswith(".src"):
            with open(os.path.join(src_dir, name)) as f:
                texts.append(f.read())
    with gzip.open(out_path, "wt") as f:
        json.dump(texts, f)
    return len(texts)


def _compile_many(job):
    cache_dir, texts = job
    from libgpuarray_b200 import api
    L = api.lib()
    fn = L.gpuarray_b200_compile_check
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_size_t),
                   ctypes.POINTER(ctypes.c_char_p)]
    bad = 0
    for t in texts:
        size = ctypes.c_size_t()
        log = ctypes.c_char_p()
        if fn(t.encode(), None, cache_dir.encode(), ctypes.byref(size), ctypes.byref(log)) != 0:
            bad += 1
    return len(texts), bad


def warm(sources_path, cache_dir=None, jobs=None):
    """Compiles every recorded variant into cache_dir; returns (compiled, failed)."""
    cache_dir = os.path.abspath(cache_dir or os.path.join(os.path.dirname(HERE), ".kernel_cache"))
    os.makedirs(cache_dir, exist_ok=True)
    with gzip.open(sources_path, "rt") as f:
        texts = json.load(f)
    jobs = max(1, jobs or os.cpu_count() or 1)
    chunks = [(cache_dir, texts[i::jobs]) for i in range(jobs)]
    if jobs == 1:
        results = [_compile_many(chunks[0])]
    else:
        with multiprocessing.get_context("spawn").Pool(jobs) as pool:
            results = pool.map(_compile_many, chunks)
    return sum(r[0] for r in results), sum(r[1] for r in results)


def main(argv):
    if len(argv) >= 3 and argv[0] == "--pack":
        print("packed %d sources into %s" % (pack(argv[1], argv[2]), argv[2]))
        return 0
    jobs = None
    if "-j" in argv:
        i = argv.index("-j")
        jobs = int(argv[i + 1])
        argv = argv[:i] + argv[i + 2:]
    if not argv:
        print(__doc__)
        return 2
    src = argv[0]
    cache = argv[1] if len(argv) > 1 else None
    done, bad = warm(src, cache, jobs)
    print("compiled %d kernel variants, %d failed" % (done, bad))
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
