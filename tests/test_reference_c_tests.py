"""Runs the reference's OWN C test programs against this library.

oracle/Makefile compiles tests/check_util.c, check_types.c, check_error.c,
check_elemwise.c and check_reduction.c of the reference, unmodified and from
where they lie, against include/ and libgpuarray.so of this repository (a
small check.h stand-in replaces libcheck). The binaries live in oracle/_ref/
(not in the history); when they are absent - the reference tree was not
mounted at build time - these tests skip. The first three need no device."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def run(name, env=None):
    exe = os.path.join(REF, name)
    if not os.path.exists(exe):
        pytest.skip("%s not built (reference tree absent at build time)" % name)
    e = dict(os.environ)
    e.update(env or {})
    e.setdefault("GPUARRAY_CACHE_PATH", os.path.join(ROOT, ".kernel_cache"))
    r = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=e,
                       timeout=600)
    assert r.returncode == 0 and "Failures: 0" in r.stdout, r.stdout
    return r.stdout


@pytest.mark.parametrize("name,count", [("check_util", 4), ("check_types", 3), ("check_error", 1)])
def test_reference_host_tests(built, name, count):
    out = run(name)
    assert "Checks: %d," % count in out


@pytest.mark.gpu
def test_reference_check_elemwise(built):
    out = run("check_elemwise", {"DEVICE": "cuda0"})
    assert "Checks: 14," in out


@pytest.mark.gpu
def test_reference_check_reduction(built):
    out = run("check_reduction", {"DEVICE": "cuda0"})
    assert "Checks: 4," in out
