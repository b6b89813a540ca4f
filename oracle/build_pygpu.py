"""Builds the reference's unmodified pygpu package against THIS library into
oracle/_ref/pygpu_site (outputs only: compiled extension modules and .pyc
files; no reference source is copied). Test infrastructure: it lets
tests/test_pygpu_dropin.py drive the engine through the reference's own Cython
bindings and Python operators. Needs the reference tree; called by
`make -C oracle`."""
import os
import py_compile
import subprocess
import sys
import sysconfig

import numpy

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
if len(sys.argv) < 2:
    raise SystemExit("usage: build_pygpu.py <reference tree>")
REF = sys.argv[1]
SITE = os.path.join(HERE, "_ref", "pygpu_site", "pygpu")
WORK = os.path.join(HERE, "_ref", "pygpu_build")
EXT = sysconfig.get_config_var("EXT_SUFFIX")


def run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise SystemExit("failed: %s\n%s" % (" ".join(cmd), r.stdout[-4000:]))


def main():
    os.makedirs(os.path.join(SITE, "tests"), exist_ok=True)
    os.makedirs(WORK, exist_ok=True)
    lib = os.path.join(ROOT, "libgpuarray_b200", "libgpuarray.so")
    for mod in ("gpuarray", "_elemwise"):
        src = os.path.join(REF, "pygpu", mod + ".pyx")
        c = os.path.join(WORK, mod + ".c")
        out = os.path.join(SITE, mod + EXT)
        if os.path.exists(out) and os.path.getmtime(out) > max(os.path.getmtime(src),
                                                               os.path.getmtime(lib)):
            continue
        run([sys.executable, "-m", "cython", "-3", "-I", REF, src, "-o", c])
        run(["/usr/bin/gcc", "-O1", "-fPIC", "-shared", "-w", "-I", os.path.join(REF, "pygpu"),
             "-I", os.path.join(ROOT, "include"), "-I", numpy.get_include(),
             "-I", sysconfig.get_paths()["include"], c, "-o", out, lib,
             "-Wl,-rpath,$ORIGIN/../../../../libgpuarray_b200"])
    for sub in ("", "tests"):
        d = os.path.join(REF, "pygpu", sub)
        for f in os.listdir(d):
            if f.endswith(".py"):
                # stored as *.pyc.bin: plain *.pyc files are filtered out when the
                # tree is shipped to a GPU box; the test renames them back
                py_compile.compile(os.path.join(d, f), cfile=os.path.join(SITE, sub, f + "c.bin"),
                                   doraise=True)
    print("pygpu built into", SITE)


if __name__ == "__main__":
    main()
