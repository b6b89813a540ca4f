"""Generates tests/golden/ref_util_golden.json by running the REFERENCE's own
compiled code: oracle/_ref/libref_util.so, which `make -C oracle ref` builds
from the reference's src/gpuarray_util.c, gpuarray_types.c, gpuarray_error.c
(and the header-only ga_float2half) where they lie. Run it where the
reference tree is mounted:

    python -m libgpuarray_b200.build && make -C oracle ref
    python tests/golden/make_golden.py

The fixture travels with the repository; tests/test_golden.py checks the CPU
oracle and the product library against it on machines without the reference.
Inputs come from numpy's PCG64 with the seeds written below.
"""
import ctypes
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402


def main():
    ref = O.ref_lib()
    if ref is None:
        raise SystemExit("oracle/_ref/libref_util.so is missing: build it from the reference tree first")
    rng = np.random.Generator(np.random.PCG64(20240607))
    out = {"source": "reference util code compiled in place (libref_util.so)", "seed": 20240607}

    # 1. gpuarray_elemwise_collapse (src/gpuarray_util.c:153-188)
    cases = []
    for _ in range(400):
        nd = int(rng.integers(1, 7))
        dims = [int(d) for d in rng.choice([1, 1, 2, 3, 4, 5, 7], size=nd)]
        strs = []
        for _k in range(int(rng.integers(1, 4))):
            s, step = [], int(rng.choice([1, 2, 4, 8]))
            for d in reversed(dims):
                s.insert(0, step)
                step *= d
            for j in range(nd):
                r = rng.random()
                if r < 0.15:
                    s[j] = 0
                elif r < 0.3:
                    s[j] = -s[j]
                elif r < 0.4:
                    s[j] *= 2
            strs.append(s)
        edims, estrs = O.collapse(dims, strs, fn=ref.gpuarray_elemwise_collapse)
        cases.append({"dims": dims, "strides": strs, "out_dims": edims, "out_strides": estrs})
    out["collapse"] = cases

    # 2. host ga_float2half (src/gpuarray/util.h:103-183): ties round away from zero
    xs = np.concatenate([
        rng.standard_normal(600).astype(np.float32) * np.float32(50),
        (rng.standard_normal(200) * 1e-6).astype(np.float32),
        np.array([0.0, -0.0, 1.0, -1.0, 65504.0, 65519.0, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25,
                  2.9831426e-08, 1 + 2.0 ** -11, 1 + 3 * 2.0 ** -11, 1.0005035, 1.0002441],
                 dtype=np.float32)])
    out["float2half"] = [[int(x.view(np.uint32)), int(ref.ref_float2half(ctypes.c_float(float(x))))]
                         for x in xs]

    # 3. type table and error strings (src/gpuarray_types.c, src/gpuarray_error.c)
    out["elsize"] = [[tc, int(ref.gpuarray_get_elsize(tc))]
                     for tc in list(range(-1, 27)) + list(range(256, 310)) + [511, 512, 1000]]
    out["error_str"] = [[code, ref.gpuarray_error_str(code).decode()]
                        for code in range(-1, 21) if code != 6]      # 6 = GA_SYS_ERROR prints errno

    path = os.path.join(HERE, "ref_util_golden.json")
    with open(path, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
