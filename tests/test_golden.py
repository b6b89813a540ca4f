"""Golden fixtures produced by the reference's own compiled util code
(tests/golden/make_golden.py ran it where the reference tree is mounted).
They pin the CPU oracle and the product's host functions on machines that do
not have the reference: dimension collapsing, float -> half conversion, the
type-size table and the error strings."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_util_golden.json")


def load():
    with open(GOLDEN) as f:
        return json.load(f)


def test_collapse_matches_the_reference_outputs(oracle, api):
    cases = load()["collapse"]
    assert len(cases) == 400
    for c in cases:
        want = (c["out_dims"], c["out_strides"])
        assert oracle.collapse(c["dims"], c["strides"]) == want
        assert oracle.collapse(c["dims"], c["strides"], fn=api.lib().gpuarray_elemwise_collapse) == want


def test_float2half_matches_the_reference_outputs_except_on_ties(oracle):
    """The reference's HOST routine rounds exact ties away from zero; its device
    kernels (and this oracle) round to even. Every other input must agree."""
    ties = 0
    for bits, ref_half in load()["float2half"]:
        x = np.array([bits], np.uint32).view(np.float32)[0]
        got = oracle.float2half_bits(float(x))
        if got != ref_half:
            # exactly halfway between two neighbouring halfs (normal or subnormal)
            lo, hi = (np.array([h], np.uint16).view(np.float16)[0] for h in (got, ref_half))
            assert abs(got - ref_half) == 1, hex(bits)
            assert abs(np.float64(x) - np.float64(lo)) == abs(np.float64(x) - np.float64(hi)), hex(bits)
            ties += 1
    assert ties == 2          # 1 + 2^-11 and 2^-25 are in the fixture


def test_type_sizes_and_error_strings_match_the_reference_outputs(api):
    g = load()
    L = api.lib()
    for tc, size in g["elsize"]:
        assert L.gpuarray_get_elsize(tc) == size, tc
    for code, text in g["error_str"]:
        assert L.gpuarray_error_str(code).decode() == text, code
