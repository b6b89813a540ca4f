"""The peer-memory exchange kernel TEMPLATE (templates/ga_exchange.cuh) executed
on the CPU: N "ranks" with NumPy buffers as their windows. On GPUs the ranks
run at the same time, one per GPU; here the two phases of the kernel are run
one after the other (push of every rank, then combine of every rank), which
exercises the slot, flag and chunk arithmetic, the fold order and the
(value, index) rule against NumPy. What it replaces in the reference is an
all-reduce (src/gpuarray_collectives_cuda_nccl.c:286-316; no pair operator
there, :158-185)."""
import ctypes
import hashlib
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SIMT = os.path.join(ROOT, "tests", "simt")
TEMPLATES = os.path.join(ROOT, "libgpuarray_b200", "csrc", "templates")
BUILD = os.path.join(ROOT, "libgpuarray_b200", "build", "simt")
MAX_RANKS, MAX_CTAS, DATA_OFF, THREADS = 16, 64, 32768, 256
NONE = np.uint64(0xFFFFFFFFFFFFFFFF)
CT = {np.dtype(np.float32): "float", np.dtype(np.float64): "double", np.dtype(np.int32): "int",
      np.dtype(np.uint8): "unsigned char", np.dtype(np.float16): "ga_half", np.dtype(np.int64): "long long"}


class Layout(ctypes.Structure):
    _fields_ = [("n", ctypes.c_ulonglong), ("seq", ctypes.c_ulonglong), ("slot_bytes", ctypes.c_ulonglong),
                ("idx_off", ctypes.c_ulonglong), ("timeout_ns", ctypes.c_ulonglong), ("key", ctypes.c_ulonglong),
                ("win", ctypes.c_ulonglong * MAX_RANKS), ("nranks", ctypes.c_uint), ("rank", ctypes.c_uint),
                ("chunk", ctypes.c_uint), ("phases", ctypes.c_uint)]


def build(dtype, pair, op):
    ct = CT[np.dtype(dtype)]
    if ct == "ga_half":
        head = ("#define GA_XC_T ga_half\n#define GA_XC_W_T float\n#define GA_XC_LOAD(x) ga_half2float(x)\n"
                "#define GA_XC_STORE(w) ga_float2half(w)\n")
    else:
        head = "#define GA_XC_T %s\n#define GA_XC_W_T %s\n#define GA_XC_LOAD(x) (x)\n#define GA_XC_STORE(w) (w)\n" % (ct, ct)
    head += "#define GA_XC_PAIR %d\n" % pair
    if pair:
        head += "#define GA_XC_MIN %d\n" % (op == "min")
    else:
        head += "#define GA_XC_OP(a, b) %s\n" % {"sum": "((a) + (b))", "prod": "((a) * (b))",
                                                  "min": "((b) < (a) ? (b) : (a))",
                                                  "max": "((b) > (a) ? (b) : (a))"}[op]
    # the stand-in cluda.h first: its include guard then keeps the device one out
    text = '#include "cluda.h"\n' + head + '#include "ga_exchange.cuh"\n' + r'''
struct simt_args { const ga__xc_layout *L; void *val; void *idx; unsigned int *status; };
static void simt_body(void *p) {
  simt_args *a = (simt_args *)p;
  ga_exchange(*a->L, (GA_XC_T *)a->val, (unsigned long long *)a->idx, a->status);
}
extern "C" void simt_launch(const void *layout, void *val, void *idx, void *status, unsigned gx) {
  simt_args a = {(const ga__xc_layout *)layout, val, idx, (unsigned int *)status};
  simt::run_grid(simt_body, &a, simt_dim3{gx, 1, 1}, simt_dim3{GA_XC_THREADS, 1, 1});
}
'''
    deps = open(os.path.join(TEMPLATES, "ga_exchange.cuh")).read() + \
        open(os.path.join(SIMT, "include", "simt_emul.h")).read() + \
        open(os.path.join(SIMT, "include", "cluda.h")).read()
    key = hashlib.sha1((text + deps).encode()).hexdigest()[:16]
    os.makedirs(BUILD, exist_ok=True)
    so = os.path.join(BUILD, "xc_%s.so" % key)
    if not os.path.exists(so):
        src = os.path.join(BUILD, "xc_%s.cpp" % key)
        with open(src, "w") as f:
            f.write(text)
        r = subprocess.run(["g++", "-std=c++17", "-O1", "-shared", "-fPIC", "-w", "-I",
                            os.path.join(SIMT, "include"), "-I", TEMPLATES, src,
                            os.path.join(SIMT, "simt_runtime.cpp"), "-o", so], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-3000:]
    return ctypes.CDLL(so)


class Ranks:
    """The windows of `nranks` ranks and the host-side arithmetic of ga_comm_exchange."""

    def __init__(self, nranks, slot_bytes=1 << 16):
        self.n = nranks
        self.slot = slot_bytes
        self.win = [np.zeros(DATA_OFF + 2 * nranks * slot_bytes, np.uint8) for _ in range(nranks)]
        self.status = [np.zeros(16, np.uint32) for _ in range(nranks)]
        self.seq = 0

    def exchange(self, lib, vals, idxs, phases=(1, 2), timeout_ns=10 ** 9, keys=None):
        n = vals[0].size
        es = vals[0].dtype.itemsize
        self.seq += 1
        ctas = min(MAX_CTAS, -(-n // THREADS))
        chunk = (-(-n // ctas) + 15) & ~15
        gx = -(-n // chunk)
        for ph in phases:
            for r in range(self.n):
                L = Layout()
                L.n, L.seq, L.slot_bytes, L.idx_off, L.timeout_ns = n, self.seq, self.slot, (n * es + 15) & ~15, timeout_ns
                for p in range(self.n):
                    L.win[p] = self.win[p].ctypes.data
                L.nranks, L.rank, L.chunk, L.phases = self.n, r, chunk, ph
                L.key = keys[r] if keys is not None else 0
                lib.simt_launch(ctypes.byref(L), ctypes.c_void_p(vals[r].ctypes.data),
                                ctypes.c_void_p(idxs[r].ctypes.data if idxs is not None else 0),
                                ctypes.c_void_p(self.status[r].ctypes.data), gx)
        return gx


def fold_pairs(vals, idxs, is_min):
    """Better value first, lower index among equals, a NaN candidate is final."""
    n = vals[0].size
    ov, oi = vals[0].copy(), np.full(n, NONE)
    for k in range(n):
        best = None
        for v, i in zip(vals, idxs):
            if i[k] == NONE:
                continue
            x = float(v[k])
            if best is None or x != x:
                take = True
            else:
                b = float(best[0])
                take = b == b and ((x < b if is_min else x > b) or (x == b and i[k] < best[1]))
            if take:
                best = (v[k], i[k])
        if best is not None:
            ov[k], oi[k] = best
    return ov, oi


def test_pairs_follow_the_single_gpu_rule(rng):
    for dtype, nranks, n, is_min in ((np.float32, 2, 1000, False), (np.float64, 8, 1024, True),
                                      (np.float16, 3, 333, False), (np.int32, 4, 70000 // 8, True)):
        lib = build(dtype, 1, "min" if is_min else "max")
        R = Ranks(nranks, slot_bytes=1 << 18)
        for rep in range(3):                          # consecutive exchanges alternate the halves
            vals = [(np.round(rng.standard_normal(n) * 2) / 2).astype(dtype) for _ in range(nranks)]
            idxs = [(rng.permutation(n * nranks)[:n] * nranks + r).astype(np.uint64) for r in range(nranks)]
            if np.dtype(dtype).kind == "f":
                vals[1][5] = np.nan                   # the shard holding element 0 delivers a NaN: final
                idxs[1][5] = 0
                vals[0][7] = np.nan                   # a shard of NaNs only: no candidate
                idxs[0][7] = NONE
                for r in range(nranks):               # signed zeros tie: the lower index wins with its sign
                    vals[r][9] = 0.0 if r % 2 else -0.0
                    vals[r][11] = 3.0                 # plain tie
            want_v, want_i = fold_pairs(vals, idxs, is_min)
            got_v = [v.copy() for v in vals]
            got_i = [i.copy() for i in idxs]
            gx = R.exchange(lib, got_v, got_i)
            assert gx == min(MAX_CTAS, -(-n // THREADS)) or gx * THREADS >= n
            for r in range(nranks):
                assert (got_i[r] == want_i).all(), (dtype, r, rep)
                assert got_v[r].tobytes() == want_v.tobytes(), (dtype, r, rep)
            assert all(int(s[0]) == 0 for s in R.status)


def test_value_only_extremes_break_ties_by_the_rank_key(rng):
    """Mode 2: no index array; equal values (+0.0 / -0.0) go to the rank with the lowest key."""
    lib = build(np.float64, 2, "max")
    nranks, n = 4, 600
    R = Ranks(nranks)
    keys = [300, 0, 100, 200]                         # rank 1 holds the first shard
    vals = [np.round(rng.standard_normal(n) * 2).astype(np.float64) / 2 for _ in range(nranks)]
    for r in range(nranks):
        vals[r][:50] = -1.0
    vals[0][3], vals[2][3] = 0.0, -0.0                # tie of zeros: key 100 (rank 2) wins, -0.0
    vals[1][4] = np.nan                               # first shard delivers a NaN: final
    vals[3][5] = -np.inf                              # a shard without candidates sends the identity
    want = np.empty(n)
    order = np.argsort(keys)
    for k in range(n):
        best = None
        for r in order:
            x = vals[r][k]
            if best is None or (best == best and x > best) or (x != x and best == best):
                best = x
        want[k] = best
    got = [v.copy() for v in vals]
    R.exchange(lib, got, None, keys=keys)
    for r in range(nranks):
        assert got[r].tobytes() == want.tobytes()
    assert np.signbit(want[3]) and want[3] == 0 and np.isnan(want[4])


def test_accumulating_operators_fold_in_rank_order(rng):
    for dtype, op, nranks, n in ((np.float64, "sum", 8, 1), (np.float32, "sum", 4, 5000), (np.float16, "sum", 3, 257),
                                 (np.float64, "prod", 2, 100), (np.uint8, "min", 5, 4097), (np.int64, "max", 2, 31)):
        lib = build(dtype, 0, op)
        R = Ranks(nranks)
        for rep in range(2):
            if np.dtype(dtype).kind == "f":
                vals = [rng.standard_normal(n).astype(dtype) for _ in range(nranks)]
            else:
                vals = [rng.integers(0, 2 if dtype == np.uint8 else 1000, n).astype(dtype) for _ in range(nranks)]
            wide = np.float32 if dtype == np.float16 else dtype
            acc = vals[0].astype(wide)
            for v in vals[1:]:
                w = v.astype(wide)
                acc = {"sum": lambda a, b: a + b, "prod": lambda a, b: a * b, "min": np.minimum,
                       "max": np.maximum}[op](acc, w)
            want = acc.astype(dtype)
            got = [v.copy() for v in vals]
            R.exchange(lib, got, None)
            for r in range(nranks):
                assert got[r].tobytes() == want.tobytes(), (dtype, op, r)


def test_a_peer_that_never_arrives_is_reported_not_waited_for(rng):
    lib = build(np.float32, 0, "sum")
    R = Ranks(2)
    vals = [np.ones(10, np.float32), np.ones(10, np.float32)]
    R.seq = 4
    # only rank 0 runs, combine phase only: the flag of rank 1 never reaches 5
    L = Layout()
    L.n, L.seq, L.slot_bytes, L.idx_off, L.timeout_ns = 10, 5, R.slot, 48, 50_000
    for p in range(2):
        L.win[p] = R.win[p].ctypes.data
    L.nranks, L.rank, L.chunk, L.phases = 2, 0, 16, 2
    lib.simt_launch(ctypes.byref(L), ctypes.c_void_p(vals[0].ctypes.data), ctypes.c_void_p(0),
                    ctypes.c_void_p(R.status[0].ctypes.data), 1)
    assert int(R.status[0][0]) == 1
