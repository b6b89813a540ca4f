"""Multi-GPU use of the engine: one process per GPU, data sharded along the
leading axis.

  * Elementwise calls and reductions that KEEP the leading axis need nothing
    beyond slicing: every rank runs the ordinary single-GPU call on its slab
    (`shard_bounds`), and the results are slabs of the global result.
  * Reductions that reduce the leading axis (or everything) produce one partial
    per rank with the final output shape; `finish_accumulate` combines them with
    a single all-reduce (SUM/PROD/MIN/MAX exist in gpucomm, reference
    src/gpuarray_collectives_cuda_nccl.c:150-185).
  * For arg-reductions NCCL has no (value, index) pair operator. `finish_minmaxarg`
    uses two all-reduces of existing operators: MAX (or MIN) on the value, then
    MIN on a candidate index that is the rank's GLOBAL flat index where its value
    equals the global extreme and the largest integer elsewhere, so the lowest
    index wins ties exactly as the single-GPU kernel does.

The functions take an `allreduce(array, op)` callable ("sum", "prod", "min",
"max"; returns the reduced array) so that the same host logic runs over
gpucomm on GPUs and over torch.distributed/gloo in the CPU tests.
"""
import numpy as np

INDEX_NONE = np.iinfo(np.int64).max


def shard_bounds(n, world, rank):
    """[lo, hi) of `n` items for `rank`: contiguous slabs, sizes differ by <= 1."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def global_flat_index(local_idx, lead_lo, lead_local, lead_axis_pos, redux_dims):
    """Translates flat indices computed on a slab into indices of the whole array.

    redux_dims: extents of the reduced axes IN reduxList ORDER for the whole
    array; lead_axis_pos: position of the sharded (leading) axis in that list;
    lead_local: slab extent along it; lead_lo: first global coordinate of the slab.
    """
    local_dims = list(redux_dims)
    local_dims[lead_axis_pos] = lead_local
    idx = np.asarray(local_idx, dtype=np.int64)
    coords = []
    rem = idx.copy()
    for d in reversed(local_dims):
        coords.append(rem % d)
        rem = rem // d
    coords = coords[::-1]
    coords[lead_axis_pos] = coords[lead_axis_pos] + lead_lo
    out = np.zeros_like(idx)
    for c, d in zip(coords, redux_dims):
        out = out * d + c
    return out


def finish_accumulate(allreduce, partial, op):
    """op in {"sum", "prod", "min", "max"}."""
    return allreduce(np.ascontiguousarray(partial), op)


def finish_minmaxarg(allreduce, local_val, local_global_idx, is_min=False):
    """Combines per-rank (value, global index) pairs; lowest index wins ties.

    NaN rule: a NaN can only be a result if it is the first reduced element of
    the whole array, i.e. has global index 0 - it is then owned by rank 0 and
    must win, so NaN values at index 0 are handled before the value all-reduce.
    """
    val = np.ascontiguousarray(local_val)
    idx = np.ascontiguousarray(local_global_idx, dtype=np.int64)
    isfloat = val.dtype.kind == "f"
    if isfloat:
        nan_first = np.isnan(val) & (idx == 0)
        # replace by the extreme so that the value reduction stays NaN-free
        fill = -np.inf if is_min else np.inf
        work = np.where(np.isnan(val), np.array(np.inf if is_min else -np.inf, val.dtype), val)
        work = np.where(nan_first, np.array(fill, val.dtype), work)
        has_nan_first = allreduce(nan_first.astype(np.int64), "max").astype(bool)
    else:
        work = val
        has_nan_first = np.zeros(val.shape, bool)
    best = allreduce(work.copy(), "min" if is_min else "max")
    cand = np.where(work == best, idx, INDEX_NONE)
    best_idx = allreduce(cand, "min")
    if isfloat:
        best = np.where(has_nan_first, np.array(np.nan, val.dtype), best)
        best_idx = np.where(has_nan_first, 0, best_idx)
    return best, best_idx


def finish_minmaxarg_packed(allreduce, local_val, local_global_idx, is_min=False):
    """The protocol GpuReduction_call_sharded runs on the device
    (csrc/ga_reduction.c, sharded_pair), restated on the host so that it can be
    tested over any all-reduce: TWO collectives instead of the three of
    finish_minmaxarg. Every global index belongs to exactly one rank, so two
    payload bits ride in the low bits of the candidate index and arrive with
    the winner: bit 0 "the value is not a NaN", bit 1 "the value is -0.0".
    A NaN can only come from the rank holding element 0 (the other shards do
    not apply the NaN-first rule) and is then the answer; it enters the value
    all-reduce as the winning infinity. local_global_idx uses
    18446744073709551615 (all ones) for "no element" (a shard of NaNs only)."""
    val = np.ascontiguousarray(local_val)
    idx = np.ascontiguousarray(local_global_idx).astype(np.uint64)
    none = np.uint64(0xFFFFFFFFFFFFFFFF)
    if val.dtype.kind == "f":
        nan = np.isnan(val)
        work = np.where(nan, np.array(-np.inf if is_min else np.inf, val.dtype), val)
        pay = np.where(nan, 0, 1).astype(np.uint64) | \
            np.where((val == 0) & np.signbit(val), 2, 0).astype(np.uint64)
    else:
        work = val
        pay = np.ones(val.shape, np.uint64)
    best = allreduce(work.copy(), "min" if is_min else "max")
    cand = np.where((work == best) & (idx != none), (idx << np.uint64(2)) | pay, none)
    r = allreduce(cand, "min")
    out_idx = (r >> np.uint64(2)).astype(np.int64)
    if val.dtype.kind == "f":
        out_val = np.where((r & np.uint64(1)) == 0, np.array(np.nan, val.dtype),
                           np.where(best == 0, np.where((r & np.uint64(2)) != 0, -np.abs(best), np.abs(best)),
                                    best)).astype(val.dtype)
    else:
        out_val = best
    return out_val, out_idx
