/* Reduction engine: one of 14 operators applied over an arbitrary set of axes
 * of a strided GpuArray.
 *
 * The reference snapshot has no such header: its only C reduction is
 * GpuArray_maxandargmax (src/gpuarray/array.h:607-644) and sum/prod/all/any
 * live in Python (pygpu/reduction.py:137-319). This interface generalises the
 * two: the object lifecycle of GpuElemwise (src/gpuarray/elemwise.h:98-140)
 * and the call arguments of GpuArray_maxandargmax.
 *
 * Semantics
 *  - Destination arrays are caller-allocated and have the non-reduced source
 *    axes in ascending order (0-d when everything is reduced). Their offsets
 *    and byte strides are honoured.
 *  - SUM, PROD, PRODNZ accumulate in the destination's type (float when the
 *    destination is GA_HALF), as pygpu's reduk template accumulates in the
 *    output dtype (pygpu/reduction.py:83-132). PRODNZ multiplies only the
 *    non-zero elements. AND, OR, XOR are bitwise and need integer or bool
 *    source and destination. ALL / ANY test "!= 0" and write 0/1.
 *  - MIN, MAX and the ARG variants use a strict comparison in reduxList order,
 *    so the FIRST extreme element wins ties (including -0.0 versus +0.0), and
 *    a NaN is produced only if it is the first reduced element: the rule of
 *    the reference kernel (src/gpuarray_reduction.c:557-606). The value
 *    destination must have the source's type; the index destination holds
 *    8-byte integers and receives the mixed-radix number of the reduced
 *    coordinates in reduxList order, last listed axis fastest.
 *  - A reduction over zero elements writes the operator's identity (0, 1,
 *    all-ones, true, false); MIN/MAX/ARG* over zero elements is GA_VALUE_ERROR.
 */
#ifndef GPUARRAY_REDUCTION_H
#define GPUARRAY_REDUCTION_H

#include <gpuarray/array.h>
#include <gpuarray/elemwise.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum _ga_reduce_op {
  GA_REDUCE_SUM = 0,
  GA_REDUCE_PROD,
  GA_REDUCE_PRODNZ,
  GA_REDUCE_MIN,
  GA_REDUCE_MAX,
  GA_REDUCE_ARGMIN,
  GA_REDUCE_ARGMAX,
  GA_REDUCE_MINANDARGMIN,
  GA_REDUCE_MAXANDARGMAX,
  GA_REDUCE_AND,
  GA_REDUCE_OR,
  GA_REDUCE_XOR,
  GA_REDUCE_ALL,
  GA_REDUCE_ANY,
  GA_REDUCE_ENDSUPPORTED
} ga_reduce_op;

typedef struct _GpuReduction GpuReduction;

/* Creates a reduction operator.
 *  ndf, ndr   hints: expected number of free and reduced axes (any rank works
 *             at call time; kernels are specialised per memory pattern, not
 *             per rank)
 *  s0TypeCode type of the source elements
 * On failure *gr is NULL and the context's error is set. */
GPUARRAY_PUBLIC int GpuReduction_new(GpuReduction **gr, gpucontext *ctx, ga_reduce_op op,
                                     unsigned ndf, unsigned ndr, int s0TypeCode, int flags);
GPUARRAY_PUBLIC void GpuReduction_free(GpuReduction *gr);

/* Runs the reduction of s0 over reduxList[0..reduxLen).
 *  d0  value destination (NULL for ARGMIN / ARGMAX)
 *  d1  index destination (NULL for value-only operators)
 * Enqueues on the context's stream and returns. */
GPUARRAY_PUBLIC int GpuReduction_call(const GpuReduction *gr, GpuArray *d0, GpuArray *d1,
                                      const GpuArray *s0, unsigned reduxLen,
                                      const int *reduxList, int flags);

/* As GpuReduction_call, for a source that is this GPU's SHARD of a larger array:
 * along the reduced axis `shard_axis` the source holds coordinates
 * [shard_lo, shard_lo + s0->dimensions[shard_axis]) of an axis of extent
 * shard_global, the other ranks of `comm` hold the rest. Every rank calls it
 * with its own shard and receives the result of the WHOLE array in its
 * destinations, everything enqueued on the context's stream with no host
 * round trip: the per-GPU kernel, then ONE exchange kernel per GPU that stores
 * the partial results into every peer's window of device memory over NVLink
 * and folds what the peers stored (csrc/templates/ga_exchange.cuh). The
 * windows are set up by the first such call on a communicator, which is
 * therefore collective and synchronises once. Where they cannot be set up on
 * every rank (ranks in one process or on several hosts, more than 16 ranks,
 * results beyond 1 MiB per rank, GPUARRAY_B200_NO_PEER_WINDOW=1) the partials
 * are combined with gpucomm_all_reduce instead (the call site of
 * src/gpuarray_collectives_cuda_nccl.c:286-316).
 *  - SUM, PROD, PRODNZ, ALL, ANY: the fold runs in rank order, so every rank
 *    ends with the same bits (one all-reduce sum / prod / min / max on the
 *    fallback path). AND, OR, XOR are folded by the exchange kernel as well;
 *    on the fallback path they return GA_UNSUPPORTED_ERROR (the collectives
 *    have no bitwise operator).
 *  - MIN, MAX and the ARG variants: the index written is the flat index in the
 *    whole reduced extent (shard offset and global radix included); the better
 *    value wins, the lower global index among equal values, so ties go exactly
 *    where they go on one GPU, the NaN-first rule and signed zeros included
 *    (on the fallback path: an all-reduce MAX/MIN of the value followed by an
 *    all-reduce MIN of a candidate index, same result).
 * A rank that does not arrive within GPUARRAY_B200_PEER_TIMEOUT_MS (default
 * 10000) makes the waiting kernels give up: they return, and later sharded
 * calls on the communicator fail with GA_COMM_ERROR
 * (gpuarray_b200_comm_peer_state in b200.h).
 * comm may be NULL (one rank: no collective), which also serves to test the
 * path on one GPU. <gpuarray/collectives.h> declares gpucomm. */
struct _gpucomm;
GPUARRAY_PUBLIC int GpuReduction_call_sharded(const GpuReduction *gr, struct _gpucomm *comm,
                                              GpuArray *d0, GpuArray *d1, const GpuArray *s0,
                                              unsigned reduxLen, const int *reduxList,
                                              int shard_axis, size_t shard_lo,
                                              size_t shard_global, int flags);

/* ---- reductions of a mapped expression over several arguments ----
 *
 *     out[kept...] = REDUCE over the reduced axes of MAP(arg0, arg1, ..., scalars)
 *
 * The C form of pygpu's ReductionKernel (pygpu/reduction.py:137-291; its test
 * pygpu/tests/test_reduction.py:57-84 reduces a[i]*b[i] with one operand
 * broadcast). Map and reduction run as ONE pass over memory.
 *  preamble     code placed before the kernel (may be NULL)
 *  map_expr     C expression in which every argument appears as a scalar
 *               variable of its own name (arrays: one element), e.g. "a * b";
 *               its value keeps its natural C type
 *  reduce_expr  C expression over `a` and `b` combining two partial results,
 *               e.g. "a + b", "max(a, b)"; it must be associative and
 *               commutative (the reference assumes the same)
 *  neutral      C expression of the neutral element, e.g. "0"
 *  out_typecode type of the destination AND of the accumulator (float when it
 *               is GA_HALF and GE_CONVERT_F16 is given)
 *  n, args      argument descriptors as for GpuElemwise_new; arrays are inputs
 *               (GE_READ), scalars are passed by value at call time
 *  flags        GE_CONVERT_F16 or 0
 * Returns NULL and sets the context's error on failure (the three expressions
 * are compiled here, so a faulty one is reported by the constructor). */
typedef struct _GpuMapReduction GpuMapReduction;

GPUARRAY_PUBLIC GpuMapReduction *GpuMapReduction_new(gpucontext *ctx, const char *preamble,
                                                     const char *map_expr,
                                                     const char *reduce_expr,
                                                     const char *neutral, int out_typecode,
                                                     unsigned int n, gpuelemwise_arg *args,
                                                     int flags);
GPUARRAY_PUBLIC void GpuMapReduction_free(GpuMapReduction *mr);

/* Runs the reduction over reduxList[0..reduxLen) of the broadcast shape of the
 * array arguments.
 *  out    caller-allocated destination: the non-reduced axes in ascending
 *         order, elements of out_typecode; offset and strides are honoured
 *  args   one entry per declared argument: GpuArray * for arrays, pointer to
 *         a host scalar of the declared type for GE_SCALAR arguments
 *  flags  GE_BROADCAST lets extents of 1 stretch; GE_PADSHAPE pads lower ranks
 *         on the left (as in GpuElemwise_call); without them every array must
 *         have the same shape
 * A reduction over zero elements writes `neutral`. */
GPUARRAY_PUBLIC int GpuMapReduction_call(GpuMapReduction *mr, GpuArray *out, void **args,
                                         unsigned int reduxLen, const int *reduxList, int flags);

#ifdef __cplusplus
}
#endif
#endif
