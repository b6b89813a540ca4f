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

#ifdef __cplusplus
}
#endif
#endif
