/* Strided N-dimensional arrays on top of gpudata.
 *
 * The struct layout is ABI (clients fill and read the fields directly); it is
 * field-for-field the reference's GpuArray (src/gpuarray/array.h:21-101).
 * Strides and the offset are in BYTES and strides may be negative. */
#ifndef GPUARRAY_ARRAY_H
#define GPUARRAY_ARRAY_H

#include <stdio.h>
#include <gpuarray/buffer.h>
#include <gpuarray/util.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct _GpuArray {
  gpudata *data;       /* device buffer (reference counted) */
  size_t *dimensions;  /* nd extents, owned by the array */
  ssize_t *strides;    /* nd byte strides, owned by the array */
  size_t offset;       /* byte offset of element [0,...,0] inside data */
  unsigned int nd;
  int flags;           /* GA_* array flags below */
  int typecode;
} GpuArray;

#define GA_C_CONTIGUOUS 0x0001
#define GA_F_CONTIGUOUS 0x0002
#define GA_ALIGNED      0x0100  /* offset and strides are multiples of the type alignment */
#define GA_WRITEABLE    0x0400
#define GA_BEHAVED      (GA_ALIGNED | GA_WRITEABLE)
#define GA_CARRAY       (GA_C_CONTIGUOUS | GA_BEHAVED)
#define GA_FARRAY       (GA_F_CONTIGUOUS | GA_BEHAVED)

typedef enum _ga_order { GA_ANY_ORDER = -1, GA_C_ORDER = 0, GA_F_ORDER = 1 } ga_order;

static inline int GpuArray_CHKFLAGS(const GpuArray *a, int flags) {
  return (a->flags & flags) == flags;
}
#define GpuArray_ISWRITEABLE(a)      GpuArray_CHKFLAGS(a, GA_WRITEABLE)
#define GpuArray_ISALIGNED(a)        GpuArray_CHKFLAGS(a, GA_ALIGNED)
#define GpuArray_ISONESEGMENT(a)     ((a)->flags & (GA_C_CONTIGUOUS | GA_F_CONTIGUOUS))
#define GpuArray_IS_C_CONTIGUOUS(a)  GpuArray_CHKFLAGS(a, GA_C_CONTIGUOUS)
#define GpuArray_IS_F_CONTIGUOUS(a)  GpuArray_CHKFLAGS(a, GA_F_CONTIGUOUS)
#define GpuArray_ISFORTRAN(a) \
  (GpuArray_CHKFLAGS(a, GA_F_CONTIGUOUS) && !GpuArray_CHKFLAGS(a, GA_C_CONTIGUOUS))
#define GpuArray_ITEMSIZE(a)         gpuarray_get_elsize((a)->typecode)

/* Recomputes the contiguity and alignment flags from dims/strides/offset,
 * keeping only GA_WRITEABLE (reference array.h:199; rules in
 * src/gpuarray_array.c:1159-1194: size-1 dimensions ignore their stride). */
/* replaces src/gpuarray/array.h:199 */
GPUARRAY_PUBLIC void GpuArray_fix_flags(GpuArray *a);

/* Allocation (reference array.h:218-269). nd == 0 makes a 0-d array. */
/* replaces src/gpuarray/array.h:218 */
GPUARRAY_PUBLIC int GpuArray_empty(GpuArray *a, gpucontext *ctx, int typecode,
                                   unsigned int nd, const size_t *dims, ga_order ord);
/* replaces src/gpuarray/array.h:239 */
GPUARRAY_PUBLIC int GpuArray_zeros(GpuArray *a, gpucontext *ctx, int typecode,
                                   unsigned int nd, const size_t *dims, ga_order ord);
/* replaces src/gpuarray/array.h:265 */
GPUARRAY_PUBLIC int GpuArray_fromdata(GpuArray *a, gpudata *data, size_t offset,
                                      int typecode, unsigned int nd, const size_t *dims,
                                      const ssize_t *strides, int writeable);

/* Views (no data movement; reference array.h:286-421). */
/* replaces src/gpuarray/array.h:286 */
GPUARRAY_PUBLIC int GpuArray_view(GpuArray *v, const GpuArray *a);
/* replaces src/gpuarray/array.h:296 */
GPUARRAY_PUBLIC int GpuArray_sync(GpuArray *a);
/* Python-style slicing: steps[i] == 0 drops dimension i at index starts[i]. */
/* replaces src/gpuarray/array.h:321 */
GPUARRAY_PUBLIC int GpuArray_index(GpuArray *r, const GpuArray *a, const ssize_t *starts,
                                   const ssize_t *stops, const ssize_t *steps);
/* replaces src/gpuarray/array.h:325 */
GPUARRAY_PUBLIC int GpuArray_index_inplace(GpuArray *a, const ssize_t *starts,
                                           const ssize_t *stops, const ssize_t *steps);
/* replaces src/gpuarray/array.h:394 */
GPUARRAY_PUBLIC int GpuArray_reshape(GpuArray *res, const GpuArray *a, unsigned int nd,
                                     const size_t *newdims, ga_order ord, int nocopy);
/* replaces src/gpuarray/array.h:398 */
GPUARRAY_PUBLIC int GpuArray_reshape_inplace(GpuArray *a, unsigned int nd,
                                             const size_t *newdims, ga_order ord);
/* new_axes == NULL reverses the axes. */
/* replaces src/gpuarray/array.h:417 */
GPUARRAY_PUBLIC int GpuArray_transpose(GpuArray *res, const GpuArray *a,
                                       const unsigned int *new_axes);
/* replaces src/gpuarray/array.h:420 */
GPUARRAY_PUBLIC int GpuArray_transpose_inplace(GpuArray *a, const unsigned int *new_axes);

/* replaces src/gpuarray/array.h:436 */
GPUARRAY_PUBLIC void GpuArray_clear(GpuArray *a);
/* replaces src/gpuarray/array.h:446 */
GPUARRAY_PUBLIC int GpuArray_share(const GpuArray *a, const GpuArray *b);
/* replaces src/gpuarray/array.h:455 */
GPUARRAY_PUBLIC gpucontext *GpuArray_context(const GpuArray *a);

/* Data movement (reference array.h:374,469-535). Typed/strided copies run
 * through the elementwise engine, like the reference's ga_extcopy
 * (src/gpuarray_array.c:42-86). */
/* replaces src/gpuarray/array.h:374 */
GPUARRAY_PUBLIC int GpuArray_setarray(GpuArray *a, const GpuArray *v);
/* replaces src/gpuarray/array.h:469 */
GPUARRAY_PUBLIC int GpuArray_move(GpuArray *dst, const GpuArray *src);
/* Host transfers need a one-segment (C or F contiguous) device array. */
/* replaces src/gpuarray/array.h:481 */
GPUARRAY_PUBLIC int GpuArray_write(GpuArray *dst, const void *src, size_t src_sz);
/* replaces src/gpuarray/array.h:494 */
GPUARRAY_PUBLIC int GpuArray_read(void *dst, size_t dst_sz, const GpuArray *src);
/* replaces src/gpuarray/array.h:506 */
GPUARRAY_PUBLIC int GpuArray_memset(GpuArray *a, int data);
/* replaces src/gpuarray/array.h:517 */
GPUARRAY_PUBLIC int GpuArray_copy(GpuArray *res, const GpuArray *a, ga_order order);
/* replaces src/gpuarray/array.h:535 */
GPUARRAY_PUBLIC int GpuArray_transfer(GpuArray *res, const GpuArray *a);
/* replaces src/gpuarray/array.h:557 */
GPUARRAY_PUBLIC int GpuArray_split(GpuArray **rs, const GpuArray *a, size_t n, size_t *p,
                                   unsigned int axis);
/* replaces src/gpuarray/array.h:575 */
GPUARRAY_PUBLIC int GpuArray_concatenate(GpuArray *r, const GpuArray **as, size_t n,
                                         unsigned int axis, int restype);
/* Gather rows of v along axis 0 (reference array.h:355). */
/* replaces src/gpuarray/array.h:355 */
GPUARRAY_PUBLIC int GpuArray_take1(GpuArray *a, const GpuArray *v, const GpuArray *i,
                                   int check_error);

/* replaces src/gpuarray/array.h:594 */
GPUARRAY_PUBLIC const char *GpuArray_error(const GpuArray *a, int err);
/* replaces src/gpuarray/array.h:603 */
GPUARRAY_PUBLIC void GpuArray_fprintf(FILE *fd, const GpuArray *a);
/* replaces src/gpuarray/array.h:605 */
GPUARRAY_PUBLIC int GpuArray_fdump(FILE *fd, const GpuArray *a);

/* Maximum and flattened index of the maximum over the axes in reduxList
 * (reference array.h:607-644, src/gpuarray_reduction.c:100-124).
 *
 * dstMax / dstArgmax have the non-reduced axes of src in ascending order
 * (0-d when every axis is reduced); dstArgmax holds 8-byte integers. The
 * index is the mixed-radix number of the reduced coordinates in reduxList
 * order, last listed axis fastest. Ties keep the first element in that
 * order (strict '>'); a NaN is returned only when it is that first element.
 * Implemented as GpuReduction MAXANDARGMAX (see reduction.h). */
/* replaces src/gpuarray/array.h:640 */
GPUARRAY_PUBLIC int GpuArray_maxandargmax(GpuArray *dstMax, GpuArray *dstArgmax,
                                          const GpuArray *src, unsigned reduxLen,
                                          const unsigned *reduxList);

#ifdef __cplusplus
}
#endif
#endif
