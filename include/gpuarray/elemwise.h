/* Elementwise engine: a C expression over named scalars, applied to every
 * element of strided, broadcastable arrays.
 *
 * Same surface as the reference's src/gpuarray/elemwise.h:28-162; flag values
 * are ABI. The kernels behind it are sm_100a templates (contiguous 128-bit
 * vectorised, collapsed-strided, broadcast, tiled transpose) with the
 * expression compiled in by NVRTC. */
#ifndef GPUARRAY_ELEMWISE_H
#define GPUARRAY_ELEMWISE_H

#include <gpuarray/buffer.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct _GpuElemwise GpuElemwise;

/* One argument of the expression (reference elemwise.h:28-68). Inside the
 * expression the argument is a scalar variable called `name` of the C type of
 * `typecode` (float when the type is GA_HALF and GE_CONVERT_F16 is set). */
typedef struct _gpuelemwise_arg {
  const char *name;
  int typecode;
  int flags;
#define GE_SCALAR 0x0001  /* passed by value at call time, not an array */
#define GE_READ   0x0002  /* loaded before the expression */
#define GE_WRITE  0x0004  /* stored after the expression */
} gpuelemwise_arg;

/* Constructor flags (reference elemwise.h:114-119). */
#define GE_NOADDR64    0x0001  /* hint only: 64-bit index kernels are still built on demand */
#define GE_CONVERT_F16 0x0002  /* compute GA_HALF arguments as float */

/* Call flags (reference elemwise.h:152-162). */
#define GE_BROADCAST  0x0100  /* size-1 input dimensions stretch to the output's */
#define GE_NOCOLLAPSE 0x0200  /* accepted; the result is the same either way */
#define GE_PADSHAPE   0x0400  /* lower-rank arguments get leading size-1 dimensions */

/* Builds the operation (reference elemwise.h:98-104, src/gpuarray_elemwise.c:604-737).
 *  preamble  code placed before the kernel (helper functions, macros); may be NULL
 *  expr      C statement(s) over the argument names, no trailing ';' needed
 *  n, args   argument descriptors, deep-copied
 *  nd        rank hint for ahead-of-time compilation; any rank works at call time
 * Returns NULL on failure with the reason in the context's error. */
/* replaces src/gpuarray/elemwise.h:98 */
GPUARRAY_PUBLIC GpuElemwise *GpuElemwise_new(gpucontext *ctx, const char *preamble,
                                             const char *expr, unsigned int n,
                                             gpuelemwise_arg *args, unsigned int nd, int flags);
/* NULL is allowed (the reference requires non-NULL). */
/* replaces src/gpuarray/elemwise.h:130 */
GPUARRAY_PUBLIC void GpuElemwise_free(GpuElemwise *ge);

/* Runs the operation (reference elemwise.h:140, src/gpuarray_elemwise.c:767-787).
 * args[i] is a GpuArray* for array arguments and a pointer to a host value of
 * the declared type for GE_SCALAR ones. The first GE_WRITE array defines the
 * shape; outputs never broadcast. Zero-size shapes succeed without a launch.
 * Returns after enqueueing on the context's stream. */
/* replaces src/gpuarray/elemwise.h:140 */
GPUARRAY_PUBLIC int GpuElemwise_call(GpuElemwise *ge, void **args, int flags);

#ifdef __cplusplus
}
#endif
#endif
