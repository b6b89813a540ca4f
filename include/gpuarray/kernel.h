/* GpuKernel: a gpukernel plus its stored argument values.
 * Follows src/gpuarray/kernel.h:20-112 of the reference. */
#ifndef GPUARRAY_KERNEL_H
#define GPUARRAY_KERNEL_H

#include <gpuarray/buffer.h>
#include <gpuarray/array.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct _GpuKernel {
  gpukernel *k;
  void **args;
} GpuKernel;

/* replaces src/gpuarray/kernel.h:54 */
GPUARRAY_PUBLIC int GpuKernel_init(GpuKernel *k, gpucontext *ctx, unsigned int count,
                                   const char **strs, const size_t *lens, const char *name,
                                   unsigned int argcount, const int *types, int flags,
                                   char **err_str);
/* replaces src/gpuarray/kernel.h:65 */
GPUARRAY_PUBLIC void GpuKernel_clear(GpuKernel *k);
/* replaces src/gpuarray/kernel.h:74 */
GPUARRAY_PUBLIC gpucontext *GpuKernel_context(GpuKernel *k);
/* replaces src/gpuarray/kernel.h:77 */
GPUARRAY_PUBLIC int GpuKernel_setarg(GpuKernel *k, unsigned int i, void *val);
/* 1-D launch shape for n work items: *ls threads per block, *gs blocks.
 * Non-zero inputs are respected. Heuristic of src/gpuarray_kernel.c:38-89. */
/* replaces src/gpuarray/kernel.h:95 */
GPUARRAY_PUBLIC int GpuKernel_sched(GpuKernel *k, size_t n, size_t *gs, size_t *ls);
/* replaces src/gpuarray/kernel.h:108 */
GPUARRAY_PUBLIC int GpuKernel_call(GpuKernel *k, unsigned int n, const size_t *gs,
                                   const size_t *ls, size_t shared, void **args);
/* replaces src/gpuarray/kernel.h:112 */
GPUARRAY_PUBLIC const char *GpuKernel_error(const GpuKernel *k, int err);

#ifdef __cplusplus
}
#endif
#endif
