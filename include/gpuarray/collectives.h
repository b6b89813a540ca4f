/* Collectives on GpuArrays (reference src/gpuarray/collectives.h:31-126,
 * src/gpuarray_array_collectives.c). Arrays must be contiguous and aligned;
 * source and destination must agree in type and element count. */
#ifndef GPUARRAY_COLLECTIVES_H
#define GPUARRAY_COLLECTIVES_H

#include <gpuarray/array.h>
#include <gpuarray/buffer_collectives.h>

#ifdef __cplusplus
extern "C" {
#endif

/* replaces src/gpuarray/collectives.h:33 */
GPUARRAY_PUBLIC int GpuArray_reduce_from(const GpuArray *src, int opcode, int root, gpucomm *comm);
/* replaces src/gpuarray/collectives.h:53 */
GPUARRAY_PUBLIC int GpuArray_reduce(const GpuArray *src, GpuArray *dest, int opcode, int root,
                                    gpucomm *comm);
/* replaces src/gpuarray/collectives.h:71 */
GPUARRAY_PUBLIC int GpuArray_all_reduce(const GpuArray *src, GpuArray *dest, int opcode,
                                        gpucomm *comm);
/* replaces src/gpuarray/collectives.h:90 */
GPUARRAY_PUBLIC int GpuArray_reduce_scatter(const GpuArray *src, GpuArray *dest, int opcode,
                                            gpucomm *comm);
/* replaces src/gpuarray/collectives.h:106 */
GPUARRAY_PUBLIC int GpuArray_broadcast(GpuArray *array, int root, gpucomm *comm);
/* replaces src/gpuarray/collectives.h:124 */
GPUARRAY_PUBLIC int GpuArray_all_gather(const GpuArray *src, GpuArray *dest, gpucomm *comm);

#ifdef __cplusplus
}
#endif
#endif
