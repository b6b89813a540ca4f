/* Multi-GPU collectives on raw buffers: one communicator per context, one
 * process per GPU, NCCL over NVLink underneath.
 *
 * Same entry points as the reference's src/gpuarray/buffer_collectives.h
 * (:30-257; implementation src/gpuarray_collectives_cuda_nccl.c). The engine
 * itself uses only gpucomm_all_reduce, to finish reductions whose reduced
 * extent is sharded over GPUs. Every call enqueues on the context's stream. */
#ifndef GPUARRAY_BUFFER_COLLECTIVES_H
#define GPUARRAY_BUFFER_COLLECTIVES_H

#include <gpuarray/buffer.h>
#include <gpuarray/config.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct _gpucomm gpucomm;

enum gpucomm_reduce_ops { GA_SUM = 0, GA_PROD = 1, GA_MAX = 2, GA_MIN = 3 };

#define GA_COMM_ID_BYTES 128
typedef struct _gpucommCliqueId { char internal[GA_COMM_ID_BYTES]; } gpucommCliqueId;

/* Blocks until all ndev ranks have joined with the same clique id. */
/* replaces src/gpuarray/buffer_collectives.h:63 */
GPUARRAY_PUBLIC int gpucomm_new(gpucomm **comm, gpucontext *ctx, gpucommCliqueId comm_id,
                                int ndev, int rank);
/* replaces src/gpuarray/buffer_collectives.h:71 */
GPUARRAY_PUBLIC void gpucomm_free(gpucomm *comm);
/* replaces src/gpuarray/buffer_collectives.h:80 */
GPUARRAY_PUBLIC const char *gpucomm_error(gpucontext *ctx);
/* replaces src/gpuarray/buffer_collectives.h:89 */
GPUARRAY_PUBLIC gpucontext *gpucomm_context(gpucomm *comm);
/* Made on one rank and distributed out of band to the others. */
/* replaces src/gpuarray/buffer_collectives.h:102 */
GPUARRAY_PUBLIC int gpucomm_gen_clique_id(gpucontext *ctx, gpucommCliqueId *comm_id);
/* replaces src/gpuarray/buffer_collectives.h:113 */
GPUARRAY_PUBLIC int gpucomm_get_count(gpucomm *comm, int *devcount);
/* replaces src/gpuarray/buffer_collectives.h:123 */
GPUARRAY_PUBLIC int gpucomm_get_rank(gpucomm *comm, int *rank);

/* count is in elements of `typecode`; supported types are GA_BYTE, GA_INT,
 * GA_UINT, GA_LONG, GA_ULONG, GA_HALF, GA_FLOAT, GA_DOUBLE. Counts above
 * INT_MAX give GA_XLARGE_ERROR, like the reference (:201-202). */
/* replaces src/gpuarray/buffer_collectives.h:148 */
GPUARRAY_PUBLIC int gpucomm_reduce(gpudata *src, size_t offsrc, gpudata *dest, size_t offdest,
                                   size_t count, int typecode, int opcode, int root,
                                   gpucomm *comm);
/* replaces src/gpuarray/buffer_collectives.h:175 */
GPUARRAY_PUBLIC int gpucomm_all_reduce(gpudata *src, size_t offsrc, gpudata *dest,
                                       size_t offdest, size_t count, int typecode, int opcode,
                                       gpucomm *comm);
/* replaces src/gpuarray/buffer_collectives.h:203 */
GPUARRAY_PUBLIC int gpucomm_reduce_scatter(gpudata *src, size_t offsrc, gpudata *dest,
                                           size_t offdest, size_t count, int typecode,
                                           int opcode, gpucomm *comm);
/* replaces src/gpuarray/buffer_collectives.h:225 */
GPUARRAY_PUBLIC int gpucomm_broadcast(gpudata *array, size_t offset, size_t count,
                                      int typecode, int root, gpucomm *comm);
/* replaces src/gpuarray/buffer_collectives.h:248 */
GPUARRAY_PUBLIC int gpucomm_all_gather(gpudata *src, size_t offsrc, gpudata *dest,
                                       size_t offdest, size_t count, int typecode,
                                       gpucomm *comm);

#ifdef __cplusplus
}
#endif
#endif
