/* Named escape hatches for code that mixes its own CUDA calls with the
 * library (reference src/gpuarray/extension.h:19-39, ext_cuda.h:20-44). */
#ifndef GPUARRAY_EXTENSIONS_H
#define GPUARRAY_EXTENSIONS_H

#include <gpuarray/config.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GPUARRAY_CUDA_CTX_NOFREE 0x10000000
#define GPUARRAY_CUDA_WAIT_READ  0x10000
#define GPUARRAY_CUDA_WAIT_WRITE 0x20000

typedef struct _GpuArrayIpcMemHandle { char priv[64]; } GpuArrayIpcMemHandle;

/* Known names: "cuda_enter", "cuda_exit", "cuda_make_ctx", "cuda_get_stream",
 * "cuda_make_buf", "cuda_get_sz", "cuda_wait", "cuda_record",
 * "cuda_get_ipc_handle", "cuda_open_ipc_handle". Unknown names give NULL. */
/* replaces src/gpuarray/extension.h:31 */
GPUARRAY_PUBLIC void *gpuarray_get_extension(const char *name);

#ifdef __cplusplus
}
#endif
#endif
