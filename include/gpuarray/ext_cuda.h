/* Typed access to the CUDA extensions (reference src/gpuarray/ext_cuda.h:20-44).
 * Include <cuda.h> first. cuda_wait / cuda_record are no-ops that return
 * GA_NO_ERROR here because every operation of a context runs on one in-order
 * stream; external work must be enqueued on cuda_get_stream(ctx) or
 * synchronised with it. */
#ifndef LIBGPU_EXT_CUDA
#define LIBGPU_EXT_CUDA

#include <cuda.h>
#include <gpuarray/config.h>
#include <gpuarray/buffer.h>
#include <gpuarray/extension.h>

#ifdef __cplusplus
extern "C" {
#endif

static void (*cuda_enter)(gpucontext *);
static void (*cuda_exit)(gpucontext *);
static gpucontext *(*cuda_make_ctx)(CUcontext, int);
static CUstream (*cuda_get_stream)(void *);
static gpudata *(*cuda_make_buf)(void *, CUdeviceptr, size_t);
static size_t (*cuda_get_sz)(gpudata *);
static int (*cuda_wait)(gpudata *, int);
static int (*cuda_record)(gpudata *, int);
static CUipcMemHandle (*cuda_get_ipc_handle)(gpudata *);
static gpudata *(*cuda_open_ipc_handle)(gpucontext *, CUipcMemHandle, size_t);

static void setup_ext_cuda(void) {
#define GA__EXT(n, T) n = (T)gpuarray_get_extension(#n)
  GA__EXT(cuda_enter, void (*)(gpucontext *));
  GA__EXT(cuda_exit, void (*)(gpucontext *));
  GA__EXT(cuda_make_ctx, gpucontext *(*)(CUcontext, int));
  GA__EXT(cuda_get_stream, CUstream (*)(void *));
  GA__EXT(cuda_make_buf, gpudata *(*)(void *, CUdeviceptr, size_t));
  GA__EXT(cuda_get_sz, size_t (*)(gpudata *));
  GA__EXT(cuda_wait, int (*)(gpudata *, int));
  GA__EXT(cuda_record, int (*)(gpudata *, int));
  GA__EXT(cuda_get_ipc_handle, CUipcMemHandle (*)(gpudata *));
  GA__EXT(cuda_open_ipc_handle, gpudata *(*)(gpucontext *, CUipcMemHandle, size_t));
#undef GA__EXT
}

#ifdef __cplusplus
}
#endif
#endif
