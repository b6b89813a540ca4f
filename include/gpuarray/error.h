/* Error codes returned by every entry point.
 *
 * Values are ABI: they are identical to the reference's enum ga_error
 * (src/gpuarray/error.h:19-42), because pygpu and Theano compare against the
 * numeric values. */
#ifndef GPUARRAY_ERROR_H
#define GPUARRAY_ERROR_H

#include <gpuarray/config.h>

#ifdef __cplusplus
extern "C" {
#endif

enum ga_error {
  GA_NO_ERROR          = 0,
  GA_MEMORY_ERROR      = 1,  /* host or device allocation failed */
  GA_VALUE_ERROR       = 2,  /* shape / rank / broadcast problem */
  GA_IMPL_ERROR        = 3,  /* CUDA driver or NVRTC failure; text in the context */
  GA_INVALID_ERROR     = 4,  /* argument that can never be valid */
  GA_UNSUPPORTED_ERROR = 5,
  GA_SYS_ERROR         = 6,  /* errno has the detail */
  GA_RUN_ERROR         = 7,
  GA_DEVSUP_ERROR      = 8,
  GA_READONLY_ERROR    = 9,
  GA_WRITEONLY_ERROR   = 10,
  GA_BLAS_ERROR        = 11,
  GA_UNALIGNED_ERROR   = 12,
  GA_COPY_ERROR        = 13,
  GA_NODEV_ERROR       = 14,
  GA_MISC_ERROR        = 15,
  GA_COMM_ERROR        = 16,
  GA_XLARGE_ERROR      = 17,
  GA_LOAD_ERROR        = 18
};

/* Static description of a code; replaces src/gpuarray_error.c:7-30. */
/* replaces src/gpuarray/error.h:49 */
GPUARRAY_PUBLIC const char *gpuarray_error_str(int err);

#ifdef __cplusplus
}
#endif
#endif
