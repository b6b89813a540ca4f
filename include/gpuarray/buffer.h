/* Contexts, device buffers and raw kernels: the thin layer over the CUDA
 * driver that the elementwise and reduction engines stand on.
 *
 * Entry points and constants follow the reference's src/gpuarray/buffer.h
 * (prototypes :56-600, property ids :604-790, use-flags :804-852) so that a
 * client compiled against the reference headers links unchanged. There is a
 * single backend ("cuda", sm_100a); names such as "opencl0:0" are refused
 * with GA_UNSUPPORTED_ERROR. */
#ifndef GPUARRAY_BUFFER_H
#define GPUARRAY_BUFFER_H

#include <gpuarray/config.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct _gpucontext gpucontext;
typedef struct _gpudata gpudata;
typedef struct _gpukernel gpukernel;
typedef struct _gpucontext_props gpucontext_props;

/* ---- enumeration (reference buffer.h:56-72) ---- */
/* replaces src/gpuarray/buffer.h:56 */
GPUARRAY_PUBLIC int gpu_get_platform_count(const char *name, unsigned int *platcount);
/* replaces src/gpuarray/buffer.h:70 */
GPUARRAY_PUBLIC int gpu_get_device_count(const char *name, unsigned int platform,
                                         unsigned int *devcount);

/* ---- context properties (reference buffer.h:89-205) ---- */
#define GA_CTX_SCHED_AUTO   0
#define GA_CTX_SCHED_SINGLE 1
#define GA_CTX_SCHED_MULTI  2

/* replaces src/gpuarray/buffer.h:89 */
GPUARRAY_PUBLIC int gpucontext_props_new(gpucontext_props **res);
/* replaces src/gpuarray/buffer.h:99 */
GPUARRAY_PUBLIC int gpucontext_props_cuda_dev(gpucontext_props *p, int devno);
/* Always fails: there is no OpenCL backend in this engine. */
/* replaces src/gpuarray/buffer.h:111 */
GPUARRAY_PUBLIC int gpucontext_props_opencl_dev(gpucontext_props *p, int platno, int devno);
/* replaces src/gpuarray/buffer.h:122 */
GPUARRAY_PUBLIC int gpucontext_props_sched(gpucontext_props *p, int sched);
/* Accepted and ignored: this engine always runs one in-order stream per context. */
/* replaces src/gpuarray/buffer.h:164 */
GPUARRAY_PUBLIC int gpucontext_props_set_single_stream(gpucontext_props *p);
/* replaces src/gpuarray/buffer.h:177 */
GPUARRAY_PUBLIC int gpucontext_props_kernel_cache(gpucontext_props *p, const char *path);
/* replaces src/gpuarray/buffer.h:192 */
GPUARRAY_PUBLIC int gpucontext_props_alloc_cache(gpucontext_props *p, size_t initial, size_t max);
/* replaces src/gpuarray/buffer.h:205 */
GPUARRAY_PUBLIC void gpucontext_props_del(gpucontext_props *p);

/* ---- context lifetime (reference buffer.h:223-265) ----
 * `name` is "cuda" (device taken from props, default 0) or "cudaN".
 * Takes ownership of `props` (may be NULL). Not thread safe. */
/* replaces src/gpuarray/buffer.h:223 */
GPUARRAY_PUBLIC int gpucontext_init(gpucontext **res, const char *name, gpucontext_props *props);
/* replaces src/gpuarray/buffer.h:236 */
GPUARRAY_PUBLIC void gpucontext_deref(gpucontext *ctx);
/* replaces src/gpuarray/buffer.h:250 */
GPUARRAY_PUBLIC int gpucontext_property(gpucontext *ctx, int prop_id, void *res);
/* Message of the last error on `ctx` (or the process-global one if NULL). */
/* replaces src/gpuarray/buffer.h:265 */
GPUARRAY_PUBLIC const char *gpucontext_error(gpucontext *ctx, int err);

/* ---- buffers (reference buffer.h:283-494) ---- */
#define GA_BUFFER_READ_WRITE 0x00
#define GA_BUFFER_DEV        0x00
#define GA_BUFFER_READ_ONLY  0x01
#define GA_BUFFER_WRITE_ONLY 0x02
#define GA_BUFFER_INIT       0x04 /* copy `data` (sz bytes of host memory) in */
#define GA_BUFFER_HOST       0x08 /* pinned host memory visible to the device */
#define GA_BUFFER_MASK       0xffff

/* replaces src/gpuarray/buffer.h:283 */
GPUARRAY_PUBLIC gpudata *gpudata_alloc(gpucontext *ctx, size_t sz, void *data, int flags, int *ret);
/* replaces src/gpuarray/buffer.h:351 */
GPUARRAY_PUBLIC void gpudata_retain(gpudata *b);
/* replaces src/gpuarray/buffer.h:363 */
GPUARRAY_PUBLIC void gpudata_release(gpudata *b);
/* 1 if the two buffers may overlap in device memory. */
/* replaces src/gpuarray/buffer.h:379 */
GPUARRAY_PUBLIC int gpudata_share(gpudata *a, gpudata *b, int *ret);
/* replaces src/gpuarray/buffer.h:396 */
GPUARRAY_PUBLIC int gpudata_move(gpudata *dst, size_t dstoff, gpudata *src, size_t srcoff, size_t sz);
/* replaces src/gpuarray/buffer.h:416 */
GPUARRAY_PUBLIC int gpudata_transfer(gpudata *dst, size_t dstoff, gpudata *src, size_t srcoff, size_t sz);
/* Blocking device->host copy; the observable synchronisation point. */
/* replaces src/gpuarray/buffer.h:432 */
GPUARRAY_PUBLIC int gpudata_read(void *dst, gpudata *src, size_t srcoff, size_t sz);
/* replaces src/gpuarray/buffer.h:448 */
GPUARRAY_PUBLIC int gpudata_write(gpudata *dst, size_t dstoff, const void *src, size_t sz);
/* Fill from dstoff to the end of the buffer with the byte `data`. */
/* replaces src/gpuarray/buffer.h:462 */
GPUARRAY_PUBLIC int gpudata_memset(gpudata *dst, size_t dstoff, int data);
/* replaces src/gpuarray/buffer.h:476 */
GPUARRAY_PUBLIC int gpudata_sync(gpudata *b);
/* replaces src/gpuarray/buffer.h:492 */
GPUARRAY_PUBLIC int gpudata_property(gpudata *buf, int prop_id, void *res);
/* replaces src/gpuarray/buffer.h:494 */
GPUARRAY_PUBLIC gpucontext *gpudata_context(gpudata *b);

/* ---- raw kernels (reference buffer.h:523-599) ----
 * The source strings are concatenated and compiled with NVRTC for sm_100a.
 * `typecodes` lists the kernel parameters; GA_BUFFER marks a gpudata*. */
/* replaces src/gpuarray/buffer.h:523 */
GPUARRAY_PUBLIC gpukernel *gpukernel_init(gpucontext *ctx, unsigned int count,
                                          const char **strings, const size_t *lengths,
                                          const char *fname, unsigned int numargs,
                                          const int *typecodes, int flags, int *ret,
                                          char **err_str);
/* replaces src/gpuarray/buffer.h:536 */
GPUARRAY_PUBLIC void gpukernel_retain(gpukernel *k);
/* replaces src/gpuarray/buffer.h:547 */
GPUARRAY_PUBLIC void gpukernel_release(gpukernel *k);
/* replaces src/gpuarray/buffer.h:562 */
GPUARRAY_PUBLIC int gpukernel_setarg(gpukernel *k, unsigned int i, void *a);
/* gs = blocks per grid dimension, ls = threads per block dimension (n <= 3).
 * args == NULL uses the values stored by gpukernel_setarg. */
/* replaces src/gpuarray/buffer.h:579 */
GPUARRAY_PUBLIC int gpukernel_call(gpukernel *k, unsigned int n, const size_t *gs,
                                   const size_t *ls, size_t shared, void **args);
/* replaces src/gpuarray/buffer.h:597 */
GPUARRAY_PUBLIC int gpukernel_property(gpukernel *k, int prop_id, void *res);
/* replaces src/gpuarray/buffer.h:599 */
GPUARRAY_PUBLIC gpucontext *gpukernel_context(gpukernel *k);

/* ---- property ids (numeric values are ABI) ---- */
#define GA_CTX_PROP_DEVNAME           1  /* char[256] */
#define GA_CTX_PROP_LMEMSIZE          3  /* size_t: shared memory per block */
#define GA_CTX_PROP_NUMPROCS          4  /* unsigned int: SM count */
#define GA_CTX_PROP_BIN_ID            7  /* const char *: "sm_100a" */
#define GA_CTX_PROP_ERRBUF            8  /* gpudata *: 8 zeroed bytes */
#define GA_CTX_PROP_TOTAL_GMEM        9  /* size_t */
#define GA_CTX_PROP_FREE_GMEM        10  /* size_t */
#define GA_CTX_PROP_NATIVE_FLOAT16   11  /* int */
#define GA_CTX_PROP_MAXGSIZE0        12  /* size_t */
#define GA_CTX_PROP_MAXGSIZE1        13
#define GA_CTX_PROP_MAXGSIZE2        14
#define GA_CTX_PROP_MAXLSIZE0        15
#define GA_CTX_PROP_MAXLSIZE1        16
#define GA_CTX_PROP_MAXLSIZE2        17
#define GA_CTX_PROP_UNIQUE_ID        19  /* char[16]: PCI bus id */
#define GA_CTX_PROP_LARGEST_MEMBLOCK 20  /* size_t */

#define GA_BUFFER_PROP_START  512
#define GA_BUFFER_PROP_CTX    512  /* gpucontext * */
#define GA_BUFFER_PROP_REFCNT 513  /* unsigned int */
#define GA_BUFFER_PROP_SIZE   514  /* size_t */

#define GA_KERNEL_PROP_START     1024
#define GA_KERNEL_PROP_CTX       1024  /* gpucontext * */
#define GA_KERNEL_PROP_MAXLSIZE  1025  /* size_t */
#define GA_KERNEL_PROP_PREFLSIZE 1026  /* size_t: warp size */
#define GA_KERNEL_PROP_NUMARGS   1027  /* unsigned int */
#define GA_KERNEL_PROP_TYPES     1028  /* const int * */

/* Feature flags for gpukernel_init (reference buffer.h:804-852). */
typedef enum _ga_usefl {
  GA_USE_SMALL   = 0x02,
  GA_USE_DOUBLE  = 0x04,
  GA_USE_COMPLEX = 0x08,  /* refused: no complex support */
  GA_USE_HALF    = 0x10,
  GA_USE_CUDA    = 0x2000,
  GA_USE_OPENCL  = 0x4000 /* refused */
} ga_usefl;

#ifdef __cplusplus
}
#endif
#endif
