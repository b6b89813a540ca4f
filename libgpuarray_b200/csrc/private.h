/* Internal declarations shared by the host sources of the B200 engine.
 *
 * Layering (bottom to top):
 *   ga_dl.c        run-time binding to libcuda / libnvrtc / libnccl
 *   ga_error.c     error records, string builder
 *   ga_types.c     type table
 *   ga_util.c      collapse, type flags
 *   ga_context.c   contexts, buffers, block cache
 *   ga_compile.c   NVRTC -> cubin -> CUfunction, with memory and disk caches
 *   ga_kernel.c    gpukernel / GpuKernel (user supplied kernels)
 *   ga_array.c     GpuArray bookkeeping and copies
 *   ga_elemwise.c  elementwise engine
 *   ga_reduction.c reduction engine
 *   ga_comm.c      NCCL collectives
 */
#ifndef GA_B200_PRIVATE_H
#define GA_B200_PRIVATE_H

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <errno.h>

#include <cuda.h>
#include <nvrtc.h>

#include <gpuarray/config.h>
#include <gpuarray/error.h>
#include <gpuarray/types.h>
#include <gpuarray/buffer.h>
#include <gpuarray/util.h>
#include <gpuarray/array.h>
#include <gpuarray/kernel.h>
#include <gpuarray/elemwise.h>
#include <gpuarray/reduction.h>
#include <gpuarray/extension.h>
#include <gpuarray/buffer_collectives.h>
#include <gpuarray/collectives.h>

#define ISSET(v, fl) (((v) & (fl)) != 0)
#define ISCLR(v, fl) (((v) & (fl)) == 0)

#define GA_HIDDEN __attribute__((visibility("hidden")))

/* ------------------------------------------------------------------ errors */

#define GA_ERR_MSGLEN 1024
typedef struct ga_error_rec {
  char msg[GA_ERR_MSGLEN];
  int code;
} ga_error_rec;

/* Used when no context is at hand (context creation, NULL arguments). */
extern GA_HIDDEN ga_error_rec *ga_global_err;

GA_HIDDEN int ga_err_set(ga_error_rec *e, int code, const char *msg);
GA_HIDDEN int ga_err_fmt(ga_error_rec *e, int code, const char *fmt, ...)
    __attribute__((format(printf, 3, 4)));
GA_HIDDEN int ga_err_sys(ga_error_rec *e, const char *what);
/* "<call>: <NAME>: <description>" as GA_IMPL_ERROR (reference src/private_cuda.h:45-50). */
GA_HIDDEN int ga_err_cuda(ga_error_rec *e, const char *call, CUresult r);

/* ---------------------------------------------------------- string builder */

typedef struct ga_strb {
  char *s;
  size_t len;
  size_t cap;
  int failed;
} ga_strb;

GA_HIDDEN void ga_strb_init(ga_strb *sb);
GA_HIDDEN void ga_strb_free(ga_strb *sb);
GA_HIDDEN void ga_strb_puts(ga_strb *sb, const char *s);
GA_HIDDEN void ga_strb_putn(ga_strb *sb, const char *s, size_t n);
GA_HIDDEN void ga_strb_printf(ga_strb *sb, const char *fmt, ...)
    __attribute__((format(printf, 2, 3)));
/* NUL-terminated view; "" if nothing was appended. */
GA_HIDDEN const char *ga_strb_cstr(ga_strb *sb);

GA_HIDDEN uint64_t ga_hash64(const void *data, size_t len, uint64_t seed);

/* ------------------------------------------------------- dynamic libraries */

/* X(name) lists: the macro-expanded name (e.g. cuMemAlloc_v2) is what is
 * looked up, so the versioned driver ABI of <cuda.h> is honoured. */
#define GA_CU_FUNCS(X)                                                              \
  X(cuInit) X(cuDriverGetVersion) X(cuGetErrorName) X(cuGetErrorString)            \
  X(cuDeviceGetCount) X(cuDeviceGet) X(cuDeviceGetName) X(cuDeviceGetAttribute)    \
  X(cuDeviceTotalMem) X(cuDeviceGetPCIBusId)                                       \
  X(cuDevicePrimaryCtxRetain) X(cuDevicePrimaryCtxRelease)                         \
  X(cuCtxPushCurrent) X(cuCtxPopCurrent) X(cuCtxGetCurrent) X(cuCtxSynchronize)    \
  X(cuCtxGetDevice)                                                                \
  X(cuStreamCreate) X(cuStreamDestroy) X(cuStreamSynchronize) X(cuStreamWaitEvent) \
  X(cuStreamIsCapturing)                                                           \
  X(cuMemAlloc) X(cuMemFree) X(cuMemHostAlloc) X(cuMemFreeHost)                    \
  X(cuMemHostGetDevicePointer) X(cuMemGetInfo) X(cuMemGetAddressRange)             \
  X(cuMemcpyHtoDAsync) X(cuMemcpyDtoHAsync) X(cuMemcpyDtoDAsync) X(cuMemcpyPeerAsync) \
  X(cuMemsetD8Async)                                                               \
  X(cuModuleLoadData) X(cuModuleUnload) X(cuModuleGetFunction)                     \
  X(cuFuncGetAttribute) X(cuFuncSetAttribute) X(cuLaunchKernel) X(cuLaunchKernelEx) \
  X(cuOccupancyMaxActiveBlocksPerMultiprocessor)                                   \
  X(cuEventCreate) X(cuEventRecord) X(cuEventSynchronize) X(cuEventElapsedTime)    \
  X(cuEventDestroy)                                                                \
  X(cuIpcGetMemHandle) X(cuIpcOpenMemHandle) X(cuIpcCloseMemHandle)

#define GA_NVRTC_FUNCS(X)                                                           \
  X(nvrtcVersion) X(nvrtcGetErrorString) X(nvrtcCreateProgram) X(nvrtcDestroyProgram) \
  X(nvrtcCompileProgram) X(nvrtcGetCUBINSize) X(nvrtcGetCUBIN)                     \
  X(nvrtcGetProgramLogSize) X(nvrtcGetProgramLog)

struct ga_cuda_api {
#define X(n) __typeof__(&n) p_##n;
  GA_CU_FUNCS(X)
#undef X
};
struct ga_nvrtc_api {
#define X(n) __typeof__(&n) p_##n;
  GA_NVRTC_FUNCS(X)
#undef X
};
extern GA_HIDDEN struct ga_cuda_api ga_cu;
extern GA_HIDDEN struct ga_nvrtc_api ga_rtc;

/* Each returns GA_NO_ERROR or GA_LOAD_ERROR (message in e). Idempotent. */
GA_HIDDEN int ga_load_cuda(ga_error_rec *e);
GA_HIDDEN int ga_load_nvrtc(ga_error_rec *e);

/* ---------------------------------------------------------------- contexts */

typedef struct ga_block {          /* one cached device allocation */
  CUdeviceptr ptr;
  size_t sz;
  struct ga_block *next;
} ga_block;

struct ga_module;                  /* ga_compile.c */

struct _gpucontext_props {
  int dev;
  int sched;
  int flags;
  char *kernel_cache_path;
  size_t max_cache_size;
  size_t initial_cache_size;
};

struct _gpucontext {
  ga_error_rec *err;
  unsigned int refcnt;
  int flags;
  int dev;                         /* CUDA ordinal */
  CUdevice cudev;
  CUcontext cu;                    /* primary context of the device */
  CUstream s;                      /* the one in-order stream */
  int own_ctx;                     /* 1: primary context retained by us */
  unsigned enter_depth;
  gpudata *errbuf;                 /* 8 zeroed bytes, GA_CTX_PROP_ERRBUF */
  /* device facts used by launch heuristics */
  unsigned int num_sms;
  size_t max_smem_block;           /* opt-in maximum shared memory per block */
  size_t smem_block;               /* default limit */
  size_t max_threads;              /* per block */
  size_t max_grid[3];
  size_t max_block[3];
  size_t l2_bytes;
  char devname[256];
  char pci_id[16];
  char bin_id[16];
  /* block cache */
  ga_block *free_blocks;
  size_t cached_bytes;
  size_t max_cached_bytes;
  /* compiled kernel cache */
  struct ga_module *modules;
  char *kernel_cache_path;
  /* engine-private helper objects created on demand (ga_array.c) */
  void *extcopy_cache;
  /* lazily created MAXANDARGMAX operators keyed by source type (ga_reduction.c) */
  void *maxandargmax_cache;
  void *take1_cache;        /* compiled gather kernels by (types, rank): ga_array.c */
  void *peer_windows;       /* exported windows of freed communicators, for reuse: ga_comm.c */
};

#define GA_BUF_EXTERNAL 0x10000    /* memory not owned (cuda_make_buf) */
#define GA_BUF_IPC      0x20000    /* opened from an IPC handle */

struct _gpudata {
  CUdeviceptr ptr;                 /* MUST stay first: &gpudata is a kernel parameter slot */
  gpucontext *ctx;                 /* MUST stay second (reference src/private.h:77-80) */
  size_t sz;                       /* size the caller asked for */
  size_t asz;                      /* size of the underlying block */
  unsigned int refcnt;
  int flags;
  void *host;                      /* GA_BUFFER_HOST: the pinned host pointer */
};

GA_HIDDEN void ga_ctx_enter(gpucontext *ctx);
GA_HIDDEN void ga_ctx_exit(gpucontext *ctx);
/* Drops one internal reference (buffers, kernels); may destroy the context. */
GA_HIDDEN void ga_ctx_unref(gpucontext *ctx);

/* -------------------------------------------------------------- compilation */

typedef struct ga_function {
  CUfunction f;
  int max_threads;                 /* CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK */
  int num_regs;
  int static_smem;
  int dependent_ok;                /* the kernel calls ga__grid_dependency_sync() before it
                                      touches memory: may launch with serialization relaxed */
} ga_function;

/* Names of the in-library header files handed to NVRTC ("cluda.h", the
 * kernel templates). Generated at build time from csrc/templates. */
extern GA_HIDDEN const char *const ga_template_names[];
extern GA_HIDDEN const char *const ga_template_sources[];
extern GA_HIDDEN const unsigned int ga_template_count;

/* Compiles `src` for sm_100a (or fetches it from the caches) and resolves the
 * kernel `fname`. `defines` is a NULL-terminated list of "-DNAME=VALUE"
 * strings (may be NULL). On a compile error returns GA_IMPL_ERROR; if
 * err_str is not NULL it receives a malloc'ed numbered listing plus the log. */
GA_HIDDEN int ga_compile(gpucontext *ctx, const char *src, const char *fname,
                         const char *const *defines, ga_function *out, char **err_str);
/* Compile only (no device needed): cubin bytes are malloc'ed into *bin. */
GA_HIDDEN int ga_compile_cubin(ga_error_rec *e, const char *src, const char *const *defines,
                               const char *cache_dir, char **bin, size_t *bin_sz,
                               char **err_str);
GA_HIDDEN void ga_modules_free(gpucontext *ctx);

/* Launch on the context stream. grid/block are CUDA dims. */
GA_HIDDEN int ga_launch(gpucontext *ctx, const ga_function *fn, const unsigned grid[3],
                        const unsigned block[3], size_t shared, void **params);

/* ------------------------------------------------------------------ kernels */

struct _gpukernel {
  gpucontext *ctx;                 /* MUST stay first (reference src/private.h:82-84) */
  unsigned int refcnt;
  ga_function fn;
  unsigned int argcount;
  int *types;
  void **args;                     /* values stored by gpukernel_setarg */
};

/* ------------------------------------------------------------------- arrays */

GA_HIDDEN int ga_array_is_c_contiguous(const GpuArray *a);
GA_HIDDEN int ga_array_is_f_contiguous(const GpuArray *a);
/* 1 when every element of `a` lies inside its buffer (bytes [0, size) of a->data). */
GA_HIDDEN int ga_array_in_bounds(const GpuArray *a);
GA_HIDDEN void ga_extcopy_cache_free(gpucontext *ctx);
GA_HIDDEN void ga_maxandargmax_cache_free(gpucontext *ctx);
GA_HIDDEN void ga_take1_cache_free(gpucontext *ctx);
GA_HIDDEN void ga_peer_windows_free(gpucontext *ctx);

/* Combination of per-GPU partial results through peer memory (ga_comm.c). */
struct _gpucomm;
enum { GA_XC_AND = 100, GA_XC_OR = 101, GA_XC_XOR = 102 }; /* beside GA_SUM .. GA_MIN */
GA_HIDDEN int ga_comm_peer_ready(struct _gpucomm *comm, size_t bytes_per_rank);
GA_HIDDEN int ga_comm_exchange(struct _gpucomm *comm, int pair, int op, int tc, CUdeviceptr val,
                               CUdeviceptr idx, size_t n, unsigned long long key);

/* Name of the C type used in kernel source for a typecode, or NULL. */
GA_HIDDEN const char *ga_ctype(int typecode);
/* 1 for the scalar types kernels can compute on (no complex, no 16-byte ints). */
GA_HIDDEN int ga_type_is_computable(int typecode);

#define GA_ADDR32_MAX   4294967295UL
#define GA_SADDR32_MIN (-2147483648L)
#define GA_SADDR32_MAX   2147483647L

#endif
