/* gpuarray_b200_sum_f32_noalloc: the split float32 sum without any allocation.
 *
 * Who needs it: code that must not call cudaMalloc/cudaFree at the moment it
 * wants a reduction - a plugin running inside another framework's memory
 * pool, a real-time loop that may not block on the driver's allocator, a host
 * thread that works between other people's stream-ordered operations. The
 * ordinary path (GpuReduction_call) keeps its partial-result buffer in a
 * gpudata that it allocates on first use and grows on demand; this entry
 * point instead owns a fixed block of device memory that is part of the
 * library image itself.
 *
 * What it runs: the same ga_rd_rows template as the engine (float32 SUM,
 * 128-bit loads, one CTA per work group, partial results published to scratch,
 * the last-arriving group combines them in split order), instantiated here at
 * build time by nvcc. The scratch - partial sums and the arrival ticket -
 * lives in `ga_noalloc_scratch`, a file-scope __device__ array of
 * GA_NOALLOC_SCRATCH_BYTES (64 KiB). Every GPU that loads the library holds
 * that block until the process exits.
 *
 * Rules for callers:
 *  - src and dst are device pointers of the CURRENT device; src is 16-byte
 *    aligned; n <= GPUARRAY_B200_NOALLOC_MAX_ELEMS, larger sizes are refused
 *    with GA_XLARGE_ERROR (text via gpucontext_error(NULL, 0));
 *  - the first call on each device looks up the device address of the scratch
 *    block (cudaGetSymbolAddress, which also makes the runtime load this
 *    module on that device). Make that first call outside of any stream
 *    capture;
 *  - all calls on a device share the one scratch block. The ticket word is
 *    cleared at the start of every call, the partial sums are overwritten
 *    before they are read; but two calls that overlap on the GPU (different
 *    streams, no dependency) race on it. Serialise them.
 */
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define GA_RD_SRC_T ga_float
#define GA_RD_X_T ga_float
#define GA_RD_ACC_T ga_float
#define GA_RD_DST_T ga_float
#define GA_RD_LOAD(raw) (raw)
#define GA_RD_STORE(a) ((GA_RD_DST_T)(a))
#define GA_RD_MAP(x) ((GA_RD_ACC_T)(x))
#define GA_RD_COMBINE(a, b) ((a) + (b))
#define GA_RD_IDENT 0
#define GA_RD_BETTER(b, a) ((b) > (a))
#define GA_RD_KIND 0
#define GA_RD_ISFLOAT 1
#define GA_RD_WRITE_VAL 1
#define GA_RD_WRITE_IDX 0
#define GA_RD_IDX_T unsigned int
#define GA_RD_VEC 4
#define GA_RD_THREADS 256
#define GA_RD_TPO 1
#define GA_RD_BY 8
#define GA_RD_GROUP 256
#define GA_RD_FLAT 0
#define GA_RD_BUILD_ROWS
#include "ga_reduce.cuh"

#include <pthread.h>

extern "C" {
#include <gpuarray/error.h>
#include <gpuarray/b200.h>
}

/* private.h is C; only these two helpers are needed from it */
struct ga_error_rec;
extern "C" int ga_err_fmt(struct ga_error_rec *e, int code, const char *fmt, ...);

#define GA_NOALLOC_MAX_SPLITS 4096
#define GA_NOALLOC_TICKET_OFFSET (GA_NOALLOC_MAX_SPLITS * 8)
#define GA_NOALLOC_SCRATCH_BYTES (64 * 1024)

/* [0, 32 KiB): partial sums, one 8-byte slot per split; then the ticket word.
 * In host code this name is only a handle for cudaGetSymbolAddress. */
static __device__ __align__(256) unsigned char ga_noalloc_scratch[GA_NOALLOC_SCRATCH_BYTES];

#define GA_NOALLOC_MAX_DEVICES 64
/* filled once per device under setup_lock, published through `ready` */
static unsigned char *scratch_of_device[GA_NOALLOC_MAX_DEVICES];
static int sms_of_device[GA_NOALLOC_MAX_DEVICES];
static int ready[GA_NOALLOC_MAX_DEVICES];
static pthread_mutex_t setup_lock = PTHREAD_MUTEX_INITIALIZER;

/* true when `p` is device (or managed) memory of device `dev`; queries the driver's
 * bookkeeping only, allocates nothing */
static int on_device(const void *p, int dev) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (at.type == cudaMemoryTypeManaged) return 1;
  return at.type == cudaMemoryTypeDevice && at.device == dev;
}

static int cuda_fail(const char *what, cudaError_t e) {
  return ga_err_fmt(NULL, GA_IMPL_ERROR, "%s: %s: %s", what, cudaGetErrorName(e),
                    cudaGetErrorString(e));
}

extern "C" GPUARRAY_PUBLIC int gpuarray_b200_sum_f32_noalloc(const float *src, size_t n,
                                                             float *dst, void *cuda_stream) {
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  cudaError_t ce;
  int dev = -1;
  unsigned char *scratch;

  if (dst == NULL || (src == NULL && n != 0))
    return ga_err_fmt(NULL, GA_INVALID_ERROR, "gpuarray_b200_sum_f32_noalloc: NULL pointer");
  if (n > GPUARRAY_B200_NOALLOC_MAX_ELEMS)
    return ga_err_fmt(NULL, GA_XLARGE_ERROR,
                      "gpuarray_b200_sum_f32_noalloc: %zu elements exceed the maximum of %llu "
                      "that the built-in scratch block is laid out for",
                      n, (unsigned long long)GPUARRAY_B200_NOALLOC_MAX_ELEMS);
  if (((uintptr_t)src & 15u) != 0)
    return ga_err_fmt(NULL, GA_UNALIGNED_ERROR,
                      "gpuarray_b200_sum_f32_noalloc: src must be 16-byte aligned");
  ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return cuda_fail("cudaGetDevice", ce);
  if (dev < 0 || dev >= GA_NOALLOC_MAX_DEVICES)
    return ga_err_fmt(NULL, GA_VALUE_ERROR, "device ordinal %d out of range", dev);

  /* nothing is queued for pointers that do not live on the current device */
  if ((n != 0 && !on_device(src, dev)) || !on_device(dst, dev))
    return ga_err_fmt(NULL, GA_VALUE_ERROR,
                      "gpuarray_b200_sum_f32_noalloc: src and dst must be device memory of the "
                      "current device (%d)", dev);

  if (!__atomic_load_n(&ready[dev], __ATOMIC_ACQUIRE)) {
    /* once per device, with that device current: the device address of the block. Two
     * threads making their first call together are serialised here. */
    void *p = NULL;
    int sms = 0;
    pthread_mutex_lock(&setup_lock);
    if (!ready[dev]) {
      ce = cudaGetSymbolAddress(&p, ga_noalloc_scratch);
      if (ce == cudaSuccess) ce = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (ce != cudaSuccess) {
        pthread_mutex_unlock(&setup_lock);
        return cuda_fail("set-up of the built-in scratch block", ce);
      }
      scratch_of_device[dev] = (unsigned char *)p;
      sms_of_device[dev] = sms;
      __atomic_store_n(&ready[dev], 1, __ATOMIC_RELEASE);
    }
    pthread_mutex_unlock(&setup_lock);
  }
  scratch = scratch_of_device[dev];

  if (n == 0) {
    ce = cudaMemsetAsync(dst, 0, sizeof(float), stream);
    return ce == cudaSuccess ? GA_NO_ERROR : cuda_fail("cudaMemsetAsync", ce);
  }

  ga__rd_layout L;
  memset(&L, 0, sizeof(L));
  L.nf_total = 1;
  L.nr_total = n;
  L.nf = 0;
  L.nr = 1;
  L.rdim[0] = n;
  L.rsrc[0] = (ga__i64)sizeof(float);
  L.inner = n;
  L.seg = (ga__u64)GA_RD_THREADS * GA_RD_VEC * 16; /* 16 vectors per thread and unit */
  if (L.seg > n) L.seg = n;
  L.nseg = (n + L.seg - 1) / L.seg;
  L.units = L.nseg;
  L.splits = (ga__u64)sms_of_device[dev] * 8;
  if (L.splits > L.units) L.splits = L.units;
  if (L.splits > GA_NOALLOC_MAX_SPLITS) L.splits = GA_NOALLOC_MAX_SPLITS;
  L.dv[0] = 1;
  L.dv[1] = 1;

  /* the ticket must read zero when the first group arrives */
  ce = cudaMemsetAsync(scratch + GA_NOALLOC_TICKET_OFFSET, 0, 256, stream);
  if (ce != cudaSuccess) return cuda_fail("cudaMemsetAsync", ce);
  ga_rd_rows<<<(unsigned)L.splits, GA_RD_THREADS, 0, stream>>>(
      L, (const char *)src, (char *)dst, (char *)NULL, (GA_RD_ACC_T *)scratch,
      (GA_RD_IDX_T *)NULL, (unsigned int *)(scratch + GA_NOALLOC_TICKET_OFFSET));
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return cuda_fail("ga_rd_rows launch", ce);
  return GA_NO_ERROR;
}
