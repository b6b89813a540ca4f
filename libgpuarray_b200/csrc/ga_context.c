/* Contexts and device buffers over the CUDA driver API.
 *
 * Stands where the reference has src/gpuarray_buffer.c (dispatch) plus the
 * context/allocation/copy half of src/gpuarray_buffer_cuda.c (:156-1071).
 * Design differences, all deliberate:
 *   - one backend, no vtable;
 *   - one in-order stream per context instead of two streams with per-buffer
 *     read/write events (:899-946): every launch and copy is enqueued on
 *     ctx->s, so ordering is by construction and a launch costs one driver
 *     call instead of ~10;
 *   - the primary context of the device is retained, so memory can be shared
 *     with other runtime-API users in the process;
 *   - freed blocks are kept in a per-context list keyed by size and reused
 *     (stream order makes immediate reuse safe), replacing the 4 MiB
 *     sub-allocator (:607-785). */
#include "private.h"

#define CU(call, args)                                              \
  do {                                                              \
    CUresult r_ = ga_cu.p_##call args;                              \
    if (r_ != CUDA_SUCCESS) {                                       \
      err = ga_err_cuda(ctx->err, #call, r_);                       \
      goto fail;                                                    \
    }                                                               \
  } while (0)

/* ----------------------------------------------------------- enumeration */

static int is_cuda_name(const char *name) {
  return name != NULL && strncmp(name, "cuda", 4) == 0;
}

int gpu_get_platform_count(const char *name, unsigned int *platcount) {
  if (!is_cuda_name(name))
    return ga_err_fmt(ga_global_err, GA_UNSUPPORTED_ERROR,
                      "Backend \"%s\" is not available (only \"cuda\")", name ? name : "(null)");
  *platcount = 1;
  return GA_NO_ERROR;
}

int gpu_get_device_count(const char *name, unsigned int platform, unsigned int *devcount) {
  int n = 0, err;
  CUresult r;
  (void)platform;
  if (!is_cuda_name(name))
    return ga_err_fmt(ga_global_err, GA_UNSUPPORTED_ERROR,
                      "Backend \"%s\" is not available (only \"cuda\")", name ? name : "(null)");
  err = ga_load_cuda(ga_global_err);
  if (err != GA_NO_ERROR) return err;
  r = ga_cu.p_cuDeviceGetCount(&n);
  if (r != CUDA_SUCCESS) return ga_err_cuda(ga_global_err, "cuDeviceGetCount", r);
  *devcount = (unsigned int)n;
  return GA_NO_ERROR;
}

/* ----------------------------------------------------------------- props */

int gpucontext_props_new(gpucontext_props **res) {
  gpucontext_props *p = calloc(1, sizeof(*p));
  if (p == NULL) return ga_err_sys(ga_global_err, "calloc");
  p->dev = -1;
  p->sched = GA_CTX_SCHED_AUTO;
  p->max_cache_size = (size_t)-1;
  *res = p;
  return GA_NO_ERROR;
}

int gpucontext_props_cuda_dev(gpucontext_props *p, int devno) {
  p->dev = devno;
  return GA_NO_ERROR;
}

int gpucontext_props_opencl_dev(gpucontext_props *p, int platno, int devno) {
  (void)p; (void)platno; (void)devno;
  return ga_err_set(ga_global_err, GA_UNSUPPORTED_ERROR, "No OpenCL backend in this library");
}

int gpucontext_props_sched(gpucontext_props *p, int sched) {
  if (sched != GA_CTX_SCHED_AUTO && sched != GA_CTX_SCHED_SINGLE && sched != GA_CTX_SCHED_MULTI)
    return ga_err_fmt(ga_global_err, GA_INVALID_ERROR, "Invalid value for sched: %d", sched);
  p->sched = sched;
  return GA_NO_ERROR;
}

int gpucontext_props_set_single_stream(gpucontext_props *p) {
  p->flags |= 1;
  return GA_NO_ERROR;
}

int gpucontext_props_kernel_cache(gpucontext_props *p, const char *path) {
  free(p->kernel_cache_path);
  p->kernel_cache_path = path ? strdup(path) : NULL;
  return GA_NO_ERROR;
}

int gpucontext_props_alloc_cache(gpucontext_props *p, size_t initial, size_t max) {
  if (initial > max)
    return ga_err_set(ga_global_err, GA_VALUE_ERROR,
                      "Initial size can't be bigger than max size");
  p->initial_cache_size = initial;
  p->max_cache_size = max;
  return GA_NO_ERROR;
}

void gpucontext_props_del(gpucontext_props *p) {
  if (p == NULL) return;
  free(p->kernel_cache_path);
  free(p);
}

/* ---------------------------------------------------------------- context */

void ga_ctx_enter(gpucontext *ctx) {
  if (ctx->enter_depth++ == 0) ga_cu.p_cuCtxPushCurrent(ctx->cu);
}

void ga_ctx_exit(gpucontext *ctx) {
  if (--ctx->enter_depth == 0) {
    CUcontext old;
    ga_cu.p_cuCtxPopCurrent(&old);
  }
}

static int dev_attr(gpucontext *ctx, CUdevice_attribute a) {
  int v = 0;
  ga_cu.p_cuDeviceGetAttribute(&v, a, ctx->cudev);
  return v;
}

/* Fills the context around an existing CUcontext (made current by caller). */
static int ctx_setup(gpucontext *ctx) {
  int err = GA_NO_ERROR, major, minor;
  size_t total = 0;

  major = dev_attr(ctx, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR);
  minor = dev_attr(ctx, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR);
  if (major != 10) {
    err = ga_err_fmt(ctx->err, GA_DEVSUP_ERROR,
                     "Device %d has compute capability %d.%d; this library only contains "
                     "sm_100a (B200) kernels", ctx->dev, major, minor);
    goto fail;
  }
  snprintf(ctx->bin_id, sizeof(ctx->bin_id), "sm_%d%da", major, minor);
  CU(cuDeviceGetName, (ctx->devname, (int)sizeof(ctx->devname), ctx->cudev));
  {
    char bus[32] = {0};
    ga_cu.p_cuDeviceGetPCIBusId(bus, (int)sizeof(bus), ctx->cudev);
    memset(ctx->pci_id, 0, sizeof(ctx->pci_id));
    memcpy(ctx->pci_id, bus, strlen(bus) < 15 ? strlen(bus) : 15);
  }
  ctx->num_sms = (unsigned)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT);
  ctx->smem_block = (size_t)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK);
  ctx->max_smem_block =
      (size_t)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN);
  ctx->max_threads = (size_t)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_MAX_THREADS_PER_BLOCK);
  ctx->max_grid[0] = (size_t)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_MAX_GRID_DIM_X);
  ctx->max_grid[1] = (size_t)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_MAX_GRID_DIM_Y);
  ctx->max_grid[2] = (size_t)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_MAX_GRID_DIM_Z);
  ctx->max_block[0] = (size_t)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_MAX_BLOCK_DIM_X);
  ctx->max_block[1] = (size_t)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_MAX_BLOCK_DIM_Y);
  ctx->max_block[2] = (size_t)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_MAX_BLOCK_DIM_Z);
  ctx->l2_bytes = (size_t)dev_attr(ctx, CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE);
  CU(cuDeviceTotalMem, (&total, ctx->cudev));
  CU(cuStreamCreate, (&ctx->s, CU_STREAM_NON_BLOCKING));
  return GA_NO_ERROR;
fail:
  return err;
}

int gpucontext_init(gpucontext **res, const char *name, gpucontext_props *props) {
  gpucontext *ctx = NULL;
  int err, dev = 0, ndev = 0, zero[2] = {0, 0};
  CUresult r;

  *res = NULL;
  if (!is_cuda_name(name)) {
    gpucontext_props_del(props);
    return ga_err_fmt(ga_global_err, GA_UNSUPPORTED_ERROR,
                      "Backend \"%s\" is not available (only \"cuda\")", name ? name : "(null)");
  }
  if (name[4] != '\0') dev = atoi(name + 4);
  else if (props != NULL && props->dev >= 0) dev = props->dev;

  err = ga_load_cuda(ga_global_err);
  if (err != GA_NO_ERROR) {
    gpucontext_props_del(props);
    return err;
  }
  r = ga_cu.p_cuDeviceGetCount(&ndev);
  if (r != CUDA_SUCCESS || dev < 0 || dev >= ndev) {
    gpucontext_props_del(props);
    return ga_err_fmt(ga_global_err, GA_NODEV_ERROR, "No CUDA device %d (%d visible)", dev, ndev);
  }

  ctx = calloc(1, sizeof(*ctx));
  if (ctx != NULL) ctx->err = calloc(1, sizeof(*ctx->err));
  if (ctx == NULL || ctx->err == NULL) {
    free(ctx);
    gpucontext_props_del(props);
    return ga_err_sys(ga_global_err, "calloc");
  }
  ctx->refcnt = 1;
  ctx->dev = dev;
  ctx->max_cached_bytes = (size_t)4 << 30;
  if (props != NULL) {
    if (props->max_cache_size != (size_t)-1) ctx->max_cached_bytes = props->max_cache_size;
    if (props->kernel_cache_path != NULL) ctx->kernel_cache_path = strdup(props->kernel_cache_path);
  }
  if (ctx->kernel_cache_path == NULL) {
    const char *env = getenv("GPUARRAY_CACHE_PATH");
    if (env != NULL && env[0] != '\0') ctx->kernel_cache_path = strdup(env);
  }
  gpucontext_props_del(props);

  r = ga_cu.p_cuDeviceGet(&ctx->cudev, dev);
  if (r == CUDA_SUCCESS) r = ga_cu.p_cuDevicePrimaryCtxRetain(&ctx->cu, ctx->cudev);
  if (r != CUDA_SUCCESS) {
    err = ga_err_cuda(ga_global_err, "cuDevicePrimaryCtxRetain", r);
    free(ctx->kernel_cache_path);
    free(ctx->err);
    free(ctx);
    return err;
  }
  ctx->own_ctx = 1;
  ga_ctx_enter(ctx);
  err = ctx_setup(ctx);
  if (err == GA_NO_ERROR) ctx->errbuf = gpudata_alloc(ctx, 8, zero, GA_BUFFER_INIT, &err);
  ga_ctx_exit(ctx);
  if (err != GA_NO_ERROR) {
    *ga_global_err = *ctx->err;
    ga_ctx_unref(ctx);
    return err;
  }
  *res = ctx;
  return GA_NO_ERROR;
}

static void ctx_destroy(gpucontext *ctx) {
  ga_block *b, *nb;
  ga_ctx_enter(ctx);
  if (ctx->s != NULL) ga_cu.p_cuStreamSynchronize(ctx->s);
  if (ctx->errbuf != NULL) {
    /* the error buffer's own reference is the one that brought us here */
    if (ctx->errbuf->ptr != 0) ga_cu.p_cuMemFree(ctx->errbuf->ptr);
    free(ctx->errbuf);
    ctx->errbuf = NULL;
  }
  ga_modules_free(ctx);
  ga_peer_windows_free(ctx);
  for (b = ctx->free_blocks; b != NULL; b = nb) {
    nb = b->next;
    ga_cu.p_cuMemFree(b->ptr);
    free(b);
  }
  ctx->free_blocks = NULL;
  if (ctx->s != NULL) ga_cu.p_cuStreamDestroy(ctx->s);
  ga_ctx_exit(ctx);
  if (ctx->own_ctx) ga_cu.p_cuDevicePrimaryCtxRelease(ctx->cudev);
  free(ctx->kernel_cache_path);
  free(ctx->err);
  free(ctx);
}

/* The context dies when the only reference left is the one held by its own
 * error buffer. */
void ga_ctx_unref(gpucontext *ctx) {
  if (--ctx->refcnt == (ctx->errbuf != NULL ? 1u : 0u)) ctx_destroy(ctx);
}

/* Drops the caller's reference. Operators the library cached on the context
 * (typed-copy kernels, the GpuArray_maxandargmax operators) are released
 * first, as the reference does with its extcopy cache
 * (src/gpuarray_buffer.c:118-126), so that they cannot keep it alive. */
void gpucontext_deref(gpucontext *ctx) {
  if (ctx == NULL) return;
  ga_ctx_enter(ctx);
  ga_extcopy_cache_free(ctx);
  ga_maxandargmax_cache_free(ctx);
  ga_take1_cache_free(ctx);
  ga_ctx_exit(ctx);
  ga_ctx_unref(ctx);
}

/* Like the reference (src/gpuarray_buffer.c:136-141) the stored message is
 * returned whatever `err` is; callers pass the code they just received. */
const char *gpucontext_error(gpucontext *ctx, int err) {
  ga_error_rec *e = ctx != NULL ? ctx->err : ga_global_err;
  (void)err;
  return e->msg;
}

GPUARRAY_PUBLIC int gpuarray_b200_error_code(gpucontext *ctx) {
  return (ctx != NULL ? ctx->err : ga_global_err)->code;
}

static int ctx_property(gpucontext *ctx, int prop_id, void *res) {
  switch (prop_id) {
  case GA_CTX_PROP_DEVNAME:
    memcpy(res, ctx->devname, sizeof(ctx->devname));
    return GA_NO_ERROR;
  case GA_CTX_PROP_LMEMSIZE:
    *(size_t *)res = ctx->smem_block;
    return GA_NO_ERROR;
  case GA_CTX_PROP_NUMPROCS:
    *(unsigned int *)res = ctx->num_sms;
    return GA_NO_ERROR;
  case GA_CTX_PROP_BIN_ID:
    *(const char **)res = ctx->bin_id;
    return GA_NO_ERROR;
  case GA_CTX_PROP_ERRBUF:
    *(gpudata **)res = ctx->errbuf;
    return GA_NO_ERROR;
  case GA_CTX_PROP_TOTAL_GMEM:
  case GA_CTX_PROP_FREE_GMEM:
  case GA_CTX_PROP_LARGEST_MEMBLOCK: {
    size_t fr = 0, tot = 0;
    CUresult r;
    ga_ctx_enter(ctx);
    r = ga_cu.p_cuMemGetInfo(&fr, &tot);
    ga_ctx_exit(ctx);
    if (r != CUDA_SUCCESS) return ga_err_cuda(ctx->err, "cuMemGetInfo", r);
    if (prop_id == GA_CTX_PROP_TOTAL_GMEM) *(size_t *)res = tot;
    else *(size_t *)res = fr + ctx->cached_bytes;
    return GA_NO_ERROR;
  }
  case GA_CTX_PROP_NATIVE_FLOAT16:
    *(int *)res = 1;
    return GA_NO_ERROR;
  case GA_CTX_PROP_MAXGSIZE0: *(size_t *)res = ctx->max_grid[0]; return GA_NO_ERROR;
  case GA_CTX_PROP_MAXGSIZE1: *(size_t *)res = ctx->max_grid[1]; return GA_NO_ERROR;
  case GA_CTX_PROP_MAXGSIZE2: *(size_t *)res = ctx->max_grid[2]; return GA_NO_ERROR;
  case GA_CTX_PROP_MAXLSIZE0: *(size_t *)res = ctx->max_block[0]; return GA_NO_ERROR;
  case GA_CTX_PROP_MAXLSIZE1: *(size_t *)res = ctx->max_block[1]; return GA_NO_ERROR;
  case GA_CTX_PROP_MAXLSIZE2: *(size_t *)res = ctx->max_block[2]; return GA_NO_ERROR;
  case GA_CTX_PROP_UNIQUE_ID:
    memcpy(res, ctx->pci_id, sizeof(ctx->pci_id));
    return GA_NO_ERROR;
  default:
    return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Invalid property %d", prop_id);
  }
}

int gpucontext_property(gpucontext *ctx, int prop_id, void *res) {
  if (prop_id >= GA_BUFFER_PROP_START)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Not a context property");
  return ctx_property(ctx, prop_id, res);
}

/* ---------------------------------------------------------------- buffers */

#define GA_ALLOC_GRANULE 512

static size_t round_alloc(size_t sz) {
  if (sz == 0) sz = 1;
  return (sz + GA_ALLOC_GRANULE - 1) / GA_ALLOC_GRANULE * GA_ALLOC_GRANULE;
}

/* Best fit among cached blocks: smallest block with sz <= size <= sz + sz/8. */
static CUdeviceptr cache_take(gpucontext *ctx, size_t sz, size_t *got) {
  ga_block **pp, **best = NULL;
  for (pp = &ctx->free_blocks; *pp != NULL; pp = &(*pp)->next) {
    size_t bs = (*pp)->sz;
    if (bs >= sz && bs - sz <= sz / 8 && (best == NULL || bs < (*best)->sz)) best = pp;
  }
  if (best != NULL) {
    ga_block *b = *best;
    CUdeviceptr p = b->ptr;
    *best = b->next;
    *got = b->sz;
    ctx->cached_bytes -= b->sz;
    free(b);
    return p;
  }
  return 0;
}

static void cache_flush(gpucontext *ctx) {
  ga_block *b, *nb;
  for (b = ctx->free_blocks; b != NULL; b = nb) {
    nb = b->next;
    ga_cu.p_cuMemFree(b->ptr);
    free(b);
  }
  ctx->free_blocks = NULL;
  ctx->cached_bytes = 0;
}

gpudata *gpudata_alloc(gpucontext *ctx, size_t sz, void *data, int flags, int *ret) {
  gpudata *b = NULL;
  int err = GA_NO_ERROR;
  size_t asz = round_alloc(sz);
  CUresult r;

  if (ISSET(flags, GA_BUFFER_INIT) && data == NULL) {
    err = ga_err_set(ctx->err, GA_VALUE_ERROR, "GA_BUFFER_INIT without data");
    goto out;
  }
  if (ISSET(flags, GA_BUFFER_READ_ONLY) && ISSET(flags, GA_BUFFER_WRITE_ONLY)) {
    err = ga_err_set(ctx->err, GA_VALUE_ERROR, "Buffer both read-only and write-only");
    goto out;
  }
  b = calloc(1, sizeof(*b));
  if (b == NULL) {
    err = ga_err_sys(ctx->err, "calloc");
    goto out;
  }
  b->ctx = ctx;
  b->refcnt = 1;
  b->flags = flags & GA_BUFFER_MASK;
  b->sz = sz;

  ga_ctx_enter(ctx);
  if (ISSET(flags, GA_BUFFER_HOST)) {
    r = ga_cu.p_cuMemHostAlloc(&b->host, asz, CU_MEMHOSTALLOC_PORTABLE | CU_MEMHOSTALLOC_DEVICEMAP);
    if (r == CUDA_SUCCESS) r = ga_cu.p_cuMemHostGetDevicePointer(&b->ptr, b->host, 0);
    if (r != CUDA_SUCCESS) err = ga_err_cuda(ctx->err, "cuMemHostAlloc", r);
  } else {
    size_t got = asz;
    b->ptr = cache_take(ctx, asz, &got);
    if (b->ptr == 0) {
      r = ga_cu.p_cuMemAlloc(&b->ptr, asz);
      if (r == CUDA_ERROR_OUT_OF_MEMORY && ctx->free_blocks != NULL) {
        ga_cu.p_cuStreamSynchronize(ctx->s);
        cache_flush(ctx);
        r = ga_cu.p_cuMemAlloc(&b->ptr, asz);
      }
      if (r != CUDA_SUCCESS) err = ga_err_cuda(ctx->err, "cuMemAlloc", r);
    }
    if (err == GA_NO_ERROR) asz = got;
  }
  b->asz = asz;
  if (err == GA_NO_ERROR && ISSET(flags, GA_BUFFER_INIT) && sz > 0) {
    if (b->host != NULL) memcpy(b->host, data, sz);
    else {
      r = ga_cu.p_cuMemcpyHtoDAsync(b->ptr, data, sz, ctx->s);
      /* `data` is the caller's and may go away after we return */
      if (r == CUDA_SUCCESS) r = ga_cu.p_cuStreamSynchronize(ctx->s);
      if (r != CUDA_SUCCESS) err = ga_err_cuda(ctx->err, "cuMemcpyHtoDAsync", r);
    }
  }
  ga_ctx_exit(ctx);
  if (err != GA_NO_ERROR) {
    if (b->ptr != 0 && b->host == NULL) {
      ga_ctx_enter(ctx);
      ga_cu.p_cuMemFree(b->ptr);
      ga_ctx_exit(ctx);
    }
    free(b);
    b = NULL;
    goto out;
  }
  ctx->refcnt++;
out:
  if (ret != NULL) *ret = err;
  return b;
}

void gpudata_retain(gpudata *b) { b->refcnt++; }

void gpudata_release(gpudata *b) {
  gpucontext *ctx;
  if (b == NULL) return;
  if (--b->refcnt != 0) return;
  ctx = b->ctx;
  ga_ctx_enter(ctx);
  if (ISSET(b->flags, GA_BUF_EXTERNAL)) {
    /* not ours */
  } else if (ISSET(b->flags, GA_BUF_IPC)) {
    ga_cu.p_cuIpcCloseMemHandle(b->ptr);
  } else if (b->host != NULL) {
    ga_cu.p_cuStreamSynchronize(ctx->s);
    ga_cu.p_cuMemFreeHost(b->host);
  } else if (b->ptr != 0) {
    ga_block *blk = NULL;
    if (ctx->cached_bytes + b->asz <= ctx->max_cached_bytes) blk = malloc(sizeof(*blk));
    if (blk != NULL) {
      blk->ptr = b->ptr;
      blk->sz = b->asz;
      blk->next = ctx->free_blocks;
      ctx->free_blocks = blk;
      ctx->cached_bytes += b->asz;
    } else {
      ga_cu.p_cuMemFree(b->ptr); /* synchronises with outstanding work */
    }
  }
  ga_ctx_exit(ctx);
  free(b);
  ga_ctx_unref(ctx);
}

int gpudata_share(gpudata *a, gpudata *b, int *ret) {
  if (ret != NULL) *ret = GA_NO_ERROR;
  if (a->ctx != b->ctx) return 0;
  if (a->ptr == b->ptr) return 1;
  return (a->ptr < b->ptr) ? (a->ptr + a->sz > b->ptr) : (b->ptr + b->sz > a->ptr);
}

static int range_ok(gpudata *b, size_t off, size_t sz) {
  return off <= b->sz && sz <= b->sz - off;
}

int gpudata_move(gpudata *dst, size_t dstoff, gpudata *src, size_t srcoff, size_t sz) {
  gpucontext *ctx = dst->ctx;
  int err = GA_NO_ERROR;
  if (src->ctx != ctx) return ga_err_set(ctx->err, GA_VALUE_ERROR, "Differing contexts");
  if (sz == 0) return GA_NO_ERROR;
  if (!range_ok(dst, dstoff, sz) || !range_ok(src, srcoff, sz))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Copy exceeds a buffer");
  ga_ctx_enter(ctx);
  CU(cuMemcpyDtoDAsync, (dst->ptr + dstoff, src->ptr + srcoff, sz, ctx->s));
fail:
  ga_ctx_exit(ctx);
  return err;
}

int gpudata_transfer(gpudata *dst, size_t dstoff, gpudata *src, size_t srcoff, size_t sz) {
  gpucontext *ctx = dst->ctx;
  int err = GA_NO_ERROR;
  if (src->ctx == ctx) return gpudata_move(dst, dstoff, src, srcoff, sz);
  if (sz == 0) return GA_NO_ERROR;
  if (!range_ok(dst, dstoff, sz) || !range_ok(src, srcoff, sz))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Copy exceeds a buffer");
  /* Both streams are ordered around the copy with events, no host wait (the
   * reference brackets both buffers the same way, src/gpuarray_buffer_cuda.c:
   * 899-946): the copy runs on the destination stream AFTER the work queued
   * so far on the source stream, and whatever the source context queues next
   * (a write to the source buffer, a reuse of its block after a release)
   * runs AFTER the copy has read it. */
  {
    CUevent ready = NULL, done = NULL;
    gpucontext *sctx = src->ctx;
    CUresult r;
    const char *what = "cuEventCreate";
    ga_ctx_enter(sctx);
    r = ga_cu.p_cuEventCreate(&ready, CU_EVENT_DISABLE_TIMING);
    if (r == CUDA_SUCCESS) what = "cuEventRecord", r = ga_cu.p_cuEventRecord(ready, sctx->s);
    ga_ctx_exit(sctx);
    if (r == CUDA_SUCCESS) {
      ga_ctx_enter(ctx);
      what = "cuStreamWaitEvent", r = ga_cu.p_cuStreamWaitEvent(ctx->s, ready, 0);
      if (r == CUDA_SUCCESS)
        what = "cuMemcpyPeerAsync",
        r = ga_cu.p_cuMemcpyPeerAsync(dst->ptr + dstoff, ctx->cu, src->ptr + srcoff, sctx->cu, sz,
                                      ctx->s);
      if (r == CUDA_SUCCESS)
        what = "cuEventCreate", r = ga_cu.p_cuEventCreate(&done, CU_EVENT_DISABLE_TIMING);
      if (r == CUDA_SUCCESS) what = "cuEventRecord", r = ga_cu.p_cuEventRecord(done, ctx->s);
      ga_ctx_exit(ctx);
    }
    if (r == CUDA_SUCCESS) {
      ga_ctx_enter(sctx);
      what = "cuStreamWaitEvent", r = ga_cu.p_cuStreamWaitEvent(sctx->s, done, 0);
      ga_ctx_exit(sctx);
    }
    /* destroying an event that is still pending is allowed: the driver frees
     * it once it has completed */
    if (ready != NULL) ga_cu.p_cuEventDestroy(ready);
    if (done != NULL) ga_cu.p_cuEventDestroy(done);
    if (r != CUDA_SUCCESS) err = ga_err_cuda(ctx->err, what, r);
    return err;
  }
}

int gpudata_read(void *dst, gpudata *src, size_t srcoff, size_t sz) {
  gpucontext *ctx = src->ctx;
  int err = GA_NO_ERROR;
  if (ISSET(src->flags, GA_BUFFER_WRITE_ONLY))
    return ga_err_set(ctx->err, GA_WRITEONLY_ERROR, "Buffer is write-only");
  if (sz == 0) return GA_NO_ERROR;
  if (!range_ok(src, srcoff, sz))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Read exceeds the buffer");
  ga_ctx_enter(ctx);
  CU(cuMemcpyDtoHAsync, (dst, src->ptr + srcoff, sz, ctx->s));
  CU(cuStreamSynchronize, (ctx->s));
fail:
  ga_ctx_exit(ctx);
  return err;
}

int gpudata_write(gpudata *dst, size_t dstoff, const void *src, size_t sz) {
  gpucontext *ctx = dst->ctx;
  int err = GA_NO_ERROR;
  if (ISSET(dst->flags, GA_BUFFER_READ_ONLY))
    return ga_err_set(ctx->err, GA_READONLY_ERROR, "Buffer is read-only");
  if (sz == 0) return GA_NO_ERROR;
  if (!range_ok(dst, dstoff, sz))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Write exceeds the buffer");
  ga_ctx_enter(ctx);
  /* For pageable sources the driver stages the bytes before returning; for
   * pinned sources the caller must keep them alive until the stream drains,
   * exactly as with the reference's asynchronous write. */
  CU(cuMemcpyHtoDAsync, (dst->ptr + dstoff, src, sz, ctx->s));
fail:
  ga_ctx_exit(ctx);
  return err;
}

int gpudata_memset(gpudata *dst, size_t dstoff, int data) {
  gpucontext *ctx = dst->ctx;
  int err = GA_NO_ERROR;
  if (dstoff > dst->sz) return ga_err_set(ctx->err, GA_VALUE_ERROR, "Offset beyond the buffer");
  if (dst->sz - dstoff == 0) return GA_NO_ERROR;
  ga_ctx_enter(ctx);
  CU(cuMemsetD8Async, (dst->ptr + dstoff, (unsigned char)data, dst->sz - dstoff, ctx->s));
fail:
  ga_ctx_exit(ctx);
  return err;
}

int gpudata_sync(gpudata *b) {
  gpucontext *ctx = b->ctx;
  int err = GA_NO_ERROR;
  ga_ctx_enter(ctx);
  CU(cuStreamSynchronize, (ctx->s));
fail:
  ga_ctx_exit(ctx);
  return err;
}

int gpudata_property(gpudata *buf, int prop_id, void *res) {
  gpucontext *ctx = buf->ctx;
  if (prop_id < GA_BUFFER_PROP_START) return ctx_property(ctx, prop_id, res);
  switch (prop_id) {
  case GA_BUFFER_PROP_CTX: *(gpucontext **)res = ctx; return GA_NO_ERROR;
  case GA_BUFFER_PROP_REFCNT: *(unsigned int *)res = buf->refcnt; return GA_NO_ERROR;
  case GA_BUFFER_PROP_SIZE: *(size_t *)res = buf->sz; return GA_NO_ERROR;
  default: return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Invalid property %d", prop_id);
  }
}

gpucontext *gpudata_context(gpudata *b) { return b->ctx; }

/* ------------------------------------------------------------- extensions */

static void ext_cuda_enter(gpucontext *ctx) { ga_ctx_enter(ctx); }
static void ext_cuda_exit(gpucontext *ctx) { ga_ctx_exit(ctx); }
static CUstream ext_cuda_get_stream(void *ctx) { return ((gpucontext *)ctx)->s; }
static size_t ext_cuda_get_sz(gpudata *d) { return d->sz; }
static int ext_cuda_wait(gpudata *d, int flags) { (void)d; (void)flags; return GA_NO_ERROR; }
static int ext_cuda_record(gpudata *d, int flags) { (void)d; (void)flags; return GA_NO_ERROR; }

/* Wraps device memory owned by someone else (e.g. a torch tensor). */
static gpudata *ext_cuda_make_buf(void *c, CUdeviceptr p, size_t sz) {
  gpucontext *ctx = (gpucontext *)c;
  gpudata *b = calloc(1, sizeof(*b));
  if (b == NULL) {
    ga_err_sys(ctx->err, "calloc");
    return NULL;
  }
  b->ptr = p;
  b->ctx = ctx;
  b->sz = sz;
  b->asz = sz;
  b->refcnt = 1;
  b->flags = GA_BUF_EXTERNAL;
  ctx->refcnt++;
  return b;
}

/* Adopts an existing CUcontext; only the primary context of a B200 works. */
static gpucontext *ext_cuda_make_ctx(CUcontext cu, int flags) {
  gpucontext *ctx;
  int err;
  CUcontext old;
  if (ga_load_cuda(ga_global_err) != GA_NO_ERROR) return NULL;
  ctx = calloc(1, sizeof(*ctx));
  if (ctx != NULL) ctx->err = calloc(1, sizeof(*ctx->err));
  if (ctx == NULL || ctx->err == NULL) {
    free(ctx);
    ga_err_sys(ga_global_err, "calloc");
    return NULL;
  }
  ctx->refcnt = 1;
  ctx->cu = cu;
  ctx->flags = flags;
  ctx->own_ctx = 0;
  ctx->max_cached_bytes = (size_t)4 << 30;
  ga_cu.p_cuCtxPushCurrent(cu);
  ga_cu.p_cuCtxGetDevice(&ctx->cudev);
  ctx->dev = (int)ctx->cudev;
  ga_cu.p_cuCtxPopCurrent(&old);
  ga_ctx_enter(ctx);
  err = ctx_setup(ctx);
  if (err == GA_NO_ERROR) {
    int zero[2] = {0, 0};
    ctx->errbuf = gpudata_alloc(ctx, 8, zero, GA_BUFFER_INIT, &err);
  }
  ga_ctx_exit(ctx);
  if (err != GA_NO_ERROR) {
    *ga_global_err = *ctx->err;
    ga_ctx_unref(ctx);
    return NULL;
  }
  return ctx;
}

static CUipcMemHandle ext_cuda_get_ipc_handle(gpudata *d) {
  CUipcMemHandle h;
  memset(&h, 0, sizeof(h));
  ga_ctx_enter(d->ctx);
  {
    CUresult r = ga_cu.p_cuIpcGetMemHandle(&h, d->ptr);
    if (r != CUDA_SUCCESS) ga_err_cuda(d->ctx->err, "cuIpcGetMemHandle", r);
  }
  ga_ctx_exit(d->ctx);
  return h;
}

static gpudata *ext_cuda_open_ipc_handle(gpucontext *ctx, CUipcMemHandle h, size_t sz) {
  gpudata *b = calloc(1, sizeof(*b));
  CUresult r;
  if (b == NULL) {
    ga_err_sys(ctx->err, "calloc");
    return NULL;
  }
  ga_ctx_enter(ctx);
  r = ga_cu.p_cuIpcOpenMemHandle(&b->ptr, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS);
  ga_ctx_exit(ctx);
  if (r != CUDA_SUCCESS) {
    ga_err_cuda(ctx->err, "cuIpcOpenMemHandle", r);
    free(b);
    return NULL;
  }
  b->ctx = ctx;
  b->sz = sz;
  b->asz = sz;
  b->refcnt = 1;
  b->flags = GA_BUF_IPC;
  ctx->refcnt++;
  return b;
}

void *gpuarray_get_extension(const char *name) {
  static const struct { const char *name; void *fn; } table[] = {
      {"cuda_enter", (void *)ext_cuda_enter},
      {"cuda_exit", (void *)ext_cuda_exit},
      {"cuda_make_ctx", (void *)ext_cuda_make_ctx},
      {"cuda_get_stream", (void *)ext_cuda_get_stream},
      {"cuda_make_buf", (void *)ext_cuda_make_buf},
      {"cuda_get_sz", (void *)ext_cuda_get_sz},
      {"cuda_wait", (void *)ext_cuda_wait},
      {"cuda_record", (void *)ext_cuda_record},
      {"cuda_get_ipc_handle", (void *)ext_cuda_get_ipc_handle},
      {"cuda_open_ipc_handle", (void *)ext_cuda_open_ipc_handle},
  };
  size_t i;
  if (name == NULL) return NULL;
  for (i = 0; i < sizeof(table) / sizeof(table[0]); i++)
    if (strcmp(name, table[i].name) == 0) return table[i].fn;
  return NULL;
}
