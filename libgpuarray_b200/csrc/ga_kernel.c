/* User-supplied kernels: gpukernel (buffer.h) and GpuKernel (kernel.h).
 *
 * The elementwise and reduction engines do not go through these objects (they
 * call ga_compile / ga_launch directly); this file keeps the reference's raw
 * kernel API (src/gpuarray_kernel.c:10-103, src/gpuarray_buffer_cuda.c
 * :1310-1552) working for clients such as pygpu.GpuKernel. */
#include "private.h"

gpukernel *gpukernel_init(gpucontext *ctx, unsigned int count, const char **strings,
                          const size_t *lengths, const char *fname, unsigned int numargs,
                          const int *typecodes, int flags, int *ret, char **err_str) {
  gpukernel *k = NULL;
  ga_strb sb;
  unsigned int i;
  int err = GA_NO_ERROR;

  ga_strb_init(&sb);
  if (err_str != NULL) *err_str = NULL;
  if (count == 0 || strings == NULL || fname == NULL) {
    err = ga_err_set(ctx->err, GA_VALUE_ERROR, "String count is 0");
    goto out;
  }
  if (ISSET(flags, GA_USE_OPENCL)) {
    err = ga_err_set(ctx->err, GA_DEVSUP_ERROR, "OpenCL kernel given to the CUDA backend");
    goto out;
  }
  if (ISSET(flags, GA_USE_COMPLEX)) {
    err = ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR, "Complex types are not supported");
    goto out;
  }
  for (i = 0; i < numargs; i++) {
    if (typecodes[i] != GA_BUFFER && !ga_type_is_computable(typecodes[i])) {
      err = ga_err_fmt(ctx->err, GA_UNSUPPORTED_ERROR, "Unsupported argument type %d (arg %u)",
                       typecodes[i], i);
      goto out;
    }
  }
  for (i = 0; i < count; i++) {
    if (lengths != NULL && lengths[i] != 0) ga_strb_putn(&sb, strings[i], lengths[i]);
    else ga_strb_puts(&sb, strings[i]);
  }
  if (sb.failed) {
    err = ga_err_set(ctx->err, GA_MEMORY_ERROR, "Out of memory assembling kernel source");
    goto out;
  }
  k = calloc(1, sizeof(*k));
  if (k != NULL) {
    k->types = calloc(numargs ? numargs : 1, sizeof(int));
    k->args = calloc(numargs ? numargs : 1, sizeof(void *));
  }
  if (k == NULL || k->types == NULL || k->args == NULL) {
    err = ga_err_sys(ctx->err, "calloc");
    goto out;
  }
  k->ctx = ctx;
  k->refcnt = 1;
  k->argcount = numargs;
  memcpy(k->types, typecodes, numargs * sizeof(int));
  err = ga_compile(ctx, ga_strb_cstr(&sb), fname, NULL, &k->fn, err_str);
  if (err != GA_NO_ERROR) goto out;
  ctx->refcnt++;
out:
  ga_strb_free(&sb);
  if (err != GA_NO_ERROR && k != NULL) {
    free(k->types);
    free(k->args);
    free(k);
    k = NULL;
  }
  if (ret != NULL) *ret = err;
  return k;
}

void gpukernel_retain(gpukernel *k) { k->refcnt++; }

void gpukernel_release(gpukernel *k) {
  unsigned int i;
  gpucontext *ctx;
  if (k == NULL || --k->refcnt != 0) return;
  ctx = k->ctx;
  for (i = 0; i < k->argcount; i++) free(k->args[i]);
  free(k->args);
  free(k->types);
  free(k);
  ga_ctx_unref(ctx);
}

int gpukernel_setarg(gpukernel *k, unsigned int i, void *a) {
  size_t sz;
  if (i >= k->argcount)
    return ga_err_fmt(k->ctx->err, GA_VALUE_ERROR, "index %u is past the number of arguments (%u)",
                      i, k->argcount);
  sz = k->types[i] == GA_BUFFER ? sizeof(CUdeviceptr) : gpuarray_get_elsize(k->types[i]);
  if (k->args[i] == NULL) {
    k->args[i] = malloc(sz < 8 ? 8 : sz);
    if (k->args[i] == NULL) return ga_err_sys(k->ctx->err, "malloc");
  }
  if (k->types[i] == GA_BUFFER) memcpy(k->args[i], &((gpudata *)a)->ptr, sizeof(CUdeviceptr));
  else memcpy(k->args[i], a, sz);
  return GA_NO_ERROR;
}

int gpukernel_call(gpukernel *k, unsigned int n, const size_t *gs, const size_t *ls,
                   size_t shared, void **args) {
  gpucontext *ctx = k->ctx;
  unsigned grid[3] = {1, 1, 1}, block[3] = {1, 1, 1};
  unsigned int i;
  size_t threads = 1;

  if (n == 0 || n > 3) return ga_err_set(ctx->err, GA_VALUE_ERROR, "Call with more than 3 dimensions");
  for (i = 0; i < n; i++) {
    if (gs[i] == 0 || ls[i] == 0 || gs[i] > ctx->max_grid[i] || ls[i] > ctx->max_block[i])
      return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Launch dimension %u out of range (%zu x %zu)", i,
                        gs[i], ls[i]);
    grid[i] = (unsigned)gs[i];
    block[i] = (unsigned)ls[i];
    threads *= ls[i];
  }
  if (threads > (size_t)k->fn.max_threads)
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Block of %zu threads exceeds the kernel limit %d",
                      threads, k->fn.max_threads);
  if (args == NULL) {
    for (i = 0; i < k->argcount; i++)
      if (k->args[i] == NULL)
        return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Argument %u was never set", i);
    args = k->args;
  }
  /* For GA_BUFFER entries of a caller-supplied list, args[i] is the gpudata*,
   * whose first member is the device pointer: it doubles as the value slot. */
  return ga_launch(ctx, &k->fn, grid, block, shared, args);
}

int gpukernel_property(gpukernel *k, int prop_id, void *res) {
  gpucontext *ctx = k->ctx;
  if (prop_id < GA_BUFFER_PROP_START) return gpucontext_property(ctx, prop_id, res);
  switch (prop_id) {
  case GA_KERNEL_PROP_CTX: *(gpucontext **)res = ctx; return GA_NO_ERROR;
  case GA_KERNEL_PROP_MAXLSIZE: *(size_t *)res = (size_t)k->fn.max_threads; return GA_NO_ERROR;
  case GA_KERNEL_PROP_PREFLSIZE: *(size_t *)res = 32; return GA_NO_ERROR;
  case GA_KERNEL_PROP_NUMARGS: *(unsigned int *)res = k->argcount; return GA_NO_ERROR;
  case GA_KERNEL_PROP_TYPES: *(const int **)res = k->types; return GA_NO_ERROR;
  default: return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Invalid property %d", prop_id);
  }
}

gpucontext *gpukernel_context(gpukernel *k) { return k->ctx; }

/* ------------------------------------------------------------- GpuKernel */

int GpuKernel_init(GpuKernel *k, gpucontext *ctx, unsigned int count, const char **strs,
                   const size_t *lens, const char *name, unsigned int argcount, const int *types,
                   int flags, char **err_str) {
  int res = GA_NO_ERROR;
  k->args = calloc(argcount ? argcount : 1, sizeof(void *));
  if (k->args == NULL) return ga_err_sys(ctx->err, "calloc");
  k->k = gpukernel_init(ctx, count, strs, lens, name, argcount, types, flags, &res, err_str);
  if (res != GA_NO_ERROR) GpuKernel_clear(k);
  return res;
}

void GpuKernel_clear(GpuKernel *k) {
  if (k->k != NULL) gpukernel_release(k->k);
  free(k->args);
  k->k = NULL;
  k->args = NULL;
}

gpucontext *GpuKernel_context(GpuKernel *k) { return gpukernel_context(k->k); }

int GpuKernel_setarg(GpuKernel *k, unsigned int i, void *val) {
  return gpukernel_setarg(k->k, i, val);
}

/* Same arithmetic as the reference heuristic: blocks of up to 512 threads in
 * warp multiples, at most 32 blocks per SM, caller-fixed values respected. */
int GpuKernel_sched(GpuKernel *k, size_t n, size_t *gs, size_t *ls) {
  gpucontext *ctx = k->k->ctx;
  const size_t warp = 32;
  size_t max_l = (size_t)k->k->fn.max_threads;
  size_t cap_g = (size_t)ctx->num_sms * 32, cap_l = 512;
  int pick_ls = 0;
  if (cap_g > ctx->max_grid[0]) cap_g = ctx->max_grid[0];
  if (cap_l > max_l) cap_l = max_l;
  if (*ls == 0) {
    pick_ls = 1;
    *ls = warp;
  }
  if (*gs == 0) {
    *gs = n == 0 ? 1 : (n - 1) / *ls + 1;
    if (*gs > cap_g) *gs = cap_g;
  }
  if (pick_ls && n > *ls * *gs) {
    *ls = (n / warp) / *gs * warp;
    if (*ls > cap_l) *ls = cap_l;
  }
  return GA_NO_ERROR;
}

int GpuKernel_call(GpuKernel *k, unsigned int n, const size_t *gs, const size_t *ls,
                   size_t shared, void **args) {
  return gpukernel_call(k->k, n, gs, ls, shared, args);
}

const char *GpuKernel_error(const GpuKernel *k, int err) {
  return gpucontext_error(gpukernel_context(k->k), err);
}
