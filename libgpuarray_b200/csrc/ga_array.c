/* GpuArray: shape/stride bookkeeping on the host plus data movement.
 *
 * Covers the entry points of the reference's src/gpuarray_array.c that the
 * elementwise/reduction path, its tests and pygpu's array class need. Views
 * (index, reshape, transpose) never touch the device. Typed or strided copies
 * are the elementwise operation "dst = src", as in the reference's ga_extcopy
 * (src/gpuarray_array.c:42-86), so they run on the same sm_100a templates as
 * every other elementwise call (vectorised, strided or tiled-transpose). */
#include "private.h"

#define MUL_SAFE_LIMIT ((size_t)1 << (sizeof(size_t) * 4))

static int mul_overflows(size_t a, size_t b) {
  return (a >= MUL_SAFE_LIMIT || b >= MUL_SAFE_LIMIT) && a > 0 && SIZE_MAX / a < b;
}

int ga_array_is_c_contiguous(const GpuArray *a) {
  size_t expect = GpuArray_ITEMSIZE(a);
  unsigned int i;
  for (i = a->nd; i > 0; i--) {
    if (a->dimensions[i - 1] != 1 && a->strides[i - 1] != (ssize_t)expect) return 0;
    expect *= a->dimensions[i - 1];
  }
  return 1;
}

int ga_array_is_f_contiguous(const GpuArray *a) {
  size_t expect = GpuArray_ITEMSIZE(a);
  unsigned int i;
  for (i = 0; i < a->nd; i++) {
    if (a->dimensions[i] != 1 && a->strides[i] != (ssize_t)expect) return 0;
    expect *= a->dimensions[i];
  }
  return 1;
}

static int array_is_aligned(const GpuArray *a) {
  size_t al = gpuarray_get_type(a->typecode)->align;
  unsigned int i;
  if (al == 0) al = 1;
  if (a->offset % al != 0) return 0;
  for (i = 0; i < a->nd; i++)
    if (a->strides[i] % (ssize_t)al != 0) return 0;
  return 1;
}

/* Host-side stand-in for a memory checker: the lowest and highest byte an
 * array can reach, from its offset, extents and byte strides, must lie inside
 * its buffer. Kernels are only launched on arrays that pass, so a wrong
 * GpuArray (hand-built with GpuArray_fromdata, say) is a host error instead of
 * a device fault. */
int ga_array_in_bounds(const GpuArray *a) {
  long long lo = (long long)a->offset, hi = (long long)a->offset;
  unsigned int i;
  if (a->data == NULL) return 0;
  for (i = 0; i < a->nd; i++) {
    long long span;
    if (a->dimensions[i] == 0) return 1; /* no element at all */
    span = (long long)(a->dimensions[i] - 1) * (long long)a->strides[i];
    if (span < 0) lo += span;
    else hi += span;
  }
  hi += (long long)gpuarray_get_elsize(a->typecode);
  return lo >= 0 && (unsigned long long)hi <= (unsigned long long)a->data->sz;
}

void GpuArray_fix_flags(GpuArray *a) {
  a->flags &= GA_WRITEABLE;
  if (ga_array_is_c_contiguous(a)) a->flags |= GA_C_CONTIGUOUS;
  if (ga_array_is_f_contiguous(a)) a->flags |= GA_F_CONTIGUOUS;
  if (array_is_aligned(a)) a->flags |= GA_ALIGNED;
}

static size_t array_nelems(const GpuArray *a) {
  size_t n = 1;
  unsigned int i;
  for (i = 0; i < a->nd; i++) n *= a->dimensions[i];
  return n;
}

/* Replaces dims/strides of `a` by copies of the given vectors. */
static int set_shape(GpuArray *a, unsigned int nd, const size_t *dims, const ssize_t *strs,
                     ga_error_rec *e) {
  size_t *d = calloc(nd ? nd : 1, sizeof(size_t));
  ssize_t *s = calloc(nd ? nd : 1, sizeof(ssize_t));
  if (d == NULL || s == NULL) {
    free(d);
    free(s);
    return ga_err_sys(e, "calloc");
  }
  if (nd > 0) {
    memcpy(d, dims, nd * sizeof(size_t));
    memcpy(s, strs, nd * sizeof(ssize_t));
  }
  free(a->dimensions);
  free(a->strides);
  a->dimensions = d;
  a->strides = s;
  a->nd = nd;
  return GA_NO_ERROR;
}

static void fill_strides(unsigned int nd, const size_t *dims, size_t elsize, ga_order ord,
                         ssize_t *strs) {
  unsigned int i;
  size_t step = elsize;
  if (ord == GA_F_ORDER) {
    for (i = 0; i < nd; i++) {
      strs[i] = (ssize_t)step;
      step *= dims[i];
    }
  } else {
    for (i = nd; i > 0; i--) {
      strs[i - 1] = (ssize_t)step;
      step *= dims[i - 1];
    }
  }
}

int GpuArray_empty(GpuArray *a, gpucontext *ctx, int typecode, unsigned int nd,
                   const size_t *dims, ga_order ord) {
  size_t bytes = gpuarray_get_elsize(typecode);
  unsigned int i;
  int err = GA_NO_ERROR;

  if (typecode == GA_SIZE || typecode == GA_SSIZE)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Cannot create array with size type");
  if (bytes == 0) return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Unknown typecode %d", typecode);
  if (ord == GA_ANY_ORDER) ord = GA_C_ORDER;
  if (ord != GA_C_ORDER && ord != GA_F_ORDER)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Invalid order");
  for (i = 0; i < nd; i++) {
    if (mul_overflows(dims[i], bytes))
      return ga_err_set(ctx->err, GA_XLARGE_ERROR,
                        "Total array size greater than addressable space");
    bytes *= dims[i];
  }
  memset(a, 0, sizeof(*a));
  a->data = gpudata_alloc(ctx, bytes, NULL, 0, &err);
  if (a->data == NULL) return err;
  a->typecode = typecode;
  a->offset = 0;
  a->nd = nd;
  a->dimensions = calloc(nd ? nd : 1, sizeof(size_t));
  a->strides = calloc(nd ? nd : 1, sizeof(ssize_t));
  if (a->dimensions == NULL || a->strides == NULL) {
    GpuArray_clear(a);
    return ga_err_sys(ctx->err, "calloc");
  }
  if (nd > 0) memcpy(a->dimensions, dims, nd * sizeof(size_t));
  fill_strides(nd, a->dimensions, gpuarray_get_elsize(typecode), ord, a->strides);
  a->flags = GA_BEHAVED | (ord == GA_F_ORDER ? GA_F_CONTIGUOUS : GA_C_CONTIGUOUS);
  if (nd <= 1) a->flags |= GA_C_CONTIGUOUS | GA_F_CONTIGUOUS;
  return GA_NO_ERROR;
}

int GpuArray_zeros(GpuArray *a, gpucontext *ctx, int typecode, unsigned int nd,
                   const size_t *dims, ga_order ord) {
  int err = GpuArray_empty(a, ctx, typecode, nd, dims, ord);
  if (err != GA_NO_ERROR) return err;
  err = gpudata_memset(a->data, a->offset, 0);
  if (err != GA_NO_ERROR) GpuArray_clear(a);
  return err;
}

int GpuArray_fromdata(GpuArray *a, gpudata *data, size_t offset, int typecode, unsigned int nd,
                      const size_t *dims, const ssize_t *strides, int writeable) {
  gpucontext *ctx = gpudata_context(data);
  int err;
  if (typecode == GA_SIZE || typecode == GA_SSIZE)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Cannot create array with size type");
  memset(a, 0, sizeof(*a));
  err = set_shape(a, nd, dims, strides, ctx->err);
  if (err != GA_NO_ERROR) return err;
  a->data = data;
  gpudata_retain(data);
  a->offset = offset;
  a->typecode = typecode;
  a->flags = writeable ? GA_WRITEABLE : 0;
  GpuArray_fix_flags(a);
  return GA_NO_ERROR;
}

int GpuArray_view(GpuArray *v, const GpuArray *a) {
  gpucontext *ctx = GpuArray_context(a);
  int err;
  memset(v, 0, sizeof(*v));
  err = set_shape(v, a->nd, a->dimensions, a->strides, ctx->err);
  if (err != GA_NO_ERROR) return err;
  v->data = a->data;
  gpudata_retain(a->data);
  v->offset = a->offset;
  v->typecode = a->typecode;
  v->flags = a->flags;
  return GA_NO_ERROR;
}

int GpuArray_sync(GpuArray *a) { return gpudata_sync(a->data); }

int GpuArray_index_inplace(GpuArray *a, const ssize_t *starts, const ssize_t *stops,
                           const ssize_t *steps) {
  gpucontext *ctx = GpuArray_context(a);
  unsigned int i, out = 0, keep = 0;
  size_t off = a->offset;
  size_t *nd_dims;
  ssize_t *nd_strs;

  if (starts == NULL || stops == NULL || steps == NULL)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Invalid slice (contains NULL)");
  for (i = 0; i < a->nd; i++)
    if (steps[i] != 0) keep++;
  nd_dims = calloc(keep ? keep : 1, sizeof(size_t));
  nd_strs = calloc(keep ? keep : 1, sizeof(ssize_t));
  if (nd_dims == NULL || nd_strs == NULL) {
    free(nd_dims);
    free(nd_strs);
    return ga_err_sys(ctx->err, "calloc");
  }
  for (i = 0; i < a->nd; i++) {
    ssize_t len = (ssize_t)a->dimensions[i];
    int bad = starts[i] < -1 || starts[i] > len;
    if (!bad && steps[i] == 0) bad = starts[i] == -1 || starts[i] >= len;
    if (!bad && steps[i] != 0)
      bad = stops[i] < -1 || stops[i] > len || (stops[i] - starts[i]) / steps[i] < 0;
    if (bad) {
      free(nd_dims);
      free(nd_strs);
      return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                        "Invalid slice value: slice(%zd, %zd, %zd) when indexing array on "
                        "dimension %u of length %zd", starts[i], stops[i], steps[i], i, len);
    }
    off += (size_t)(starts[i] * a->strides[i]);
    if (steps[i] != 0) {
      nd_strs[out] = steps[i] * a->strides[i];
      nd_dims[out] = (size_t)((stops[i] - starts[i] + steps[i] - (steps[i] < 0 ? -1 : 1)) / steps[i]);
      out++;
    }
  }
  free(a->dimensions);
  free(a->strides);
  a->dimensions = nd_dims;
  a->strides = nd_strs;
  a->nd = keep;
  a->offset = off;
  GpuArray_fix_flags(a);
  return GA_NO_ERROR;
}

int GpuArray_index(GpuArray *r, const GpuArray *a, const ssize_t *starts, const ssize_t *stops,
                   const ssize_t *steps) {
  int err = GpuArray_view(r, a);
  if (err != GA_NO_ERROR) return err;
  err = GpuArray_index_inplace(r, starts, stops, steps);
  if (err != GA_NO_ERROR) GpuArray_clear(r);
  return err;
}

/* Tries to express `newdims` over the existing memory. Groups of old axes and
 * groups of new axes with equal element counts are matched left to right; a
 * group can be re-split only if its old axes are contiguous among themselves
 * in the requested order. GA_COPY_ERROR when a copy would be needed. */
int GpuArray_reshape_inplace(GpuArray *a, unsigned int nd, const size_t *newdims, ga_order ord) {
  gpucontext *ctx = GpuArray_context(a);
  size_t elsize = GpuArray_ITEMSIZE(a);
  size_t oldn = array_nelems(a), newn = 1;
  ssize_t *ns;
  unsigned int i, oi = 0, ni = 0;
  int err;

  if (ord == GA_ANY_ORDER) ord = (GpuArray_ISFORTRAN(a) && a->nd > 1) ? GA_F_ORDER : GA_C_ORDER;
  for (i = 0; i < nd; i++) {
    if (mul_overflows(newdims[i], newn))
      return ga_err_set(ctx->err, GA_XLARGE_ERROR,
                        "Output array size greater than addressable space");
    newn *= newdims[i];
  }
  if (newn != oldn)
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "New shape differs in total size");

  ns = calloc(nd ? nd : 1, sizeof(ssize_t));
  if (ns == NULL) return ga_err_sys(ctx->err, "calloc");

  if ((ord == GA_C_ORDER && GpuArray_CHKFLAGS(a, GA_C_CONTIGUOUS)) ||
      (ord == GA_F_ORDER && GpuArray_CHKFLAGS(a, GA_F_CONTIGUOUS)) || newn == 0) {
    fill_strides(nd, newdims, elsize, ord, ns);
  } else {
    while (ni < nd && oi < a->nd) {
      unsigned int oj = oi + 1, nj = ni + 1, k;
      size_t op = a->dimensions[oi], np = newdims[ni];
      while (np != op) {
        if (np < op) np *= newdims[nj++];
        else op *= a->dimensions[oj++];
      }
      for (k = oi; k + 1 < oj; k++) {
        int ok = ord == GA_F_ORDER
                     ? a->strides[k + 1] == (ssize_t)a->dimensions[k] * a->strides[k]
                     : a->strides[k] == (ssize_t)a->dimensions[k + 1] * a->strides[k + 1];
        if (!ok) {
          free(ns);
          return ga_err_set(ctx->err, GA_COPY_ERROR,
                            "Copy is needed but disallowed by parameters");
        }
      }
      if (ord == GA_F_ORDER) {
        ns[ni] = a->strides[oi];
        for (k = ni + 1; k < nj; k++) ns[k] = ns[k - 1] * (ssize_t)newdims[k - 1];
      } else {
        ns[nj - 1] = a->strides[oj - 1];
        for (k = nj - 1; k > ni; k--) ns[k - 1] = ns[k] * (ssize_t)newdims[k];
      }
      ni = nj;
      oi = oj;
    }
    /* trailing size-1 axes of the new shape */
    for (i = ni; i < nd; i++)
      ns[i] = ord == GA_F_ORDER && i > 0 ? ns[i - 1] * (ssize_t)newdims[i - 1] : (ssize_t)elsize;
  }
  err = set_shape(a, nd, newdims, ns, ctx->err);
  free(ns);
  if (err != GA_NO_ERROR) return err;
  GpuArray_fix_flags(a);
  return GA_NO_ERROR;
}

int GpuArray_reshape(GpuArray *res, const GpuArray *a, unsigned int nd, const size_t *newdims,
                     ga_order ord, int nocopy) {
  int err = GpuArray_view(res, a);
  if (err != GA_NO_ERROR) return err;
  err = GpuArray_reshape_inplace(res, nd, newdims, ord);
  if (err == GA_COPY_ERROR && !nocopy) {
    GpuArray_clear(res);
    err = GpuArray_copy(res, a, ord);
    if (err != GA_NO_ERROR) return err;
    err = GpuArray_reshape_inplace(res, nd, newdims, ord);
  }
  if (err != GA_NO_ERROR) GpuArray_clear(res);
  return err;
}

int GpuArray_transpose_inplace(GpuArray *a, const unsigned int *new_axes) {
  gpucontext *ctx = GpuArray_context(a);
  size_t *d = calloc(a->nd ? a->nd : 1, sizeof(size_t));
  ssize_t *s = calloc(a->nd ? a->nd : 1, sizeof(ssize_t));
  unsigned int i, k;
  if (d == NULL || s == NULL) {
    free(d);
    free(s);
    return ga_err_set(ctx->err, GA_MEMORY_ERROR, "Out of memory");
  }
  for (i = 0; i < a->nd; i++) {
    unsigned int from = new_axes == NULL ? a->nd - 1 - i : new_axes[i];
    if (from >= a->nd) {
      free(d);
      free(s);
      return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Axis %u out of range in transpose", from);
    }
    for (k = 0; new_axes != NULL && k < i; k++)
      if (new_axes[k] == from) {
        free(d);
        free(s);
        return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                          "Repeated axes in transpose: new_axes[%u] == new_axes[%u] == %u", i, k,
                          from);
      }
    d[i] = a->dimensions[from];
    s[i] = a->strides[from];
  }
  free(a->dimensions);
  free(a->strides);
  a->dimensions = d;
  a->strides = s;
  GpuArray_fix_flags(a);
  return GA_NO_ERROR;
}

int GpuArray_transpose(GpuArray *res, const GpuArray *a, const unsigned int *new_axes) {
  int err = GpuArray_view(res, a);
  if (err != GA_NO_ERROR) return err;
  err = GpuArray_transpose_inplace(res, new_axes);
  if (err != GA_NO_ERROR) GpuArray_clear(res);
  return err;
}

void GpuArray_clear(GpuArray *a) {
  if (a->data != NULL) gpudata_release(a->data);
  free(a->dimensions);
  free(a->strides);
  memset(a, 0, sizeof(*a));
}

int GpuArray_share(const GpuArray *a, const GpuArray *b) {
  if (a->data != b->data) return 0;
  return gpudata_share(a->data, b->data, NULL);
}

gpucontext *GpuArray_context(const GpuArray *a) { return gpudata_context(a->data); }

/* ------------------------------------------------------------ typed copies */

typedef struct extcopy_entry {
  int itype, otype;
  GpuElemwise *ge;
  struct extcopy_entry *next;
} extcopy_entry;

void ga_extcopy_cache_free(gpucontext *ctx) {
  extcopy_entry *e = (extcopy_entry *)ctx->extcopy_cache, *n;
  ctx->extcopy_cache = NULL;
  for (; e != NULL; e = n) {
    n = e->next;
    GpuElemwise_free(e->ge);
    free(e);
  }
}

/* dst[...] = (dst type)src[...] over arbitrary strides; src may broadcast. */
static int extcopy(GpuArray *dst, const GpuArray *src) {
  gpucontext *ctx = GpuArray_context(dst);
  extcopy_entry *e;
  void *args[2];

  if (ctx != GpuArray_context(src))
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "src and dst context differ");
  for (e = (extcopy_entry *)ctx->extcopy_cache; e != NULL; e = e->next)
    if (e->itype == src->typecode && e->otype == dst->typecode) break;
  if (e == NULL) {
    gpuelemwise_arg ga[2];
    ga[0].name = "src";
    ga[0].typecode = src->typecode;
    ga[0].flags = GE_READ;
    ga[1].name = "dst";
    ga[1].typecode = dst->typecode;
    ga[1].flags = GE_WRITE;
    e = calloc(1, sizeof(*e));
    if (e == NULL) return ga_err_sys(ctx->err, "calloc");
    e->ge = GpuElemwise_new(ctx, "", "dst = src", 2, ga, 0, GE_CONVERT_F16);
    if (e->ge == NULL) {
      free(e);
      return ctx->err->code;
    }
    e->itype = src->typecode;
    e->otype = dst->typecode;
    e->next = (extcopy_entry *)ctx->extcopy_cache;
    ctx->extcopy_cache = e;
  }
  args[0] = (void *)src;
  args[1] = (void *)dst;
  return GpuElemwise_call(e->ge, args, GE_BROADCAST);
}

int GpuArray_setarray(GpuArray *a, const GpuArray *v) {
  gpucontext *ctx = GpuArray_context(a);
  GpuArray tv;
  ssize_t *strs;
  unsigned int i, off;
  int err, plain = 1;

  if (a->nd < v->nd)
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Dimension error. a->nd = %u, v->nd = %u", a->nd,
                      v->nd);
  if (!GpuArray_ISWRITEABLE(a))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Destination array not writable");
  if (!GpuArray_ISALIGNED(v) || !GpuArray_ISALIGNED(a))
    return ga_err_set(ctx->err, GA_UNALIGNED_ERROR, "One of the inputs is unaligned");
  off = a->nd - v->nd;
  for (i = 0; i < v->nd; i++) {
    if (v->dimensions[i] == a->dimensions[i + off]) continue;
    if (v->dimensions[i] != 1)
      return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                        "Shape error. v->dimensions[%u] = %zu, a->dimensions[%u + %u] = %zu", i,
                        v->dimensions[i], i, off, a->dimensions[i + off]);
    plain = 0;
  }
  if (plain && a->nd == v->nd && a->typecode == v->typecode && GpuArray_ISONESEGMENT(a) &&
      GpuArray_ISONESEGMENT(v) && GpuArray_ISFORTRAN(a) == GpuArray_ISFORTRAN(v))
    return gpudata_move(a->data, a->offset, v->data, v->offset,
                        array_nelems(a) * GpuArray_ITEMSIZE(a));

  /* present v with a's rank and extents; broadcast axes get stride 0 */
  strs = calloc(a->nd ? a->nd : 1, sizeof(ssize_t));
  if (strs == NULL) return ga_err_set(ctx->err, GA_MEMORY_ERROR, "Out of memory");
  for (i = off; i < a->nd; i++)
    if (v->dimensions[i - off] == a->dimensions[i]) strs[i] = v->strides[i - off];
  tv = *v;
  tv.nd = a->nd;
  tv.dimensions = a->dimensions;
  tv.strides = strs;
  if (tv.nd != 0) GpuArray_fix_flags(&tv);
  err = extcopy(a, &tv);
  free(strs);
  return err;
}

int GpuArray_move(GpuArray *dst, const GpuArray *src) {
  gpucontext *ctx = GpuArray_context(dst);
  unsigned int i;
  if (!GpuArray_ISWRITEABLE(dst))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Destination array (dst) not writeable");
  if (!GpuArray_ISALIGNED(src))
    return ga_err_set(ctx->err, GA_UNALIGNED_ERROR, "Source array (src) not aligned");
  if (!GpuArray_ISALIGNED(dst))
    return ga_err_set(ctx->err, GA_UNALIGNED_ERROR, "Destination array (dst) not aligned");
  if (src->nd != dst->nd)
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Dimension mismatch. src->nd = %u, dst->nd = %u",
                      src->nd, dst->nd);
  for (i = 0; i < src->nd; i++)
    if (src->dimensions[i] != dst->dimensions[i])
      return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                        "Dimension mismatch. src->dimensions[%u] = %zu, dst->dimensions[%u] = %zu",
                        i, src->dimensions[i], i, dst->dimensions[i]);
  if (!GpuArray_ISONESEGMENT(dst) || !GpuArray_ISONESEGMENT(src) ||
      GpuArray_ISFORTRAN(dst) != GpuArray_ISFORTRAN(src) || dst->typecode != src->typecode)
    return extcopy(dst, src);
  return gpudata_move(dst->data, dst->offset, src->data, src->offset,
                      array_nelems(dst) * GpuArray_ITEMSIZE(dst));
}

int GpuArray_write(GpuArray *dst, const void *src, size_t src_sz) {
  gpucontext *ctx = GpuArray_context(dst);
  if (!GpuArray_ISWRITEABLE(dst))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Destination array (dst) not writeable");
  if (!GpuArray_ISONESEGMENT(dst))
    return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR, "Destination array (dst) not one segment");
  return gpudata_write(dst->data, dst->offset, src, src_sz);
}

int GpuArray_read(void *dst, size_t dst_sz, const GpuArray *src) {
  gpucontext *ctx = GpuArray_context(src);
  if (!GpuArray_ISONESEGMENT(src))
    return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR, "Array (src) not one segment");
  return gpudata_read(dst, src->data, src->offset, dst_sz);
}

int GpuArray_memset(GpuArray *a, int data) {
  gpucontext *ctx = GpuArray_context(a);
  if (!GpuArray_ISONESEGMENT(a))
    return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR, "Array (a) not one segment");
  return gpudata_memset(a->data, a->offset, data);
}

int GpuArray_copy(GpuArray *res, const GpuArray *a, ga_order order) {
  int err = GpuArray_empty(res, GpuArray_context(a), a->typecode, a->nd, a->dimensions, order);
  if (err != GA_NO_ERROR) return err;
  err = GpuArray_move(res, a);
  if (err != GA_NO_ERROR) GpuArray_clear(res);
  return err;
}

int GpuArray_transfer(GpuArray *res, const GpuArray *a) {
  gpucontext *ctx = GpuArray_context(res);
  if (!GpuArray_ISONESEGMENT(res))
    return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR, "Array (res) not one segment");
  if (!GpuArray_ISONESEGMENT(a))
    return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR, "Array (a) not one segment");
  if (res->typecode != a->typecode)
    return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR, "typecode mismatch");
  return gpudata_transfer(res->data, res->offset, a->data, a->offset,
                          array_nelems(a) * GpuArray_ITEMSIZE(a));
}

int GpuArray_split(GpuArray **rs, const GpuArray *a, size_t n, size_t *p, unsigned int axis) {
  gpucontext *ctx = GpuArray_context(a);
  ssize_t *lo, *hi, *st;
  size_t i, done = 0;
  int err = GA_NO_ERROR;
  if (axis >= a->nd) return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Invalid axis %u", axis);
  lo = calloc(a->nd, sizeof(ssize_t));
  hi = calloc(a->nd, sizeof(ssize_t));
  st = calloc(a->nd, sizeof(ssize_t));
  if (lo == NULL || hi == NULL || st == NULL) {
    free(lo);
    free(hi);
    free(st);
    return ga_err_sys(ctx->err, "calloc");
  }
  for (i = 0; i < a->nd; i++) {
    hi[i] = (ssize_t)a->dimensions[i];
    st[i] = 1;
  }
  for (i = 0; i <= n; i++) {
    lo[axis] = i > 0 ? (ssize_t)p[i - 1] : 0;
    hi[axis] = i < n ? (ssize_t)p[i] : (ssize_t)a->dimensions[axis];
    err = GpuArray_index(rs[i], a, lo, hi, st);
    if (err != GA_NO_ERROR) break;
    done++;
  }
  free(lo);
  free(hi);
  free(st);
  if (err != GA_NO_ERROR)
    for (i = 0; i < done; i++) GpuArray_clear(rs[i]);
  return err;
}

int GpuArray_concatenate(GpuArray *r, const GpuArray **as, size_t n, unsigned int axis,
                         int restype) {
  gpucontext *ctx = GpuArray_context(as[0]);
  unsigned int nd = as[0]->nd, d;
  size_t *dims, *keep_dims, keep_off, i;
  int keep_flags, err = GA_NO_ERROR;

  if (axis >= nd)
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Invalid axis. axis = %u, as[0]->nd = %u", axis, nd);
  dims = calloc(nd, sizeof(size_t));
  if (dims == NULL) return ga_err_set(ctx->err, GA_MEMORY_ERROR, "Out of memory");
  memcpy(dims, as[0]->dimensions, nd * sizeof(size_t));
  for (i = 0; i < n && err == GA_NO_ERROR; i++) {
    if (!GpuArray_ISALIGNED(as[i]))
      err = ga_err_fmt(ctx->err, GA_UNALIGNED_ERROR, "Unaligned array (as[%zu]).", i);
    else if (as[i]->nd != nd)
      err = ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                       "Shape mismatch. as[%zu]->nd = %u, as[0]->nd = %u", i, as[i]->nd, nd);
    for (d = 0; d < nd && err == GA_NO_ERROR && i > 0; d++) {
      if (d == axis) dims[d] += as[i]->dimensions[d];
      else if (dims[d] != as[i]->dimensions[d])
        err = ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                         "Dimension mismatch. as[%zu]->dimensions[%u] = %zu, "
                         "as[0]->dimensions[%u] = %zu", i, d, as[i]->dimensions[d], d, dims[d]);
    }
  }
  if (err == GA_NO_ERROR) err = GpuArray_empty(r, ctx, restype, nd, dims, GA_ANY_ORDER);
  free(dims);
  if (err != GA_NO_ERROR) return err;

  /* slide a window of each input's extent along `axis` of the result */
  keep_off = r->offset;
  keep_dims = r->dimensions;
  keep_flags = r->flags;
  for (i = 0; i < n; i++) {
    r->dimensions = as[i]->dimensions;
    GpuArray_fix_flags(r);
    err = extcopy(r, as[i]);
    if (err != GA_NO_ERROR) break;
    r->offset += (size_t)(r->strides[axis] * (ssize_t)as[i]->dimensions[axis]);
  }
  r->offset = keep_off;
  r->dimensions = keep_dims;
  r->flags = keep_flags;
  if (err != GA_NO_ERROR) GpuArray_clear(r);
  return err;
}

/* a[k, ...] = v[i[k], ...]: gather along axis 0 (reference
 * src/gpuarray_array.c:425-546). `a` and `i` are C-contiguous, `v` may have
 * any strides. With check_error the error word is read back (a host
 * synchronisation) and an out-of-range index gives GA_VALUE_ERROR. */
typedef struct take1_entry {
  int a_tc, v_tc, i_tc;
  unsigned int nd;
  ga_function fn;
  struct take1_entry *next;
} take1_entry;

void ga_take1_cache_free(gpucontext *ctx) {
  take1_entry *e = (take1_entry *)ctx->take1_cache, *n;
  ctx->take1_cache = NULL;
  for (; e != NULL; e = n) {
    n = e->next;
    free(e);
  }
}

int GpuArray_take1(GpuArray *a, const GpuArray *v, const GpuArray *i, int check_error) {
  gpucontext *ctx = GpuArray_context(a);
  ga_strb sb;
  ga_function fn;
  unsigned long long blob[2 + 2 * 16];
  unsigned grid[3] = {1, 1, 1}, block[3] = {256, 1, 1};
  CUdeviceptr p_r, p_v, p_i, p_e;
  void *params[5];
  size_t n0, n1 = 1;
  unsigned int j;
  int err, kerr = 0;

  if (!GpuArray_ISWRITEABLE(a))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Destination array not writeable");
  if (!GpuArray_ISALIGNED(a) || !GpuArray_ISALIGNED(v) || !GpuArray_ISALIGNED(i))
    return ga_err_set(ctx->err, GA_UNALIGNED_ERROR, "Not all arrays are aligned");
  if (!ga_array_in_bounds(a) || !ga_array_in_bounds(v) || !ga_array_in_bounds(i))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "An array reaches outside its buffer");
  if (!GpuArray_IS_C_CONTIGUOUS(a))
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "Destination array (a) not C-contiguous");
  if (!GpuArray_IS_C_CONTIGUOUS(i))
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "Index array (i) not C-contiguous");
  if (v->nd == 0 || a->nd == 0 || i->nd != 1 || a->nd != v->nd || v->nd > 16)
    return ga_err_fmt(ctx->err, GA_INVALID_ERROR,
                      "Dimension mismatch. v->nd = %u, a->nd = %u, i->nd = %u", v->nd, a->nd, i->nd);
  if (a->dimensions[0] != i->dimensions[0])
    return ga_err_fmt(ctx->err, GA_INVALID_ERROR,
                      "Dimension mismatch. a->dimensions[0] = %zu, i->dimensions[0] = %zu",
                      a->dimensions[0], i->dimensions[0]);
  for (j = 1; j < v->nd; j++) {
    if (a->dimensions[j] != v->dimensions[j])
      return ga_err_fmt(ctx->err, GA_INVALID_ERROR,
                        "Dimension mismatch. a->dimensions[%u] = %zu, v->dimensions[%u] = %zu", j,
                        a->dimensions[j], j, v->dimensions[j]);
    n1 *= v->dimensions[j];
  }
  n0 = i->dimensions[0];
  if (!ga_type_is_computable(a->typecode) || !ga_type_is_computable(v->typecode) ||
      !ga_type_is_computable(i->typecode) || i->typecode == GA_FLOAT || i->typecode == GA_DOUBLE ||
      i->typecode == GA_HALF)
    return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR, "Unsupported element or index type");
  if (n0 == 0 || n1 == 0) return GA_NO_ERROR;

  {
    /* the gather kernel of this (types, rank): built once per context, so that a call
     * costs no source generation, hashing or module look-up */
    take1_entry *te;
    for (te = (take1_entry *)ctx->take1_cache; te != NULL; te = te->next)
      if (te->a_tc == a->typecode && te->v_tc == v->typecode && te->i_tc == i->typecode &&
          te->nd == v->nd)
        break;
    if (te == NULL) {
      ga_strb_init(&sb);
      ga_strb_printf(&sb,
                     "#include \"cluda.h\"\n#define GA_TK_R_T %s\n#define GA_TK_V_T %s\n"
                     "#define GA_TK_I_T %s\n#define GA_TK_ND %u\n#include \"ga_take1.cuh\"\n",
                     ga_ctype(a->typecode), ga_ctype(v->typecode), ga_ctype(i->typecode), v->nd);
      if (sb.failed) {
        ga_strb_free(&sb);
        return ga_err_set(ctx->err, GA_MEMORY_ERROR, "Out of memory");
      }
      err = ga_compile(ctx, ga_strb_cstr(&sb), "ga_take1", NULL, &fn, NULL);
      ga_strb_free(&sb);
      if (err != GA_NO_ERROR) return err;
      fn.dependent_ok = 1;
      te = calloc(1, sizeof(*te));
      if (te == NULL) return ga_err_sys(ctx->err, "calloc");
      te->a_tc = a->typecode;
      te->v_tc = v->typecode;
      te->i_tc = i->typecode;
      te->nd = v->nd;
      te->fn = fn;
      te->next = (take1_entry *)ctx->take1_cache;
      ctx->take1_cache = te;
    }
    fn = te->fn;
  }

  blob[0] = n0;
  blob[1] = n1;
  for (j = 0; j < v->nd; j++) {
    blob[2 + j] = v->dimensions[j];
    blob[2 + v->nd + j] = (unsigned long long)(long long)v->strides[j];
  }
  p_r = a->data->ptr + a->offset;
  p_v = v->data->ptr + v->offset;
  p_i = i->data->ptr + i->offset;
  p_e = ctx->errbuf->ptr;
  params[0] = blob;
  params[1] = &p_r;
  params[2] = &p_v;
  params[3] = &p_i;
  params[4] = &p_e;
  grid[0] = (unsigned)((n1 + 255) / 256 > 65535 ? 65535 : (n1 + 255) / 256);
  grid[1] = (unsigned)(n0 > 65535 ? 65535 : n0);
  err = ga_launch(ctx, &fn, grid, block, 0, params);
  if (err == GA_NO_ERROR && check_error) {
    err = gpudata_read(&kerr, ctx->errbuf, 0, sizeof(int));
    if (err == GA_NO_ERROR && kerr != 0) {
      kerr = 0;
      gpudata_write(ctx->errbuf, 0, &kerr, sizeof(int));
      err = ga_err_set(ctx->err, GA_VALUE_ERROR, "Index out of bounds");
    }
  }
  return err;
}

const char *GpuArray_error(const GpuArray *a, int err) {
  return gpucontext_error(gpudata_context(a->data), err);
}

void GpuArray_fprintf(FILE *fd, const GpuArray *a) {
  unsigned int i;
  fprintf(fd, "GpuArray <%p, data: %p> nd=%u typecode=%d itemsize=%zu offset=%zu\n", (void *)a,
          (void *)a->data, a->nd, a->typecode, GpuArray_ITEMSIZE(a), a->offset);
  fprintf(fd, "\tdims:");
  for (i = 0; i < a->nd; i++) fprintf(fd, " %zu", a->dimensions[i]);
  fprintf(fd, "\n\tstrides:");
  for (i = 0; i < a->nd; i++) fprintf(fd, " %zd", a->strides[i]);
  fprintf(fd, "\n\tflags:%s%s%s%s\n", (a->flags & GA_C_CONTIGUOUS) ? " C_CONTIGUOUS" : "",
          (a->flags & GA_F_CONTIGUOUS) ? " F_CONTIGUOUS" : "",
          (a->flags & GA_ALIGNED) ? " ALIGNED" : "", (a->flags & GA_WRITEABLE) ? " WRITEABLE" : "");
}

int GpuArray_fdump(FILE *fd, const GpuArray *a) {
  gpucontext *ctx = GpuArray_context(a);
  size_t elsize = GpuArray_ITEMSIZE(a), n = array_nelems(a), k;
  char *buf, *p;
  int err;
  buf = calloc((n * elsize) != 0 ? n * elsize : 1, 1);
  if (buf == NULL) return ga_err_set(ctx->err, GA_MEMORY_ERROR, "Out of memory");
  err = GpuArray_read(buf, n * elsize, a);
  for (k = 0, p = buf; err == GA_NO_ERROR && k < n; k++, p += elsize) {
    fprintf(fd, "[%zu] = ", k);
    switch (a->typecode) {
    case GA_UINT: fprintf(fd, "%u", *(unsigned int *)p); break;
    case GA_INT: fprintf(fd, "%d", *(int *)p); break;
    case GA_LONG: fprintf(fd, "%lld", (long long)*(int64_t *)p); break;
    case GA_ULONG: fprintf(fd, "%llu", (unsigned long long)*(uint64_t *)p); break;
    case GA_FLOAT: fprintf(fd, "%f", *(float *)p); break;
    case GA_DOUBLE: fprintf(fd, "%f", *(double *)p); break;
    default:
      fprintf(fd, "<unsupported data type %d>\n", a->typecode);
      err = ga_err_fmt(ctx->err, GA_UNSUPPORTED_ERROR, "Unsupported data type for dump: %d",
                       a->typecode);
      continue;
    }
    fprintf(fd, "\n");
  }
  free(buf);
  return err;
}
