/* Map-reduce engine: GpuMapReduction_new / _call / _free.
 *
 *     out[kept...] = REDUCE over the reduced axes of MAP(arg0, arg1, ..., scalars)
 *
 * Host side of what the reference does in Python for its ReductionKernel
 * (pygpu/reduction.py:137-291: a map expression over several arguments, a
 * reduce expression over `a` and `b`, a neutral element; arguments broadcast
 * against each other when the call asks for it, pygpu/tools.py:68-168). The
 * argument descriptors and the call flags are GpuElemwise's
 * (src/gpuarray/elemwise.h:28-68, :98-140); the axis list and the
 * caller-allocated destination follow GpuArray_maxandargmax
 * (src/gpuarray/array.h:607-644).
 *
 * A call: broadcast the array arguments to one shape; split the axes into kept
 * and reduced; collapse each set over ALL arguments at once (two neighbouring
 * axes merge only if every argument, and for kept axes the destination, agrees);
 * order the reduced axes by memory distance; pick one of three kernel shapes
 * (templates/ga_mapreduce.cuh) from the innermost strides; one launch.
 */
#include "private.h"

#define MR_MAXD 6
#define MR_THREADS 256
#define MR_BY 8
#define MR_MAXARR 16

enum { MR_ROWS = 0, MR_COLS = 1, MR_GENERAL = 2 };

typedef struct mr_variant {
  int shape, vec, group, tpo;
  unsigned long long modes; /* 2 bits per array argument */
  ga_function fn;
  struct mr_variant *next;
} mr_variant;

struct _GpuMapReduction {
  gpucontext *ctx;
  char *preamble, *map_expr, *reduce_expr, *neutral;
  gpuelemwise_arg *args;
  unsigned int n, narray;
  int out_tc, flags;
  unsigned int min_elsize, max_elsize;
  mr_variant *variants;
  gpudata *scratch, *tickets;
  size_t scratch_sz, tickets_sz;
  void **params;
};

/* Field order matches struct ga__mr_layout up to `tiles`; the two stride tables
 * follow with the argument count of the operator. */
typedef struct mr_head {
  unsigned long long nf_total, nr_total, nf, nr;
  unsigned long long fdim[MR_MAXD];
  long long fdst[MR_MAXD];
  unsigned long long rdim[MR_MAXD];
  unsigned long long splits, inner, seg, nseg, units, tiles;
} mr_head;

typedef struct mr_layout {
  mr_head h;
  long long str[2 * MR_MAXARR * MR_MAXD]; /* fsrc[narray][MAXD] then rsrc[narray][MAXD] */
} mr_layout;

static int is_array(const gpuelemwise_arg *a) { return ISCLR(a->flags, GE_SCALAR); }

static const char *compute_type(const GpuMapReduction *mr, int tc) {
  if (tc == GA_HALF && ISSET(mr->flags, GE_CONVERT_F16)) return "ga_float";
  return ga_ctype(tc);
}

/* ---------------------------------------------------------------- codegen */

static char *gen_source(const GpuMapReduction *mr, const mr_variant *v) {
  ga_strb sb;
  unsigned int j, k;
  const char *dst_t = ga_ctype(mr->out_tc), *acc_t = compute_type(mr, mr->out_tc);
  ga_strb_init(&sb);
  ga_strb_puts(&sb, "#include \"cluda.h\"\n");
  if (mr->preamble != NULL) ga_strb_puts(&sb, mr->preamble);
  ga_strb_puts(&sb, "\n#define GA_EW_ARRAYS(X)");
  for (j = 0, k = 0; j < mr->n; j++) {
    const gpuelemwise_arg *a = &mr->args[j];
    if (!is_array(a)) continue;
    ga_strb_printf(&sb, " \\\n  X(%u, %s, %s, %s, 1, 0, %d)", k, a->name, ga_ctype(a->typecode),
                   compute_type(mr, a->typecode), (int)((v->modes >> (2 * k)) & 3));
    k++;
  }
  ga_strb_puts(&sb, "\n#define GA_EW_SCALARS(X)");
  for (j = 0; j < mr->n; j++) {
    const gpuelemwise_arg *a = &mr->args[j];
    if (is_array(a)) continue;
    ga_strb_printf(&sb, " \\\n  X(%s, %s)", a->name, ga_ctype(a->typecode));
  }
  ga_strb_printf(&sb, "\n#define GA_EW_NARR %u\n", mr->narray);
  /* the map expression sees every argument as a scalar of its own name; its
   * value keeps its natural C type, as in `acc = REDUCE(acc, MAP)` */
  ga_strb_puts(&sb, "static __device__ __forceinline__ auto ga_mr_map(");
  for (j = 0; j < mr->n; j++)
    if (is_array(&mr->args[j]))
      ga_strb_printf(&sb, "const %s %s, ", compute_type(mr, mr->args[j].typecode), mr->args[j].name);
  for (j = 0; j < mr->n; j++)
    if (!is_array(&mr->args[j]))
      ga_strb_printf(&sb, "const %s %s, ", ga_ctype(mr->args[j].typecode), mr->args[j].name);
  ga_strb_printf(&sb, "int ga__unused) {\n  return (%s);\n}\n", mr->map_expr);
  ga_strb_printf(&sb,
                 "#define GA_MR_ACC_T %s\n#define GA_MR_DST_T %s\n"
                 "#define GA_MR_REDUCE(a, b) ((GA_MR_ACC_T)(%s))\n#define GA_MR_NEUTRAL (%s)\n"
                 "#define GA_MR_STORE(v) %s\n"
                 "#define GA_MR_VEC %d\n#define GA_MR_THREADS %d\n#define GA_MR_GROUP %d\n"
                 "#define GA_MR_BY %d\n#define GA_MR_TPO %d\n#define %s\n"
                 "#include \"ga_mapreduce.cuh\"\n",
                 acc_t, dst_t, mr->reduce_expr, mr->neutral,
                 (mr->out_tc == GA_HALF && ISSET(mr->flags, GE_CONVERT_F16))
                     ? "ga_float2half((float)(v))" : "((GA_MR_DST_T)(v))",
                 v->vec, MR_THREADS, v->group ? v->group : MR_THREADS, MR_BY, v->tpo ? v->tpo : 1,
                 v->shape == MR_ROWS ? "GA_MR_BUILD_ROWS"
                 : v->shape == MR_COLS ? "GA_MR_BUILD_COLS" : "GA_MR_BUILD_GENERAL");
  if (sb.failed) {
    ga_strb_free(&sb);
    return NULL;
  }
  return sb.s;
}

static const char *const mr_entry[] = {"ga_mr_rows", "ga_mr_cols", "ga_mr_general"};

static mr_variant *get_variant(GpuMapReduction *mr, const mr_variant *want, int *err) {
  mr_variant *v;
  char *src, *listing = NULL;
  for (v = mr->variants; v != NULL; v = v->next)
    if (v->shape == want->shape && v->vec == want->vec && v->group == want->group &&
        v->tpo == want->tpo && v->modes == want->modes)
      return v;
  v = malloc(sizeof(*v));
  if (v == NULL) {
    *err = ga_err_sys(mr->ctx->err, "malloc");
    return NULL;
  }
  *v = *want;
  src = gen_source(mr, v);
  if (src == NULL) {
    free(v);
    *err = ga_err_set(mr->ctx->err, GA_MISC_ERROR, "Formatting error creating kernel source");
    return NULL;
  }
  *err = ga_compile(mr->ctx, src, mr_entry[v->shape], NULL, &v->fn,
                    getenv("GPUARRAY_B200_DEBUG") ? &listing : NULL);
  if (listing != NULL) {
    fprintf(stderr, "%s\n", listing);
    free(listing);
  }
  free(src);
  if (*err != GA_NO_ERROR) {
    free(v);
    return NULL;
  }
  v->fn.dependent_ok = 1;
  v->next = mr->variants;
  mr->variants = v;
  return v;
}

/* Test hook: the source of one variant, without a device; caller frees. */
GPUARRAY_PUBLIC char *gpuarray_b200_mapreduction_source(const char *preamble, const char *map_expr,
                                                        const char *reduce_expr,
                                                        const char *neutral, int out_tc,
                                                        unsigned int n, gpuelemwise_arg *args,
                                                        int flags, int shape, int vec, int group,
                                                        int tpo, unsigned long long modes) {
  GpuMapReduction mr;
  mr_variant v;
  unsigned int i;
  memset(&mr, 0, sizeof(mr));
  memset(&v, 0, sizeof(v));
  mr.preamble = (char *)preamble;
  mr.map_expr = (char *)map_expr;
  mr.reduce_expr = (char *)reduce_expr;
  mr.neutral = (char *)neutral;
  mr.out_tc = out_tc;
  mr.args = args;
  mr.n = n;
  mr.flags = flags;
  for (i = 0; i < n; i++)
    if (is_array(&args[i])) mr.narray++;
  v.shape = shape;
  v.vec = vec;
  v.group = group;
  v.tpo = tpo;
  v.modes = modes;
  return gen_source(&mr, &v);
}

/* ------------------------------------------------------------ construction */

GpuMapReduction *GpuMapReduction_new(gpucontext *ctx, const char *preamble, const char *map_expr,
                                     const char *reduce_expr, const char *neutral,
                                     int out_typecode, unsigned int n, gpuelemwise_arg *args,
                                     int flags) {
  GpuMapReduction *mr;
  unsigned int i;
  int err = GA_NO_ERROR;

  if (map_expr == NULL || reduce_expr == NULL || neutral == NULL || n == 0 || args == NULL) {
    ga_err_set(ctx->err, GA_VALUE_ERROR, "GpuMapReduction_new: NULL expression or arguments");
    return NULL;
  }
  if (!ga_type_is_computable(out_typecode)) {
    ga_err_fmt(ctx->err, GA_UNSUPPORTED_ERROR, "Output type %d is not supported", out_typecode);
    return NULL;
  }
  mr = calloc(1, sizeof(*mr));
  if (mr == NULL) {
    ga_err_sys(ctx->err, "calloc");
    return NULL;
  }
  mr->ctx = ctx;
  ctx->refcnt++;
  mr->flags = flags;
  mr->n = n;
  mr->out_tc = out_typecode;
  mr->map_expr = strdup(map_expr);
  mr->reduce_expr = strdup(reduce_expr);
  mr->neutral = strdup(neutral);
  if (preamble != NULL) mr->preamble = strdup(preamble);
  mr->args = calloc(n, sizeof(gpuelemwise_arg));
  mr->params = calloc(n + 5, sizeof(void *));
  if (mr->map_expr == NULL || mr->reduce_expr == NULL || mr->neutral == NULL ||
      (preamble != NULL && mr->preamble == NULL) || mr->args == NULL || mr->params == NULL) {
    ga_err_sys(ctx->err, "strdup");
    goto fail;
  }
  mr->min_elsize = 16;
  mr->max_elsize = 1;
  for (i = 0; i < n; i++) {
    size_t es = gpuarray_get_elsize(args[i].typecode);
    if (args[i].name == NULL) {
      ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Argument %u has no name", i);
      goto fail;
    }
    if (!ga_type_is_computable(args[i].typecode)) {
      ga_err_fmt(ctx->err, GA_UNSUPPORTED_ERROR, "Argument %u (%s): type %d is not supported", i,
                 args[i].name, args[i].typecode);
      goto fail;
    }
    if (is_array(&args[i]) && ISSET(args[i].flags, GE_WRITE)) {
      ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                 "Argument %u (%s): a map-reduction only reads its arguments", i, args[i].name);
      goto fail;
    }
    mr->args[i].typecode = args[i].typecode;
    mr->args[i].flags = args[i].flags;
    mr->args[i].name = strdup(args[i].name);
    if (mr->args[i].name == NULL) {
      ga_err_sys(ctx->err, "strdup");
      goto fail;
    }
    if (is_array(&args[i])) {
      mr->narray++;
      if (es < mr->min_elsize) mr->min_elsize = (unsigned)es;
      if (es > mr->max_elsize) mr->max_elsize = (unsigned)es;
    }
  }
  if (mr->narray == 0) {
    /* the reference refuses this too (pygpu/reduction.py:175-178) */
    ga_err_set(ctx->err, GA_VALUE_ERROR, "A map-reduction needs at least one array argument");
    goto fail;
  }
  if (mr->narray > MR_MAXARR) {
    ga_err_fmt(ctx->err, GA_UNSUPPORTED_ERROR, "More than %d array arguments", MR_MAXARR);
    goto fail;
  }
  /* Build the scalar general kernel now: it validates the three expressions, so
   * a bad one is reported by the constructor, like GpuElemwise_new does. */
  {
    mr_variant want;
    memset(&want, 0, sizeof(want));
    want.shape = MR_GENERAL;
    want.vec = 1;
    want.tpo = 32;
    if (get_variant(mr, &want, &err) == NULL) goto fail;
  }
  return mr;
fail:
  GpuMapReduction_free(mr);
  return NULL;
}

void GpuMapReduction_free(GpuMapReduction *mr) {
  mr_variant *v, *nv;
  gpucontext *ctx;
  unsigned int i;
  if (mr == NULL) return;
  ctx = mr->ctx;
  for (v = mr->variants; v != NULL; v = nv) {
    nv = v->next;
    free(v);
  }
  if (mr->args != NULL)
    for (i = 0; i < mr->n; i++) free((void *)mr->args[i].name);
  if (mr->scratch != NULL) gpudata_release(mr->scratch);
  if (mr->tickets != NULL) gpudata_release(mr->tickets);
  free(mr->args);
  free(mr->params);
  free(mr->preamble);
  free(mr->map_expr);
  free(mr->reduce_expr);
  free(mr->neutral);
  free(mr);
  if (ctx != NULL) ga_ctx_unref(ctx);
}

/* -------------------------------------------------------------------- call */

static long long ll_abs(long long v) { return v < 0 ? -v : v; }

static int ensure_scratch(GpuMapReduction *mr, size_t bytes, size_t ticket_bytes) {
  int err = GA_NO_ERROR;
  if (bytes > mr->scratch_sz) {
    if (mr->scratch != NULL) gpudata_release(mr->scratch);
    mr->scratch_sz = 0;
    mr->scratch = gpudata_alloc(mr->ctx, bytes, NULL, 0, &err);
    if (mr->scratch == NULL) return err;
    mr->scratch_sz = bytes;
  }
  if (ticket_bytes > mr->tickets_sz) {
    /* counters start at zero and every launch hands them back at zero */
    if (mr->tickets != NULL) gpudata_release(mr->tickets);
    mr->tickets_sz = 0;
    if (ticket_bytes < 4096) ticket_bytes = 4096;
    mr->tickets = gpudata_alloc(mr->ctx, ticket_bytes, NULL, 0, &err);
    if (mr->tickets == NULL) return err;
    err = gpudata_memset(mr->tickets, 0, 0);
    if (err != GA_NO_ERROR) return err;
    mr->tickets_sz = ticket_bytes;
  }
  return GA_NO_ERROR;
}

/* The normalised problem of one call. */
typedef struct mr_problem {
  unsigned int nd;                      /* broadcast rank */
  size_t dims[64];
  long long str[MR_MAXARR][64];         /* broadcast byte strides per array argument */
  unsigned long long base[MR_MAXARR];   /* address of element 0 per array argument */
  size_t elsize[MR_MAXARR];
} mr_problem;

/* One array argument as the shape logic sees it. */
typedef struct mr_arr {
  unsigned int nd;
  const size_t *dims;
  const ssize_t *strides;
  unsigned long long base;
} mr_arr;

/* Broadcast shape of the array arguments (pygpu/tools.py:68-168 with
 * broadcast=True: extents must agree or be 1; lower ranks pad on the left when
 * GE_PADSHAPE is given, as in GpuElemwise_call). `arrs` holds the array
 * arguments in declaration order. Pure host arithmetic. */
static int broadcast_shapes(const GpuMapReduction *mr, ga_error_rec *e, const mr_arr *arrs,
                            int flags, mr_problem *P) {
  unsigned int i, j, k, nd = 0;
  for (k = 0; k < mr->narray; k++) {
    if (arrs[k].nd > 64) return ga_err_set(e, GA_UNSUPPORTED_ERROR, "More than 64 dimensions");
    if (k == 0) nd = arrs[k].nd;
    else if (arrs[k].nd != nd) {
      if (ISCLR(flags, GE_PADSHAPE))
        return ga_err_fmt(e, GA_VALUE_ERROR, "Array argument %u has differing nd = %u", k,
                          arrs[k].nd);
      if (arrs[k].nd > nd) nd = arrs[k].nd;
    }
  }
  P->nd = nd;
  for (j = 0; j < nd; j++) P->dims[j] = 1;
  for (k = 0; k < mr->narray; k++) {
    const unsigned int pad = nd - arrs[k].nd;
    for (j = pad; j < nd; j++)
      if (arrs[k].dims[j - pad] != 1 && P->dims[j] == 1) P->dims[j] = arrs[k].dims[j - pad];
  }
  for (k = 0; k < mr->narray; k++) { /* a zero extent anywhere makes the whole axis empty */
    const unsigned int pad = nd - arrs[k].nd;
    for (j = pad; j < nd; j++)
      if (arrs[k].dims[j - pad] == 0) P->dims[j] = 0;
  }
  for (i = 0, k = 0; i < mr->n; i++) {
    unsigned int pad;
    if (!is_array(&mr->args[i])) continue;
    pad = nd - arrs[k].nd;
    for (j = 0; j < nd; j++) {
      size_t vd = j < pad ? 1 : arrs[k].dims[j - pad];
      if (vd != P->dims[j] && (vd != 1 || ISCLR(flags, GE_BROADCAST)))
        return ga_err_fmt(e, GA_VALUE_ERROR,
                          "Mismatched dimension %u for input %u (expected %zu got %zu)", j, i,
                          P->dims[j], vd);
      P->str[k][j] = (vd == 1 || j < pad) ? 0 : (long long)arrs[k].strides[j - pad];
    }
    P->base[k] = arrs[k].base;
    P->elsize[k] = gpuarray_get_elsize(mr->args[i].typecode);
    k++;
  }
  return GA_NO_ERROR;
}

/* Validates the array arguments of a call and describes them for the shape logic. */
static int gather_args(GpuMapReduction *mr, void **args, mr_arr *arrs) {
  gpucontext *ctx = mr->ctx;
  unsigned int i, k;
  for (i = 0, k = 0; i < mr->n; i++) {
    const GpuArray *v;
    if (!is_array(&mr->args[i])) {
      if (args[i] == NULL) return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Argument %u is NULL", i);
      continue;
    }
    v = (const GpuArray *)args[i];
    if (v == NULL) return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Argument %u is NULL", i);
    if (v->typecode != mr->args[i].typecode)
      return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Argument %u has type %d, declared %d", i,
                        v->typecode, mr->args[i].typecode);
    if (GpuArray_context(v) != ctx)
      return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Argument %u belongs to another context", i);
    if (!GpuArray_ISALIGNED(v))
      return ga_err_fmt(ctx->err, GA_UNALIGNED_ERROR, "Argument %u is not aligned", i);
    if (!ga_array_in_bounds(v))
      return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Argument %u reaches outside its buffer", i);
    arrs[k].nd = v->nd;
    arrs[k].dims = v->dimensions;
    arrs[k].strides = v->strides;
    arrs[k].base = (unsigned long long)(v->data->ptr + v->offset);
    k++;
  }
  return GA_NO_ERROR;
}

static long long *fsrc_of(mr_layout *L, unsigned k) { return &L->str[(size_t)k * MR_MAXD]; }
static long long *rsrc_of(mr_layout *L, unsigned narray, unsigned k) {
  return &L->str[((size_t)narray + k) * MR_MAXD];
}

static int normalise(const GpuMapReduction *mr, ga_error_rec *e, const mr_problem *P,
                     const ssize_t *out_strides, const unsigned char *red, mr_layout *L) {
  const unsigned na = mr->narray;
  unsigned int j, k, n, kd = 0;
  memset(L, 0, sizeof(*L));
  L->h.nf_total = 1;
  L->h.nr_total = 1;

  /* kept axes, ascending; destination axis kd pairs with the kd-th kept axis */
  for (j = 0, n = 0; j < P->nd; j++) {
    long long sd;
    int merge;
    if (red[j]) continue;
    L->h.nf_total *= P->dims[j];
    sd = out_strides[kd];
    kd++;
    if (P->dims[j] == 1) continue;
    merge = n > 0 && L->h.fdst[n - 1] == (long long)P->dims[j] * sd;
    for (k = 0; k < na && merge; k++)
      if (fsrc_of(L, k)[n - 1] != (long long)P->dims[j] * P->str[k][j]) merge = 0;
    if (merge) {
      L->h.fdim[n - 1] *= P->dims[j];
      L->h.fdst[n - 1] = sd;
      for (k = 0; k < na; k++) fsrc_of(L, k)[n - 1] = P->str[k][j];
      continue;
    }
    if (n == MR_MAXD)
      return ga_err_fmt(e, GA_UNSUPPORTED_ERROR,
                        "More than %d kept dimensions remain after collapsing", MR_MAXD);
    L->h.fdim[n] = P->dims[j];
    L->h.fdst[n] = sd;
    for (k = 0; k < na; k++) fsrc_of(L, k)[n] = P->str[k][j];
    n++;
  }
  L->h.nf = n;

  /* reduced axes, traversed in memory order (largest total |stride| outermost) */
  {
    unsigned int ax[64], m = 0, i;
    unsigned long long key[64];
    for (j = 0; j < P->nd; j++) {
      if (!red[j]) continue;
      L->h.nr_total *= P->dims[j];
      if (P->dims[j] == 1) continue;
      ax[m] = j;
      key[m] = 0;
      for (k = 0; k < na; k++) key[m] += (unsigned long long)ll_abs(P->str[k][j]);
      m++;
    }
    for (i = 1; i < m; i++) { /* stable insertion sort, descending key */
      unsigned int ta = ax[i], q = i;
      unsigned long long tk = key[i];
      while (q > 0 && key[q - 1] < tk) {
        ax[q] = ax[q - 1];
        key[q] = key[q - 1];
        q--;
      }
      ax[q] = ta;
      key[q] = tk;
    }
    for (i = 0, n = 0; i < m; i++) {
      int merge = n > 0;
      j = ax[i];
      for (k = 0; k < na && merge; k++)
        if (rsrc_of(L, na, k)[n - 1] != (long long)P->dims[j] * P->str[k][j]) merge = 0;
      if (merge) {
        L->h.rdim[n - 1] *= P->dims[j];
        for (k = 0; k < na; k++) rsrc_of(L, na, k)[n - 1] = P->str[k][j];
        continue;
      }
      if (n == MR_MAXD)
        return ga_err_fmt(e, GA_UNSUPPORTED_ERROR,
                          "More than %d reduced dimensions remain after collapsing", MR_MAXD);
      L->h.rdim[n] = P->dims[j];
      for (k = 0; k < na; k++) rsrc_of(L, na, k)[n] = P->str[k][j];
      n++;
    }
    L->h.nr = n;
  }
  return GA_NO_ERROR;
}

/* every stride of argument k except the innermost one of its own kind is a
 * multiple of m, and so is its base address */
static int arg_aligned(const mr_layout *L, const mr_problem *P, unsigned na, unsigned k,
                       long long m, int skip_kept_inner, int skip_red_inner) {
  unsigned d;
  const long long *f = &L->str[(size_t)k * MR_MAXD], *r = &L->str[((size_t)na + k) * MR_MAXD];
  if (P->base[k] % (unsigned long long)m != 0) return 0;
  for (d = 0; d < L->h.nf; d++)
    if (!(skip_kept_inner && d + 1 == L->h.nf) && f[d] % m != 0) return 0;
  for (d = 0; d < L->h.nr; d++)
    if (!(skip_red_inner && d + 1 == L->h.nr) && r[d] % m != 0) return 0;
  return 1;
}

/* Kernel shape, access modes, split and launch geometry. Pure host arithmetic. */
static void mr_plan(const GpuMapReduction *mr, const mr_problem *P, mr_layout *L, mr_variant *want,
                    unsigned grid[3], unsigned block[3], unsigned num_sms) {
  const unsigned na = mr->narray;
  unsigned k, vec0;
  int rows_ok, cols_ok, any;
  size_t bytes_per_elem = 0;
  grid[0] = grid[1] = grid[2] = 1;
  block[0] = MR_THREADS;
  block[1] = block[2] = 1;
  memset(want, 0, sizeof(*want));
  want->vec = 1;
  want->tpo = 1;
  want->group = MR_THREADS;
  L->h.splits = 1;
  L->h.seg = L->h.inner = 0;
  L->h.nseg = 1;
  L->h.units = 1;
  L->h.tiles = 1;
  for (k = 0; k < na; k++) bytes_per_elem += P->elsize[k];
  vec0 = 16 / mr->min_elsize;
  while (vec0 > 1 && vec0 * mr->max_elsize > 64) vec0 /= 2;

  rows_ok = L->h.nr_total > 0 && L->h.nr >= 1;
  for (k = 0, any = 0; k < na && rows_ok; k++) {
    long long s = L->str[((size_t)na + k) * MR_MAXD + (L->h.nr - 1)];
    if (s == (long long)P->elsize[k]) any = 1;
    else if (s != 0) rows_ok = 0;
  }
  rows_ok = rows_ok && any;
  cols_ok = !rows_ok && L->h.nr_total > 0 && L->h.nf >= 1 && L->h.fdim[L->h.nf - 1] >= 16;
  for (k = 0, any = 0; k < na && cols_ok; k++) {
    long long s = L->str[(size_t)k * MR_MAXD + (L->h.nf - 1)];
    if (s == (long long)P->elsize[k]) any = 1;
    else if (s != 0) cols_ok = 0;
  }
  cols_ok = cols_ok && any;

  if (rows_ok) {
    unsigned vec = vec0;
    unsigned long long nvrow, rows_outer, target_groups, s;
    want->shape = MR_ROWS;
    L->h.inner = L->h.rdim[L->h.nr - 1];
    rows_outer = L->h.nr_total / L->h.inner;
    /* vector loads need every contiguous argument aligned, row starts included */
    for (;;) {
      int ok = 1;
      for (k = 0; k < na && ok; k++) {
        long long s_in = L->str[((size_t)na + k) * MR_MAXD + (L->h.nr - 1)];
        long long vb = (long long)(P->elsize[k] * vec > 16 ? 16 : P->elsize[k] * vec);
        if (s_in != 0 && !arg_aligned(L, P, na, k, vb, 0, 1)) ok = 0;
      }
      if (ok || vec == 1) break;
      vec /= 2;
    }
    want->vec = (int)vec;
    for (k = 0; k < na; k++) {
      long long s_in = L->str[((size_t)na + k) * MR_MAXD + (L->h.nr - 1)];
      want->modes |= (unsigned long long)(s_in == 0 ? 2 : 1) << (2 * k);
    }
    nvrow = L->h.inner / vec;
    L->h.seg = L->h.inner;
    L->h.nseg = 1;
    L->h.units = rows_outer;
    if (L->h.nf_total >= (unsigned long long)num_sms * 16) want->group = 32;
    else if (L->h.nf_total >= (unsigned long long)num_sms * 4 && nvrow >= 1024) want->group = MR_THREADS;
    else {
      /* few outputs: split the reduced extent over several groups per output */
      unsigned long long seg, cap;
      want->group = (nvrow >= 2048 && L->h.nf_total < (unsigned long long)num_sms * 4) ? MR_THREADS : 32;
      seg = (unsigned long long)want->group * vec * 16;
      if (seg < L->h.inner) {
        L->h.seg = seg;
        L->h.nseg = (L->h.inner + seg - 1) / seg;
        L->h.units = rows_outer * L->h.nseg;
      }
      target_groups = want->group == MR_THREADS ? (unsigned long long)num_sms * 4
                                                : (unsigned long long)num_sms * 32 * (MR_THREADS / 32);
      s = (target_groups + L->h.nf_total - 1) / L->h.nf_total;
      /* a group's share should stay above ~24 KiB per warp (ramp and finish cost) */
      cap = L->h.nr_total * bytes_per_elem / ((want->group == 32 ? 24u : 96u) << 10);
      if (cap < 1) cap = 1;
      if (s > cap) s = cap;
      if (s > L->h.units) s = L->h.units;
      if (s > (1u << 20)) s = 1u << 20;
      L->h.splits = s ? s : 1;
    }
    if (L->h.seg >= 0x7fffffffULL) { /* a run beyond 32-bit indexing is cut even without a split */
      L->h.seg = (unsigned long long)want->group * vec * 16 * 1024;
      L->h.nseg = (L->h.inner + L->h.seg - 1) / L->h.seg;
      L->h.units = rows_outer * L->h.nseg;
    }
    {
      unsigned gpb = MR_THREADS / (unsigned)want->group;
      unsigned long long nwork = L->h.nf_total * L->h.splits, blocks = (nwork + gpb - 1) / gpb;
      unsigned long long capb = (unsigned long long)num_sms * 64;
      if (blocks > capb) blocks = capb; /* groups loop over their work items */
      grid[0] = (unsigned)(blocks ? blocks : 1);
    }
  } else if (cols_ok) {
    unsigned vec = vec0 > 4 ? 4 : vec0;
    unsigned long long ko, nwork, s;
    want->shape = MR_COLS;
    L->h.inner = L->h.fdim[L->h.nf - 1];
    for (;;) {
      int ok = L->h.inner % vec == 0;
      for (k = 0; k < na && ok; k++) {
        long long s_in = L->str[(size_t)k * MR_MAXD + (L->h.nf - 1)];
        long long vb = (long long)(P->elsize[k] * vec > 16 ? 16 : P->elsize[k] * vec);
        if (s_in != 0 && !arg_aligned(L, P, na, k, vb, 1, 0)) ok = 0;
      }
      if (ok || vec == 1) break;
      vec /= 2;
    }
    want->vec = (int)vec;
    for (k = 0; k < na; k++) {
      long long s_in = L->str[(size_t)k * MR_MAXD + (L->h.nf - 1)];
      want->modes |= (unsigned long long)(s_in == 0 ? 2 : 1) << (2 * k);
    }
    L->h.tiles = (L->h.inner + 32ULL * vec - 1) / (32ULL * vec);
    ko = L->h.nf_total / L->h.inner;
    nwork = ko * L->h.tiles;
    s = ((unsigned long long)num_sms * 3 + nwork - 1) / nwork;
    if (s > (L->h.nr_total + MR_BY * 8 - 1) / (MR_BY * 8)) s = (L->h.nr_total + MR_BY * 8 - 1) / (MR_BY * 8);
    if (s > 1024) s = 1024;
    L->h.splits = s ? s : 1;
    L->h.units = nwork;
    grid[0] = nwork > 0x7fffffffULL ? 0x7fffffffu : (unsigned)nwork;
    grid[1] = (unsigned)L->h.splits;
    block[0] = 32;
    block[1] = MR_BY;
  } else {
    unsigned long long gpb, blocks;
    want->shape = MR_GENERAL;
    if (L->h.nr_total >= 2048 && L->h.nf_total < 4096) want->tpo = MR_THREADS;
    else if (L->h.nr_total >= 64) want->tpo = 32;
    gpb = MR_THREADS / (unsigned)want->tpo;
    blocks = (L->h.nf_total + gpb - 1) / gpb;
    if (blocks > (unsigned long long)num_sms * 256) blocks = (unsigned long long)num_sms * 256;
    grid[0] = (unsigned)(blocks ? blocks : 1);
  }
}

int GpuMapReduction_call(GpuMapReduction *mr, GpuArray *out, void **args, unsigned int reduxLen,
                         const int *reduxList, int flags) {
  gpucontext *ctx;
  mr_problem P;
  mr_layout L;
  mr_variant want, *v;
  unsigned char red[64];
  unsigned grid[3], block[3], i, j, k, p = 0, ndd;
  CUdeviceptr p_dst, p_val = 0, p_tic = 0, ptrs[MR_MAXARR];
  int err;

  if (mr == NULL) return GA_INVALID_ERROR;
  ctx = mr->ctx;
  if (out == NULL || args == NULL)
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "GpuMapReduction_call: NULL argument");
  {
    mr_arr arrs[MR_MAXARR];
    err = gather_args(mr, args, arrs);
    if (err != GA_NO_ERROR) return err;
    err = broadcast_shapes(mr, ctx->err, arrs, flags, &P);
    if (err != GA_NO_ERROR) return err;
  }
  if (reduxLen == 0 || reduxList == NULL)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Reduction is along no axes");
  if (reduxLen > P.nd)
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "More reduction axes than dimensions");
  memset(red, 0, sizeof(red));
  for (i = 0; i < reduxLen; i++) {
    if (reduxList[i] < 0 || (unsigned)reduxList[i] >= P.nd)
      return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Reduction axis %d out of range", reduxList[i]);
    if (red[reduxList[i]])
      return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Reduction axis %d listed twice", reduxList[i]);
    red[reduxList[i]] = 1;
  }
  ndd = P.nd - reduxLen;
  if (out->nd != ndd)
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Destination has %u dimensions, expected %u",
                      out->nd, ndd);
  for (j = 0, k = 0; j < P.nd; j++) {
    if (red[j]) continue;
    if (out->dimensions[k] != P.dims[j])
      return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                        "Destination dimension %u is %zu but axis %u has %zu", k,
                        out->dimensions[k], j, P.dims[j]);
    k++;
  }
  if (out->typecode != mr->out_tc)
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Destination has type %d, the operator writes %d",
                      out->typecode, mr->out_tc);
  if (GpuArray_context(out) != ctx)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Destination belongs to another context");
  if (!GpuArray_ISWRITEABLE(out))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Destination is not writeable");
  if (!GpuArray_ISALIGNED(out))
    return ga_err_set(ctx->err, GA_UNALIGNED_ERROR, "Destination is not aligned");
  if (!ga_array_in_bounds(out))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Destination reaches outside its buffer");

  err = normalise(mr, ctx->err, &P, out->strides, red, &L);
  if (err != GA_NO_ERROR) return err;
  if (L.h.nf_total == 0) return GA_NO_ERROR;
  mr_plan(mr, &P, &L, &want, grid, block, ctx->num_sms);
  v = get_variant(mr, &want, &err);
  if (v == NULL) return err;
  if (L.h.splits > 1) {
    size_t cells = (size_t)L.h.splits * (size_t)L.h.nf_total;
    size_t nticket = want.shape == MR_COLS ? (size_t)L.h.units : (size_t)L.h.nf_total;
    err = ensure_scratch(mr, cells * 8, nticket * sizeof(unsigned int));
    if (err != GA_NO_ERROR) return err;
    p_val = mr->scratch->ptr;
    p_tic = mr->tickets->ptr;
  }
  /* the kernel's parameter block is the head followed by the two stride tables
   * of exactly `narray` rows each: a prefix of L */
  p_dst = out->data->ptr + out->offset;
  for (k = 0; k < mr->narray; k++) ptrs[k] = (CUdeviceptr)P.base[k];
  mr->params[p++] = &L;
  mr->params[p++] = &p_dst;
  mr->params[p++] = &p_val;
  mr->params[p++] = &p_tic;
  for (k = 0; k < mr->narray; k++) mr->params[p++] = &ptrs[k];
  for (i = 0; i < mr->n; i++)
    if (!is_array(&mr->args[i])) mr->params[p++] = args[i];
  return ga_launch(ctx, &v->fn, grid, block, 0, mr->params);
}

/* Test and tooling hook: what GpuMapReduction_call would decide for array
 * arguments given by rank, extents, byte strides and the address of their
 * first element, on a device with num_sms multiprocessors, without any device.
 * args[i] gives typecodes and GE_* flags (names may be NULL); the destination
 * is taken as C-contiguous with elements of out_tc. out[0..13] = kernel shape
 * (0 rows, 1 cols, 2 general), vector width, group, threads per output, access
 * modes (2 bits per array), splits, seg, nseg, units, grid x, grid y, block x,
 * block y, outputs. The parameter block the kernel would receive is copied
 * into `layout` (cap bytes available, *used = its size). */
GPUARRAY_PUBLIC int gpuarray_b200_mapreduction_plan(int out_tc, unsigned int n,
                                                    const gpuelemwise_arg *args,
                                                    const unsigned int *nds,
                                                    const size_t *const *dims,
                                                    const ssize_t *const *strides,
                                                    const unsigned long long *bases,
                                                    unsigned int reduxLen, const int *reduxList,
                                                    int call_flags, unsigned int num_sms,
                                                    unsigned long long *out, void *layout,
                                                    size_t cap, size_t *used) {
  GpuMapReduction mr;
  mr_arr arrs[MR_MAXARR];
  mr_problem P;
  mr_layout L;
  mr_variant want;
  unsigned char red[64];
  ssize_t ostr[64];
  unsigned grid[3], block[3], i, k, kd;
  size_t step, need;
  int err;
  memset(&mr, 0, sizeof(mr));
  mr.args = (gpuelemwise_arg *)args;
  mr.n = n;
  mr.out_tc = out_tc;
  mr.min_elsize = 16;
  mr.max_elsize = 1;
  for (i = 0, k = 0; i < n; i++) {
    size_t es = gpuarray_get_elsize(args[i].typecode);
    if (!is_array(&args[i])) continue;
    if (k == MR_MAXARR) return ga_err_set(ga_global_err, GA_UNSUPPORTED_ERROR, "Too many arrays");
    arrs[k].nd = nds[i];
    arrs[k].dims = dims[i];
    arrs[k].strides = strides[i];
    arrs[k].base = bases[i];
    if (es < mr.min_elsize) mr.min_elsize = (unsigned)es;
    if (es > mr.max_elsize) mr.max_elsize = (unsigned)es;
    k++;
  }
  mr.narray = k;
  if (k == 0) return ga_err_set(ga_global_err, GA_VALUE_ERROR, "No array argument");
  err = broadcast_shapes(&mr, ga_global_err, arrs, call_flags, &P);
  if (err != GA_NO_ERROR) return err;
  if (reduxLen == 0 || reduxLen > P.nd)
    return ga_err_set(ga_global_err, GA_VALUE_ERROR, "Bad number of reduction axes");
  memset(red, 0, sizeof(red));
  for (i = 0; i < reduxLen; i++) {
    if (reduxList[i] < 0 || (unsigned)reduxList[i] >= P.nd || red[reduxList[i]])
      return ga_err_set(ga_global_err, GA_INVALID_ERROR, "Bad reduction axis");
    red[reduxList[i]] = 1;
  }
  for (i = 0, kd = 0; i < P.nd; i++)
    if (!red[i]) kd++;
  step = gpuarray_get_elsize(out_tc);
  for (i = P.nd, k = kd; i > 0; i--) {
    if (red[i - 1]) continue;
    ostr[--k] = (ssize_t)step;
    step *= P.dims[i - 1];
  }
  err = normalise(&mr, ga_global_err, &P, ostr, red, &L);
  if (err != GA_NO_ERROR) return err;
  memset(out, 0, 14 * sizeof(*out));
  out[13] = L.h.nf_total;
  if (L.h.nf_total == 0) return GA_NO_ERROR;
  mr_plan(&mr, &P, &L, &want, grid, block, num_sms);
  out[0] = (unsigned long long)want.shape;
  out[1] = (unsigned long long)want.vec;
  out[2] = (unsigned long long)want.group;
  out[3] = (unsigned long long)want.tpo;
  out[4] = want.modes;
  out[5] = L.h.splits;
  out[6] = L.h.seg;
  out[7] = L.h.nseg;
  out[8] = L.h.units;
  out[9] = grid[0];
  out[10] = grid[1];
  out[11] = block[0];
  out[12] = block[1];
  need = sizeof(mr_head) + 2 * (size_t)mr.narray * MR_MAXD * sizeof(long long);
  if (layout != NULL) {
    if (cap < need) return ga_err_set(ga_global_err, GA_VALUE_ERROR, "Layout buffer too small");
    memcpy(layout, &L, need);
  }
  if (used != NULL) *used = need;
  return GA_NO_ERROR;
}
