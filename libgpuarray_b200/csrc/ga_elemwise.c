/* Elementwise engine: GpuElemwise_new / _call / _free.
 *
 * Host side of the path that the reference implements in
 * src/gpuarray_elemwise.c. The argument checking, broadcasting and collapsing
 * rules are the reference's (check_contig :547-576, check_basic :272-383);
 * what differs is everything after them:
 *   - kernels are instances of three hand-written sm_100a templates
 *     (templates/ga_ew_contig.cuh, ga_ew_strided.cuh, ga_ew_transpose.cuh)
 *     with the user's expression compiled in as an inlined function;
 *   - variants are built on first use and keyed by what actually changes the
 *     code (vector width, rank, index width, per-argument access mode), not
 *     one kernel per rank and address width built eagerly (:672-730);
 *   - device pointers are passed with the array offset already applied, and
 *     shape/stride data travels as one kernel parameter block, so a call is a
 *     single cuLaunchKernel.
 */
#include "private.h"

#define GA_EW_THREADS 256
#define GA_EW_MAX_ND 16

typedef struct ew_variant {
  int kind;              /* 0 contig, 1 strided, 2 transpose */
  int ept;
  int unroll;
  unsigned int nd;
  int idx32;             /* bit 0: 32-bit element indices; bit 1: 32-bit byte offsets too */
  unsigned long long modes; /* 2 bits per array */
  int tp, tq, pwi;       /* transpose: tile edges, P positions per thread */
  ga_function fn;
  struct ew_variant *next;
} ew_variant;

struct _GpuElemwise {
  gpucontext *ctx;
  char *expr;
  char *preamble;
  gpuelemwise_arg *args;
  unsigned int n;        /* arguments */
  unsigned int narray;
  int flags;
  int ept;               /* elements per thread-chunk giving 16-byte accesses */
  unsigned int min_elsize, max_elsize;
  ew_variant *variants;
  /* call-time scratch, sized for `nd_cap` dimensions */
  unsigned int nd_cap;
  size_t *dims;
  ssize_t **strides;     /* narray vectors */
  unsigned long long *blob;
  size_t blob_words;
  void **params;
  /* dry run (gpuarray_b200_elemwise_plan): choose, record, launch nothing */
  int dry;
  ew_variant dry_variant;
  unsigned dry_grid[3], dry_block[3];
};

static int is_array(const gpuelemwise_arg *a) { return ISCLR(a->flags, GE_SCALAR); }
static int is_output(const gpuelemwise_arg *a) { return ISSET(a->flags, GE_WRITE); }

/* Tuning knobs for experiments: GPUARRAY_B200_EW="unroll,gridcap_per_sm"
 * (unroll 0 = the default rule). */
static void ew_tuning(int *unroll, unsigned *gridcap_per_sm) {
  static int parsed = 0, t_unroll = 0;
  static unsigned t_cap = 0;
  if (!parsed) {
    const char *env = getenv("GPUARRAY_B200_EW");
    if (env != NULL) sscanf(env, "%d,%u", &t_unroll, &t_cap);
    if (t_unroll < 0 || t_unroll > 8) t_unroll = 0;
    parsed = 1;
  }
  *unroll = t_unroll;
  *gridcap_per_sm = t_cap;
}

/* Vectors a thread of the contiguous kernel has in flight. Measured on B200:
 * four for 4- and 8-byte elements; two when a vector holds 8 or 16 narrow
 * elements, whose unpacked values otherwise cost too many registers (uint8:
 * 43 us instead of 59 us for 2^27 elements; float16: 19.2 instead of 20.4). */
static int contig_unroll(const GpuElemwise *ge, int ept) {
  int u;
  unsigned cap;
  ew_tuning(&u, &cap);
  (void)ge;
  if (u > 0) return u;
  return ept >= 8 ? 2 : 4;
}

/* ---------------------------------------------------------------- codegen */

static const char *compute_type(const GpuElemwise *ge, const gpuelemwise_arg *a) {
  if (a->typecode == GA_HALF && ISSET(ge->flags, GE_CONVERT_F16)) return "ga_float";
  return ga_ctype(a->typecode);
}

/* Everything up to (not including) the #include of a template. */
static void gen_prologue(const GpuElemwise *ge, ga_strb *sb, const ew_variant *v) {
  unsigned int j, k;
  ga_strb_puts(sb, "#include \"cluda.h\"\n");
  {
    /* experiments: GPUARRAY_B200_EW_DEFINES="NAME=VALUE;NAME=VALUE" puts #define lines in
     * front of the template (its #ifndef defaults then stand back) */
    const char *extra = getenv("GPUARRAY_B200_EW_DEFINES");
    while (extra != NULL && *extra != '\0') {
      const char *end = strchr(extra, ';'), *eq;
      size_t len = end != NULL ? (size_t)(end - extra) : strlen(extra);
      eq = memchr(extra, '=', len);
      if (eq != NULL) {
        ga_strb_puts(sb, "#define ");
        ga_strb_putn(sb, extra, (size_t)(eq - extra));
        ga_strb_puts(sb, " ");
        ga_strb_putn(sb, eq + 1, len - (size_t)(eq - extra) - 1);
        ga_strb_puts(sb, "\n");
      }
      extra = end != NULL ? end + 1 : NULL;
    }
  }
  if (ge->preamble != NULL) ga_strb_puts(sb, ge->preamble);
  ga_strb_puts(sb, "\n#define GA_EW_ARRAYS(X)");
  for (j = 0, k = 0; j < ge->n; j++) {
    const gpuelemwise_arg *a = &ge->args[j];
    if (!is_array(a)) continue;
    ga_strb_printf(sb, " \\\n  X(%u, %s, %s, %s, %d, %d, %d)", k, a->name, ga_ctype(a->typecode),
                   compute_type(ge, a), ISSET(a->flags, GE_READ) ? 1 : 0, is_output(a) ? 1 : 0,
                   (int)((v->modes >> (2 * k)) & 3));
    k++;
  }
  ga_strb_puts(sb, "\n#define GA_EW_SCALARS(X)");
  for (j = 0; j < ge->n; j++) {
    const gpuelemwise_arg *a = &ge->args[j];
    if (is_array(a)) continue;
    ga_strb_printf(sb, " \\\n  X(%s, %s)", a->name, ga_ctype(a->typecode));
  }
  ga_strb_printf(sb,
                 "\n#define GA_EW_EPT %d\n#define GA_EW_UNROLL %d\n#define GA_EW_THREADS %d\n"
                 "#define GA_EW_IDX %s\n#define GA_EW_IDX32 %d\n#define GA_EW_OFF32 %d\n"
                 "#define GA_EW_ND %u\n#define GA_EW_NARR %u\n",
                 v->ept, v->unroll, GA_EW_THREADS, v->idx32 ? "unsigned int" : "size_t",
                 v->idx32 & 1, (v->idx32 >> 1) & 1, v->nd ? v->nd : 1,
                 ge->narray ? ge->narray : 1);
  if (v->kind == 2) /* unroll == 2 marks the cp.async + ldmatrix build of the tiled transpose */
    ga_strb_printf(sb, "#define GA_EW_TP %d\n#define GA_EW_TQ %d\n#define GA_EW_PWI %d\n"
                       "#define GA_EW_LDSM %d\n", v->tp, v->tq,
                   v->unroll == 2 ? 1 : (v->pwi > 0 ? v->pwi : 1), v->unroll == 2 ? 1 : 0);

  /* The expression sees each argument as a scalar variable of its own name. */
  ga_strb_puts(sb, "static __device__ __forceinline__ void ga_ew_apply(");
  for (j = 0; j < ge->n; j++) {
    const gpuelemwise_arg *a = &ge->args[j];
    if (is_array(a)) ga_strb_printf(sb, "%s &%s, ", compute_type(ge, a), a->name);
  }
  for (j = 0; j < ge->n; j++) {
    const gpuelemwise_arg *a = &ge->args[j];
    if (!is_array(a)) ga_strb_printf(sb, "%s %s, ", ga_ctype(a->typecode), a->name);
  }
  ga_strb_puts(sb, "int ga__unused) {\n");
  ga_strb_puts(sb, ge->expr);
  ga_strb_puts(sb, ";\n}\n");
}

static const char *const kind_header[] = {"ga_ew_contig.cuh", "ga_ew_strided.cuh",
                                          "ga_ew_transpose.cuh"};
static const char *const kind_entry[] = {"ga_ew_contig", "ga_ew_strided", "ga_ew_transpose"};

static char *gen_source(const GpuElemwise *ge, const ew_variant *v) {
  ga_strb sb;
  ga_strb_init(&sb);
  gen_prologue(ge, &sb, v);
  ga_strb_printf(&sb, "#include \"%s\"\n", kind_header[v->kind]);
  if (sb.failed) {
    ga_strb_free(&sb);
    return NULL;
  }
  return sb.s;
}

static ew_variant *get_variant(GpuElemwise *ge, const ew_variant *want, int *err) {
  ew_variant *v;
  char *src, *listing = NULL;
  if (ge->dry) {
    ge->dry_variant = *want;
    ge->dry_variant.next = NULL;
    return &ge->dry_variant;
  }
  for (v = ge->variants; v != NULL; v = v->next)
    if (v->kind == want->kind && v->ept == want->ept && v->unroll == want->unroll &&
        v->nd == want->nd && v->idx32 == want->idx32 && v->modes == want->modes &&
        v->tp == want->tp && v->tq == want->tq && v->pwi == want->pwi)
      return v;
  v = malloc(sizeof(*v));
  if (v == NULL) {
    *err = ga_err_sys(ge->ctx->err, "malloc");
    return NULL;
  }
  *v = *want;
  src = gen_source(ge, v);
  if (src == NULL) {
    free(v);
    *err = ga_err_set(ge->ctx->err, GA_MISC_ERROR, "Formatting error creating kernel source");
    return NULL;
  }
  *err = ga_compile(ge->ctx, src, kind_entry[v->kind], NULL, &v->fn,
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
  v->next = ge->variants;
  ge->variants = v;
  return v;
}

/* Test hook: the source that would be compiled for a given variant, without
 * touching a device. kind 0/1/2; modes packs 2 bits per array. Caller frees. */
GPUARRAY_PUBLIC char *gpuarray_b200_elemwise_source(const char *preamble, const char *expr,
                                                    unsigned int n, gpuelemwise_arg *args,
                                                    int flags, int kind, int ept, int unroll,
                                                    unsigned int nd, int idx32,
                                                    unsigned long long modes, int tp, int tq) {
  GpuElemwise ge;
  ew_variant v;
  unsigned int i;
  memset(&ge, 0, sizeof(ge));
  memset(&v, 0, sizeof(v));
  ge.expr = (char *)expr;
  ge.preamble = (char *)preamble;
  ge.args = args;
  ge.n = n;
  ge.flags = flags;
  for (i = 0; i < n; i++)
    if (is_array(&args[i])) ge.narray++;
  v.kind = kind;
  v.ept = ept;
  v.unroll = unroll;
  v.nd = nd;
  v.idx32 = idx32;
  v.modes = modes;
  v.tp = tp;
  v.tq = tq;
  v.pwi = 1;
  for (i = 0; i < n; i++) {
    size_t es = gpuarray_get_elsize(args[i].typecode);
    if (is_array(&args[i]) && es < 4 && (int)(4 / es) > v.pwi) v.pwi = (int)(4 / es);
  }
  return gen_source(&ge, &v);
}

/* ------------------------------------------------------------ construction */

static int grow_scratch(GpuElemwise *ge, unsigned int nd) {
  unsigned int i, cap = ge->nd_cap ? ge->nd_cap : 8;
  size_t *d;
  while (cap < nd) cap *= 2;
  if (cap == ge->nd_cap) return 0;
  d = realloc(ge->dims, cap * sizeof(size_t));
  if (d == NULL) return -1;
  ge->dims = d;
  for (i = 0; i < ge->narray; i++) {
    ssize_t *s = realloc(ge->strides[i], cap * sizeof(ssize_t));
    if (s == NULL) return -1;
    ge->strides[i] = s;
  }
  ge->nd_cap = cap;
  return 0;
}

GpuElemwise *GpuElemwise_new(gpucontext *ctx, const char *preamble, const char *expr,
                             unsigned int n, gpuelemwise_arg *args, unsigned int nd, int flags) {
  GpuElemwise *ge;
  unsigned int i;
  int err = GA_NO_ERROR;

  if (expr == NULL || (n > 0 && args == NULL)) {
    ga_err_set(ctx->err, GA_VALUE_ERROR, "GpuElemwise_new: NULL expression or arguments");
    return NULL;
  }
  ge = calloc(1, sizeof(*ge));
  if (ge == NULL) {
    ga_err_sys(ctx->err, "calloc");
    return NULL;
  }
  ge->ctx = ctx;
  ctx->refcnt++; /* the operator keeps its context alive */
  ge->flags = flags;
  ge->n = n;
  ge->expr = strdup(expr);
  if (preamble != NULL) ge->preamble = strdup(preamble);
  ge->args = calloc(n ? n : 1, sizeof(gpuelemwise_arg));
  if (ge->expr == NULL || (preamble != NULL && ge->preamble == NULL) || ge->args == NULL) {
    ga_err_sys(ctx->err, "strdup");
    goto fail;
  }
  ge->min_elsize = 16;
  ge->max_elsize = 1;
  for (i = 0; i < n; i++) {
    size_t es = gpuarray_get_elsize(args[i].typecode);
    if (args[i].name == NULL) {
      ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Argument %u has no name", i);
      goto fail;
    }
    if (!ga_type_is_computable(args[i].typecode)) {
      ga_err_fmt(ctx->err, GA_UNSUPPORTED_ERROR,
                 "Argument %u (%s): type %d is not supported (complex and 16-byte integer types "
                 "have no CUDA representation)", i, args[i].name, args[i].typecode);
      goto fail;
    }
    ge->args[i].typecode = args[i].typecode;
    ge->args[i].flags = args[i].flags;
    ge->args[i].name = strdup(args[i].name);
    if (ge->args[i].name == NULL) {
      ga_err_sys(ctx->err, "strdup");
      goto fail;
    }
    if (is_array(&args[i])) {
      ge->narray++;
      if (es < ge->min_elsize) ge->min_elsize = (unsigned)es;
      if (es > ge->max_elsize) ge->max_elsize = (unsigned)es;
    }
  }
  if (ge->narray > 30) {
    ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR, "More than 30 array arguments");
    goto fail;
  }
  if (ge->narray == 0) ge->min_elsize = ge->max_elsize = 4;
  /* 16 bytes for the narrowest argument, at most 64 for the widest */
  ge->ept = (int)(16 / ge->min_elsize);
  while (ge->ept > 1 && (unsigned)ge->ept * ge->max_elsize > 64) ge->ept /= 2;

  ge->strides = calloc(ge->narray ? ge->narray : 1, sizeof(ssize_t *));
  ge->params = calloc(n + 2, sizeof(void *));
  if (ge->strides == NULL || ge->params == NULL || grow_scratch(ge, nd > 8 ? nd : 8) != 0) {
    ga_err_sys(ctx->err, "calloc");
    goto fail;
  }

  /* Build the vectorised contiguous kernel now: it validates the expression,
   * so a bad one is reported here as in the reference (:672-688). */
  {
    ew_variant want;
    unsigned cap;
    memset(&want, 0, sizeof(want));
    want.kind = 0;
    want.ept = ge->ept;
    ew_tuning(&want.unroll, &cap);
    want.unroll = contig_unroll(ge, want.ept);
    want.idx32 = 1;
    if (get_variant(ge, &want, &err) == NULL) goto fail;
  }
  return ge;
fail:
  GpuElemwise_free(ge);
  return NULL;
}

void GpuElemwise_free(GpuElemwise *ge) {
  unsigned int i;
  ew_variant *v, *nv;
  if (ge == NULL) return;
  for (v = ge->variants; v != NULL; v = nv) {
    nv = v->next;
    free(v);
  }
  if (ge->strides != NULL)
    for (i = 0; i < ge->narray; i++) free(ge->strides[i]);
  if (ge->args != NULL)
    for (i = 0; i < ge->n; i++) free((void *)ge->args[i].name);
  free(ge->strides);
  free(ge->dims);
  free(ge->args);
  free(ge->params);
  free(ge->blob);
  free(ge->preamble);
  free(ge->expr);
  {
    gpucontext *ctx = ge->ctx;
    free(ge);
    if (ctx != NULL) ga_ctx_unref(ctx);
  }
}

/* ------------------------------------------------------------------- calls */

static CUdeviceptr array_base(const GpuArray *a) { return a->data->ptr + a->offset; }

static int ew_launch(GpuElemwise *ge, const ew_variant *v, const unsigned grid[3],
                     const unsigned block[3]) {
  if (ge->dry) {
    memcpy(ge->dry_grid, grid, sizeof(ge->dry_grid));
    memcpy(ge->dry_block, block, sizeof(ge->dry_block));
    return GA_NO_ERROR;
  }
  return ga_launch(ge->ctx, &v->fn, grid, block, 0, ge->params);
}

/* The contiguous fast path applies when every array has the same shape and
 * they are all C- or all F-contiguous (reference check_contig). Returns 1 and
 * the element count if so. */
static int check_contig(const GpuElemwise *ge, void **args, size_t *n_out) {
  const GpuArray *first = NULL, *v;
  unsigned int i, j;
  int c_ok = 1, f_ok = 1;
  size_t n = 1;
  for (i = 0; i < ge->n; i++) {
    if (!is_array(&ge->args[i])) continue;
    v = (const GpuArray *)args[i];
    if (first == NULL) {
      first = v;
      for (j = 0; j < v->nd; j++) n *= v->dimensions[j];
    } else {
      if (v->nd != first->nd) return 0;
      for (j = 0; j < v->nd; j++)
        if (v->dimensions[j] != first->dimensions[j]) return 0;
    }
    c_ok &= GpuArray_IS_C_CONTIGUOUS(v) != 0;
    f_ok &= GpuArray_IS_F_CONTIGUOUS(v) != 0;
  }
  if (first == NULL || !(c_ok || f_ok)) return 0;
  *n_out = n;
  return 1;
}

static int call_contig(GpuElemwise *ge, void **args, size_t n) {
  gpucontext *ctx = ge->ctx;
  ew_variant want, *v;
  CUdeviceptr ptrs[32];
  unsigned int i, k = 0, p = 0, capsm;
  unsigned grid[3] = {1, 1, 1}, block[3] = {GA_EW_THREADS, 1, 1};
  int err = GA_NO_ERROR, aligned = 1;
  size_t nvec, per_block, blocks;

  memset(&want, 0, sizeof(want));
  want.kind = 0;
  ew_tuning(&want.unroll, &capsm);
  for (i = 0; i < ge->n; i++) {
    if (!is_array(&ge->args[i])) continue;
    ptrs[k] = array_base((const GpuArray *)args[i]);
    if (ptrs[k] % 16 != 0) aligned = 0;
    k++;
  }
  want.ept = aligned ? ge->ept : 1;
  want.unroll = contig_unroll(ge, want.ept);
  want.idx32 = n < ((size_t)1 << 31);
  v = get_variant(ge, &want, &err);
  if (v == NULL) return err;

  ge->params[p++] = &n;
  for (i = 0, k = 0; i < ge->n; i++)
    if (is_array(&ge->args[i])) ge->params[p++] = &ptrs[k++];
  for (i = 0; i < ge->n; i++)
    if (!is_array(&ge->args[i])) ge->params[p++] = args[i];

  nvec = n / (size_t)v->ept;
  per_block = (size_t)GA_EW_THREADS * (size_t)v->unroll;
  blocks = (nvec + per_block - 1) / per_block;
  if (blocks == 0) blocks = 1;
  if (capsm != 0 && blocks > (size_t)capsm * ctx->num_sms) blocks = (size_t)capsm * ctx->num_sms;
  if (blocks > 0x7fffffffu) blocks = 0x7fffffffu;
  grid[0] = (unsigned)blocks;
  return ew_launch(ge, v, grid, block);
}

static void make_div32(unsigned int d, unsigned int out[4]) {
  unsigned int l = 0;
  unsigned long long m;
  while (l < 32 && ((unsigned long long)1 << l) < d) l++;
  m = ((((unsigned long long)1 << l) - d) << 32) / d + 1;
  out[0] = d;
  out[1] = (unsigned int)m;
  out[2] = l < 1 ? l : 1;
  out[3] = l > 0 ? l - 1 : 0;
}

/* Shape agreement, broadcasting and collapsing (reference check_basic). On
 * success ge->dims / ge->strides hold the collapsed problem. */
static int check_basic(GpuElemwise *ge, void **args, int flags, size_t *n_out,
                       unsigned int *nd_out) {
  gpucontext *ctx = ge->ctx;
  const GpuArray *shape_src = NULL, *v;
  unsigned int i, j, p, nd = 0, seen = 0;
  size_t n = 1;

  for (i = 0; i < ge->n; i++) {
    if (!is_array(&ge->args[i])) continue;
    v = (const GpuArray *)args[i];
    if (seen == 0) nd = v->nd;
    else if (v->nd != nd) {
      if (ISCLR(flags, GE_PADSHAPE))
        return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Arg %u has differing nd = %u", i, v->nd);
      if (v->nd > nd) nd = v->nd;
    }
    seen++;
    if (shape_src == NULL && is_output(&ge->args[i])) shape_src = v;
  }
  if (shape_src == NULL) return ga_err_set(ctx->err, GA_VALUE_ERROR, "No output arrays");
  if (nd > ge->nd_cap && grow_scratch(ge, nd) != 0) return ga_err_sys(ctx->err, "realloc");
  if (shape_src->nd != nd) {
    /* an output of lower rank would have to broadcast */
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                      "Output has nd = %u but the operation has nd = %u", shape_src->nd, nd);
  }
  memcpy(ge->dims, shape_src->dimensions, nd * sizeof(size_t));

  for (i = 0, p = 0; i < ge->n; i++) {
    unsigned int pad;
    if (!is_array(&ge->args[i])) continue;
    v = (const GpuArray *)args[i];
    pad = nd - v->nd;
    for (j = 0; j < nd; j++) {
      size_t vd = j < pad ? 1 : v->dimensions[j - pad];
      ssize_t vs = j < pad ? 0 : v->strides[j - pad];
      if (vd != ge->dims[j] &&
          (ISCLR(flags, GE_BROADCAST) || is_output(&ge->args[i]) || vd != 1))
        return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                          "Mismatched dimension %u for input %u (expected %zu got %zu)", j, i,
                          ge->dims[j], vd);
      ge->strides[p][j] = vd == 1 ? 0 : vs;
    }
    p++;
  }
  for (j = 0; j < nd; j++) n *= ge->dims[j];
  if (nd > 1) gpuarray_elemwise_collapse(ge->narray, &nd, ge->dims, ge->strides);
  *n_out = n;
  *nd_out = nd;
  return GA_NO_ERROR;
}

static int ensure_blob(GpuElemwise *ge, size_t words) {
  if (words > ge->blob_words) {
    unsigned long long *b = realloc(ge->blob, words * sizeof(*b));
    if (b == NULL) return -1;
    ge->blob = b;
    ge->blob_words = words;
  }
  return 0;
}

static int call_transpose(GpuElemwise *ge, void **args, size_t n, unsigned int nd, int *handled);

static int call_strided(GpuElemwise *ge, void **args, size_t n, unsigned int nd) {
  gpucontext *ctx = ge->ctx;
  ew_variant want, *v;
  CUdeviceptr ptrs[32];
  unsigned int i, j, k, p = 0, nout, capsm;
  unsigned grid[3] = {1, 1, 1}, block[3] = {GA_EW_THREADS, 1, 1};
  int err = GA_NO_ERROR, handled = 0;
  size_t inner, cpr, rows, nchunks, words, blocks;
  unsigned long long *w;

  if (nd == 0) return ga_err_set(ctx->err, GA_VALUE_ERROR, "nd == 0");
  if (nd > GA_EW_MAX_ND)
    return ga_err_fmt(ctx->err, GA_UNSUPPORTED_ERROR,
                      "%u dimensions remain after collapsing; at most %d are supported", nd,
                      GA_EW_MAX_ND);

  err = call_transpose(ge, args, n, nd, &handled);
  if (handled) return err;

  memset(&want, 0, sizeof(want));
  want.kind = 1;
  want.nd = nd;
  want.ept = ge->ept;
  want.unroll = 1;
  ew_tuning(&want.unroll, &capsm);
  want.unroll = 1;
  inner = ge->dims[nd - 1];
  cpr = (inner + (size_t)want.ept - 1) / (size_t)want.ept;
  rows = n / inner;
  nchunks = rows * cpr;
  want.idx32 = n < ((size_t)1 << 31) && nchunks < ((size_t)1 << 31);

  for (i = 0, k = 0; i < ge->n; i++) {
    const gpuelemwise_arg *a = &ge->args[i];
    size_t es, vb;
    ssize_t is;
    unsigned long long mode = 0;
    if (!is_array(a)) continue;
    ptrs[k] = array_base((const GpuArray *)args[i]);
    es = gpuarray_get_elsize(a->typecode);
    vb = es * (size_t)want.ept;
    if (vb > 16) vb = 16;
    is = ge->strides[k][nd - 1];
    if (is == 0 && !is_output(a)) mode = 2;
    else if (is == (ssize_t)es && inner % (size_t)want.ept == 0 && ptrs[k] % vb == 0) {
      mode = 1;
      for (j = 0; j + 1 < nd; j++)
        if (ge->strides[k][j] % (ssize_t)vb != 0) mode = 0;
    }
    want.modes |= mode << (2 * k);
    k++;
  }
  if (want.idx32) {
    /* 32-bit byte offsets when no argument spans 2 GiB */
    int small = 1;
    for (k = 0; k < ge->narray && small; k++) {
      unsigned long long span = 64;
      for (j = 0; j < nd; j++) {
        ssize_t st = ge->strides[k][j];
        span += (unsigned long long)(ge->dims[j] - 1) * (unsigned long long)(st < 0 ? -st : st);
      }
      if (span >= 0x7fffffffULL) small = 0;
    }
    if (small) want.idx32 |= 2;
  }
  v = get_variant(ge, &want, &err);
  if (v == NULL) return err;

  /* parameter block: see struct ga__ew_layout in ga_ew_strided.cuh */
  nout = nd > 1 ? nd - 1 : 1;
  words = 3 + nout + 2 + 2 * nout + (size_t)(ge->narray ? ge->narray : 1) * nd;
  if (ensure_blob(ge, words) != 0) return ga_err_sys(ctx->err, "realloc");
  w = ge->blob;
  memset(w, 0, words * sizeof(*w));
  w[0] = nchunks;
  w[1] = inner;
  w[2] = cpr;
  for (j = 0; j + 1 < nd; j++) w[3 + j] = ge->dims[j];
  if (want.idx32) {
    make_div32((unsigned)cpr, (unsigned int *)&w[3 + nout]);
    for (j = 0; j + 1 < nd; j++)
      make_div32((unsigned)ge->dims[j], (unsigned int *)&w[3 + nout + 2 + 2 * j]);
  }
  for (k = 0; k < ge->narray; k++)
    for (j = 0; j < nd; j++)
      w[3 + nout + 2 + 2 * nout + (size_t)k * nd + j] = (unsigned long long)(long long)ge->strides[k][j];

  ge->params[p++] = w;
  for (i = 0, k = 0; i < ge->n; i++)
    if (is_array(&ge->args[i])) ge->params[p++] = &ptrs[k++];
  for (i = 0; i < ge->n; i++)
    if (!is_array(&ge->args[i])) ge->params[p++] = args[i];

  blocks = (nchunks + GA_EW_THREADS - 1) / GA_EW_THREADS;
  if (blocks == 0) blocks = 1;
  /* measured on B200: CTAs that handle a single chunk per thread are bound by
   * the CTA launch rate when the kernel mostly writes (broadcast of two small
   * inputs into 134 MB: 35 us uncapped, 21-22 us at 16-32 CTAs per SM) */
  if (capsm == 0) capsm = 32;
  if (blocks > (size_t)capsm * ctx->num_sms) blocks = (size_t)capsm * ctx->num_sms;
  if (blocks > 0x7fffffffu) blocks = 0x7fffffffu;
  grid[0] = (unsigned)blocks;
  return ew_launch(ge, v, grid, block);
}

/* Tiled transpose: taken when some pure input is contiguous along a dimension
 * P other than the innermost one (Q) and would otherwise be gathered element
 * by element. Sets *handled when the call was dispatched here. */
static int call_transpose(GpuElemwise *ge, void **args, size_t n, unsigned int nd, int *handled) {
  gpucontext *ctx = ge->ctx;
  ew_variant want, *v;
  CUdeviceptr ptrs[32];
  unsigned int i, j, k, p = 0, q = nd - 1, pdim_ax = nd, nout, best_votes = 0;
  unsigned grid[3] = {1, 1, 1}, block[3] = {GA_EW_THREADS, 1, 1};
  unsigned long long *w, tiles_p, tiles_q, nouter, ntiles;
  size_t words, smem = 0;
  int err = GA_NO_ERROR, tile;
  (void)n;

  *handled = 0;
  if (nd < 2 || getenv("GPUARRAY_B200_NO_TRANSPOSE") != NULL) return GA_NO_ERROR;
  /* vote for the dimension along which gathered inputs are contiguous */
  for (j = 0; j + 1 < nd; j++) {
    unsigned votes = 0;
    for (i = 0, k = 0; i < ge->n; i++) {
      const gpuelemwise_arg *a = &ge->args[i];
      ssize_t es;
      if (!is_array(a)) continue;
      es = (ssize_t)gpuarray_get_elsize(a->typecode);
      if (!is_output(a) && ge->strides[k][j] == es && ge->strides[k][q] != es &&
          ge->strides[k][q] != 0)
        votes++;
      k++;
    }
    if (votes > best_votes) {
      best_votes = votes;
      pdim_ax = j;
    }
  }
  if (best_votes == 0 || ge->dims[pdim_ax] < 16 || ge->dims[q] < 16) return GA_NO_ERROR;

  memset(&want, 0, sizeof(want));
  want.kind = 2;
  want.nd = nd;
  want.ept = ge->ept;
  want.unroll = 1;
  want.idx32 = 0;
  for (i = 0, k = 0; i < ge->n; i++) {
    const gpuelemwise_arg *a = &ge->args[i];
    size_t es, vb;
    ssize_t sq, sp;
    unsigned long long mode = 0;
    if (!is_array(a)) continue;
    ptrs[k] = array_base((const GpuArray *)args[i]);
    es = gpuarray_get_elsize(a->typecode);
    vb = es * (size_t)want.ept > 16 ? 16 : es * (size_t)want.ept;
    sq = ge->strides[k][q];
    sp = ge->strides[k][pdim_ax];
    if (!is_output(a) && sp == (ssize_t)es && sq != (ssize_t)es && sq != 0) mode = 3;
    else if (sq == 0 && !is_output(a)) mode = 2;
    else if (sq == (ssize_t)es && ge->dims[q] % (size_t)want.ept == 0 && ptrs[k] % vb == 0) {
      mode = 1;
      for (j = 0; j + 1 < nd; j++)
        if (ge->strides[k][j] % (ssize_t)vb != 0) mode = 0;
    }
    want.modes |= mode << (2 * k);
    k++;
  }
  /* P positions per thread: one 32-bit shared-memory word of the narrowest
   * staged type */
  want.pwi = 1;
  for (i = 0, k = 0; i < ge->n; i++) {
    if (!is_array(&ge->args[i])) continue;
    if (((want.modes >> (2 * k)) & 3) == 3) {
      size_t es = gpuarray_get_elsize(ge->args[i].typecode);
      if (es < 4 && (int)(4 / es) > want.pwi) want.pwi = (int)(4 / es);
    }
    k++;
  }
  /* Tile: as wide along P as the contiguous extent allows (up to 256), so
   * the staged reads are long contiguous bursts; 64 along Q; shrink until the
   * staged tiles fit the 48 KiB of static shared memory. */
  {
    int tp = 32, tq = 64, tpmax = 256, ldsm = want.ept == 8 && getenv("GPUARRAY_B200_NO_LDSM") == NULL;
    /* measured on B200: 256 x 64 for 2-byte staged elements (cfg4: 35.8 us,
     * 128 x 64: 38.3); 128 x 32 for 4 bytes and more (fp32 8192 x 4096
     * transpose: 49.0 us, 128 x 64: 53.2) */
    for (i = 0, k = 0; i < ge->n; i++) {
      if (!is_array(&ge->args[i])) continue;
      if (((want.modes >> (2 * k)) & 3) == 3) {
        if (gpuarray_get_elsize(ge->args[i].typecode) >= 4) {
          tpmax = 128;
          tq = 32;
        }
        if (gpuarray_get_elsize(ge->args[i].typecode) != 2) ldsm = 0;
      }
      k++;
    }
    if (tq < want.ept) tq = want.ept;
    while (tp < tpmax && (size_t)tp < ge->dims[pdim_ax]) tp *= 2;
    /* Every staged input has 2-byte elements: asynchronous 16-byte copies into swizzled
     * rows and transposing matrix loads (ga_ew_transpose.cuh, GA_EW_LDSM). Tiles of
     * 256 x 32: measured on B200 (cfg4, one tile per CTA) 32.4 us against 33.1 us for
     * 256 x 64, and 36.1 us for the word-staged build. */
    if (ldsm && tp >= 64) {
      tq = 32;
      want.unroll = 2;
      want.pwi = 1;
    }
    for (;;) {
      smem = 0;
      for (i = 0, k = 0; i < ge->n; i++) {
        if (!is_array(&ge->args[i])) continue;
        if (((want.modes >> (2 * k)) & 3) == 3) {
          size_t es = gpuarray_get_elsize(ge->args[i].typecode);
          size_t wsz = es > 4 ? 8 : 4, pw = es < 4 ? 4 / es : 1;
          smem += want.unroll == 2 ? (size_t)tq * (size_t)tp * 2
                                   : (size_t)tq * ((size_t)tp / pw + 1) * wsz;
        }
        k++;
      }
      if (smem <= 40 * 1024) break;
      if (tp > (want.unroll == 2 ? 64 : 32)) tp /= 2;
      else if (tq > 32) tq /= 2;
      else break;
    }
    tile = smem <= 46 * 1024 ? 64 : 0;
    want.tp = tp;
    want.tq = tq;
  }
  if (tile == 0 || want.tq % want.ept != 0 || want.tp % want.pwi != 0) return GA_NO_ERROR;
  {
    /* experiment knob: GPUARRAY_B200_EWT="tp,tq" (tq a multiple of the chunk) */
    const char *env = getenv("GPUARRAY_B200_EWT");
    int etp = 0, etq = 0;
    if (env != NULL && sscanf(env, "%d,%d", &etp, &etq) == 2 && etp >= 8 && etq >= want.ept &&
        etq % want.ept == 0 && (want.unroll != 2 || (etp % 64 == 0 && etq % 32 == 0))) {
      want.tp = etp;
      want.tq = etq;
    }
  }
  v = get_variant(ge, &want, &err);
  *handled = 1;
  if (v == NULL) return err;

  nout = nd > 2 ? nd - 2 : 1;
  words = 5 + nout + 2 * (size_t)ge->narray + (size_t)ge->narray * nout;
  if (ensure_blob(ge, words) != 0) return ga_err_sys(ctx->err, "realloc");
  w = ge->blob;
  memset(w, 0, words * sizeof(*w));
  tiles_p = (ge->dims[pdim_ax] + (size_t)want.tp - 1) / (size_t)want.tp;
  tiles_q = (ge->dims[q] + (size_t)want.tq - 1) / (size_t)want.tq;
  nouter = 1;
  for (j = 0, k = 0; j < nd; j++) {
    if (j == pdim_ax || j == q) continue;
    w[5 + k++] = ge->dims[j];
    nouter *= ge->dims[j];
  }
  w[0] = ge->dims[pdim_ax];
  w[1] = ge->dims[q];
  w[2] = tiles_p;
  w[3] = tiles_q;
  w[4] = nouter;
  for (k = 0; k < ge->narray; k++) {
    unsigned int oi = 0;
    w[5 + nout + k] = (unsigned long long)(long long)ge->strides[k][pdim_ax];
    w[5 + nout + ge->narray + k] = (unsigned long long)(long long)ge->strides[k][q];
    for (j = 0; j < nd; j++) {
      if (j == pdim_ax || j == q) continue;
      w[5 + nout + 2 * (size_t)ge->narray + (size_t)k * nout + oi++] =
          (unsigned long long)(long long)ge->strides[k][j];
    }
  }
  ge->params[p++] = w;
  for (i = 0, k = 0; i < ge->n; i++)
    if (is_array(&ge->args[i])) ge->params[p++] = &ptrs[k++];
  for (i = 0; i < ge->n; i++)
    if (!is_array(&ge->args[i])) ge->params[p++] = args[i];
  ntiles = tiles_p * tiles_q * nouter;
  grid[0] = ntiles > 0x7fffffffULL ? 0x7fffffffu : (unsigned)ntiles;
  return ew_launch(ge, v, grid, block);
}

/* Test and tooling hook: the shape work of GpuElemwise_call (contiguous fast
 * path test, rank padding, broadcast, output-defines-shape, dimension
 * collapsing) on plain shape / byte-stride lists, without any device.
 *   n            number of arguments; args[i] gives typecode and GE_* flags
 *   nds[i], dims[i], strides[i]   rank, extents, byte strides of array i
 *                (ignored for GE_SCALAR arguments)
 * Returns the GA_* code the call would return up to this point. out[0] = path
 * (0 contiguous kernel, 1 strided/transposing kernels), out[1] = element count,
 * out[2] = rank after collapsing (1 for the contiguous path), then that many
 * collapsed extents, then per array argument that many collapsed byte strides
 * (strided path only). `out` must hold 3 + 8 + 8 * n words. */
GPUARRAY_PUBLIC int gpuarray_b200_elemwise_shapes(unsigned int n, const gpuelemwise_arg *args,
                                                  const unsigned int *nds,
                                                  const size_t *const *dims,
                                                  const ssize_t *const *strides, int call_flags,
                                                  long long *out) {
  struct _gpucontext fake;
  GpuElemwise ge;
  GpuArray arrs[32];
  void *ptrs[32];
  unsigned int i, j, k, nd = 0;
  size_t cnt = 0;
  int err;
  if (n > 32) return ga_err_set(ga_global_err, GA_UNSUPPORTED_ERROR, "More than 32 arguments");
  memset(&fake, 0, sizeof(fake));
  fake.err = ga_global_err;
  memset(&ge, 0, sizeof(ge));
  ge.ctx = &fake;
  ge.args = (gpuelemwise_arg *)args;
  ge.n = n;
  for (i = 0; i < n; i++) {
    ptrs[i] = &arrs[i];
    if (!is_array(&args[i])) continue;
    ge.narray++;
    memset(&arrs[i], 0, sizeof(arrs[i]));
    arrs[i].nd = nds[i];
    arrs[i].dimensions = (size_t *)dims[i];
    arrs[i].strides = (ssize_t *)strides[i];
    arrs[i].typecode = args[i].typecode;
    arrs[i].flags = GA_ALIGNED | GA_WRITEABLE;
    GpuArray_fix_flags(&arrs[i]);
  }
  ge.strides = calloc(ge.narray ? ge.narray : 1, sizeof(ssize_t *));
  if (ge.strides == NULL || grow_scratch(&ge, 8) != 0) {
    err = ga_err_sys(ga_global_err, "calloc");
    goto done;
  }
  if (check_contig(&ge, ptrs, &cnt)) {
    out[0] = 0;
    out[1] = (long long)cnt;
    out[2] = 1;
    out[3] = (long long)cnt;
    err = GA_NO_ERROR;
    goto done;
  }
  err = check_basic(&ge, ptrs, call_flags, &cnt, &nd);
  if (err != GA_NO_ERROR) goto done;
  if (nd > 8) {
    err = ga_err_set(ga_global_err, GA_UNSUPPORTED_ERROR, "More than 8 dimensions remain");
    goto done;
  }
  out[0] = 1;
  out[1] = (long long)cnt;
  out[2] = (long long)nd;
  for (j = 0; j < nd; j++) out[3 + j] = (long long)ge.dims[j];
  for (k = 0; k < ge.narray; k++)
    for (j = 0; j < nd; j++) out[3 + nd + k * nd + j] = (long long)ge.strides[k][j];
done:
  if (ge.strides != NULL)
    for (k = 0; k < ge.narray; k++) free(ge.strides[k]);
  free(ge.strides);
  free(ge.dims);
  return err;
}

/* Test and tooling hook: everything GpuElemwise_call decides for a call -
 * kernel, widths, per-argument access modes, tile, launch geometry - computed
 * on the host alone for arrays described by rank, extents, byte strides and the
 * address of their first element (alignment only; nothing is dereferenced).
 * obj_flags are the GpuElemwise_new flags (GE_CONVERT_F16 ...), call_flags the
 * GpuElemwise_call flags. out[0..15] = kernel (0 contiguous, 1 strided, 2
 * tiled transpose), elements per thread chunk, chunks in flight, rank after
 * collapsing, index width bits (1: 32-bit indices, 2: 32-bit row offsets),
 * access modes (2 bits per array: 0 gather, 1 vector, 2 broadcast, 3 staged
 * through shared memory), tile P, tile Q, P positions per thread, grid x/y/z,
 * block x/y/z, element count. blob_out (may be NULL) receives the layout
 * parameter block of the strided / transposing kernels, *blob_words its length
 * in 8-byte words. */
GPUARRAY_PUBLIC int gpuarray_b200_elemwise_plan(unsigned int n, const gpuelemwise_arg *args,
                                                const unsigned int *nds,
                                                const size_t *const *dims,
                                                const ssize_t *const *strides,
                                                const unsigned long long *bases, int obj_flags,
                                                int call_flags, unsigned int num_sms,
                                                unsigned long long *out,
                                                unsigned long long *blob_out, size_t blob_cap,
                                                size_t *blob_words) {
  struct _gpucontext fake;
  struct _gpudata bufs[32];
  GpuElemwise ge;
  GpuArray arrs[32];
  void *ptrs[32];
  unsigned int i, k, nd = 0;
  size_t cnt = 0;
  int err;
  if (n > 32) return ga_err_set(ga_global_err, GA_UNSUPPORTED_ERROR, "More than 32 arguments");
  memset(&fake, 0, sizeof(fake));
  fake.err = ga_global_err;
  fake.num_sms = num_sms;
  memset(&ge, 0, sizeof(ge));
  ge.ctx = &fake;
  ge.args = (gpuelemwise_arg *)args;
  ge.n = n;
  ge.flags = obj_flags;
  ge.dry = 1;
  ge.min_elsize = 16;
  ge.max_elsize = 1;
  for (i = 0; i < n; i++) {
    size_t es = gpuarray_get_elsize(args[i].typecode);
    ptrs[i] = &arrs[i];
    if (!is_array(&args[i])) continue;
    ge.narray++;
    if (es < ge.min_elsize) ge.min_elsize = (unsigned)es;
    if (es > ge.max_elsize) ge.max_elsize = (unsigned)es;
    memset(&bufs[i], 0, sizeof(bufs[i]));
    bufs[i].ptr = (CUdeviceptr)bases[i];
    bufs[i].ctx = &fake;
    bufs[i].sz = bufs[i].asz = (size_t)-1;
    bufs[i].refcnt = 1;
    memset(&arrs[i], 0, sizeof(arrs[i]));
    arrs[i].data = &bufs[i];
    arrs[i].nd = nds[i];
    arrs[i].dimensions = (size_t *)dims[i];
    arrs[i].strides = (ssize_t *)strides[i];
    arrs[i].typecode = args[i].typecode;
    arrs[i].flags = GA_ALIGNED | GA_WRITEABLE;
    GpuArray_fix_flags(&arrs[i]);
  }
  if (ge.narray == 0) ge.min_elsize = ge.max_elsize = 4;
  ge.ept = (int)(16 / ge.min_elsize);
  while (ge.ept > 1 && (unsigned)ge.ept * ge.max_elsize > 64) ge.ept /= 2;
  ge.strides = calloc(ge.narray ? ge.narray : 1, sizeof(ssize_t *));
  ge.params = calloc(n + 2, sizeof(void *));
  if (ge.strides == NULL || ge.params == NULL || grow_scratch(&ge, 8) != 0) {
    err = ga_err_sys(ga_global_err, "calloc");
    goto done;
  }
  if (check_contig(&ge, ptrs, &cnt)) {
    err = cnt == 0 ? GA_NO_ERROR : call_contig(&ge, ptrs, cnt);
  } else {
    err = check_basic(&ge, ptrs, call_flags, &cnt, &nd);
    if (err == GA_NO_ERROR && cnt != 0) err = call_strided(&ge, ptrs, cnt, nd);
  }
  if (err != GA_NO_ERROR) goto done;
  memset(out, 0, 16 * sizeof(*out));
  out[15] = cnt;
  if (cnt != 0) {
    const ew_variant *v = &ge.dry_variant;
    out[0] = (unsigned long long)v->kind;
    out[1] = (unsigned long long)v->ept;
    out[2] = (unsigned long long)v->unroll;
    out[3] = v->nd;
    out[4] = (unsigned long long)v->idx32;
    out[5] = v->modes;
    out[6] = (unsigned long long)v->tp;
    out[7] = (unsigned long long)v->tq;
    out[8] = (unsigned long long)v->pwi;
    for (k = 0; k < 3; k++) {
      out[9 + k] = ge.dry_grid[k];
      out[12 + k] = ge.dry_block[k];
    }
    /* the layout parameter block of the strided / transposing kernels */
    if (blob_words != NULL) *blob_words = v->kind == 0 ? 0 : ge.blob_words;
    if (blob_out != NULL && v->kind != 0) {
      if (ge.blob_words > blob_cap) {
        err = ga_err_set(ga_global_err, GA_VALUE_ERROR, "Layout buffer too small");
        goto done;
      }
      memcpy(blob_out, ge.blob, ge.blob_words * sizeof(*blob_out));
    }
  }
done:
  if (ge.strides != NULL)
    for (k = 0; k < ge.narray; k++) free(ge.strides[k]);
  free(ge.strides);
  free(ge.dims);
  free(ge.params);
  free(ge.blob);
  return err;
}

int GpuElemwise_call(GpuElemwise *ge, void **args, int flags) {
  gpucontext *ctx = ge->ctx;
  size_t n = 0;
  unsigned int nd = 0, i;
  int err;

  for (i = 0; i < ge->n; i++) {
    if (args[i] == NULL) return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Argument %u is NULL", i);
    if (is_array(&ge->args[i])) {
      const GpuArray *a = (const GpuArray *)args[i];
      if (a->typecode != ge->args[i].typecode)
        return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                          "Argument %u (%s) has type %d but the operation was built for %d", i,
                          ge->args[i].name, a->typecode, ge->args[i].typecode);
      if (GpuArray_context(a) != ctx)
        return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Argument %u belongs to another context", i);
      if (!GpuArray_ISALIGNED(a))
        return ga_err_fmt(ctx->err, GA_UNALIGNED_ERROR, "Argument %u is not aligned", i);
      if (is_output(&ge->args[i]) && !GpuArray_ISWRITEABLE(a))
        return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Output argument %u is not writeable", i);
      if (!ga_array_in_bounds(a))
        return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                          "Argument %u (%s) reaches outside its buffer", i, ge->args[i].name);
    }
  }
  if (check_contig(ge, args, &n)) {
    if (n == 0) return GA_NO_ERROR;
    return call_contig(ge, args, n);
  }
  err = check_basic(ge, args, flags, &n, &nd);
  if (err != GA_NO_ERROR) return err;
  if (n == 0) return GA_NO_ERROR;
  return call_strided(ge, args, n, nd);
}
