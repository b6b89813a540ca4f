/* Reduction engine: GpuReduction_new / _call / _free and GpuArray_maxandargmax.
 *
 * Host side of what the reference does in src/gpuarray_reduction.c (argument
 * checks :198-261, axis bookkeeping :268-295 and :616-626, launch-shape search
 * :673-776, five device allocations per call :782-834) and, for sum / prod /
 * all / any, in pygpu/reduction.py:137-319. Differences:
 *   - the axes are first normalised: size-1 axes vanish, kept axes and reduced
 *     axes are collapsed separately (a kept pair merges only if source and both
 *     destinations agree; a reduced pair only if memory order and flat-index
 *     weight agree), and reduced axes are traversed in MEMORY order while every
 *     element carries its flat index in reduxList order, so any axis list gets
 *     coalesced traffic and the reference's index/tie semantics;
 *   - one of three fixed kernel shapes (templates/ga_reduce.cuh) is picked from
 *     the normalised strides instead of solving for a launch factorisation;
 *   - shapes, strides and weights travel in one kernel parameter block: no
 *     allocation or host-to-device copy per call. The only device scratch is
 *     the partial buffer of two-pass reductions, kept by the operator object.
 */
#include "private.h"

#define RD_MAXD 8
#define RD_THREADS 256
#define RD_BY 8

enum { SHAPE_ROWS = 0, SHAPE_COLS = 1, SHAPE_GENERAL = 2 };

typedef struct rd_variant {
  int shape, vec, idx64, tpo, dst_tc, write_val, write_idx, group, flat, mu, onerun, fast8, lazy;
  int simple; /* rows: lean one-run-per-warp loop */
  int tiny;   /* rows: runs of 1-8 vectors back to back, walked as one flat array of vectors */
  int by;     /* cols: row lanes per CTA (0 = RD_BY) */
  int ctas_per_sm; /* CTAs of RD_THREADS threads the compiled kernel fits on an SM */
  ga_function fn;
  struct rd_variant *next;
} rd_variant;

struct _GpuReduction {
  gpucontext *ctx;
  ga_reduce_op op;
  int src_tc;
  int kind;              /* 0 accumulate, 1 (value, index) pairs */
  rd_variant *variants;
  gpudata *scratch;      /* partial results of split reductions */
  size_t scratch_sz;
  gpudata *tickets;      /* arrival counters, zero between launches */
  size_t tickets_sz;
  /* helpers of sharded (value, index) calls, built on first use */
  GpuReduction *sh_pair; /* MIN/MAXANDARG* operator that produces the local pair */
  GpuElemwise *sh_e1, *sh_e2, *sh_e3;
  int sh_e3_key;         /* (has value << 8) | (has index << 9) | index typecode of sh_e3 */
};

/* Normalised problem; field order matches struct ga__rd_layout. */
typedef struct rd_layout {
  unsigned long long nf_total, nr_total, nf, nr;
  unsigned long long fdim[RD_MAXD];
  long long fsrc[RD_MAXD], fdst0[RD_MAXD], fdst1[RD_MAXD];
  unsigned long long rdim[RD_MAXD];
  long long rsrc[RD_MAXD];
  unsigned long long rmul[RD_MAXD];
  unsigned long long splits, inner, seg, nseg, units, tiles;
  unsigned int dv[4];
  unsigned long long ioff, early, nan_first;
} rd_layout;

/* One reduced axis of the source is a shard of a longer axis held by several
 * GPUs: this rank's slab starts at coordinate `lo` of `global` along it. */
typedef struct rd_shard {
  int axis;
  unsigned long long lo, global;
} rd_shard;

static int op_is_pair(ga_reduce_op op) {
  return op == GA_REDUCE_MIN || op == GA_REDUCE_MAX || op == GA_REDUCE_ARGMIN ||
         op == GA_REDUCE_ARGMAX || op == GA_REDUCE_MINANDARGMIN || op == GA_REDUCE_MAXANDARGMAX;
}
static int op_is_min(ga_reduce_op op) {
  return op == GA_REDUCE_MIN || op == GA_REDUCE_ARGMIN || op == GA_REDUCE_MINANDARGMIN;
}
static int op_writes_val(ga_reduce_op op) {
  return op != GA_REDUCE_ARGMIN && op != GA_REDUCE_ARGMAX;
}
static int op_writes_idx(ga_reduce_op op) {
  return op == GA_REDUCE_ARGMIN || op == GA_REDUCE_ARGMAX || op == GA_REDUCE_MINANDARGMIN ||
         op == GA_REDUCE_MAXANDARGMAX;
}
static int tc_is_float(int tc) { return tc == GA_FLOAT || tc == GA_DOUBLE || tc == GA_HALF; }
static int tc_is_unsigned(int tc) {
  return tc == GA_BOOL || tc == GA_UBYTE || tc == GA_USHORT || tc == GA_UINT || tc == GA_ULONG ||
         tc == GA_SIZE;
}
static int tc_is_index(int tc) {
  return tc == GA_LONG || tc == GA_ULONG || tc == GA_SIZE || tc == GA_SSIZE;
}

/* ---------------------------------------------------------------- codegen */

static const char *extreme_literal(int tc, int lowest) {
  if (tc_is_float(tc)) return lowest ? "(-INFINITY)" : "INFINITY";
  if (tc_is_unsigned(tc)) {
    if (lowest) return "0";
    switch (gpuarray_get_elsize(tc)) {
    case 1: return "255";
    case 2: return "65535";
    case 4: return "4294967295U";
    default: return "18446744073709551615ULL";
    }
  }
  switch (gpuarray_get_elsize(tc)) {
  case 1: return lowest ? "(-128)" : "127";
  case 2: return lowest ? "(-32768)" : "32767";
  case 4: return lowest ? "(-2147483647 - 1)" : "2147483647";
  default: return lowest ? "(-9223372036854775807LL - 1)" : "9223372036854775807LL";
  }
}

static char *gen_source(const GpuReduction *gr, const rd_variant *v) {
  ga_strb sb;
  const char *src_t = ga_ctype(gr->src_tc);
  const char *x_t = gr->src_tc == GA_HALF ? "float" : src_t;
  const char *acc_t, *dst_t = ga_ctype(v->dst_tc);
  const char *map = "((GA_RD_ACC_T)(x))", *combine = "((a) + (b))", *ident = "0";

  ga_strb_init(&sb);
  if (gr->kind == 1) acc_t = x_t;
  else if (gr->op == GA_REDUCE_ALL || gr->op == GA_REDUCE_ANY) acc_t = "ga_ubyte";
  else acc_t = v->dst_tc == GA_HALF ? "float" : dst_t;

  switch (gr->op) {
  case GA_REDUCE_SUM: break;
  case GA_REDUCE_PROD: combine = "((a) * (b))"; ident = "1"; break;
  case GA_REDUCE_PRODNZ:
    map = "((x) == 0 ? (GA_RD_ACC_T)1 : (GA_RD_ACC_T)(x))";
    combine = "((a) * (b))";
    ident = "1";
    break;
  case GA_REDUCE_AND: combine = "((a) & (b))"; ident = "(~(GA_RD_ACC_T)0)"; break;
  case GA_REDUCE_OR: combine = "((a) | (b))"; break;
  case GA_REDUCE_XOR: combine = "((a) ^ (b))"; break;
  case GA_REDUCE_ALL: map = "((x) != 0)"; combine = "((a) && (b))"; ident = "1"; break;
  case GA_REDUCE_ANY: map = "((x) != 0)"; combine = "((a) || (b))"; break;
  default: ident = extreme_literal(gr->src_tc, !op_is_min(gr->op)); break;
  }
  ga_strb_puts(&sb, "#include \"cluda.h\"\n");
  ga_strb_printf(&sb, "#define GA_RD_SRC_T %s\n#define GA_RD_X_T %s\n#define GA_RD_ACC_T %s\n"
                      "#define GA_RD_DST_T %s\n", src_t, x_t, acc_t, dst_t);
  ga_strb_printf(&sb, "#define GA_RD_LOAD(raw) %s\n",
                 gr->src_tc == GA_HALF ? "ga_half2float(raw)" : "(raw)");
  ga_strb_printf(&sb, "#define GA_RD_STORE(a) %s\n",
                 v->dst_tc == GA_HALF ? "ga_float2half((float)(a))" : "((GA_RD_DST_T)(a))");
  ga_strb_printf(&sb, "#define GA_RD_MAP(x) %s\n#define GA_RD_COMBINE(a, b) %s\n"
                      "#define GA_RD_IDENT %s\n#define GA_RD_BETTER(b, a) %s\n",
                 map, combine, ident, op_is_min(gr->op) ? "((b) < (a))" : "((b) > (a))");
  /* float16 sums accumulated in float: widen-and-add in one instruction */
  if (gr->op == GA_REDUCE_SUM && gr->src_tc == GA_HALF &&
      (v->dst_tc == GA_HALF || v->dst_tc == GA_FLOAT))
    ga_strb_puts(&sb, "#define GA_RD_ADD_RAW(acc, raw) ga__add_f32_f16((acc), (raw))\n");
  if (gr->kind == 1) {
    const int mn = op_is_min(gr->op);
    if (gr->src_tc == GA_DOUBLE)
      ga_strb_printf(&sb, "#define GA_RD_PICK(a, b) %s((a), (b))\n", mn ? "fmin" : "fmax");
    else if (tc_is_float(gr->src_tc))
      ga_strb_printf(&sb, "#define GA_RD_PICK(a, b) %s((a), (b))\n", mn ? "fminf" : "fmaxf");
    else
      ga_strb_printf(&sb, "#define GA_RD_PICK(a, b) ((a) %s (b) ? (a) : (b))\n", mn ? "<" : ">");
  }
  {
    /* experiments: GPUARRAY_B200_RD_DEFINES="NAME=VALUE;NAME=VALUE" puts #define lines in
     * front of the template (its #ifndef defaults then stand back) */
    const char *extra = getenv("GPUARRAY_B200_RD_DEFINES");
    while (extra != NULL && *extra != '\0') {
      const char *end = strchr(extra, ';'), *eq;
      size_t len = end != NULL ? (size_t)(end - extra) : strlen(extra);
      eq = memchr(extra, '=', len);
      if (eq != NULL) {
        ga_strb_puts(&sb, "#define ");
        ga_strb_putn(&sb, extra, (size_t)(eq - extra));
        ga_strb_puts(&sb, " ");
        ga_strb_putn(&sb, eq + 1, len - (size_t)(eq - extra) - 1);
        ga_strb_puts(&sb, "\n");
      }
      extra = end != NULL ? end + 1 : NULL;
    }
  }
  ga_strb_printf(&sb, "#define GA_RD_KIND %d\n#define GA_RD_ISFLOAT %d\n#define GA_RD_WRITE_VAL %d\n"
                      "#define GA_RD_WRITE_IDX %d\n#define GA_RD_IDX_T %s\n#define GA_RD_VEC %d\n"
                      "#define GA_RD_THREADS %d\n#define GA_RD_TPO %d\n"
                      "#define GA_RD_BY %d\n#define GA_RD_GROUP %d\n#define GA_RD_FLAT %d\n"
                      "#define GA_RD_MU %d\n#define GA_RD_ONERUN %d\n#define GA_RD_FAST8 %d\n#define GA_RD_LAZY %d\n"
                      "#define GA_RD_SIMPLE %d\n#define GA_RD_UNROLL %d\n#define GA_RD_TINY %d\n"
                      "#define %s\n"
                      "#include \"ga_reduce.cuh\"\n",
                 gr->kind, tc_is_float(gr->src_tc), v->write_val, v->write_idx,
                 v->idx64 ? "unsigned long long" : "unsigned int", v->vec, RD_THREADS, v->tpo,
                 v->by ? v->by : RD_BY, v->group ? v->group : RD_THREADS, v->flat, v->mu ? v->mu : 1,
                 v->onerun, v->fast8, v->lazy, v->simple, gr->kind == 1 ? 8 : 4, v->tiny,
                 v->shape == SHAPE_ROWS   ? "GA_RD_BUILD_ROWS"
                 : v->shape == SHAPE_COLS ? "GA_RD_BUILD_COLS"
                                          : "GA_RD_BUILD_GENERAL");
  if (sb.failed) {
    ga_strb_free(&sb);
    return NULL;
  }
  return sb.s;
}

static const char *const shape_entry[] = {"ga_rd_rows", "ga_rd_cols", "ga_rd_general"};

static rd_variant *get_variant(GpuReduction *gr, const rd_variant *want, int *err) {
  rd_variant *v;
  char *src, *listing = NULL;
  for (v = gr->variants; v != NULL; v = v->next)
    if (v->shape == want->shape && v->vec == want->vec && v->idx64 == want->idx64 &&
        v->tpo == want->tpo && v->dst_tc == want->dst_tc &&
        v->write_val == want->write_val && v->write_idx == want->write_idx &&
        v->group == want->group && v->flat == want->flat && v->mu == want->mu &&
        v->onerun == want->onerun && v->fast8 == want->fast8 && v->lazy == want->lazy &&
        v->simple == want->simple && v->by == want->by && v->tiny == want->tiny)
      return v;
  v = malloc(sizeof(*v));
  if (v == NULL) {
    *err = ga_err_sys(gr->ctx->err, "malloc");
    return NULL;
  }
  *v = *want;
  src = gen_source(gr, v);
  if (src == NULL) {
    free(v);
    *err = ga_err_set(gr->ctx->err, GA_MISC_ERROR, "Formatting error creating kernel source");
    return NULL;
  }
  *err = ga_compile(gr->ctx, src, shape_entry[v->shape], NULL, &v->fn,
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
  {
    int n = 0;
    ga_ctx_enter(gr->ctx);
    if (ga_cu.p_cuOccupancyMaxActiveBlocksPerMultiprocessor(&n, v->fn.f, RD_THREADS, 0) != CUDA_SUCCESS)
      n = 0;
    ga_ctx_exit(gr->ctx);
    v->ctas_per_sm = n;
  }
  v->next = gr->variants;
  gr->variants = v;
  return v;
}

/* Split row reductions by warps: trims the split count so that the grid ends on a full
 * or nearly full wave of resident CTAs. `slots` = CTAs the device holds at once (SMs x the
 * compiled kernel's occupancy). A grid a little over a whole number of waves runs its last
 * CTAs on a mostly idle device. Measured on B200, fp32, sums: (256, 64, 4096) over (0, 2),
 * 64 outputs: 1360 CTAs (2.3 waves) 53.0 us, 1184 (2.0) 48.6 us, 592 (1.0) 46.4 us, 744 (1.26)
 * 52.5 us; (512, 512, 256) over (1, 2): 1344 CTAs (2.27 waves) 51.1 us, 1088 (1.84) 46.6 us,
 * 1216 (2.05) 55.0 us, 640 (1.08) 57.5 us. Only ever lowers the count, by a third at most;
 * grids within one wave are left alone. */
static void rd_fit_waves(rd_layout *L, const rd_variant *v, unsigned grid[3], unsigned long long slots) {
  unsigned long long gpb, s, best = 0;
  if (v->shape != SHAPE_ROWS || v->onerun || L->splits <= 1 || slots == 0 || v->group <= 0) return;
  gpb = (unsigned long long)(RD_THREADS / v->group);
  if ((L->nf_total * L->splits + gpb - 1) / gpb <= slots) return;
  for (s = L->splits; s >= 1 && s * 3 >= L->splits * 2; s--) {
    const unsigned long long ctas = (L->nf_total * s + gpb - 1) / gpb, rem = ctas % slots;
    if (rem == 0 || rem * 10 >= slots * 7) {
      best = s;
      break;
    }
  }
  if (best == 0 || best == L->splits) return;
  L->splits = best;
  grid[0] = (unsigned)((L->nf_total * best + gpb - 1) / gpb);
}

/* Test hook: what rd_fit_waves makes of a split row reduction of `outputs` outputs planned
 * with `splits` splits and `group` threads per work item on a device that holds `slots` CTAs
 * at once. Returns the trimmed split count; *ctas receives the grid size. */
GPUARRAY_PUBLIC unsigned long long gpuarray_b200_reduction_fit_waves(unsigned long long outputs,
                                                                     unsigned long long splits,
                                                                     int group,
                                                                     unsigned long long slots,
                                                                     unsigned int *ctas) {
  rd_layout L;
  rd_variant v;
  unsigned grid[3] = {0, 1, 1};
  memset(&L, 0, sizeof(L));
  memset(&v, 0, sizeof(v));
  L.nf_total = outputs;
  L.splits = splits;
  v.shape = SHAPE_ROWS;
  v.group = group;
  grid[0] = (unsigned)((outputs * splits + (unsigned long long)(RD_THREADS / group) - 1) /
                       (unsigned long long)(RD_THREADS / group));
  rd_fit_waves(&L, &v, grid, slots);
  if (ctas != NULL) *ctas = grid[0];
  return L.splits;
}

/* Test hook: source of one reduction kernel variant; caller frees. */
GPUARRAY_PUBLIC char *gpuarray_b200_reduction_source(int op, int src_tc, int dst_tc, int shape,
                                                     int vec, int idx64, int tpo, int group) {
  GpuReduction gr;
  rd_variant v;
  memset(&gr, 0, sizeof(gr));
  memset(&v, 0, sizeof(v));
  gr.op = (ga_reduce_op)op;
  gr.src_tc = src_tc;
  gr.kind = op_is_pair(gr.op);
  v.shape = shape;
  v.vec = vec;
  v.idx64 = idx64;
  v.tpo = tpo;
  v.group = group & 0xffff; /* bits 16-19: runs at once, bit 20: one-run mode, bit 21: flattened,
                               bit 22: lean one-run-per-warp loop, bit 23: flat walk of tiny runs,
                               bits 24-29: row lanes (cols) */
  v.mu = (group >> 16) & 0xf;
  v.onerun = (group >> 20) & 1;
  v.flat = (group >> 21) & 1;
  v.simple = (group >> 22) & 1;
  v.tiny = (group >> 23) & 1;
  v.by = (group >> 24) & 0x3f;
  v.dst_tc = dst_tc;
  v.write_val = op_writes_val(gr.op);
  v.write_idx = op_writes_idx(gr.op);
  return gen_source(&gr, &v);
}

/* ------------------------------------------------------------ construction */

int GpuReduction_new(GpuReduction **out, gpucontext *ctx, ga_reduce_op op, unsigned ndf,
                     unsigned ndr, int s0TypeCode, int flags) {
  GpuReduction *gr;
  (void)ndf; (void)ndr; (void)flags;
  if (out == NULL) return ga_err_set(ctx->err, GA_INVALID_ERROR, "GpuReduction_new: NULL result");
  *out = NULL;
  if ((int)op < 0 || op >= GA_REDUCE_ENDSUPPORTED)
    return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Unknown reduction operator %d", (int)op);
  if (!ga_type_is_computable(s0TypeCode) || s0TypeCode == GA_SIZE || s0TypeCode == GA_SSIZE)
    return ga_err_fmt(ctx->err, GA_UNSUPPORTED_ERROR, "Unsupported source type %d", s0TypeCode);
  if ((op == GA_REDUCE_AND || op == GA_REDUCE_OR || op == GA_REDUCE_XOR) &&
      tc_is_float(s0TypeCode))
    return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR,
                      "Bitwise reductions need an integer or bool source");
  gr = calloc(1, sizeof(*gr));
  if (gr == NULL) return ga_err_sys(ctx->err, "calloc");
  gr->ctx = ctx;
  gr->op = op;
  gr->src_tc = s0TypeCode;
  gr->kind = op_is_pair(op);
  ctx->refcnt++;
  *out = gr;
  return GA_NO_ERROR;
}

void GpuReduction_free(GpuReduction *gr) {
  rd_variant *v, *nv;
  gpucontext *ctx;
  if (gr == NULL) return;
  ctx = gr->ctx;
  for (v = gr->variants; v != NULL; v = nv) {
    nv = v->next;
    free(v);
  }
  if (gr->scratch != NULL) gpudata_release(gr->scratch);
  if (gr->tickets != NULL) gpudata_release(gr->tickets);
  GpuReduction_free(gr->sh_pair);
  GpuElemwise_free(gr->sh_e1);
  GpuElemwise_free(gr->sh_e2);
  GpuElemwise_free(gr->sh_e3);
  free(gr);
  ga_ctx_unref(ctx);
}

/* ------------------------------------------------------------ normalisation */

static int check_dst(gpucontext *ctx, const GpuArray *d, const GpuArray *s, const unsigned char *red,
                     unsigned ndd, const char *what) {
  unsigned i, k = 0;
  if (d->nd != ndd)
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "%s has %u dimensions, expected %u", what, d->nd,
                      ndd);
  for (i = 0; i < s->nd; i++) {
    if (red[i]) continue;
    if (d->dimensions[k] != s->dimensions[i])
      return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                        "%s dimension %u is %zu but source axis %u has %zu", what, k,
                        d->dimensions[k], i, s->dimensions[i]);
    k++;
  }
  if (GpuArray_context(d) != ctx)
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "%s belongs to another context", what);
  if (!GpuArray_ISWRITEABLE(d))
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "%s is not writeable", what);
  if (!GpuArray_ISALIGNED(d))
    return ga_err_fmt(ctx->err, GA_UNALIGNED_ERROR, "%s is not aligned", what);
  if (!ga_array_in_bounds(d))
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "%s reaches outside its buffer", what);
  return GA_NO_ERROR;
}

static long long ll_abs(long long v) { return v < 0 ? -v : v; }

/* Fills nf/nr, dims, strides, weights and totals of `L`. */
static int normalise(int kind, ga_error_rec *e, rd_layout *L, const GpuArray *d0,
                     const GpuArray *d1, const GpuArray *s, const unsigned char *red,
                     unsigned reduxLen, const int *reduxList, const rd_shard *sh,
                     unsigned long long *span) {
  unsigned i, k, n;
  unsigned long long mul;

  memset(L, 0, sizeof(*L));
  L->nf_total = 1;
  L->nr_total = 1;
  L->nan_first = (sh == NULL || sh->lo == 0) ? 1 : 0;

  /* kept axes, ascending; destination axis k pairs with the k-th kept axis */
  for (i = 0, k = 0, n = 0; i < s->nd; i++) {
    long long s0, sd0, sd1;
    if (red[i]) continue;
    L->nf_total *= s->dimensions[i];
    s0 = s->strides[i];
    sd0 = d0 != NULL ? d0->strides[k] : 0;
    sd1 = d1 != NULL ? d1->strides[k] : 0;
    k++;
    if (s->dimensions[i] == 1) continue;
    if (n > 0 && L->fsrc[n - 1] == (long long)s->dimensions[i] * s0 &&
        L->fdst0[n - 1] == (long long)s->dimensions[i] * sd0 &&
        L->fdst1[n - 1] == (long long)s->dimensions[i] * sd1) {
      L->fdim[n - 1] *= s->dimensions[i];
      L->fsrc[n - 1] = s0;
      L->fdst0[n - 1] = sd0;
      L->fdst1[n - 1] = sd1;
      continue;
    }
    if (n == RD_MAXD)
      return ga_err_fmt(e, GA_UNSUPPORTED_ERROR,
                        "More than %d kept dimensions remain after collapsing", RD_MAXD);
    L->fdim[n] = s->dimensions[i];
    L->fsrc[n] = s0;
    L->fdst0[n] = sd0;
    L->fdst1[n] = sd1;
    n++;
  }
  L->nf = n;

  /* reduced axes with their weight in the flat index (last listed fastest) */
  {
    unsigned long long dim[64], w[64];
    long long str[64];
    unsigned m = 0;
    mul = 1;
    for (i = reduxLen; i > 0; i--) {
      unsigned ax = (unsigned)reduxList[i - 1];
      size_t dsz = s->dimensions[ax];
      const int sharded = sh != NULL && sh->axis == (int)ax;
      L->nr_total *= dsz;
      /* the flat index counts in the extents of the WHOLE array: a sharded axis
       * weighs its global extent, and the slab's first coordinate is an offset */
      if (sharded && kind == 1) L->ioff = sh->lo * mul;
      if (dsz != 1) {
        if (m == 64)
          return ga_err_set(e, GA_UNSUPPORTED_ERROR, "More than 64 reduced axes");
        dim[m] = dsz;
        str[m] = s->strides[ax];
        w[m] = kind == 1 ? mul : 0;
        m++;
      }
      mul *= sharded ? sh->global : dsz;
    }
    if (span != NULL) *span = mul; /* flat indices run over [0, span) */
    /* traversal order = memory order: largest |stride| outermost (stable insertion sort) */
    for (i = 1; i < m; i++) {
      unsigned long long td = dim[i], tw = w[i];
      long long ts = str[i];
      unsigned j = i;
      while (j > 0 && ll_abs(str[j - 1]) < ll_abs(ts)) {
        dim[j] = dim[j - 1];
        str[j] = str[j - 1];
        w[j] = w[j - 1];
        j--;
      }
      dim[j] = td;
      str[j] = ts;
      w[j] = tw;
    }
    for (i = 0, n = 0; i < m; i++) {
      if (n > 0 && L->rsrc[n - 1] == (long long)dim[i] * str[i] &&
          L->rmul[n - 1] == dim[i] * w[i]) {
        L->rdim[n - 1] *= dim[i];
        L->rsrc[n - 1] = str[i];
        L->rmul[n - 1] = w[i];
        continue;
      }
      if (n == RD_MAXD)
        return ga_err_fmt(e, GA_UNSUPPORTED_ERROR,
                          "More than %d reduced dimensions remain after collapsing", RD_MAXD);
      L->rdim[n] = dim[i];
      L->rsrc[n] = str[i];
      L->rmul[n] = w[i];
      n++;
    }
    L->nr = n;
  }
  return GA_NO_ERROR;
}

/* -------------------------------------------------------------------- call */

static int ensure_scratch(GpuReduction *gr, size_t bytes, size_t ticket_bytes) {
  int err = GA_NO_ERROR;
  if (bytes > gr->scratch_sz) {
    if (gr->scratch != NULL) gpudata_release(gr->scratch);
    gr->scratch_sz = 0;
    gr->scratch = gpudata_alloc(gr->ctx, bytes, NULL, 0, &err);
    if (gr->scratch == NULL) return err;
    gr->scratch_sz = bytes;
  }
  if (ticket_bytes > gr->tickets_sz) {
    /* counters start at zero and every launch hands them back at zero */
    if (gr->tickets != NULL) gpudata_release(gr->tickets);
    gr->tickets_sz = 0;
    if (ticket_bytes < 4096) ticket_bytes = 4096;
    gr->tickets = gpudata_alloc(gr->ctx, ticket_bytes, NULL, 0, &err);
    if (gr->tickets == NULL) return err;
    err = gpudata_memset(gr->tickets, 0, 0);
    if (err != GA_NO_ERROR) return err;
    gr->tickets_sz = ticket_bytes;
  }
  return GA_NO_ERROR;
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

static int all_multiple(const long long *v, unsigned n, long long m) {
  unsigned i;
  for (i = 0; i < n; i++)
    if (v[i] % m != 0) return 0;
  return 1;
}

/* Tuning for experiments: GPUARRAY_B200_RD="ctas_per_sm,seg_vectors,cta_min_vectors,
 * cols_ctas_per_sm (0 = the lanes rule),onerun_ctas_per_sm,onerun_loads_per_lane,
 * onerun_outputs_at_once,lazy_index (0/1),lazy_min_vectors_per_lane,cols_row_lanes (0 = rule),
 * lean_rows (0/1),cols_early_rows,lazy_min_vectors_per_lane_short_runs,
 * outputs_per_sm_from_which_a_warp_owns_an_output,
 * warps_per_sm_wanted_when_2_or_4_warps_share_a_run (0 = a CTA per run),
 * trim_splits_to_whole_waves (0/1),flat_walk_of_tiny_runs (0/1)". The
 * defaults are the best of sweeps on a B200. */
static unsigned rd_cols_ctas_per_sm = 0, rd_cols_by = 0;
static unsigned rd_simple = 1, rd_cols_early = 4, rd_lazy_onerun_min = 8, rd_warp_rows_per_sm = 16, rd_subcta = 24;
static unsigned rd_wave_fit = 1, rd_tiny = 1;
static unsigned rd_onerun_ctas_per_sm = 3, rd_onerun_lpl = 4, rd_onerun_mu = 0, rd_lazy = 1, rd_lazy_min = 32;

static void rd_tuning(unsigned *ctas_per_sm, unsigned *seg_vecs, unsigned *warp_bytes) {
  static int parsed = 0;
  static unsigned t_ctas = 32, t_seg = 16, t_warp = 0x7fffffff;
  *warp_bytes = t_warp;
  if (!parsed) {
    const char *env = getenv("GPUARRAY_B200_RD");
    if (env != NULL)
      sscanf(env, "%u,%u,%u,%u,%u,%u,%u,%u,%u,%u,%u,%u,%u,%u,%u,%u,%u", &t_ctas, &t_seg, &t_warp, &rd_cols_ctas_per_sm,
             &rd_onerun_ctas_per_sm, &rd_onerun_lpl, &rd_onerun_mu, &rd_lazy, &rd_lazy_min,
             &rd_cols_by, &rd_simple, &rd_cols_early, &rd_lazy_onerun_min, &rd_warp_rows_per_sm,
             &rd_subcta, &rd_wave_fit, &rd_tiny);
    *warp_bytes = t_warp;
    if (t_ctas == 0) t_ctas = 32;
    if (t_seg == 0) t_seg = 8;
    parsed = 1;
  }
  *ctas_per_sm = t_ctas;
  *seg_vecs = t_seg;
}

/* What the planner needs to know besides the normalised layout. */
typedef struct rd_plan_in {
  ga_error_rec *e;
  int kind;
  ga_reduce_op op;
  int src_tc, dst_tc, need_val, need_idx;
  unsigned num_sms;
  unsigned long long p_src; /* address of the source's first element (alignment only) */
  unsigned long long idx_span; /* flat indices run over [0, idx_span): the reduced element
                                  count, or that of the whole array when the source is a shard */
} rd_plan_in;

/* Chooses the kernel variant, the split of the reduced extent and the launch
 * geometry for a normalised problem. Pure host arithmetic: no device, no
 * allocation (gpuarray_b200_reduction_plan exposes it to tests). */
static int rd_plan(const rd_plan_in *in, rd_layout *L, rd_variant *want, unsigned grid[3],
                   unsigned block[3]) {
  unsigned ctas_per_sm, seg_vecs, cta_min_vecs;
  size_t elsize = gpuarray_get_elsize(in->src_tc), target;
  grid[0] = grid[1] = grid[2] = 1;
  block[0] = RD_THREADS;
  block[1] = block[2] = 1;
  rd_tuning(&ctas_per_sm, &seg_vecs, &cta_min_vecs);
  target = (size_t)in->num_sms * ctas_per_sm;

  memset(want, 0, sizeof(*want));
  want->dst_tc = in->dst_tc;
  want->write_val = in->need_val;
  want->write_idx = in->need_idx;
  want->idx64 = L->nr_total >= 0xffffffffULL || in->idx_span >= 0xffffffffULL;
  want->vec = 1;
  want->tpo = 1;
  L->splits = 1;

  if (L->nr_total > 0 && L->nr >= 1 && L->rsrc[L->nr - 1] == (long long)elsize &&
      L->rdim[L->nr - 1] >= 2) {
    /* --- contiguous reduced run --- */
    unsigned vec = (unsigned)(16 / elsize);
    unsigned long long rows_outer = L->nr_total / L->rdim[L->nr - 1];
    want->shape = SHAPE_ROWS;
    if (vec > 1 && in->p_src % 16 == 0 && all_multiple(L->fsrc, (unsigned)L->nf, 16) &&
        all_multiple(L->rsrc, (unsigned)L->nr - 1, 16))
      want->vec = (int)vec;
    L->inner = L->rdim[L->nr - 1];
    {
      unsigned long long nvrow = L->inner / (unsigned)want->vec, groups_target, nwork, blocks, share;
      unsigned gpb;
      /* Who shares a work item, and whether the reduced extent is split:
       *  - plenty of outputs: a warp per output, no split;
       *  - a moderate number of outputs with long runs: a CTA per output;
       *  - few outputs: split the reduced extent (CTAs when the runs are long
       *    and the outputs very few, which also keeps the partial count low). */
      int need_split = 0;
      /* loads one lane of a warp issues per run: short runs need help to keep
       * enough bytes in flight (see the kernel's comment) */
      unsigned long long nload = nvrow + (L->inner % (unsigned)want->vec != 0);
      if (rd_tiny && rows_outer == 1 && nload <= 8 && (nload & (nload - 1)) == 0 && elsize > 1 &&
          (unsigned long long)want->vec * elsize == 16 && L->inner % (unsigned)want->vec == 0 &&
          L->nf == 1 && L->fsrc[0] == (long long)(L->inner * elsize) &&
          L->nf_total * nload < 0x7fffffffULL && !(in->kind == 0 && elsize == 8)) {
        /* runs of 16-128 bytes, back to back: the flat walk (GA_RD_TINY in the template).
         * Measured on B200, 256 MiB, against the short-run path below: fp32 rows of 4: MAX
         * 98.6 -> 54.0 us, SUM 59.8 -> 51.1 us; rows of 16: ARGMAX 58.8 -> 49.7 us, MAX AND
         * ARGMAX 65.4 -> 57.2 us, SUM 45.2 -> 44.6 us; rows of 32: 55.4 / 57.6 / 60.7 / 47.2 ->
         * 52.2 / 51.6 / 56.7 / 44.1 us; fp16 rows of 32: MAX AND ARGMAX 86.7 -> 64.0 us; fp64
         * rows of 8: MAX 63.4 -> 53.4 us but SUM 47.6 -> 51.8 us (two 64-bit shuffle steps for
         * two adds), hence the exception. */
        unsigned long long vectors = L->nf_total * nload;
        want->tiny = 1;
        want->group = (int)nload;
        want->mu = 1;
        L->seg = L->inner;
        L->nseg = 1;
        L->units = 1;
        blocks = (vectors + 4ULL * RD_THREADS - 1) / (4ULL * RD_THREADS);
        if (blocks > (unsigned long long)in->num_sms * 8) blocks = (unsigned long long)in->num_sms * 8;
        grid[0] = (unsigned)blocks;
        goto rows_done;
      }
      if (rows_outer == 1 && nload <= 256) {
        unsigned g = 1, lpl;
        while (g < 32 && g * rd_onerun_lpl < nload) g *= 2;
        lpl = (unsigned)((nload + g - 1) / g);
        want->onerun = 1;
        want->group = (int)g;
        /* outputs a group works on at once. Measured on B200 (fp32, 256 MiB, rows of 16 ..
         * 1024): MIN / MAX / ARGMIN / ARGMAX - one destination, a light state - gain from 4
         * (rows of 16: 60.4 -> 54.8 us, of 512: 56.6 -> 55.0 us) except with two lanes per
         * row (32 columns: 55.5 -> 57.0 us) and with the values-only scan of longer rows
         * (1024 columns: 51.5 -> 54.7 us); value AND index (67 - 74 us against 60) and sums
         * (rows of 16: 44.9 -> 50.2 us) lose: their four states no longer fit the registers
         * three CTAs per SM leave. */
        want->mu = rd_onerun_mu                                                        ? (int)rd_onerun_mu
                   : lpl <= 2                                                          ? 4
                   : (in->kind == 1 && !(in->need_val && in->need_idx) && lpl <= 4 && g != 2) ? 4
                                                                                       : 2;
        L->seg = L->inner;
        L->nseg = 1;
        L->units = 1;
        gpb = RD_THREADS / g;
        blocks = (L->nf_total + (unsigned long long)gpb * (unsigned)want->mu - 1) /
                 ((unsigned long long)gpb * (unsigned)want->mu);
        if (rd_onerun_ctas_per_sm && blocks > (unsigned long long)in->num_sms * rd_onerun_ctas_per_sm)
          blocks = (unsigned long long)in->num_sms * rd_onerun_ctas_per_sm;
        grid[0] = (unsigned)blocks;
        goto rows_done;
      }
      want->flat = nvrow < 16;
      want->mu = want->flat ? 1 : nload <= 64 ? 4 : nload <= 256 ? 2 : 1;
      if (nvrow >= cta_min_vecs) want->group = RD_THREADS;
      else if (L->nf_total >= (unsigned long long)in->num_sms * rd_warp_rows_per_sm) want->group = 32;
      else if (L->nf_total >= (unsigned long long)in->num_sms * 4 && nvrow >= 1024) {
        /* A moderate number of long runs: a warp per run would leave the SMs with too few
         * warps to cover DRAM latency, a CTA per run makes every CTA short-lived. Two or
         * four warps share a run when that gives at least 24 warps per SM. Measured on
         * B200, MAXANDARGMAX of fp32 (2048, 32000) (the 8-GPU shard of the headline):
         * 54.5 us with a warp or a CTA per row; see the profile notes for the shared form. */
        unsigned g = 64;
        while (g < RD_THREADS && L->nf_total * (g / 32) < (unsigned long long)in->num_sms * rd_subcta) g *= 2;
        want->group = (int)(rd_subcta ? g : RD_THREADS);
      }
      else {
        /* warps, unless long runs would leave them either too few or with
         * shares too short to be worth a ticket (see the cap below) */
        unsigned long long s_w = ((unsigned long long)target * (RD_THREADS / 32) + L->nf_total - 1) /
                                 L->nf_total;
        unsigned long long cap_w = L->nr_total * elsize / (24u << 10);
        if (cap_w < 1) cap_w = 1;
        if (s_w > cap_w) s_w = cap_w;
        need_split = 1;
        want->group = (nvrow >= 2048 && (L->nf_total < (unsigned long long)in->num_sms ||
                                        L->nf_total * s_w < (unsigned long long)in->num_sms * 16))
                         ? RD_THREADS : 32;
      }
      if (want->group > 32) want->flat = 0, want->mu = 1;
      gpb = RD_THREADS / (unsigned)want->group;
      /* measured on B200: whole-CTA groups run best as a few long-lived CTAs
       * per SM, warp groups as many (a full complement of resident warps) */
      groups_target = want->group == RD_THREADS ? (unsigned long long)in->num_sms * 4
                                               : (unsigned long long)target * gpb;
      L->seg = L->inner;
      L->nseg = 1;
      L->units = rows_outer;
      if (need_split) {
        unsigned long long s;
        if (!want->flat) {
          unsigned long long seg = (unsigned long long)want->group * vec * seg_vecs;
          if (seg < L->inner) {
            L->seg = seg;
            L->nseg = (L->inner + seg - 1) / seg;
            L->units = rows_outer * L->nseg;
          }
        }
        s = (groups_target + L->nf_total - 1) / L->nf_total;
        if (want->group == 32) {
          /* measured on B200: a warp's share should stay above ~24 KiB, or the
           * ramp of each share and the ticketed finish outweigh the parallelism */
          unsigned long long cap = L->nr_total * elsize / (24u << 10);
          if (cap < 1) cap = 1;
          if (s > cap) s = cap;
        }
        if (s > L->units) s = L->units;
        if (s > 1u << 20) s = 1u << 20;
        L->splits = s ? s : 1;
      }
      if (L->seg >= 0x7fffffffULL) {
        /* a single run longer than 32-bit indexing: cut it even without splitting */
        L->seg = (unsigned long long)want->group * vec * seg_vecs * 1024;
        L->nseg = (L->inner + L->seg - 1) / L->seg;
        L->units = rows_outer * L->nseg;
      }
      make_div32((unsigned int)(nvrow ? nvrow : 1), L->dv);
      share = (L->units / L->splits + 1) * (nvrow + 1);
      if (want->flat && share >= 0xffffffffULL)
        return ga_err_set(in->e, GA_XLARGE_ERROR, "Reduction share exceeds 32-bit indexing");
      nwork = L->nf_total * L->splits;
      blocks = (nwork + gpb - 1) / gpb;
      grid[0] = blocks > 0x7fffffffULL ? 0x7fffffffu : (unsigned)blocks;
    rows_done:;
    }
  } else if (L->nr_total > 0 && L->nf >= 1 && L->fsrc[L->nf - 1] == (long long)elsize &&
             L->fdim[L->nf - 1] >= 16) {
    /* --- contiguous kept run --- */
    unsigned vec = (unsigned)(16 / elsize);
    unsigned long long ko, nwork, s;
    if (vec > 4) vec = 4;
    want->shape = SHAPE_COLS;
    L->inner = L->fdim[L->nf - 1];
    while (vec > 1 && !(L->inner % vec == 0 && in->p_src % (vec * elsize) == 0 &&
                        all_multiple(L->fsrc, (unsigned)L->nf - 1, (long long)(vec * elsize)) &&
                        all_multiple(L->rsrc, (unsigned)L->nr, (long long)(vec * elsize))))
      vec /= 2;
    want->vec = (int)vec;
    L->tiles = (L->inner + 32ULL * vec - 1) / (32ULL * vec);
    ko = L->nf_total / L->inner;
    nwork = ko * L->tiles;
    {
      /* Row lanes per CTA (by) times splits = the row lanes that share one column tile.
       * Measured on B200 (fp32 4096 x 4096 over axis 0, 32 tiles): what counts is that
       * every thread walks about 16 rows and that the whole grid is resident at once
       * (2048 threads per SM); 16 lanes x 16 splits 14.1 us, 32 x 8 14.3 us, 8 x 32 14.4 us,
       * 8 x 14 17.2 us, 32 x 10 (two waves) 18.9 us. 16 lanes keep the shared exchange of
       * the widest states (16 bytes x 4 x 32 x 16) within the static limit. */
      unsigned long long lanes_fit = ((unsigned long long)in->num_sms * 64) / nwork; /* warps */
      unsigned long long lanes_want = (L->nr_total + 15) / 16, lanes;
      unsigned by = rd_cols_by ? rd_cols_by : RD_BY;
      if (rd_cols_by == 0 && lanes_want >= 128 && lanes_fit >= 32) by = 16;
      lanes = lanes_want < lanes_fit ? lanes_want : lanes_fit;
      if (rd_cols_ctas_per_sm != 0) /* experiment knob: CTAs per SM instead */
        lanes = (((unsigned long long)in->num_sms * rd_cols_ctas_per_sm + nwork - 1) / nwork) * by;
      s = lanes / by;
      if (s < 1) s = 1;
      if (s > (L->nr_total + by * 8 - 1) / (by * 8)) s = (L->nr_total + by * 8 - 1) / (by * 8);
      if (s > 1024) s = 1024;
      want->by = (int)by;
      block[1] = by;
      /* L2 hints ahead of the dependency wait: one reduced dimension, no outer kept
       * position, fully vectorised rows (so every tile row starts on 16 bytes). Measured
       * on B200 (fp32 4096 x 4096 over axis 0, 16 lanes x 16 splits): 14.2 -> 13.4 us with
       * 4 rows per lane; 8 rows give the same, 16 rows and hints issued AFTER the wait
       * are slower than none. */
      if (L->nr == 1 && ko == 1 && (size_t)vec * elsize == 16 && rd_cols_early != 0)
        L->early = rd_cols_early;
      /* the lean walk: one reduced dimension, one contiguous kept run, 32-bit counters */
      if (rd_simple && L->nr == 1 && ko == 1 && L->nr_total < 0x7fffffffULL &&
          L->inner < 0x7fffffffULL)
        want->simple = 1;
    }
    L->splits = s ? s : 1;
    L->units = nwork; /* tickets: one per column tile */
    grid[0] = nwork > 0x7fffffffULL ? 0x7fffffffu : (unsigned)nwork;
    grid[1] = (unsigned)L->splits;
    block[0] = 32;
  } else {
    /* --- arbitrary strides --- */
    unsigned long long groups_per_block, blocks;
    want->shape = SHAPE_GENERAL;
    if (L->nr_total >= 2048 && L->nf_total < 4096) want->tpo = RD_THREADS;
    else if (L->nr_total >= 64) want->tpo = 32;
    groups_per_block = RD_THREADS / (unsigned)want->tpo;
    blocks = (L->nf_total + groups_per_block - 1) / groups_per_block;
    if (blocks > (unsigned long long)target * 8) blocks = (unsigned long long)target * 8;
    grid[0] = (unsigned)(blocks ? blocks : 1);
  }

  /* (value, index) operators over long runs scan values only (GA_RD_LAZY). Measured on
   * B200: 32 KiB fp32 rows (64 vectors per lane) 49.7 -> 46.2 us for 268 MB, the headline's
   * 128 KB rows 321.7 -> 316.5 us; 8 KiB fp64 runs (16 per lane) lose 6 % to the extra
   * look at the winning vector, hence the threshold. */
  if (in->kind == 1 && want->shape == SHAPE_ROWS && !want->onerun && !want->flat && want->mu <= 1 &&
      rd_lazy && L->seg / (unsigned)want->vec / (unsigned)(want->group ? want->group : RD_THREADS) >= rd_lazy_min)
    want->lazy = 1;
  /* ... and over one short run per output when a lane sees many vectors. Measured on B200: with
   * 4 vectors per lane the second look at the winning vector costs more than the scan saves
   * (ARGMAX of fp32 (2^17, 512): 57.4 -> 59.3 us; MAX of (2^22, 16): 60.0 -> 64.5 us), hence
   * the threshold of 8. */
  if (in->kind == 1 && want->shape == SHAPE_ROWS && want->onerun && rd_lazy && want->vec > 1 &&
      L->inner / (unsigned)want->vec / (unsigned)want->group >= rd_lazy_onerun_min)
    want->lazy = 1;
  /* one run per output, a warp each, nothing split: the lean loop (GA_RD_SIMPLE). Measured on
   * B200, fp32 4096 x 4096 over axis 1, launches back to back: 13.8 -> see the profile notes */
  if (want->shape == SHAPE_ROWS && rd_simple && want->group == 32 && L->splits == 1 && L->nr == 1 &&
      L->nseg == 1 && !want->onerun && !want->flat && want->mu <= 1 && !want->lazy &&
      L->nf_total < 0xffffffffULL && L->inner < 0x7fffffffULL)
    want->simple = 1;
  /* whole-word arithmetic on vectors of 1-byte elements (see ga__fold_lanes) */
  if (elsize == 1 && want->vec % 4 == 0 && want->shape == SHAPE_ROWS) {
    if (in->op == GA_REDUCE_SUM && !tc_is_float(want->dst_tc) &&
        gpuarray_get_elsize(want->dst_tc) >= 4)
      want->fast8 = in->src_tc == GA_BYTE ? 1 : 2;
    else if (in->op == GA_REDUCE_ANY) want->fast8 = 3;
    else if (in->op == GA_REDUCE_ALL) want->fast8 = 4;
  }
  return GA_NO_ERROR;
}

/* Test and tooling hook: the plan GpuReduction_call would make for a source of
 * the given shape and byte strides on a device with `num_sms` SMs, without any
 * device. Destinations are taken as C-contiguous. `base` stands for the
 * address of the source's first element (its alignment decides vector width).
 * out[0..23] = shape (0 rows, 1 cols, 2 general), vec, group, flat, runs at
 * once, one-run mode, lazy index, byte folding, threads per output (general),
 * 64-bit index, splits, seg, nseg, units, grid x, grid y, block x, block y
 * (cols: row lanes per CTA), outputs, reduced elements per output, lean rows
 * loop, three spare words. Returns a GA_* code. */
static int plan_worker(int op, int src_tc, int dst_tc, unsigned int nd, const size_t *dims,
                       const ssize_t *strides, unsigned int reduxLen, const int *reduxList,
                       unsigned long long base, unsigned int num_sms, unsigned long long *out,
                       rd_layout *layout_out) {
  GpuArray s, d, di;
  size_t ddims[64];
  ssize_t dstr[64], distr[64];
  unsigned char red[64];
  rd_layout L;
  rd_variant want;
  rd_plan_in in;
  unsigned grid[3], block[3], i, k;
  size_t step;
  int err;
  if (nd == 0 || nd > 64 || reduxLen == 0 || reduxLen > nd || (int)op < 0 ||
      op >= GA_REDUCE_ENDSUPPORTED)
    return ga_err_set(ga_global_err, GA_INVALID_ERROR, "Invalid rank, axis count or operator");
  memset(red, 0, sizeof(red));
  for (i = 0; i < reduxLen; i++) {
    if (reduxList[i] < 0 || (unsigned)reduxList[i] >= nd || red[reduxList[i]])
      return ga_err_set(ga_global_err, GA_INVALID_ERROR, "Bad reduction axis");
    red[reduxList[i]] = 1;
  }
  memset(&s, 0, sizeof(s));
  memset(&d, 0, sizeof(d));
  s.nd = nd;
  s.dimensions = (size_t *)dims;
  s.strides = (ssize_t *)strides;
  for (i = 0, k = 0; i < nd; i++)
    if (!red[i]) ddims[k++] = dims[i];
  step = gpuarray_get_elsize(dst_tc);
  for (i = k; i > 0; i--) {
    dstr[i - 1] = (ssize_t)step;
    step *= ddims[i - 1];
  }
  d.nd = k;
  d.dimensions = ddims;
  d.strides = dstr;
  step = 8; /* the index destination holds 8-byte integers */
  for (i = k; i > 0; i--) {
    distr[i - 1] = (ssize_t)step;
    step *= ddims[i - 1];
  }
  memset(&di, 0, sizeof(di));
  di.nd = k;
  di.dimensions = ddims;
  di.strides = distr;
  memset(&in, 0, sizeof(in));
  in.e = ga_global_err;
  in.op = (ga_reduce_op)op;
  in.kind = op_is_pair(in.op);
  in.src_tc = src_tc;
  in.dst_tc = dst_tc;
  in.need_val = op_writes_val(in.op);
  in.need_idx = op_writes_idx(in.op);
  in.num_sms = num_sms;
  in.p_src = base;
  err = normalise(in.kind, in.e, &L, in.need_val ? &d : NULL, in.need_idx ? &di : NULL, &s, red,
                  reduxLen, reduxList, NULL, &in.idx_span);
  if (err != GA_NO_ERROR) return err;
  memset(out, 0, 24 * sizeof(*out));
  out[18] = L.nf_total;
  out[19] = L.nr_total;
  if (L.nf_total == 0 || L.nr_total == 0) return GA_NO_ERROR;
  err = rd_plan(&in, &L, &want, grid, block);
  if (err != GA_NO_ERROR) return err;
  out[0] = (unsigned long long)want.shape;
  out[1] = (unsigned long long)want.vec;
  out[2] = (unsigned long long)(want.group ? want.group : RD_THREADS);
  out[3] = (unsigned long long)want.flat;
  out[4] = (unsigned long long)(want.mu ? want.mu : 1);
  out[5] = (unsigned long long)want.onerun;
  out[6] = (unsigned long long)want.lazy;
  out[7] = (unsigned long long)want.fast8;
  out[8] = (unsigned long long)want.tpo;
  out[9] = (unsigned long long)want.idx64;
  out[10] = L.splits;
  out[11] = L.seg;
  out[12] = L.nseg;
  out[13] = L.units;
  out[14] = grid[0];
  out[15] = grid[1];
  out[16] = block[0];
  out[17] = block[1];
  out[20] = (unsigned long long)want.simple;
  out[21] = (unsigned long long)want.tiny;
  if (layout_out != NULL) *layout_out = L;
  return GA_NO_ERROR;
}

GPUARRAY_PUBLIC int gpuarray_b200_reduction_plan(int op, int src_tc, int dst_tc, unsigned int nd,
                                                 const size_t *dims, const ssize_t *strides,
                                                 unsigned int reduxLen, const int *reduxList,
                                                 unsigned long long base, unsigned int num_sms,
                                                 unsigned long long *out) {
  return plan_worker(op, src_tc, dst_tc, nd, dims, strides, reduxLen, reduxList, base, num_sms, out,
                     NULL);
}

/* As gpuarray_b200_reduction_plan, and also copies the parameter block the
 * kernel would receive (struct ga__rd_layout of ga_reduce.cuh) into `layout`
 * (`cap` bytes available); *used receives its size. For tools that run the
 * kernel templates outside the library. */
GPUARRAY_PUBLIC int gpuarray_b200_reduction_layout(int op, int src_tc, int dst_tc, unsigned int nd,
                                                   const size_t *dims, const ssize_t *strides,
                                                   unsigned int reduxLen, const int *reduxList,
                                                   unsigned long long base, unsigned int num_sms,
                                                   unsigned long long *out, void *layout,
                                                   size_t cap, size_t *used) {
  rd_layout L;
  int err;
  memset(&L, 0, sizeof(L));
  if (cap < sizeof(L)) return ga_err_set(ga_global_err, GA_VALUE_ERROR, "Layout buffer too small");
  err = plan_worker(op, src_tc, dst_tc, nd, dims, strides, reduxLen, reduxList, base, num_sms, out,
                    &L);
  if (err != GA_NO_ERROR) return err;
  memcpy(layout, &L, sizeof(L));
  if (used != NULL) *used = sizeof(L);
  return GA_NO_ERROR;
}

static int rd_call(const GpuReduction *cgr, GpuArray *d0, GpuArray *d1, const GpuArray *s0,
                   unsigned reduxLen, const int *reduxList, int flags, const rd_shard *sh) {
  GpuReduction *gr = (GpuReduction *)cgr;
  gpucontext *ctx;
  unsigned char red[64];
  rd_layout L;
  rd_variant want, *v1;
  unsigned i, ndd;
  unsigned grid[3] = {1, 1, 1}, block[3] = {RD_THREADS, 1, 1};
  int err = GA_NO_ERROR, need_val, need_idx;
  unsigned long long idx_span = 0;
  CUdeviceptr p_src, p_d0 = 0, p_d1 = 0, p_val = 0, p_idx = 0, p_tic = 0;
  void *params[7];
  (void)flags;

  if (gr == NULL) return GA_INVALID_ERROR;
  ctx = gr->ctx;
  if (s0 == NULL) return ga_err_set(ctx->err, GA_INVALID_ERROR, "Source array is NULL");
  if (s0->nd == 0 || s0->nd > 64 || reduxLen == 0 || reduxLen > s0->nd || reduxList == NULL)
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "Invalid rank or reduction axis count");
  if (s0->typecode != gr->src_tc)
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR,
                      "Source has type %d but the operator was built for %d", s0->typecode,
                      gr->src_tc);
  if (GpuArray_context(s0) != ctx)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Source belongs to another context");
  if (!GpuArray_ISALIGNED(s0)) return ga_err_set(ctx->err, GA_UNALIGNED_ERROR, "Source is not aligned");
  if (!ga_array_in_bounds(s0))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Source reaches outside its buffer");
  memset(red, 0, sizeof(red));
  for (i = 0; i < reduxLen; i++) {
    if (reduxList[i] < 0 || (unsigned)reduxList[i] >= s0->nd)
      return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Reduction axis %d out of range", reduxList[i]);
    if (red[reduxList[i]])
      return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Reduction axis %d listed twice", reduxList[i]);
    red[reduxList[i]] = 1;
  }
  ndd = s0->nd - reduxLen;
  need_val = op_writes_val(gr->op);
  need_idx = op_writes_idx(gr->op);
  if (need_val && d0 == NULL)
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "Value destination is NULL");
  if (need_idx && d1 == NULL)
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "Index destination is NULL");
  if (!need_val) d0 = NULL;
  if (!need_idx) d1 = NULL;
  if (d0 != NULL) {
    err = check_dst(ctx, d0, s0, red, ndd, "Value destination");
    if (err != GA_NO_ERROR) return err;
    if (gr->kind == 1 && d0->typecode != s0->typecode)
      return ga_err_set(ctx->err, GA_VALUE_ERROR,
                        "min/max destination must have the source's type");
    if (!ga_type_is_computable(d0->typecode) || d0->typecode == GA_SIZE || d0->typecode == GA_SSIZE)
      return ga_err_fmt(ctx->err, GA_UNSUPPORTED_ERROR, "Unsupported destination type %d",
                        d0->typecode);
    if ((gr->op == GA_REDUCE_AND || gr->op == GA_REDUCE_OR || gr->op == GA_REDUCE_XOR) &&
        tc_is_float(d0->typecode))
      return ga_err_set(ctx->err, GA_VALUE_ERROR, "Bitwise reductions need an integer destination");
  }
  if (d1 != NULL) {
    err = check_dst(ctx, d1, s0, red, ndd, "Index destination");
    if (err != GA_NO_ERROR) return err;
    if (!tc_is_index(d1->typecode))
      return ga_err_set(ctx->err, GA_VALUE_ERROR, "Index destination must hold 8-byte integers");
  }

  if (sh != NULL && (sh->axis < 0 || (unsigned)sh->axis >= s0->nd || !red[sh->axis] ||
                     sh->lo + s0->dimensions[sh->axis] > sh->global))
    return ga_err_set(ctx->err, GA_VALUE_ERROR,
                      "The sharded axis must be a reduced axis and the slab must lie inside it");
  err = normalise(gr->kind, ctx->err, &L, d0, d1, s0, red, reduxLen, reduxList, sh, &idx_span);
  if (err != GA_NO_ERROR) return err;
  if (L.nf_total == 0) return GA_NO_ERROR;
  if (L.nr_total == 0 && gr->kind == 1)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "min/max over zero elements");

  p_src = s0->data->ptr + s0->offset;
  if (d0 != NULL) p_d0 = d0->data->ptr + d0->offset;
  if (d1 != NULL) p_d1 = d1->data->ptr + d1->offset;
  {
    rd_plan_in in;
    in.e = ctx->err;
    in.kind = gr->kind;
    in.op = gr->op;
    in.src_tc = gr->src_tc;
    in.dst_tc = d0 != NULL ? d0->typecode : gr->src_tc;
    in.need_val = need_val;
    in.need_idx = need_idx;
    in.num_sms = ctx->num_sms;
    in.p_src = p_src;
    in.idx_span = idx_span;
    err = rd_plan(&in, &L, &want, grid, block);
    if (err != GA_NO_ERROR) return err;
  }
  v1 = get_variant(gr, &want, &err);
  if (v1 == NULL) return err;
  if (rd_wave_fit) rd_fit_waves(&L, v1, grid, (unsigned long long)ctx->num_sms * (unsigned)v1->ctas_per_sm);
  if (L.splits > 1) {
    /* scratch: values [outputs][splits], indices [outputs][splits], tickets */
    size_t cells = (size_t)L.splits * (size_t)L.nf_total;
    size_t nticket = want.shape == SHAPE_COLS ? (size_t)L.units : (size_t)L.nf_total;
    err = ensure_scratch(gr, cells * 16, nticket * sizeof(unsigned int));
    if (err != GA_NO_ERROR) return err;
    p_val = gr->scratch->ptr;
    p_idx = gr->scratch->ptr + cells * 8;
    p_tic = gr->tickets->ptr;
  }
  params[0] = &L;
  params[1] = &p_src;
  params[2] = &p_d0;
  params[3] = &p_d1;
  params[4] = &p_val;
  params[5] = &p_idx;
  params[6] = &p_tic;
  return ga_launch(ctx, &v1->fn, grid, block, 0, params);
}

int GpuReduction_call(const GpuReduction *gr, GpuArray *d0, GpuArray *d1, const GpuArray *s0,
                      unsigned reduxLen, const int *reduxList, int flags) {
  return rd_call(gr, d0, d1, s0, reduxLen, reduxList, flags, NULL);
}

/* ------------------------------------------ reduced extent sharded over GPUs */

/* In-place all-reduce of a contiguous array (no-op without a communicator). */
static int sh_all_reduce(GpuArray *a, int opcode, gpucomm *comm) {
  if (comm == NULL) return GA_NO_ERROR;
  return GpuArray_all_reduce(a, a, opcode, comm);
}

static int sh_elemwise(gpucontext *ctx, GpuElemwise **slot, const char *expr, unsigned n,
                       gpuelemwise_arg *args, int convert_f16) {
  if (*slot != NULL) return GA_NO_ERROR;
  *slot = GpuElemwise_new(ctx, "", expr, n, args, 0, convert_f16 ? GE_CONVERT_F16 : 0);
  return *slot != NULL ? GA_NO_ERROR : ctx->err->code;
}

/* (value, index) operators when ONE reduced axis is sharded over the ranks of
 * `comm`: the reference's collectives have no pair operator
 * (src/gpuarray_collectives_cuda_nccl.c:158-185: sum, prod, max, min), so the
 * combination is two all-reduces of existing operators around three small
 * elementwise kernels, everything enqueued on the context's stream with no
 * host round trip:
 *   1. the local kernel writes (v, i): i already is the flat index in the WHOLE
 *      reduced extent (the shard's offset and the global radix are folded into
 *      the kernel's index weights); a shard that does not hold element 0 does
 *      not apply the NaN-first rule;
 *   2. w = v with a NaN (only possible on the rank that holds element 0, where
 *      it is the final answer) replaced by the winning infinity; p = payload
 *      bits of v: bit 0 "not a NaN", bit 1 "negative zero";
 *   3. all-reduce MAX (MIN) of w                                   -> best
 *   4. c = (w == best and i valid) ? (i << 2 | p) : all-ones
 *   5. all-reduce MIN of c: the lowest global index wins ties, and since every
 *      index belongs to exactly one rank the two payload bits of the winner
 *      travel with it                                              -> r
 *   6. index = r >> 2; value = NaN if payload bit 0 is clear, else best with
 *      the winner's sign when best is zero.
 * Bit-exact with the single-GPU kernel on the whole array, ties, NaN-first and
 * signed zeros included (the NaN written is the canonical quiet NaN). */
static size_t sh_count(const GpuArray *a) {
  size_t n = 1;
  unsigned int k;
  for (k = 0; k < a->nd; k++) n *= a->dimensions[k];
  return n;
}

/* The same over the communicator's peer windows (ga_comm.c,
 * templates/ga_exchange.cuh): the local kernel writes (v, i) with global
 * indices, ONE more launch pushes them into every peer's window over NVLink
 * and folds the peers' pairs - better value first, then lower index; a NaN can
 * only come from the shard that holds element 0 and is then the answer. The
 * winner's own bits are written, so signed zeros need no side channel. */
static int sharded_pair_peer(GpuReduction *gr, gpucomm *comm, GpuArray *d0, GpuArray *d1,
                             const GpuArray *s0, unsigned reduxLen, const int *reduxList,
                             const rd_shard *sh) {
  gpucontext *ctx = gr->ctx;
  const GpuArray *shape_of = d0 != NULL ? d0 : d1;
  const size_t n = sh_count(shape_of);
  GpuArray v, i, *pv = d0, *pi = d1;
  int have_v = 0, have_i = 0, err;

  if (d0 == NULL || !ga_array_is_c_contiguous(d0) || !GpuArray_ISALIGNED(d0) ||
      d0->typecode != gr->src_tc) {
    err = GpuArray_empty(&v, ctx, gr->src_tc, shape_of->nd, shape_of->dimensions, GA_C_ORDER);
    if (err != GA_NO_ERROR) return err;
    have_v = 1;
    pv = &v;
  }
  if (d1 == NULL || !ga_array_is_c_contiguous(d1) || !GpuArray_ISALIGNED(d1) ||
      gpuarray_get_elsize(d1->typecode) != 8) {
    err = GpuArray_empty(&i, ctx, GA_ULONG, shape_of->nd, shape_of->dimensions, GA_C_ORDER);
    if (err != GA_NO_ERROR) goto done;
    have_i = 1;
    pi = &i;
  }
  err = rd_call(gr->sh_pair, pv, pi, s0, reduxLen, reduxList, 0, sh);
  if (err != GA_NO_ERROR) goto done;
  err = ga_comm_exchange(comm, 1, op_is_min(gr->op) ? GA_MIN : GA_MAX, gr->src_tc,
                         pv->data->ptr + pv->offset, pi->data->ptr + pi->offset, n, 0);
  if (err != GA_NO_ERROR) goto done;
  if (have_v && d0 != NULL) err = GpuArray_move(d0, &v);
  if (err == GA_NO_ERROR && have_i && d1 != NULL) err = GpuArray_move(d1, &i);
done:
  if (have_v) GpuArray_clear(&v);
  if (have_i) GpuArray_clear(&i);
  return err;
}

static int sharded_pair(GpuReduction *gr, gpucomm *comm, GpuArray *d0, GpuArray *d1,
                        const GpuArray *s0, unsigned reduxLen, const int *reduxList,
                        const rd_shard *sh) {
  gpucontext *ctx = gr->ctx;
  const int is_min = op_is_min(gr->op), isf = tc_is_float(gr->src_tc), tc = gr->src_tc;
  const int half = tc == GA_HALF;
  const GpuArray *shape_of = d0 != NULL ? d0 : d1;
  GpuArray v, i, w, p, c;
  int have[5] = {0, 0, 0, 0, 0}, err, k;
  void *args[5];

  if (gr->sh_pair == NULL) {
    err = GpuReduction_new(&gr->sh_pair, ctx, is_min ? GA_REDUCE_MINANDARGMIN : GA_REDUCE_MAXANDARGMAX,
                           0, 0, tc, 0);
    if (err != GA_NO_ERROR) return err;
  }
  if (comm != NULL) {
    const size_t n = sh_count(shape_of);
    const size_t need = ((n * gpuarray_get_elsize(tc) + 15) & ~(size_t)15) + n * 8;
    if (ga_comm_peer_ready(comm, need))
      return sharded_pair_peer(gr, comm, d0, d1, s0, reduxLen, reduxList, sh);
  }
#define SH_TMP(arr, slot, typecode)                                                            \
  err = GpuArray_empty(&arr, ctx, typecode, shape_of->nd, shape_of->dimensions, GA_C_ORDER);   \
  if (err != GA_NO_ERROR) goto done;                                                           \
  have[slot] = 1;
  SH_TMP(v, 0, tc)
  SH_TMP(i, 1, GA_ULONG)
  SH_TMP(c, 4, GA_ULONG)
  err = rd_call(gr->sh_pair, &v, &i, s0, reduxLen, reduxList, 0, sh);
  if (err != GA_NO_ERROR) goto done;

  if (isf) {
    gpuelemwise_arg a1[3] = {{"v", tc, GE_READ}, {"w", tc, GE_WRITE}, {"p", GA_UBYTE, GE_WRITE}};
    SH_TMP(w, 2, tc)
    SH_TMP(p, 3, GA_UBYTE)
    err = sh_elemwise(ctx, &gr->sh_e1,
                      is_min ? "w = (v != v) ? -INFINITY : v; "
                               "p = ((v != v) ? 0 : 1) | ((v == 0 && signbit(v)) ? 2 : 0)"
                             : "w = (v != v) ? INFINITY : v; "
                               "p = ((v != v) ? 0 : 1) | ((v == 0 && signbit(v)) ? 2 : 0)",
                      3, a1, half);
    if (err != GA_NO_ERROR) goto done;
    args[0] = &v; args[1] = &w; args[2] = &p;
    err = GpuElemwise_call(gr->sh_e1, args, 0);
    if (err != GA_NO_ERROR) goto done;
  }
  {
    GpuArray *best = isf ? &w : &v; /* the all-reduce runs in place */
    GpuArray wl; /* the local values, kept for step 4 */
    int have_wl = 0;
    if (comm != NULL) {
      err = GpuArray_copy(&wl, best, GA_C_ORDER);
      if (err != GA_NO_ERROR) goto done;
      have_wl = 1;
      err = sh_all_reduce(best, is_min ? GA_MIN : GA_MAX, comm);
    }
    if (err == GA_NO_ERROR) {
      if (isf) {
        gpuelemwise_arg a2[5] = {{"w", tc, GE_READ}, {"b", tc, GE_READ}, {"i", GA_ULONG, GE_READ},
                                 {"p", GA_UBYTE, GE_READ}, {"c", GA_ULONG, GE_WRITE}};
        err = sh_elemwise(ctx, &gr->sh_e2,
                          "c = (w == b && i != 18446744073709551615ULL) ? ((i << 2) | p) "
                          ": 18446744073709551615ULL", 5, a2, half);
        args[0] = have_wl ? &wl : best; args[1] = best; args[2] = &i; args[3] = &p; args[4] = &c;
      } else {
        gpuelemwise_arg a2[4] = {{"w", tc, GE_READ}, {"b", tc, GE_READ}, {"i", GA_ULONG, GE_READ},
                                 {"c", GA_ULONG, GE_WRITE}};
        err = sh_elemwise(ctx, &gr->sh_e2,
                          "c = (w == b && i != 18446744073709551615ULL) ? ((i << 2) | 1) "
                          ": 18446744073709551615ULL", 4, a2, 0);
        args[0] = have_wl ? &wl : best; args[1] = best; args[2] = &i; args[3] = &c;
      }
      if (err == GA_NO_ERROR) err = GpuElemwise_call(gr->sh_e2, args, 0);
    }
    if (have_wl) GpuArray_clear(&wl);
    if (err != GA_NO_ERROR) goto done;
    err = sh_all_reduce(&c, GA_MIN, comm);
    if (err != GA_NO_ERROR) goto done;
    {
      /* step 6, written straight into the caller's destinations (any strides) */
      gpuelemwise_arg a3[4];
      unsigned n3 = 0;
      const int key = (d0 != NULL ? 1 << 8 : 0) | (d1 != NULL ? 1 << 9 : 0) |
                      (d1 != NULL ? d1->typecode : 0);
      char expr[256];
      a3[n3].name = "b"; a3[n3].typecode = tc; a3[n3].flags = GE_READ; args[n3++] = best;
      a3[n3].name = "r"; a3[n3].typecode = GA_ULONG; a3[n3].flags = GE_READ; args[n3++] = &c;
      expr[0] = '\0';
      if (d0 != NULL) {
        a3[n3].name = "o"; a3[n3].typecode = tc; a3[n3].flags = GE_WRITE; args[n3++] = d0;
        strcat(expr, isf ? "o = ((r & 1) == 0) ? NAN : ((b == 0) ? ((r & 2) ? -fabs(b) : fabs(b)) : b)"
                         : "o = b");
      }
      if (d1 != NULL) {
        a3[n3].name = "j"; a3[n3].typecode = d1->typecode; a3[n3].flags = GE_WRITE; args[n3++] = d1;
        strcat(expr, d0 != NULL ? "; j = r >> 2" : "j = r >> 2");
      }
      if (gr->sh_e3 != NULL && gr->sh_e3_key != key) {
        GpuElemwise_free(gr->sh_e3);
        gr->sh_e3 = NULL;
      }
      err = sh_elemwise(ctx, &gr->sh_e3, expr, n3, a3, half);
      if (err != GA_NO_ERROR) goto done;
      gr->sh_e3_key = key;
      err = GpuElemwise_call(gr->sh_e3, args, 0);
    }
  }
done:
#undef SH_TMP
  {
    GpuArray *tmp[5] = {&v, &i, &w, &p, &c};
    for (k = 0; k < 5; k++)
      if (have[k]) GpuArray_clear(tmp[k]);
  }
  return err;
}

int GpuReduction_call_sharded(const GpuReduction *cgr, gpucomm *comm, GpuArray *d0, GpuArray *d1,
                              const GpuArray *s0, unsigned reduxLen, const int *reduxList,
                              int shard_axis, size_t shard_lo, size_t shard_global, int flags) {
  GpuReduction *gr = (GpuReduction *)cgr;
  gpucontext *ctx;
  rd_shard sh;
  int err, opcode;
  if (gr == NULL) return GA_INVALID_ERROR;
  ctx = gr->ctx;
  if (s0 == NULL) return ga_err_set(ctx->err, GA_INVALID_ERROR, "Source array is NULL");
  if (shard_axis < 0 || (unsigned)shard_axis >= s0->nd)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "The sharded axis is out of range");
  sh.axis = shard_axis;
  sh.lo = shard_lo;
  sh.global = shard_global;
  if (gr->kind == 1) {
    if (!op_writes_val(gr->op)) d0 = NULL;
    if (!op_writes_idx(gr->op)) d1 = NULL;
    if (d0 == NULL && d1 == NULL)
      return ga_err_set(ctx->err, GA_INVALID_ERROR, "Destination is NULL");
    if ((op_writes_val(gr->op) && d0 == NULL) || (op_writes_idx(gr->op) && d1 == NULL))
      return ga_err_set(ctx->err, GA_INVALID_ERROR, "Destination is NULL");
    if (comm != NULL && d1 == NULL &&
        (!tc_is_float(gr->src_tc) || (reduxLen > 0 && reduxList[0] == shard_axis)) &&
        ga_comm_peer_ready(comm, sh_count(d0) * gpuarray_get_elsize(gr->src_tc) + 32)) {
      /* (+ 32: the rank's key follows the values in its slot, 16-byte aligned)
       * MIN / MAX without an index: the value-only kernel, then the exchange with the
       * shard's first coordinate as the tie-break key. When the sharded axis is the
       * slowest reduced one, every element of a lower shard precedes every element of a
       * higher one, so "equal values go to the lower shard" is the single-GPU rule (it
       * only shows between +0.0 and -0.0; integers have no distinguishable ties). */
      GpuArray tmp, *part = d0;
      const int use_tmp = !(GpuArray_IS_C_CONTIGUOUS(d0) || GpuArray_IS_F_CONTIGUOUS(d0)) ||
                          !GpuArray_ISALIGNED(d0) || d0->typecode != gr->src_tc;
      if (use_tmp) {
        err = GpuArray_empty(&tmp, ctx, gr->src_tc, d0->nd, d0->dimensions, GA_C_ORDER);
        if (err != GA_NO_ERROR) return err;
        part = &tmp;
      }
      err = rd_call(gr, part, NULL, s0, reduxLen, reduxList, flags, &sh);
      if (err == GA_NO_ERROR)
        err = ga_comm_exchange(comm, 2, op_is_min(gr->op) ? GA_MIN : GA_MAX, gr->src_tc,
                               part->data->ptr + part->offset, 0, sh_count(part),
                               (unsigned long long)shard_lo);
      if (err == GA_NO_ERROR && use_tmp) err = GpuArray_move(d0, &tmp);
      if (use_tmp) GpuArray_clear(&tmp);
      return err;
    }
    return sharded_pair(gr, comm, d0, d1, s0, reduxLen, reduxList, &sh);
  }
  /* accumulating operators: per-GPU partial of the final shape, ONE all-reduce */
  switch (gr->op) {
  case GA_REDUCE_SUM: opcode = GA_SUM; break;
  case GA_REDUCE_PROD: case GA_REDUCE_PRODNZ: opcode = GA_PROD; break;
  case GA_REDUCE_ALL: opcode = GA_MIN; break; /* destinations hold 0 / 1 */
  case GA_REDUCE_ANY: opcode = GA_MAX; break;
  case GA_REDUCE_AND: opcode = GA_XC_AND; break; /* peer windows only, checked below */
  case GA_REDUCE_OR: opcode = GA_XC_OR; break;
  case GA_REDUCE_XOR: opcode = GA_XC_XOR; break;
  default:
    return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR, "Operator cannot be combined across GPUs");
  }
  if (d0 == NULL) return ga_err_set(ctx->err, GA_INVALID_ERROR, "Value destination is NULL");
  if (opcode >= GA_XC_AND &&
      (comm == NULL || !ga_comm_peer_ready(comm, sh_count(d0) * gpuarray_get_elsize(d0->typecode))))
    return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR,
                      "Bitwise reductions are combined across GPUs through the communicator's peer "
                      "windows only: the collectives offer sum, prod, min and max");
  {
    GpuArray tmp, view;
    GpuArray *part = d0;
    int use_tmp = !(GpuArray_IS_C_CONTIGUOUS(d0) || GpuArray_IS_F_CONTIGUOUS(d0)) ||
                  !GpuArray_ISALIGNED(d0);
    if (use_tmp) {
      err = GpuArray_empty(&tmp, ctx, d0->typecode, d0->nd, d0->dimensions, GA_C_ORDER);
      if (err != GA_NO_ERROR) return err;
      part = &tmp;
    }
    err = rd_call(gr, part, NULL, s0, reduxLen, reduxList, flags, &sh);
    if (err == GA_NO_ERROR && comm != NULL &&
        ga_comm_peer_ready(comm, sh_count(part) * gpuarray_get_elsize(part->typecode))) {
      /* one launch over the peer windows; every rank folds in rank order */
      err = ga_comm_exchange(comm, 0, opcode, part->typecode == GA_BOOL ? GA_UBYTE : part->typecode,
                             part->data->ptr + part->offset, 0, sh_count(part), 0);
    } else if (err == GA_NO_ERROR && comm != NULL) {
      if (part->typecode == GA_BOOL) { /* the collectives know no bool: same bytes as unsigned */
        err = GpuArray_view(&view, part);
        if (err == GA_NO_ERROR) {
          view.typecode = GA_UBYTE;
          err = GpuArray_all_reduce(&view, &view, opcode, comm);
          GpuArray_clear(&view);
        }
      } else {
        err = GpuArray_all_reduce(part, part, opcode, comm);
      }
    }
    if (err == GA_NO_ERROR && use_tmp) err = GpuArray_move(d0, &tmp);
    if (use_tmp) GpuArray_clear(&tmp);
  }
  return err;
}

/* ------------------------------------------------- GpuArray_maxandargmax */

typedef struct mam_entry {
  int tc;
  GpuReduction *gr;
  struct mam_entry *next;
} mam_entry;

void ga_maxandargmax_cache_free(gpucontext *ctx) {
  mam_entry *e = (mam_entry *)ctx->maxandargmax_cache, *n;
  ctx->maxandargmax_cache = NULL;
  for (; e != NULL; e = n) {
    n = e->next;
    GpuReduction_free(e->gr);
    free(e);
  }
}

int GpuArray_maxandargmax(GpuArray *dstMax, GpuArray *dstArgmax, const GpuArray *src,
                          unsigned reduxLen, const unsigned *reduxList) {
  gpucontext *ctx;
  mam_entry *e;
  int axes[64], err;
  unsigned i;

  if (dstMax == NULL || dstArgmax == NULL || src == NULL || reduxList == NULL || src->data == NULL)
    return ga_err_set(ga_global_err, GA_INVALID_ERROR, "GpuArray_maxandargmax: NULL argument");
  ctx = GpuArray_context(src);
  if (src->nd == 0 || reduxLen == 0 || reduxLen > src->nd || reduxLen > 64)
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "Invalid rank or reduction axis count");
  for (i = 0; i < reduxLen; i++) {
    if (reduxList[i] >= src->nd)
      return ga_err_fmt(ctx->err, GA_INVALID_ERROR, "Reduction axis %u out of range", reduxList[i]);
    axes[i] = (int)reduxList[i];
  }
  for (e = (mam_entry *)ctx->maxandargmax_cache; e != NULL; e = e->next)
    if (e->tc == src->typecode) break;
  if (e == NULL) {
    e = calloc(1, sizeof(*e));
    if (e == NULL) return ga_err_sys(ctx->err, "calloc");
    err = GpuReduction_new(&e->gr, ctx, GA_REDUCE_MAXANDARGMAX, 0, 0, src->typecode, 0);
    if (err != GA_NO_ERROR) {
      free(e);
      return err;
    }
    e->tc = src->typecode;
    e->next = (mam_entry *)ctx->maxandargmax_cache;
    ctx->maxandargmax_cache = e;
  }
  return GpuReduction_call(e->gr, dstMax, dstArgmax, src, reduxLen, axes, 0);
}
