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
} rd_layout;

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
  if (gr->kind == 1) {
    const int mn = op_is_min(gr->op);
    if (gr->src_tc == GA_DOUBLE)
      ga_strb_printf(&sb, "#define GA_RD_PICK(a, b) %s((a), (b))\n", mn ? "fmin" : "fmax");
    else if (tc_is_float(gr->src_tc))
      ga_strb_printf(&sb, "#define GA_RD_PICK(a, b) %s((a), (b))\n", mn ? "fminf" : "fmaxf");
    else
      ga_strb_printf(&sb, "#define GA_RD_PICK(a, b) ((a) %s (b) ? (a) : (b))\n", mn ? "<" : ">");
  }
  ga_strb_printf(&sb, "#define GA_RD_KIND %d\n#define GA_RD_ISFLOAT %d\n#define GA_RD_WRITE_VAL %d\n"
                      "#define GA_RD_WRITE_IDX %d\n#define GA_RD_IDX_T %s\n#define GA_RD_VEC %d\n"
                      "#define GA_RD_THREADS %d\n#define GA_RD_TPO %d\n"
                      "#define GA_RD_BY %d\n#define GA_RD_GROUP %d\n#define GA_RD_FLAT %d\n"
                      "#define GA_RD_MU %d\n#define GA_RD_ONERUN %d\n#define GA_RD_FAST8 %d\n#define GA_RD_LAZY %d\n"
                      "#define %s\n"
                      "#include \"ga_reduce.cuh\"\n",
                 gr->kind, tc_is_float(gr->src_tc), v->write_val, v->write_idx,
                 v->idx64 ? "unsigned long long" : "unsigned int", v->vec, RD_THREADS, v->tpo,
                 RD_BY, v->group ? v->group : RD_THREADS, v->flat, v->mu ? v->mu : 1, v->onerun, v->fast8, v->lazy,
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
        v->onerun == want->onerun && v->fast8 == want->fast8 && v->lazy == want->lazy)
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
  v->next = gr->variants;
  gr->variants = v;
  return v;
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
  v.group = group & 0xffff; /* bits 16-19: runs at once, bit 20: one-run mode, bit 21: flattened */
  v.mu = (group >> 16) & 0xf;
  v.onerun = (group >> 20) & 1;
  v.flat = (group >> 21) & 1;
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
                     unsigned reduxLen, const int *reduxList) {
  unsigned i, k, n;
  unsigned long long mul;

  memset(L, 0, sizeof(*L));
  L->nf_total = 1;
  L->nr_total = 1;

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
      L->nr_total *= dsz;
      if (dsz != 1) {
        if (m == 64)
          return ga_err_set(e, GA_UNSUPPORTED_ERROR, "More than 64 reduced axes");
        dim[m] = dsz;
        str[m] = s->strides[ax];
        w[m] = kind == 1 ? mul : 0;
        m++;
      }
      mul *= dsz;
    }
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
 * cols_ctas_per_sm,onerun_ctas_per_sm,onerun_loads_per_lane,onerun_outputs_at_once,
 * lazy_index (0/1),lazy_min_vectors_per_lane". The
 * defaults are the best of sweeps on a B200. */
static unsigned rd_cols_ctas_per_sm = 3;
static unsigned rd_onerun_ctas_per_sm = 3, rd_onerun_lpl = 4, rd_onerun_mu = 0, rd_lazy = 1, rd_lazy_min = 32;

static void rd_tuning(unsigned *ctas_per_sm, unsigned *seg_vecs, unsigned *warp_bytes) {
  static int parsed = 0;
  static unsigned t_ctas = 32, t_seg = 16, t_warp = 0x7fffffff;
  *warp_bytes = t_warp;
  if (!parsed) {
    const char *env = getenv("GPUARRAY_B200_RD");
    if (env != NULL)
      sscanf(env, "%u,%u,%u,%u,%u,%u,%u,%u,%u", &t_ctas, &t_seg, &t_warp, &rd_cols_ctas_per_sm,
             &rd_onerun_ctas_per_sm, &rd_onerun_lpl, &rd_onerun_mu, &rd_lazy, &rd_lazy_min);
    if (rd_cols_ctas_per_sm == 0) rd_cols_ctas_per_sm = 3;
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
  want->idx64 = L->nr_total >= 0xffffffffULL;
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
      if (rows_outer == 1 && nload <= 256) {
        unsigned g = 1, lpl;
        while (g < 32 && g * rd_onerun_lpl < nload) g *= 2;
        lpl = (unsigned)((nload + g - 1) / g);
        want->onerun = 1;
        want->group = (int)g;
        want->mu = rd_onerun_mu ? (int)rd_onerun_mu : lpl <= 2 ? 4 : 2;
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
      else if (L->nf_total >= (unsigned long long)in->num_sms * 16) want->group = 32;
      else if (L->nf_total >= (unsigned long long)in->num_sms * 4 && nvrow >= 1024)
        want->group = RD_THREADS;
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
      if (want->group == RD_THREADS) want->flat = 0, want->mu = 1;
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
    s = ((unsigned long long)in->num_sms * rd_cols_ctas_per_sm + nwork - 1) / nwork;
    if (s > (L->nr_total + RD_BY * 8 - 1) / (RD_BY * 8)) s = (L->nr_total + RD_BY * 8 - 1) / (RD_BY * 8);
    if (s > 1024) s = 1024;
    L->splits = s ? s : 1;
    L->units = nwork; /* tickets: one per column tile */
    grid[0] = nwork > 0x7fffffffULL ? 0x7fffffffu : (unsigned)nwork;
    grid[1] = (unsigned)L->splits;
    block[0] = 32;
    block[1] = RD_BY;
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
 * out[0..19] = shape (0 rows, 1 cols, 2 general), vec, group, flat, runs at
 * once, one-run mode, lazy index, byte folding, threads per output (general),
 * 64-bit index, splits, seg, nseg, units, grid x, grid y, block x, block y,
 * outputs, reduced elements per output. Returns a GA_* code. */
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
                  reduxLen, reduxList);
  if (err != GA_NO_ERROR) return err;
  memset(out, 0, 20 * sizeof(*out));
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

int GpuReduction_call(const GpuReduction *cgr, GpuArray *d0, GpuArray *d1, const GpuArray *s0,
                      unsigned reduxLen, const int *reduxList, int flags) {
  GpuReduction *gr = (GpuReduction *)cgr;
  gpucontext *ctx;
  unsigned char red[64];
  rd_layout L;
  rd_variant want, *v1;
  unsigned i, ndd;
  unsigned grid[3] = {1, 1, 1}, block[3] = {RD_THREADS, 1, 1};
  int err = GA_NO_ERROR, need_val, need_idx;
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

  err = normalise(gr->kind, ctx->err, &L, d0, d1, s0, red, reduxLen, reduxList);
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
    err = rd_plan(&in, &L, &want, grid, block);
    if (err != GA_NO_ERROR) return err;
  }
  v1 = get_variant(gr, &want, &err);
  if (v1 == NULL) return err;
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
