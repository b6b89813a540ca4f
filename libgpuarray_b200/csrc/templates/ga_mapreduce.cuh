/* Reduction of a mapped expression over several broadcastable arguments:
 *
 *     out[kept...] = REDUCE over the reduced axes of MAP(arg0, arg1, ..., scalars)
 *
 * This is what pygpu's ReductionKernel computes (pygpu/reduction.py:33-134:
 * `acc = REDUCE(acc, MAP)` per element, a block per output with a
 * shared-memory tree, one div/mod per dimension, per argument, per element).
 * Here the map and the reduction share ONE pass over HBM, and the traversal is
 * picked from the arguments' strides like the one-array reductions of
 * ga_reduce.cuh:
 *
 *   ga_mr_rows     the innermost reduced dimension is contiguous (or broadcast)
 *                  in every array argument: a warp or a CTA owns one
 *                  (output, split) pair and streams 128-bit loads along it
 *   ga_mr_cols     the innermost KEPT dimension is contiguous (or broadcast):
 *                  a thread owns GA_MR_VEC adjacent outputs and walks down the
 *                  reduced extent; blockDim.y row lanes, gridDim.y splits
 *   ga_mr_general  anything else: GA_MR_TPO threads per output decode every
 *                  element's offsets
 *
 * Split reductions finish like ga_reduce.cuh's: every group stores its
 * partial, takes a ticket, and the last arriver combines all partials in split
 * order (nobody waits; results are bitwise repeatable).
 *
 * The including translation unit defines GA_EW_ARRAYS(X) / GA_EW_SCALARS(X) /
 * GA_EW_NARR exactly as for the elementwise templates (per array: index, name,
 * storage type S, type C seen by the expression, read, write, access mode),
 * the function ga_mr_map(args..., scalars..., 0) returning the mapped value,
 * and GA_MR_ACC_T, GA_MR_DST_T, GA_MR_REDUCE(a, b), GA_MR_NEUTRAL,
 * GA_MR_STORE(acc), GA_MR_VEC, GA_MR_THREADS, GA_MR_GROUP (rows: 32 or
 * GA_MR_THREADS), GA_MR_BY (cols), GA_MR_TPO (general) and one of
 * GA_MR_BUILD_ROWS / _COLS / _GENERAL.
 * Access modes: 1 = contiguous along the fast dimension and aligned (vector
 * loads), 2 = stride 0 along it (one load, replicated), 0 = gathered.
 */
#include "ga_ew_common.cuh"

/* the operator vocabulary of ga_reduce.cuh, for its states, shuffles, block
 * reduction, tickets and L2 loads */
#define GA_RD_SRC_T GA_MR_ACC_T
#define GA_RD_X_T GA_MR_ACC_T
#define GA_RD_ACC_T GA_MR_ACC_T
#define GA_RD_DST_T GA_MR_DST_T
#define GA_RD_LOAD(raw) (raw)
#define GA_RD_STORE(a) GA_MR_STORE(a)
#define GA_RD_MAP(x) (x)
#define GA_RD_COMBINE(a, b) GA_MR_REDUCE(a, b)
#define GA_RD_IDENT GA_MR_NEUTRAL
#define GA_RD_BETTER(b, a) (0)
#define GA_RD_KIND 0
#define GA_RD_ISFLOAT 0
#define GA_RD_WRITE_VAL 1
#define GA_RD_WRITE_IDX 0
#define GA_RD_IDX_T unsigned int
#define GA_RD_VEC GA_MR_VEC
#define GA_RD_THREADS GA_MR_THREADS
#include "ga_reduce.cuh"

#define GA_MR_MAXD 6

/* Mirrors the block marshalled by fill_layout() in ga_mapredux.c. */
struct ga__mr_layout {
  ga__u64 nf_total, nr_total;    /* outputs; reduced elements per output */
  ga__u64 nf, nr;                /* kept / reduced dimension counts */
  ga__u64 fdim[GA_MR_MAXD];      /* kept extents, outermost first */
  ga__i64 fdst[GA_MR_MAXD];      /* their byte strides in the destination */
  ga__u64 rdim[GA_MR_MAXD];      /* reduced extents in traversal order */
  ga__u64 splits;                /* groups (rows) / gridDim.y (cols) sharing one output */
  ga__u64 inner;                 /* rows: contiguous reduced run; cols: contiguous kept run */
  ga__u64 seg, nseg, units;      /* rows: elements per unit, units per run, units per output */
  ga__u64 tiles;                 /* cols: column tiles per contiguous kept run */
  ga__i64 fsrc[GA_EW_NARR][GA_MR_MAXD]; /* byte strides of the kept dims per argument */
  ga__i64 rsrc[GA_EW_NARR][GA_MR_MAXD]; /* ... of the reduced dims */
};

#define GA__MP_ARR(k, n, S, C, R, W, M) , const char *n##_p
#define GA__MP_SC(n, T) , T n##_s
#define GA__MARG_SC(n, T) n##_s,

/* per-argument running byte offsets */
#define GA__MOFF_DECL(k, n, S, C, R, W, M) ga__i64 n##_fo = 0;
#define GA__MOFF_FSTEP(k, n, S, C, R, W, M) n##_fo += (ga__i64)c_ * L.fsrc[k][d];
#define GA__MROW_DECL(k, n, S, C, R, W, M) ga__i64 n##_ro = 0;
#define GA__MROW_STEP(k, n, S, C, R, W, M) n##_ro += (ga__i64)c_ * L.rsrc[k][d];

/* byte offsets of output `o` in every argument: decode the kept coordinates once */
#define GA__MR_KEPT_OFFSETS(o_)                                   \
  GA_EW_ARRAYS(GA__MOFF_DECL)                                     \
  {                                                               \
    ga__u64 q_ = (o_);                                            \
    for (int d = (int)L.nf - 1; d >= 0; d--) {                    \
      const ga__u64 qq_ = d > 0 ? q_ / L.fdim[d] : 0;             \
      const ga__u64 c_ = q_ - qq_ * L.fdim[d];                    \
      q_ = qq_;                                                   \
      GA_EW_ARRAYS(GA__MOFF_FSTEP)                                \
    }                                                             \
  }

/* byte offsets of reduced position r_ over the reduced dims [0, nd_) */
#define GA__MR_ROW_OFFSETS(r_, nd_)                               \
  GA_EW_ARRAYS(GA__MROW_DECL)                                     \
  {                                                               \
    ga__u64 q_ = (r_);                                            \
    for (int d = (int)(nd_) - 1; d >= 0; d--) {                   \
      const ga__u64 qq_ = d > 0 ? q_ / L.rdim[d] : 0;             \
      const ga__u64 c_ = q_ - qq_ * L.rdim[d];                    \
      q_ = qq_;                                                   \
      GA_EW_ARRAYS(GA__MROW_STEP)                                 \
    }                                                             \
  }

static __device__ __forceinline__ void ga__mr_store(const ga__mr_layout &L, char *dst,
                                                    const ga__u64 o, const GA_MR_ACC_T v) {
  ga__i64 off = 0;
  ga__u64 q = o;
  for (int d = (int)L.nf - 1; d >= 0; d--) {
    const ga__u64 qq = d > 0 ? q / L.fdim[d] : 0;
    off += (ga__i64)(q - qq * L.fdim[d]) * L.fdst[d];
    q = qq;
  }
  *reinterpret_cast<GA_MR_DST_T *>(dst + off) = GA_MR_STORE(v);
}

/* ------------------------------------------------------------------ rows */
#if defined(GA_MR_BUILD_ROWS)
/* vector i of the run (mode 1), the run's single value (mode 2), or GA_MR_VEC
 * gathered elements (mode 0) */
#define GA__MR_VDECL(k, n, S, C, R, W, M) C n##_c[GA_MR_VEC];
#define GA__MR_VLOAD(k, n, S, C, R, W, M)                                                   \
  if (M == 1) {                                                                              \
    ga__load_run<C, S, GA_MR_VEC>(reinterpret_cast<const S *>(n##_rp) + (size_t)e0_, n##_c); \
  } else if (M == 2) {                                                                       \
    _Pragma("unroll") for (int j = 0; j < GA_MR_VEC; j++) n##_c[j] = n##_b;                  \
  } else {                                                                                   \
    _Pragma("unroll") for (int j = 0; j < GA_MR_VEC; j++)                                    \
      n##_c[j] = ga__conv<C, S>::in(*reinterpret_cast<const S *>(                            \
          n##_rp + (ga__i64)(e0_ + (unsigned)j) * n##_is));                                  \
  }
#define GA__MR_VARG(k, n, S, C, R, W, M) n##_c[j],
/* one element e_ of the run */
#define GA__MR_SARG(k, n, S, C, R, W, M)                                                     \
  ((M == 2) ? n##_b                                                                          \
            : ga__conv<C, S>::in(*reinterpret_cast<const S *>(n##_rp + (ga__i64)e_ * n##_is))),
#define GA__MR_RUN_SETUP(k, n, S, C, R, W, M)                                                \
  const ga__i64 n##_is = L.rsrc[k][nro];                                                     \
  const char *const n##_rp = n##_p + n##_fo + n##_ro + (ga__i64)seg0 * n##_is;               \
  const C n##_b = (M == 2) ? ga__conv<C, S>::in(*reinterpret_cast<const S *>(n##_rp)) : C();

extern "C" __global__ void __launch_bounds__(GA_MR_THREADS)
ga_mr_rows(const __grid_constant__ ga__mr_layout L, char *dst, GA_MR_ACC_T *pval,
           unsigned int *tickets GA_EW_ARRAYS(GA__MP_ARR) GA_EW_SCALARS(GA__MP_SC)) {
  ga__grid_dependency_sync();
#if GA_MR_GROUP > 32
  __shared__ ga__state sm[32];
  __shared__ int sm_last;
#endif
  const ga__u64 nwork = L.nf_total * L.splits;
  const int nro = (int)L.nr - 1;
  const unsigned lane = threadIdx.x % GA_MR_GROUP;
  const ga__u64 group = ((ga__u64)blockIdx.x * GA_MR_THREADS + threadIdx.x) / GA_MR_GROUP;
  const ga__u64 ngroups = (ga__u64)gridDim.x * (GA_MR_THREADS / GA_MR_GROUP);
  const ga__u64 rounds = (nwork + ngroups - 1) / ngroups;

  for (ga__u64 it = 0; it < rounds; it++) {
    const ga__u64 w = group + it * ngroups;
    const bool live = w < nwork;
    ga__u64 o = live ? w : 0, split = 0;
    if (L.splits > 1) {
      const ga__u64 ww = o;
      o = ww / L.splits;
      split = ww - o * L.splits;
    }
    ga__state st[GA_MR_VEC];
#pragma unroll
    for (int j = 0; j < GA_MR_VEC; j++) st[j] = ga__init();

    if (live) {
      const ga__u64 ub = split * L.units / L.splits, ue = (split + 1) * L.units / L.splits;
      GA__MR_KEPT_OFFSETS(o)
      for (ga__u64 u = ub; u < ue; u++) {
        ga__u64 r = u, g = 0;
        if (L.nseg > 1) {
          r = u / L.nseg;
          g = u - r * L.nseg;
        }
        GA__MR_ROW_OFFSETS(r, nro)
        const ga__u64 seg0 = g * L.seg;
        const unsigned int len = (unsigned int)((L.inner - seg0 < L.seg) ? (L.inner - seg0) : L.seg);
        const unsigned int nv = len / GA_MR_VEC;
        GA_EW_ARRAYS(GA__MR_RUN_SETUP)
#pragma unroll 4
        for (unsigned int i = lane; i < nv; i += GA_MR_GROUP) {
          const unsigned int e0_ = i * GA_MR_VEC;
          GA_EW_ARRAYS(GA__MR_VDECL)
          GA_EW_ARRAYS(GA__MR_VLOAD)
#pragma unroll
          for (int j = 0; j < GA_MR_VEC; j++)
            st[j].v = GA_MR_REDUCE(st[j].v, ga_mr_map(GA_EW_ARRAYS(GA__MR_VARG)
                                                          GA_EW_SCALARS(GA__MARG_SC) 0));
        }
        for (unsigned int e_ = nv * GA_MR_VEC + lane; e_ < len; e_ += GA_MR_GROUP)
          st[0].v = GA_MR_REDUCE(st[0].v, ga_mr_map(GA_EW_ARRAYS(GA__MR_SARG)
                                                    GA_EW_SCALARS(GA__MARG_SC) 0));
      }
    }
#pragma unroll
    for (int j = 1; j < GA_MR_VEC; j++) ga__merge(st[0], st[j]);
#if GA_MR_GROUP > 32
    const ga__state tot = ga__block_reduce(st[0], sm, threadIdx.x, GA_MR_THREADS);
#else
    const ga__state tot = ga__warp_reduce(st[0]);
#endif
    if (L.splits == 1) {
      if (live && lane == 0) ga__mr_store(L, dst, o, tot.v);
#if GA_MR_GROUP > 32
      __syncthreads();
#endif
    } else {
      int last = 0;
      if (live && lane == 0) {
        pval[o * L.splits + split] = tot.v;
        last = ga__take_ticket(&tickets[o], (unsigned int)L.splits) ? 1 : 0;
      }
#if GA_MR_GROUP > 32
      if (lane == 0) sm_last = last;
      __syncthreads();
      last = sm_last;
#else
      last = __shfl_sync(0xffffffffu, last, 0);
#endif
      ga__state fin = ga__init();
      if (last) {
        /* a lane combines its partials in increasing split order; the lanes are
         * then merged in the fixed order of the tree below */
        for (ga__u64 sp = lane; sp < L.splits; sp += GA_MR_GROUP) {
          ga__state t;
          t.v = ga__ldcg(&pval[o * L.splits + sp]);
          ga__merge(fin, t);
        }
      }
#if GA_MR_GROUP > 32
      fin = ga__block_reduce(fin, sm, threadIdx.x, GA_MR_THREADS);
      __syncthreads();
#else
      fin = ga__warp_reduce(fin);
#endif
      if (last && lane == 0) ga__mr_store(L, dst, o, fin.v);
    }
  }
}
#endif

/* ------------------------------------------------------------------ cols */
#if defined(GA_MR_BUILD_COLS)
/* GA_MR_VEC adjacent outputs of one reduced position */
#define GA__MC_VDECL(k, n, S, C, R, W, M) C n##_c[GA_MR_VEC];
#define GA__MC_VLOAD(k, n, S, C, R, W, M)                                                   \
  {                                                                                          \
    const char *a_ = n##_p + n##_fo + n##_ro;                                                \
    if (M == 1) {                                                                            \
      ga__load_run<C, S, GA_MR_VEC>(reinterpret_cast<const S *>(a_), n##_c);                 \
    } else if (M == 2) {                                                                     \
      const C t_ = ga__conv<C, S>::in(*reinterpret_cast<const S *>(a_));                     \
      _Pragma("unroll") for (int j = 0; j < GA_MR_VEC; j++) n##_c[j] = t_;                   \
    } else {                                                                                 \
      _Pragma("unroll") for (int j = 0; j < GA_MR_VEC; j++)                                  \
        n##_c[j] = ga__conv<C, S>::in(                                                       \
            *reinterpret_cast<const S *>(a_ + (ga__i64)j * L.fsrc[k][L.nf - 1]));            \
    }                                                                                        \
  }
#define GA__MC_VARG(k, n, S, C, R, W, M) n##_c[j],
#define GA__MC_COLOFF(k, n, S, C, R, W, M) n##_fo += (ga__i64)col0 * L.fsrc[k][L.nf - 1];

extern "C" __global__ void __launch_bounds__(32 * GA_MR_BY)
ga_mr_cols(const __grid_constant__ ga__mr_layout L, char *dst, GA_MR_ACC_T *pval,
           unsigned int *tickets GA_EW_ARRAYS(GA__MP_ARR) GA_EW_SCALARS(GA__MP_SC)) {
  ga__grid_dependency_sync();
  __shared__ ga__state sm[GA_MR_BY][GA_MR_VEC][32];
  __shared__ int sm_last;
  const unsigned tx = threadIdx.x, ty = threadIdx.y;
  const ga__u64 kc = L.inner;
  const ga__u64 ko_total = L.nf_total / kc;
  const ga__u64 nwork = ko_total * L.tiles;
  const ga__u64 split = blockIdx.y;
  const ga__u64 nblk = (L.nr_total + GA_MR_BY - 1) / GA_MR_BY;

  for (ga__u64 w = blockIdx.x; w < nwork; w += gridDim.x) {
    ga__u64 ko = 0, tile = w;
    if (ko_total > 1) {
      ko = w / L.tiles;
      tile = w - ko * L.tiles;
    }
    const ga__u64 col0 = (tile * 32 + tx) * GA_MR_VEC;
    const bool live = col0 < kc;      /* kc is a multiple of GA_MR_VEC (host) */
    const ga__u64 o0 = ko * kc + col0;
    ga__state st[GA_MR_VEC];
#pragma unroll
    for (int j = 0; j < GA_MR_VEC; j++) st[j] = ga__init();

    if (live) {
      /* offsets of the outer kept position ko (kept dims but the innermost), plus the column */
      GA_EW_ARRAYS(GA__MOFF_DECL)
      {
        ga__u64 q_ = ko;
        for (int d = (int)L.nf - 2; d >= 0; d--) {
          const ga__u64 qq_ = d > 0 ? q_ / L.fdim[d] : 0;
          const ga__u64 c_ = q_ - qq_ * L.fdim[d];
          q_ = qq_;
          GA_EW_ARRAYS(GA__MOFF_FSTEP)
        }
      }
      GA_EW_ARRAYS(GA__MC_COLOFF)
      const unsigned int cnt =
          (nblk > split) ? (unsigned int)((nblk - split + L.splits - 1) / L.splits) : 0u;
#pragma unroll 4
      for (unsigned int n = 0; n < cnt; n++) {
        const ga__u64 jr = ((ga__u64)n * L.splits + split) * GA_MR_BY + ty;
        if (jr >= L.nr_total) break;
        GA__MR_ROW_OFFSETS(jr, L.nr)
        GA_EW_ARRAYS(GA__MC_VDECL)
        GA_EW_ARRAYS(GA__MC_VLOAD)
#pragma unroll
        for (int j = 0; j < GA_MR_VEC; j++)
          st[j].v = GA_MR_REDUCE(st[j].v, ga_mr_map(GA_EW_ARRAYS(GA__MC_VARG)
                                                    GA_EW_SCALARS(GA__MARG_SC) 0));
      }
    }
#pragma unroll
    for (int k = 0; k < GA_MR_VEC; k++) sm[ty][k][tx] = st[k];
    __syncthreads();
    if (ty < GA_MR_VEC && live) {
      ga__state tot = sm[0][ty][tx];
#pragma unroll
      for (int y = 1; y < GA_MR_BY; y++) ga__merge(tot, sm[y][ty][tx]);
      if (L.splits == 1) ga__mr_store(L, dst, o0 + ty, tot.v);
      else pval[split * L.nf_total + o0 + ty] = tot.v;
    }
    if (L.splits > 1) {
      __syncthreads();
      if (tx == 0 && ty == 0) sm_last = ga__take_ticket(&tickets[w], (unsigned int)L.splits) ? 1 : 0;
      __syncthreads();
      if (sm_last) {
        ga__state fin[GA_MR_VEC];
#pragma unroll
        for (int k = 0; k < GA_MR_VEC; k++) fin[k] = ga__init();
        if (live) {
          for (ga__u64 sp = ty; sp < L.splits; sp += GA_MR_BY) {
#pragma unroll
            for (int k = 0; k < GA_MR_VEC; k++) {
              ga__state t;
              t.v = ga__ldcg(&pval[sp * L.nf_total + o0 + k]);
              ga__merge(fin[k], t);
            }
          }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GA_MR_VEC; k++) sm[ty][k][tx] = fin[k];
        __syncthreads();
        if (ty < GA_MR_VEC && live) {
          ga__state tot = sm[0][ty][tx];
#pragma unroll
          for (int y = 1; y < GA_MR_BY; y++) ga__merge(tot, sm[y][ty][tx]);
          ga__mr_store(L, dst, o0 + ty, tot.v);
        }
      }
    }
    __syncthreads();
  }
}
#endif

/* --------------------------------------------------------------- general */
#if defined(GA_MR_BUILD_GENERAL)
#define GA__MG_ARG(k, n, S, C, R, W, M) \
  ga__conv<C, S>::in(*reinterpret_cast<const S *>(n##_p + n##_fo + n##_ro)),

extern "C" __global__ void __launch_bounds__(GA_MR_THREADS)
ga_mr_general(const __grid_constant__ ga__mr_layout L, char *dst, GA_MR_ACC_T *pval,
              unsigned int *tickets GA_EW_ARRAYS(GA__MP_ARR) GA_EW_SCALARS(GA__MP_SC)) {
  ga__grid_dependency_sync();
#if GA_MR_TPO > 32
  __shared__ ga__state sm[32];
#endif
  const unsigned lane = threadIdx.x % GA_MR_TPO;
  const ga__u64 group = ((ga__u64)blockIdx.x * GA_MR_THREADS + threadIdx.x) / GA_MR_TPO;
  const ga__u64 ngroups = (ga__u64)gridDim.x * (GA_MR_THREADS / GA_MR_TPO);
  const ga__u64 rounds = (L.nf_total + ngroups - 1) / ngroups;

  for (ga__u64 it = 0; it < rounds; it++) {
    const ga__u64 o = group + it * ngroups;
    const bool live = o < L.nf_total;
    ga__state st = ga__init();
    if (live) {
      GA__MR_KEPT_OFFSETS(o)
      for (ga__u64 jr = lane; jr < L.nr_total; jr += GA_MR_TPO) {
        GA__MR_ROW_OFFSETS(jr, L.nr)
        st.v = GA_MR_REDUCE(st.v, ga_mr_map(GA_EW_ARRAYS(GA__MG_ARG) GA_EW_SCALARS(GA__MARG_SC) 0));
      }
    }
#if GA_MR_TPO == 32
    st = ga__warp_reduce(st);
#elif GA_MR_TPO > 32
    st = ga__block_reduce(st, sm, threadIdx.x, GA_MR_THREADS);
    __syncthreads();
#endif
    if (live && lane == 0) ga__mr_store(L, dst, o, st.v);
  }
}
#endif
