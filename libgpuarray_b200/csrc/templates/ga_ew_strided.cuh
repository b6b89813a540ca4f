/* Strided / broadcast elementwise kernel over GA_EW_ND collapsed dimensions.
 *
 * Replaces the per-rank kernels of the reference's gen_elemwise_basic_kernel
 * (src/gpuarray_elemwise.c:123-250), which decode every element index with
 * nd-1 run-time divisions and issue one scalar access per element. Here a
 * thread owns a chunk of GA_EW_EPT consecutive positions of the innermost
 * dimension, so the index is decoded once per chunk (with multiply-high
 * division when indices fit 32 bits), and each argument is accessed in the
 * way its innermost stride allows:
 *   mode 1  stride == element size, aligned: 128-bit loads/stores
 *   mode 2  stride == 0 (broadcast input): one load, replicated
 *   mode 0  anything else: one scalar access per element
 * Byte offsets are always 64-bit.
 *
 * Needs the definitions listed in ga_ew_contig.cuh plus GA_EW_ND,
 * GA_EW_NARR, GA_EW_IDX32 (0/1), GA_EW_OFF32 (0/1).
 */
#include "ga_ew_common.cuh"

#ifndef GA_EW_OFF32
#define GA_EW_OFF32 0
#endif
#define GA_EW_NOUT ((GA_EW_ND > 1) ? (GA_EW_ND - 1) : 1)

/* Mirrors the block the host marshals in ga_elemwise.c (all 8-byte units). */
struct ga__ew_layout {
  unsigned long long nchunks;          /* rows * cpr */
  unsigned long long inner;            /* extent of the innermost dimension */
  unsigned long long cpr;              /* chunks per row = ceil(inner / EPT) */
  unsigned long long dims[GA_EW_NOUT]; /* outer extents, outermost first */
  ga__div32 div_cpr;
  ga__div32 div_dims[GA_EW_NOUT];
  long long str[GA_EW_NARR][GA_EW_ND]; /* byte strides */
};

#define GA__P_ARR(k, n, S, C, R, W, M) , char *n##_p
#define GA__P_SC(n, T) , T n##_s
/* byte offset of a row: 32-bit arithmetic when the host found that no argument
 * spans 2 GiB (one multiply-add per dimension instead of a 64-bit product) */
#if GA_EW_OFF32
typedef int ga__ew_off;
#else
typedef long long ga__ew_off;
#endif
#define GA__DECL(k, n, S, C, R, W, M) C n##_c[GA_EW_EPT]; ga__ew_off n##_off = 0;
#define GA__STEP(k, n, S, C, R, W, M) n##_off += (ga__ew_off)pos * (ga__ew_off)L.str[k][d];
#define GA__STEP0(k, n, S, C, R, W, M) n##_off += (ga__ew_off)r * (ga__ew_off)L.str[k][0];
#define GA__ARG_ARR(k, n, S, C, R, W, M) n##_c[e],
#define GA__ARG_SC(n, T) n##_s,

#define GA__LOAD(k, n, S, C, R, W, M)                                                      \
  if (R) {                                                                                 \
    const char *b_ = n##_p + n##_off;                                                      \
    if (M == 1) {                                                                          \
      ga__load_run<C, S, GA_EW_EPT>(                                                       \
          reinterpret_cast<const S *>(b_ + (long long)w0 * (long long)sizeof(S)), n##_c);  \
    } else if (M == 2) {                                                                   \
      const C t_ = ga__conv<C, S>::in(*reinterpret_cast<const S *>(b_));                   \
      _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++) n##_c[e] = t_;                 \
    } else {                                                                               \
      const long long s_ = L.str[k][GA_EW_ND - 1];                                         \
      _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++)                                \
        if (w0 + e < W_)                                                                   \
          n##_c[e] = ga__conv<C, S>::in(                                                   \
              *reinterpret_cast<const S *>(b_ + (long long)(w0 + e) * s_));                \
    }                                                                                      \
  }

#define GA__STORE(k, n, S, C, R, W, M)                                                     \
  if (W) {                                                                                 \
    char *b_ = n##_p + n##_off;                                                            \
    if (M == 1) {                                                                          \
      ga__store_run<C, S, GA_EW_EPT>(                                                      \
          reinterpret_cast<S *>(b_ + (long long)w0 * (long long)sizeof(S)), n##_c);        \
    } else {                                                                               \
      const long long s_ = L.str[k][GA_EW_ND - 1];                                         \
      _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++)                                \
        if (w0 + e < W_)                                                                   \
          *reinterpret_cast<S *>(b_ + (long long)(w0 + e) * s_) =                          \
              ga__conv<C, S>::out(n##_c[e]);                                               \
    }                                                                                      \
  }

extern "C" __global__ void __launch_bounds__(GA_EW_THREADS)
ga_ew_strided(const __grid_constant__ ga__ew_layout L
              GA_EW_ARRAYS(GA__P_ARR) GA_EW_SCALARS(GA__P_SC)) {
  ga__grid_dependency_sync();
  const GA_EW_IDX nchunks = (GA_EW_IDX)L.nchunks;
  const GA_EW_IDX W_ = (GA_EW_IDX)L.inner;
  const GA_EW_IDX nthr = (GA_EW_IDX)gridDim.x * GA_EW_THREADS;

  for (GA_EW_IDX c = (GA_EW_IDX)blockIdx.x * GA_EW_THREADS + threadIdx.x; c < nchunks;
       c += nthr) {
    GA_EW_ARRAYS(GA__DECL)
#if GA_EW_IDX32
    GA_EW_IDX r = ga__divide(c, L.div_cpr);
#else
    GA_EW_IDX r = c / (GA_EW_IDX)L.cpr;
#endif
    const GA_EW_IDX w0 = (c - r * (GA_EW_IDX)L.cpr) * GA_EW_EPT;
#if GA_EW_ND > 1
#pragma unroll
    for (int d = GA_EW_ND - 2; d >= 1; d--) {
#if GA_EW_IDX32
      const GA_EW_IDX q = ga__divide(r, L.div_dims[d]);
#else
      const GA_EW_IDX q = r / (GA_EW_IDX)L.dims[d];
#endif
      const GA_EW_IDX pos = r - q * (GA_EW_IDX)L.dims[d];
      r = q;
      GA_EW_ARRAYS(GA__STEP)
    }
    GA_EW_ARRAYS(GA__STEP0)
#endif
    GA_EW_ARRAYS(GA__LOAD)
#pragma unroll
    for (int e = 0; e < GA_EW_EPT; e++)
      ga_ew_apply(GA_EW_ARRAYS(GA__ARG_ARR) GA_EW_SCALARS(GA__ARG_SC) 0);
    GA_EW_ARRAYS(GA__STORE)
  }
}
