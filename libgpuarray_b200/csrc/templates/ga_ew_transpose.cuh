/* Tiled-transpose elementwise kernel: arguments disagree on which collapsed
 * dimension is contiguous in memory (e.g. an NHWC view combined into an NCHW
 * output).
 *
 * With the reference's strided kernel (src/gpuarray_elemwise.c:123-250) such a
 * call reads one element per 32-byte sector for every argument that is not
 * contiguous along the innermost dimension. Here a CTA owns a GA_EW_TP x
 * GA_EW_TQ tile over (P, Q): Q is the innermost collapsed dimension (the
 * orientation the expression is evaluated and outputs are written in), P the
 * dimension along which the "mode 3" inputs are contiguous. Those inputs are
 * read with 128-bit loads along P into shared memory and read back along Q,
 * so both sides of the transpose move full 128-byte lines.
 *
 * Per-argument mode (last field of GA_EW_ARRAYS):
 *   3  input contiguous along P: staged through shared memory
 *   1  contiguous along Q and aligned: 128-bit access, GA_EW_EPT elements
 *   2  input with stride 0 along Q: one scalar load per thread chunk
 *   0  anything else: scalar access with its own strides
 *
 * Needs the definitions listed in ga_ew_contig.cuh plus GA_EW_ND (>= 2),
 * GA_EW_NARR, GA_EW_TP, GA_EW_TQ.
 */
#include "ga_ew_common.cuh"

#define GA_EWT_NOUT ((GA_EW_ND > 2) ? (GA_EW_ND - 2) : 1)

/* Mirrors the block marshalled by call_transpose() in ga_elemwise.c. */
struct ga__ewt_layout {
  unsigned long long pdim, qdim, tiles_p, tiles_q, nouter;
  unsigned long long odims[GA_EWT_NOUT];       /* remaining dims, outermost first */
  long long strp[GA_EW_NARR], strq[GA_EW_NARR]; /* byte strides along P and Q */
  long long stro[GA_EW_NARR][GA_EWT_NOUT];      /* byte strides of the remaining dims */
};

/* shared-memory row pitch in elements: odd number of 32-bit words when possible */
#define GA__PITCH(S) (GA_EW_TP + ((sizeof(S) >= 4) ? 1 : (4 / sizeof(S))))

#define GA__P_ARR(k, n, S, C, R, W, M) , char *n##_p
#define GA__P_SC(n, T) , T n##_s
#define GA__ARG_ARR(k, n, S, C, R, W, M) n##_c[e],
#define GA__ARG_SC(n, T) n##_s,

#define GA__SMEM(k, n, S, C, R, W, M) \
  __shared__ S n##_sm[(M == 3) ? GA_EW_TQ : 1][(M == 3) ? GA__PITCH(S) : 1];

#define GA__BASE(k, n, S, C, R, W, M) long long n##_base = 0;
#define GA__BASE_STEP(k, n, S, C, R, W, M) n##_base += (long long)pos * L.stro[k][d];

/* stage a mode-3 input: vectors along P, rows along Q */
#define GA__STAGE(k, n, S, C, R, W, M)                                                        \
  if (M == 3) {                                                                               \
    constexpr int VP = (16 / sizeof(S)) < GA_EW_TP ? (16 / sizeof(S)) : GA_EW_TP;             \
    constexpr int PV = GA_EW_TP / VP; /* vectors per tile row */                              \
    const char *g_ = n##_p + n##_base + (long long)p0 * L.strp[k] + (long long)q0 * L.strq[k]; \
    const bool al_ = (((unsigned long long)g_) % (VP * sizeof(S)) == 0) &&                    \
                     (L.strq[k] % (long long)(VP * sizeof(S)) == 0);                          \
    for (int i_ = threadIdx.x; i_ < GA_EW_TQ * PV; i_ += GA_EW_THREADS) {                     \
      const int q_ = i_ / PV, pv_ = (i_ - q_ * PV) * VP;                                      \
      if ((unsigned long long)q_ < qn) {                                                      \
        const S *src_ = reinterpret_cast<const S *>(g_ + (long long)q_ * L.strq[k]) + pv_;    \
        if (al_ && (unsigned long long)(pv_ + VP) <= pn) {                                    \
          const ga__pack<S, VP> t_ = *reinterpret_cast<const ga__pack<S, VP> *>(src_);        \
          _Pragma("unroll") for (int j_ = 0; j_ < VP; j_++) n##_sm[q_][pv_ + j_] = t_.v[j_]; \
        } else {                                                                              \
          _Pragma("unroll") for (int j_ = 0; j_ < VP; j_++)                                   \
            if ((unsigned long long)(pv_ + j_) < pn) n##_sm[q_][pv_ + j_] = src_[j_];         \
        }                                                                                     \
      }                                                                                       \
    }                                                                                         \
  }

#define GA__DECL(k, n, S, C, R, W, M) C n##_c[GA_EW_EPT];

#define GA__LOAD(k, n, S, C, R, W, M)                                                         \
  if (R) {                                                                                    \
    if (M == 3) {                                                                             \
      _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++)                                   \
        n##_c[e] = ga__conv<C, S>::in(n##_sm[ql + e][pl]);                                    \
    } else {                                                                                  \
      const char *b_ = n##_p + n##_base + (long long)(p0 + pl) * L.strp[k];                   \
      if (M == 1) {                                                                           \
        ga__load_run<C, S, GA_EW_EPT>(                                                        \
            reinterpret_cast<const S *>(b_ + (long long)(q0 + ql) * (long long)sizeof(S)),    \
            n##_c);                                                                           \
      } else if (M == 2) {                                                                    \
        const C t_ = ga__conv<C, S>::in(*reinterpret_cast<const S *>(b_));                    \
        _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++) n##_c[e] = t_;                  \
      } else {                                                                                \
        _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++)                                 \
          if ((unsigned long long)(ql + e) < qn)                                              \
            n##_c[e] = ga__conv<C, S>::in(*reinterpret_cast<const S *>(                       \
                b_ + (long long)(q0 + ql + e) * L.strq[k]));                                  \
      }                                                                                       \
    }                                                                                         \
  }

#define GA__STORE(k, n, S, C, R, W, M)                                                        \
  if (W) {                                                                                    \
    char *b_ = n##_p + n##_base + (long long)(p0 + pl) * L.strp[k];                           \
    if (M == 1) {                                                                             \
      ga__store_run<C, S, GA_EW_EPT>(                                                         \
          reinterpret_cast<S *>(b_ + (long long)(q0 + ql) * (long long)sizeof(S)), n##_c);    \
    } else {                                                                                  \
      _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++)                                   \
        if ((unsigned long long)(ql + e) < qn)                                                \
          *reinterpret_cast<S *>(b_ + (long long)(q0 + ql + e) * L.strq[k]) =                 \
              ga__conv<C, S>::out(n##_c[e]);                                                  \
    }                                                                                         \
  }

extern "C" __global__ void __launch_bounds__(GA_EW_THREADS)
ga_ew_transpose(const __grid_constant__ ga__ewt_layout L
                GA_EW_ARRAYS(GA__P_ARR) GA_EW_SCALARS(GA__P_SC)) {
  GA_EW_ARRAYS(GA__SMEM)
  const unsigned long long ntiles = L.tiles_p * L.tiles_q * L.nouter;
  constexpr int QG = GA_EW_TQ / GA_EW_EPT; /* thread chunks per tile column */

  for (unsigned long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    /* tile coordinates: Q tiles fastest, then P tiles, then the outer index */
    unsigned long long r = t / L.tiles_q;
    const unsigned long long q0 = (t - r * L.tiles_q) * GA_EW_TQ;
    unsigned long long o = r / L.tiles_p;
    const unsigned long long p0 = (r - o * L.tiles_p) * GA_EW_TP;
    const unsigned long long pn = (L.pdim - p0 < GA_EW_TP) ? (L.pdim - p0) : GA_EW_TP;
    const unsigned long long qn = (L.qdim - q0 < GA_EW_TQ) ? (L.qdim - q0) : GA_EW_TQ;
    GA_EW_ARRAYS(GA__BASE)
#if GA_EW_ND > 2
#pragma unroll
    for (int d = GA_EW_ND - 3; d >= 0; d--) {
      const unsigned long long qq = o / L.odims[d];
      const unsigned long long pos = o - qq * L.odims[d];
      o = qq;
      GA_EW_ARRAYS(GA__BASE_STEP)
    }
#endif
    GA_EW_ARRAYS(GA__STAGE)
    __syncthreads();
    for (int it = threadIdx.x; it < GA_EW_TP * QG; it += GA_EW_THREADS) {
      const int pl = it / QG;
      const int ql = (it - pl * QG) * GA_EW_EPT;
      if ((unsigned long long)pl < pn && (unsigned long long)ql < qn) {
        GA_EW_ARRAYS(GA__DECL)
        GA_EW_ARRAYS(GA__LOAD)
#pragma unroll
        for (int e = 0; e < GA_EW_EPT; e++)
          ga_ew_apply(GA_EW_ARRAYS(GA__ARG_ARR) GA_EW_SCALARS(GA__ARG_SC) 0);
        GA_EW_ARRAYS(GA__STORE)
      }
    }
    __syncthreads();
  }
}
