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
 * so both sides of the transpose move whole cache lines.
 *
 * Shared memory holds 32-bit words (GA_EW_PW = 4 / element size elements per
 * word for 1- and 2-byte types) in rows of TP/PW + 1 words. The odd pitch
 * makes both phases free of bank conflicts: staging writes the four words of
 * a 128-bit load from 8 lanes x 4 rows, evaluation reads one word per row
 * from 4 row-chunks x 8 word-columns. A thread evaluates the expression on
 * GA_EW_PWI adjacent P positions x GA_EW_EPT consecutive Q positions and
 * stores GA_EW_PWI vectors of GA_EW_EPT elements.
 *
 * Per-argument mode (last field of GA_EW_ARRAYS):
 *   3  input contiguous along P: staged through shared memory
 *   1  contiguous along Q and aligned: 128-bit access, GA_EW_EPT elements
 *   2  input with stride 0 along Q: one scalar load per P position
 *   0  anything else: scalar access with its own strides
 *
 * GA_EW_LDSM = 1 (every staged input has 2-byte elements, GA_EW_EPT == 8, TP a
 * multiple of 64, TQ of 32): the tile goes to shared memory with 16-byte
 * asynchronous copies (cp.async, no registers in between) into unpadded rows
 * whose 16-byte chunks are XOR-swizzled by the row, and comes back with
 * ldmatrix.x4.trans: one instruction hands a thread 8 consecutive Q positions
 * of one P position, i.e. one 128-bit store. A warp covers 8 P positions x 32
 * Q positions per step. Both the copies (8 lanes fill one 128-byte row
 * segment) and the matrix loads (the 8 rows of a matrix are 8 distinct chunk
 * columns) are free of bank conflicts.
 *
 * Needs the definitions listed in ga_ew_contig.cuh plus GA_EW_ND (>= 2),
 * GA_EW_NARR, GA_EW_TP, GA_EW_TQ, GA_EW_PWI (P positions per thread; 1 with
 * GA_EW_LDSM).
 */
#include "ga_ew_common.cuh"

#ifndef GA_EW_LDSM
#define GA_EW_LDSM 0
#endif

#define GA_EWT_NOUT ((GA_EW_ND > 2) ? (GA_EW_ND - 2) : 1)

/* Mirrors the block marshalled by call_transpose() in ga_elemwise.c. */
struct ga__ewt_layout {
  unsigned long long pdim, qdim, tiles_p, tiles_q, nouter;
  unsigned long long odims[GA_EWT_NOUT];       /* remaining dims, outermost first */
  long long strp[GA_EW_NARR], strq[GA_EW_NARR]; /* byte strides along P and Q */
  long long stro[GA_EW_NARR][GA_EWT_NOUT];      /* byte strides of the remaining dims */
};

/* shared-memory word for storage type S and elements per word */
template <int BYTES> struct ga__word { typedef unsigned int type; };
template <> struct ga__word<8> { typedef unsigned long long type; };
#define GA__W(S) typename ga__word<(sizeof(S) > 4 ? 8 : 4)>::type
#define GA__WT(S) ga__word<(sizeof(S) > 4 ? 8 : 4)>::type
#define GA__PW(S) ((sizeof(S) < 4) ? (4 / (int)sizeof(S)) : 1)
#define GA__PITCHW(S) (GA_EW_TP / GA__PW(S) + 1)

/* Which (row, 128-bit vector) of the tile a staging slot touches. A warp
 * covers 4 rows x 8 vectors when the row has a multiple of 8 vectors: its
 * four 32-bit stores per lane then hit 32 distinct banks (rows are an odd
 * number of words apart), and each row still receives 128 contiguous bytes. */
template <int PV>
static __device__ __forceinline__ void ga__stage_map(const int i, int &q, int &v) {
  if (PV % 8 == 0 && GA_EW_TQ % 4 == 0) {
    const int lane = i & 31, blk = i >> 5;
    const int rq = blk / (PV / 8), vb = blk - rq * (PV / 8);
    q = rq * 4 + (lane >> 3);
    v = vb * 8 + (lane & 7);
  } else {
    q = i / PV;
    v = i - q * PV;
  }
}

#define GA__P_ARR(k, n, S, C, R, W, M) , char *n##_p
#define GA__P_SC(n, T) , T n##_s
#define GA__ARG_ARR(k, n, S, C, R, W, M) n##_c[kk][e],
#define GA__ARG_SC(n, T) n##_s,

#if GA_EW_LDSM
/* chunk swizzle of tile row q: the 8 rows one ldmatrix matrix takes (q = 8a + 2m + b for
 * a = 0..3, b = 0..1, fixed m) get 8 different values */
static __device__ __forceinline__ int ga__swz(const int q) { return (((q >> 3) & 3) << 1) | (q & 1); }
#define GA__SMEM(k, n, S, C, R, W, M) \
  alignas(128) __shared__ unsigned char n##_sm[(M == 3) ? GA_EW_TQ * GA_EW_TP * 2 : 16];
#else
#define GA__SMEM(k, n, S, C, R, W, M) \
  __shared__ GA__WT(S) n##_sm[(M == 3) ? GA_EW_TQ : 1][(M == 3) ? GA__PITCHW(S) : 1];
#endif

#define GA__BASE(k, n, S, C, R, W, M) long long n##_base = 0;
#define GA__BASE_STEP(k, n, S, C, R, W, M) n##_base += (long long)pos * L.stro[k][d];
#define GA__BASE_FIN(k, n, S, C, R, W, M) \
  char *const n##_t = n##_p + n##_base + (long long)p0 * L.strp[k] + (long long)q0 * L.strq[k];

#if GA_EW_LDSM
/* stage a mode-3 input: 16-byte asynchronous copies along P into swizzled rows */
#define GA__STAGE(k, n, S, C, R, W, M)                                                        \
  if (M == 3) {                                                                               \
    constexpr int CH = GA_EW_TP / 8; /* 16-byte chunks per tile row */                        \
    const long long sq_ = L.strq[k];                                                          \
    const bool al_ = (((unsigned long long)n##_t) % 16 == 0) && (sq_ % 16 == 0) &&            \
                     (pn == GA_EW_TP);                                                        \
    if (al_) {                                                                                \
      _Pragma("unroll") for (int k_ = 0; k_ < (GA_EW_TQ * CH + GA_EW_THREADS - 1) / GA_EW_THREADS; k_++) { \
        const int i_ = threadIdx.x + k_ * GA_EW_THREADS;                                      \
        const int q_ = i_ / CH, c_ = i_ - q_ * CH;                                            \
        if (i_ < GA_EW_TQ * CH && q_ < qn)                                                    \
          ga__cp_async16(n##_sm + q_ * (GA_EW_TP * 2) + ((c_ ^ ga__swz(q_)) << 4),            \
                         n##_t + (long long)q_ * sq_ + c_ * 16);                              \
      }                                                                                       \
    } else {                                                                                  \
      for (int i_ = threadIdx.x; i_ < GA_EW_TQ * GA_EW_TP; i_ += GA_EW_THREADS) {             \
        const int q_ = i_ / GA_EW_TP, p_ = i_ - q_ * GA_EW_TP;                                \
        if (q_ < qn && p_ < pn)                                                               \
          *reinterpret_cast<S *>(n##_sm + q_ * (GA_EW_TP * 2) +                               \
                                 (((p_ >> 3) ^ ga__swz(q_)) << 4) + (p_ & 7) * 2) =           \
              *reinterpret_cast<const S *>(n##_t + (long long)q_ * sq_ + p_ * 2);             \
      }                                                                                       \
    }                                                                                         \
  }
/* the thread's 8 consecutive Q positions of P position pl, by one transposing matrix load
 * (executed by every lane, in or out of range: the addresses stay inside the tile) */
#define GA__LOAD3(k, n, S, C, R, W, M)                                                        \
  if (R && M == 3) {                                                                          \
    const int lane_ = threadIdx.x & 31, m_ = lane_ >> 3, rho_ = lane_ & 7;                    \
    const int q_ = qbase + 8 * (rho_ >> 1) + 2 * m_ + (rho_ & 1);                             \
    unsigned int r_[4];                                                                       \
    ga__ldsm_x4_trans(n##_sm + q_ * (GA_EW_TP * 2) + (((pl >> 3) ^ ga__swz(q_)) << 4), r_);   \
    _Pragma("unroll") for (int j_ = 0; j_ < 4; j_++) {                                        \
      S two_[2];                                                                              \
      memcpy(two_, &r_[j_], 4);                                                               \
      n##_c[0][2 * j_] = ga__conv<C, S>::in(two_[0]);                                         \
      n##_c[0][2 * j_ + 1] = ga__conv<C, S>::in(two_[1]);                                     \
    }                                                                                         \
  }
#else
/* stage a mode-3 input: 128-bit loads along P, one row per Q position */
#define GA__STAGE(k, n, S, C, R, W, M)                                                        \
  if (M == 3) {                                                                               \
    typedef GA__WT(S) W_;                                                                     \
    constexpr int VP = 16 / (int)sizeof(S);      /* elements per 128-bit load */              \
    constexpr int WV = 16 / (int)sizeof(W_);     /* words per 128-bit load */                 \
    constexpr int PV = (GA_EW_TP + VP - 1) / VP; /* loads per tile row */                     \
    const long long sq_ = L.strq[k];                                                          \
    const bool al_ = (((unsigned long long)n##_t) % 16 == 0) && (sq_ % 16 == 0) &&            \
                     (pn == GA_EW_TP) && (GA_EW_TP % VP == 0);                                \
    if (al_) {                                                                                \
      /* all loads of the thread first, then the shared-memory stores */                     \
      constexpr int NV = (GA_EW_TQ * PV + GA_EW_THREADS - 1) / GA_EW_THREADS;                 \
      ga__pack<W_, WV> r_[NV];                                                                \
      _Pragma("unroll") for (int k_ = 0; k_ < NV; k_++) {                                     \
        const int i_ = threadIdx.x + k_ * GA_EW_THREADS;                                      \
        int q_, v_;                                                                           \
        ga__stage_map<PV>(i_, q_, v_);                                                        \
        if (i_ < GA_EW_TQ * PV && q_ < qn)                                                    \
          r_[k_] = *reinterpret_cast<const ga__pack<W_, WV> *>(                               \
              n##_t + (long long)q_ * sq_ + v_ * 16);                                         \
      }                                                                                       \
      _Pragma("unroll") for (int k_ = 0; k_ < NV; k_++) {                                     \
        const int i_ = threadIdx.x + k_ * GA_EW_THREADS;                                      \
        int q_, v_;                                                                           \
        ga__stage_map<PV>(i_, q_, v_);                                                        \
        if (i_ < GA_EW_TQ * PV && q_ < qn) {                                                  \
          _Pragma("unroll") for (int j_ = 0; j_ < WV; j_++)                                   \
            n##_sm[q_][v_ * WV + j_] = r_[k_].v[j_];                                          \
        }                                                                                     \
      }                                                                                       \
    } else {                                                                                  \
      for (int i_ = threadIdx.x; i_ < GA_EW_TQ * GA_EW_TP; i_ += GA_EW_THREADS) {             \
        const int q_ = i_ / GA_EW_TP, p_ = i_ - q_ * GA_EW_TP;                                \
        if (q_ < qn && p_ < pn)                                                               \
          reinterpret_cast<S *>(&n##_sm[q_][0])[p_] =                                         \
              *reinterpret_cast<const S *>(n##_t + (long long)q_ * sq_ + p_ * (int)sizeof(S)); \
      }                                                                                       \
    }                                                                                         \
  }

#endif /* GA_EW_LDSM */

#define GA__DECL(k, n, S, C, R, W, M) C n##_c[GA_EW_PWI][GA_EW_EPT];

#if GA_EW_LDSM
#define GA__LOAD_STAGED(k, n, S, C, R, W, M) /* done by GA__LOAD3 before the range test */
#else
#define GA__LOAD_STAGED(k, n, S, C, R, W, M)                                                  \
  {                                                                                           \
    typedef GA__WT(S) W_;                                                                     \
    constexpr int PW = GA__PW(S);                                                             \
    _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++) {                                   \
      _Pragma("unroll") for (int w_ = 0; w_ < GA_EW_PWI / PW; w_++) {                         \
        const W_ word_ = n##_sm[ql + e][pl / PW + w_];                                        \
        S tmp_[PW];                                                                           \
        memcpy(tmp_, &word_, sizeof(W_));                                                     \
        _Pragma("unroll") for (int j_ = 0; j_ < PW; j_++)                                     \
          n##_c[w_ * PW + j_][e] = ga__conv<C, S>::in(tmp_[j_]);                              \
      }                                                                                       \
    }                                                                                         \
  }
#endif

#define GA__LOAD(k, n, S, C, R, W, M)                                                         \
  if (R) {                                                                                    \
    if (M == 3) {                                                                             \
      GA__LOAD_STAGED(k, n, S, C, R, W, M)                                                    \
    } else {                                                                                  \
      _Pragma("unroll") for (int kk = 0; kk < GA_EW_PWI; kk++) {                              \
        if (pl + kk < pn) {                                                                   \
          const char *b_ = n##_t + (long long)(pl + kk) * L.strp[k];                          \
          if (M == 1) {                                                                       \
            ga__load_run<C, S, GA_EW_EPT>(                                                    \
                reinterpret_cast<const S *>(b_ + ql * (int)sizeof(S)), n##_c[kk]);            \
          } else if (M == 2) {                                                                \
            const C t_ = ga__conv<C, S>::in(*reinterpret_cast<const S *>(b_));                \
            _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++) n##_c[kk][e] = t_;          \
          } else {                                                                            \
            _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++)                             \
              if (ql + e < qn)                                                                \
                n##_c[kk][e] = ga__conv<C, S>::in(                                            \
                    *reinterpret_cast<const S *>(b_ + (long long)(ql + e) * L.strq[k]));      \
          }                                                                                   \
        }                                                                                     \
      }                                                                                       \
    }                                                                                         \
  }

#define GA__STORE(k, n, S, C, R, W, M)                                                        \
  if (W) {                                                                                    \
    _Pragma("unroll") for (int kk = 0; kk < GA_EW_PWI; kk++) {                                \
      if (pl + kk < pn) {                                                                     \
        char *b_ = n##_t + (long long)(pl + kk) * L.strp[k];                                  \
        if (M == 1) {                                                                         \
          ga__store_run<C, S, GA_EW_EPT>(reinterpret_cast<S *>(b_ + ql * (int)sizeof(S)),     \
                                         n##_c[kk]);                                          \
        } else {                                                                              \
          _Pragma("unroll") for (int e = 0; e < GA_EW_EPT; e++)                               \
            if (ql + e < qn)                                                                  \
              *reinterpret_cast<S *>(b_ + (long long)(ql + e) * L.strq[k]) =                  \
                  ga__conv<C, S>::out(n##_c[kk][e]);                                          \
        }                                                                                     \
      }                                                                                       \
    }                                                                                         \
  }

#ifndef GA_EWT_EARLY
#define GA_EWT_EARLY 0 /* 1: the rows of the CTA's first tile of every staged input are asked into L2
                          before the wait for the previous kernel of the stream (see ga__prefetch_l2).
                          Measured on B200 and left off: fp16 NHWC -> NCHW bias + ReLU 32.6 -> 34.0 us.
                          What does pay is waiting only after the first tile's coordinates and
                          addresses have been worked out from the kernel parameters: 33.0 -> 32.6 us
                          there, 49.5 -> 45.3 us for a transposed fp32 (8192, 4096) view */
#endif
/* thread q_ < qn asks for row q_ of the tile (pn elements along P, whole 16-byte pieces) */
#define GA__EARLY(k, n, S, C, R, W, M)                                                        \
  if (R && M == 3) {                                                                          \
    const unsigned int nb_ = ((unsigned int)pn * (unsigned int)sizeof(S)) & ~15u;             \
    const char *row_ = n##_t + (long long)threadIdx.x * L.strq[k];                            \
    if ((int)threadIdx.x < qn && nb_ != 0 && ((unsigned long long)row_) % 16 == 0)            \
      ga__prefetch_l2(row_, nb_);                                                             \
  }

extern "C" __global__ void __launch_bounds__(GA_EW_THREADS)
ga_ew_transpose(const __grid_constant__ ga__ewt_layout L
                GA_EW_ARRAYS(GA__P_ARR) GA_EW_SCALARS(GA__P_SC)) {
  GA_EW_ARRAYS(GA__SMEM)
  bool ga__waited = false; /* the wait for the previous kernel comes after the first tile's
                              addresses are known (they depend on kernel parameters only) */
  const unsigned long long ntiles = L.tiles_p * L.tiles_q * L.nouter;
  constexpr int QG = GA_EW_TQ / GA_EW_EPT; /* Q chunks per tile */
  constexpr int PG = GA_EW_TP / GA_EW_PWI; /* P groups per tile */
  constexpr int QL = QG < 4 ? QG : 4;      /* Q chunks side by side inside a warp */

  for (unsigned long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    /* tile coordinates: Q tiles fastest, then P tiles, then the outer index */
    unsigned long long r = t / L.tiles_q;
    const unsigned long long q0 = (t - r * L.tiles_q) * GA_EW_TQ;
    unsigned long long o = r / L.tiles_p;
    const unsigned long long p0 = (r - o * L.tiles_p) * GA_EW_TP;
    const int pn = (int)((L.pdim - p0 < GA_EW_TP) ? (L.pdim - p0) : GA_EW_TP);
    const int qn = (int)((L.qdim - q0 < GA_EW_TQ) ? (L.qdim - q0) : GA_EW_TQ);
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
    GA_EW_ARRAYS(GA__BASE_FIN)
    if (!ga__waited) {
#if GA_EWT_EARLY
      GA_EW_ARRAYS(GA__EARLY)
#endif
      ga__grid_dependency_sync();
      ga__waited = true;
    }
    GA_EW_ARRAYS(GA__STAGE)
#if GA_EW_LDSM
    ga__cp_async_wait_all();
    __syncthreads();
    {
      /* a warp step: 8 P positions (one 16-byte chunk column) x 32 Q positions */
      constexpr int NG = GA_EW_TP / 8, NUNITS = NG * (GA_EW_TQ / 32);
      const int lane = threadIdx.x & 31;
#pragma unroll 2
      for (int u = threadIdx.x >> 5; u < NUNITS; u += GA_EW_THREADS / 32) {
        const int g_ = u % NG, qbase = (u / NG) * 32;
        const int pl = 8 * g_ + (lane >> 2), ql = qbase + 8 * (lane & 3);
        GA_EW_ARRAYS(GA__DECL)
        GA_EW_ARRAYS(GA__LOAD3)
        if (pl < pn && ql < qn) {
          GA_EW_ARRAYS(GA__LOAD)
#pragma unroll
          for (int e = 0; e < GA_EW_EPT; e++) {
            constexpr int kk = 0;
            ga_ew_apply(GA_EW_ARRAYS(GA__ARG_ARR) GA_EW_SCALARS(GA__ARG_SC) 0);
          }
          GA_EW_ARRAYS(GA__STORE)
        }
      }
    }
#else
    __syncthreads();
    for (int it = threadIdx.x; it < PG * QG; it += GA_EW_THREADS) {
      /* lanes: QL chunks along Q x 8 groups along P (see the header comment) */
      const int a_ = it % QL, b_i = it / QL;
      const int pl = (b_i % PG) * GA_EW_PWI;
      const int ql = (a_ + QL * (b_i / PG)) * GA_EW_EPT;
      if (pl < pn && ql < qn) {
        GA_EW_ARRAYS(GA__DECL)
        GA_EW_ARRAYS(GA__LOAD)
#pragma unroll
        for (int kk = 0; kk < GA_EW_PWI; kk++) {
#pragma unroll
          for (int e = 0; e < GA_EW_EPT; e++)
            ga_ew_apply(GA_EW_ARRAYS(GA__ARG_ARR) GA_EW_SCALARS(GA__ARG_SC) 0);
        }
        GA_EW_ARRAYS(GA__STORE)
      }
    }
#endif
    __syncthreads();
  }
  if (!ga__waited) ga__grid_dependency_sync(); /* a CTA without a tile */
}
