/* Reduction kernels for sm_100a: three traversal shapes over one operator
 * vocabulary.
 *
 * They replace (a) the reference's maxandargmax kernel, where ONE thread
 * walks the whole reduced extent of its output serially
 * (src/gpuarray_reduction.c:520-607), and (b) pygpu's reduk template, a block
 * per output with a shared-memory tree and a div/mod per element
 * (pygpu/reduction.py:33-134). Here the reduced extent itself is spread over
 * threads, warps, CTAs and - when there are few outputs - over several work
 * groups per output. Each group publishes its partial result and takes a
 * ticket; the group that draws the last ticket combines all partials in
 * split order and writes the output. Nobody waits (no spinning, so nothing
 * can hang), the combination order is fixed (results are bitwise repeatable)
 * and the whole reduction is one launch.
 *
 *   ga_rd_rows     the innermost reduced dimension is contiguous in memory:
 *                  a CTA streams 128-bit loads along it, warp shuffles then
 *                  one shared-memory hop finish the CTA's share
 *   ga_rd_cols     the innermost KEPT dimension is contiguous: a thread owns
 *                  GA_RD_VEC adjacent outputs and walks down the reduced
 *                  extent; blockDim.y row-lanes and gridDim.y splits share it
 *   ga_rd_general  any strides: GA_RD_TPO threads per output decode each
 *                  element's offset
 *
 * Operators. GA_RD_KIND 0: acc = COMBINE(acc, MAP(x)) from IDENT (sum, prod,
 * prodnz, and, or, xor, all, any). GA_RD_KIND 1: (value, flat index) pairs
 * for min/max/arg*: `b` replaces `a` when BETTER(b.v, a.v) or when the values
 * compare equal and b has the smaller flat index - the first occurrence in
 * reduxList order wins, +0.0 and -0.0 tie, and a NaN never wins by
 * comparison. The single case in which the reference kernel returns a NaN -
 * the very first reduced element is one (:557-561, :583-586) - is applied
 * when the final value is written.
 *
 * The including translation unit defines (all by the host, ga_reduction.c):
 *   GA_RD_SRC_T   storage type of a source element
 *   GA_RD_X_T     type after GA_RD_LOAD (float for ga_half, else SRC_T)
 *   GA_RD_ACC_T   accumulator (kind 0) or compared value type (kind 1)
 *   GA_RD_DST_T   storage type of the value destination
 *   GA_RD_LOAD(raw) GA_RD_STORE(acc) GA_RD_MAP(x) GA_RD_COMBINE(a,b)
 *   GA_RD_IDENT GA_RD_BETTER(b,a) GA_RD_KIND GA_RD_ISFLOAT
 *   GA_RD_WRITE_VAL GA_RD_WRITE_IDX GA_RD_IDX_T GA_RD_VEC GA_RD_THREADS
 *   GA_RD_TPO GA_RD_BY GA_RD_GROUP (rows: 32, 64, 128 or GA_RD_THREADS) GA_RD_FLAT
 */
#include "cluda.h"

#ifndef GA_RD_MU
#define GA_RD_MU 1 /* rows: runs (or, with GA_RD_ONERUN, outputs) a group loads from at once */
#endif
#ifndef GA_RD_FAST8
#define GA_RD_FAST8 0 /* 1-byte elements folded a 32-bit word at a time: 1 signed sum,
                         2 unsigned sum, 3 any, 4 all */
#endif
#ifndef GA_RD_LAZY
#define GA_RD_LAZY 0 /* rows, (value, index) operators: scan values only, recover the index
                        afterwards; needs GA_RD_PICK(a, b) = the better of two values */
#endif
#ifndef GA_RD_ONERUN
#define GA_RD_ONERUN 0 /* rows: every output is one short contiguous run and nothing is split */
#endif
#ifndef GA_RD_ROWS_EARLY
#define GA_RD_ROWS_EARLY 64 /* rows, GA_RD_SIMPLE: bytes per lane (a multiple of 16) of the warp's first
                               run to ask into L2 before the dependency wait; 0 = none. Measured on
                               B200, fp32 4096 x 4096 over axis 1, launches back to back: 0: 13.5 us,
                               64: 13.3 us, 128: 13.3 us, 256: 14.1 us, 512: 16.1 us */
#endif
#ifndef GA_RD_TINY
#define GA_RD_TINY 0 /* rows: every output is one run of 1, 2, 4 or 8 full vectors and the runs lie
                        back to back: the source is walked as ONE flat array of vectors,
                        GA_RD_GROUP (= vectors per run) adjacent lanes share an output */
#endif
#ifndef GA_RD_SIMPLE
#define GA_RD_SIMPLE 0 /* rows: every output is ONE contiguous run owned by one warp, nothing is
                          split, fewer than 2^32 outputs: a lean loop with 32-bit indices */
#endif
#ifndef GA_RD_UNROLL
#define GA_RD_UNROLL 8 /* vectors a thread has in flight in the streaming loops. The host asks for 4
                          with accumulating operators: the leftover iterations of an unrolled loop
                          go one load per memory round trip, and runs of a few KiB leave a lane a
                          dozen vectors (fp16 (64, 256, 56, 56) over (0, 2, 3): 25.0 -> 20.9 us;
                          fp32 4096 x 4096 over axis 0: 14.7 -> 13.65 us); (value, index) operators
                          keep 8 (argmax over axis 0 of 8192 x 8192: 53.7 us against 55.8 with 4) */
#endif
#ifndef GA_RD_MINB
#define GA_RD_MINB 0 /* rows, cols: CTAs per SM the register allocation must leave room for
                        (0 = no constraint). Small grids ask for twice their own residency so
                        that the NEXT launch of the stream finds free slots while this one runs
                        (programmatic dependent launch). */
#endif

#define GA_RD_MAXD 8
static constexpr int ga__rd_unroll = GA_RD_UNROLL; /* `#pragma unroll` takes a constant, not a macro */
typedef unsigned long long ga__u64;
typedef long long ga__i64;

/* Mirrors the block marshalled by fill_layout() in ga_reduction.c. */
struct ga__rd_layout {
  ga__u64 nf_total;          /* number of outputs */
  ga__u64 nr_total;          /* reduced elements per output */
  ga__u64 nf, nr;            /* kept / reduced dimension counts */
  ga__u64 fdim[GA_RD_MAXD];  /* kept extents, outermost first */
  ga__i64 fsrc[GA_RD_MAXD];  /* byte strides of the kept dims in src */
  ga__i64 fdst0[GA_RD_MAXD]; /* ... in the value destination */
  ga__i64 fdst1[GA_RD_MAXD]; /* ... in the index destination */
  ga__u64 rdim[GA_RD_MAXD];  /* reduced extents in traversal order */
  ga__i64 rsrc[GA_RD_MAXD];  /* their byte strides in src */
  ga__u64 rmul[GA_RD_MAXD];  /* their weight in the flat (reduxList-order) index */
  ga__u64 splits;            /* CTAs (rows) / gridDim.y (cols) sharing one output */
  ga__u64 inner;             /* rows: contiguous reduced run; cols: contiguous kept run */
  ga__u64 seg;               /* rows: elements per unit of work */
  ga__u64 nseg;              /* rows: units per run */
  ga__u64 units;             /* rows: units per output */
  ga__u64 tiles;             /* cols: column tiles per contiguous kept run */
  unsigned int dv[4];        /* rows: divisor, multiplier, shifts for idx / (inner / VEC) */
  ga__u64 ioff;              /* added to every flat index written (a shard's offset in the
                                whole reduced extent; 0 otherwise) */
  ga__u64 early;             /* cols: reduced positions whose tile row a row lane asks into L2
                                before waiting for the previous kernel (0 = none) */
  ga__u64 nan_first;         /* 1: a NaN in the first reduced element is the result (the
                                reference's rule); 0 for a shard that does not hold the first
                                element of the whole reduced extent */
};

/* exact n / d for 32-bit n with the constants the host derived from d */
static __device__ __forceinline__ unsigned int ga__rd_divide(unsigned int n, const unsigned int *k) {
  const unsigned int t = __umulhi(k[1], n);
  return (t + ((n - t) >> k[2])) >> k[3];
}

struct ga__state {
  GA_RD_ACC_T v;
#if GA_RD_KIND == 1
  GA_RD_IDX_T i;
#endif
};

#define GA__IDX_NONE (~(GA_RD_IDX_T)0)

static __device__ __forceinline__ ga__state ga__init() {
  ga__state s;
  s.v = (GA_RD_ACC_T)(GA_RD_IDENT);
#if GA_RD_KIND == 1
  s.i = GA__IDX_NONE;
#endif
  return s;
}

/* fold one source element (already through GA_RD_LOAD) with flat index f */
static __device__ __forceinline__ void ga__take(ga__state &s, const GA_RD_X_T x, const GA_RD_IDX_T f) {
#if GA_RD_KIND == 0
  s.v = GA_RD_COMBINE(s.v, GA_RD_MAP(x));
#else
  if (GA_RD_BETTER(x, s.v) || (x == s.v && f < s.i)) {
    s.v = x;
    s.i = f;
  }
#endif
}

/* fold one source element as stored; operators that can consume the storage form
 * directly define GA_RD_ADD_RAW(acc, raw) (float16 sums: one mixed-precision add instead
 * of a conversion and an add, same value) */
static __device__ __forceinline__ void ga__take_raw(ga__state &s, const GA_RD_SRC_T raw,
                                                    const GA_RD_IDX_T f) {
#if defined(GA_RD_ADD_RAW) && GA_RD_KIND == 0
  s.v = GA_RD_ADD_RAW(s.v, raw);
#else
  ga__take(s, GA_RD_LOAD(raw), f);
#endif
}

static __device__ __forceinline__ void ga__merge(ga__state &a, const ga__state &b) {
#if GA_RD_KIND == 0
  a.v = GA_RD_COMBINE(a.v, b.v);
#else
  if (GA_RD_BETTER(b.v, a.v) || (b.v == a.v && b.i < a.i)) a = b;
#endif
}

template <typename T>
static __device__ __forceinline__ T ga__shfl_down(const T v, const int delta) {
  if (sizeof(T) <= 4) {
    unsigned int w = 0;
    memcpy(&w, &v, sizeof(T));
    w = __shfl_down_sync(0xffffffffu, w, delta);
    T r;
    memcpy(&r, &w, sizeof(T));
    return r;
  } else {
    unsigned long long w;
    memcpy(&w, &v, sizeof(T));
    w = __shfl_down_sync(0xffffffffu, w, delta);
    T r;
    memcpy(&r, &w, sizeof(T));
    return r;
  }
}

/* W adjacent lanes (W a power of two, aligned) combine in a fixed order; the
 * result is valid in the first of them */
template <int W>
static __device__ __forceinline__ ga__state ga__lanes_reduce(ga__state s) {
#pragma unroll
  for (int d = W / 2; d > 0; d >>= 1) {
    ga__state t;
    t.v = ga__shfl_down(s.v, d);
#if GA_RD_KIND == 1
    t.i = ga__shfl_down(s.i, d);
#endif
    ga__merge(s, t);
  }
  return s;
}

/* result valid in lane 0 */
static __device__ __forceinline__ ga__state ga__warp_reduce(ga__state s) {
  return ga__lanes_reduce<32>(s);
}

/* result valid in thread 0 of the CTA; `sm` holds one state per warp */
static __device__ __forceinline__ ga__state ga__block_reduce(ga__state s, ga__state *sm,
                                                             const unsigned tid,
                                                             const unsigned nthreads) {
  s = ga__warp_reduce(s);
  if ((tid & 31u) == 0) sm[tid >> 5] = s;
  __syncthreads();
  if (tid < 32) {
    s = tid < (nthreads >> 5) ? sm[tid] : ga__init();
    s = ga__warp_reduce(s);
  }
  return s;
}

/* A group of W consecutive warps of the CTA (W a power of two; W = all of them gives the
 * CTA-wide reduction) combines in a fixed order; the result is valid in the group's first
 * thread. Every thread of the CTA must call it (one barrier inside; the caller places
 * another before `sm` is reused). `sm` holds one state per warp of the CTA. */
template <int W>
static __device__ __forceinline__ ga__state ga__group_reduce(ga__state s, ga__state *sm,
                                                             const unsigned tid) {
  s = ga__warp_reduce(s);
  if ((tid & 31u) == 0) sm[tid >> 5] = s;
  __syncthreads();
  if (tid % (32 * W) == 0) {
#pragma unroll
    for (int k = 1; k < W; k++) ga__merge(s, sm[(tid >> 5) + k]);
  }
  return s;
}

/* byte offset of output `o` through one stride vector of the kept dims */
static __device__ __forceinline__ ga__i64 ga__foff(const ga__rd_layout &L, const ga__i64 *str,
                                                   ga__u64 o) {
  ga__i64 off = 0;
  if (L.nf_total <= 0xffffffffULL) { /* 32-bit division is several times cheaper */
    unsigned int o32 = (unsigned int)o;
    for (int d = (int)L.nf - 1; d > 0; d--) {
      const unsigned int fd = (unsigned int)L.fdim[d], q = o32 / fd;
      off += (ga__i64)(o32 - q * fd) * str[d];
      o32 = q;
    }
    if (L.nf > 0) off += (ga__i64)o32 * str[0];
    return off;
  }
  for (int d = (int)L.nf - 1; d > 0; d--) {
    const ga__u64 q = o / L.fdim[d];
    off += (ga__i64)(o - q * L.fdim[d]) * str[d];
    o = q;
  }
  if (L.nf > 0) off += (ga__i64)o * str[0];
  return off;
}

/* final result of output `o` */
static __device__ __forceinline__ void ga__emit(const ga__rd_layout &L, const char *src, char *d0,
                                                char *d1, const ga__u64 o, ga__state s) {
#if GA_RD_KIND == 1 && GA_RD_ISFLOAT
  {
    const GA_RD_SRC_T raw = *reinterpret_cast<const GA_RD_SRC_T *>(src + ga__foff(L, L.fsrc, o));
    const GA_RD_X_T first = GA_RD_LOAD(raw);
    if (L.nan_first != 0 && first != first) {
      s.v = first;
      s.i = 0;
    }
  }
#endif
#if GA_RD_WRITE_VAL
  *reinterpret_cast<GA_RD_DST_T *>(d0 + ga__foff(L, L.fdst0, o)) = GA_RD_STORE(s.v);
#endif
#if GA_RD_KIND == 1 && GA_RD_WRITE_IDX
  /* "no element" (a shard of NaNs only) stays all-ones whatever the offset */
  *reinterpret_cast<ga__u64 *>(d1 + ga__foff(L, L.fdst1, o)) =
      (s.i == GA__IDX_NONE) ? ~(ga__u64)0 : (ga__u64)s.i + L.ioff;
#endif
}

/* ga__emit for callers that still hold the first reduced element of the output in a
 * register (its raw form): spares the load - and the wait for it at the end of every
 * output - that ga__emit spends on the NaN-first rule */
static __device__ __forceinline__ void ga__emit_with_first(const ga__rd_layout &L, char *d0, char *d1,
                                                           const ga__u64 o, ga__state s,
                                                           const GA_RD_SRC_T first_raw) {
#if GA_RD_KIND == 1 && GA_RD_ISFLOAT
  {
    const GA_RD_X_T first = GA_RD_LOAD(first_raw);
    if (L.nan_first != 0 && first != first) {
      s.v = first;
      s.i = 0;
    }
  }
#endif
#if GA_RD_WRITE_VAL
  *reinterpret_cast<GA_RD_DST_T *>(d0 + ga__foff(L, L.fdst0, o)) = GA_RD_STORE(s.v);
#endif
#if GA_RD_KIND == 1 && GA_RD_WRITE_IDX
  *reinterpret_cast<ga__u64 *>(d1 + ga__foff(L, L.fdst1, o)) =
      (s.i == GA__IDX_NONE) ? ~(ga__u64)0 : (ga__u64)s.i + L.ioff;
#endif
}

/* ga__emit when there is ONE kept dimension (the lean column walk): for accumulating
 * operators the offset is a single multiply - no coordinate decoding, no first-element
 * check - which also spares the kernel a spill */
static __device__ __forceinline__ void ga__emit_lean(const ga__rd_layout &L, const char *src,
                                                     char *d0, char *d1, const unsigned int o,
                                                     const ga__state &s) {
#if GA_RD_KIND == 0
  *reinterpret_cast<GA_RD_DST_T *>(d0 + (ga__i64)o * L.fdst0[0]) = GA_RD_STORE(s.v);
#else
  ga__emit(L, src, d0, d1, o, s);
#endif
}

template <typename T>
static __device__ __forceinline__ T ga__ldcg(const T *p) {
  T r;
  if (sizeof(T) == 1) {
    const unsigned char w = __ldcg(reinterpret_cast<const unsigned char *>(p));
    memcpy(&r, &w, 1);
  } else if (sizeof(T) == 2) {
    const unsigned short w = __ldcg(reinterpret_cast<const unsigned short *>(p));
    memcpy(&r, &w, 2);
  } else if (sizeof(T) == 4) {
    const unsigned int w = __ldcg(reinterpret_cast<const unsigned int *>(p));
    memcpy(&r, &w, 4);
  } else {
    const unsigned long long w = __ldcg(reinterpret_cast<const unsigned long long *>(p));
    memcpy(&r, &w, 8);
  }
  return r;
}

/* N bytes from L2, N a multiple of the alignment of p, in the widest pieces */
template <int N>
static __device__ __forceinline__ void ga__ldcg_block(void *dst, const void *p) {
  if (N % 16 == 0) {
#pragma unroll
    for (int i = 0; i < N / 16; i++) {
      const uint4 w = __ldcg(reinterpret_cast<const uint4 *>(p) + i);
      memcpy(static_cast<char *>(dst) + 16 * i, &w, 16);
    }
  } else if (N % 8 == 0) {
#pragma unroll
    for (int i = 0; i < N / 8; i++) {
      const uint2 w = __ldcg(reinterpret_cast<const uint2 *>(p) + i);
      memcpy(static_cast<char *>(dst) + 8 * i, &w, 8);
    }
  } else if (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N / 4; i++) {
      const unsigned int w = __ldcg(reinterpret_cast<const unsigned int *>(p) + i);
      memcpy(static_cast<char *>(dst) + 4 * i, &w, 4);
    }
  } else if (N % 2 == 0) {
#pragma unroll
    for (int i = 0; i < N / 2; i++) {
      const unsigned short w = __ldcg(reinterpret_cast<const unsigned short *>(p) + i);
      memcpy(static_cast<char *>(dst) + 2 * i, &w, 2);
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; i++)
      static_cast<unsigned char *>(dst)[i] = __ldcg(reinterpret_cast<const unsigned char *>(p) + i);
  }
}

static __device__ __forceinline__ void ga__put_partial(const ga__rd_layout &L, GA_RD_ACC_T *pval,
                                                       GA_RD_IDX_T *pidx, const ga__u64 split,
                                                       const ga__u64 o, const ga__state &s) {
  pval[o * L.splits + split] = s.v; /* [output][split] */
#if GA_RD_KIND == 1
  pidx[o * L.splits + split] = s.i;
#endif
}

/* partial `split` of output `o`, read from L2 (ld.global.cg): other CTAs wrote
 * it, and the ticket's fence/atomic pair ordered those writes before us */
static __device__ __forceinline__ ga__state ga__get_partial(const ga__rd_layout &L,
                                                            const GA_RD_ACC_T *pval,
                                                            const GA_RD_IDX_T *pidx,
                                                            const ga__u64 split, const ga__u64 o) {
  ga__state t;
  t.v = ga__ldcg(&pval[o * L.splits + split]);
#if GA_RD_KIND == 1
  t.i = ga__ldcg(&pidx[o * L.splits + split]);
#endif
  return t;
}

/* One thread of a group calls this after the group's partial is stored.
 * Returns true for the group that arrived last at `ticket`; that group then
 * owns every partial of the output. The counter is left at zero for the next
 * launch. */
static __device__ __forceinline__ bool ga__take_ticket(unsigned int *ticket,
                                                       const unsigned int nsplits) {
  __threadfence();
  const unsigned int seen = atomicAdd(ticket, 1u);
  if (seen + 1u != nsplits) return false;
  *ticket = 0u;
  __threadfence();
  return true;
}

#if GA_RD_FAST8
/* 1-byte elements that are only ever folded a word at a time: the vector is
 * declared as words. Declared as N bytes and copied into words afterwards, the
 * compiler splits the 128-bit load into 16 byte values and glues them together
 * again (about 28 extract / insert instructions per vector: the int8 sum of
 * 2^28 elements ran at 52 % ALU-pipe utilisation and 4.2 TB/s). */
template <int N>
struct alignas(N >= 16 ? 16 : N) ga__rd_pack {
  unsigned int w[N / 4];
};
#else
template <int N>
struct alignas((sizeof(GA_RD_SRC_T) * N >= 16) ? 16 : sizeof(GA_RD_SRC_T) * N) ga__rd_pack {
  GA_RD_SRC_T v[N];
};
#endif

#if GA_RD_FAST8
/* A vector of 1-byte elements folded into ONE state with word arithmetic
 * instead of element by element: sums with a 4-way byte dot product against
 * ones (exact: a vector's sum fits 32 bits by far), ANY with an OR of the
 * words, ALL with the classic has-a-zero-byte test. Same results as the
 * per-element form; about a tenth of the instructions. */
static __device__ __forceinline__ void ga__fold_words(ga__state &s,
                                                      const ga__rd_pack<GA_RD_VEC> &t) {
  const unsigned int *w = t.w;
#if GA_RD_FAST8 == 1
  int acc = 0;
#pragma unroll
  for (int i = 0; i < GA_RD_VEC / 4; i++) acc = __dp4a((int)w[i], 0x01010101, acc);
  s.v = GA_RD_COMBINE(s.v, (GA_RD_ACC_T)acc);
#elif GA_RD_FAST8 == 2
  unsigned int acc = 0;
#pragma unroll
  for (int i = 0; i < GA_RD_VEC / 4; i++) acc = __dp4a(w[i], 0x01010101u, acc);
  s.v = GA_RD_COMBINE(s.v, (GA_RD_ACC_T)acc);
#elif GA_RD_FAST8 == 3
  unsigned int acc = 0;
#pragma unroll
  for (int i = 0; i < GA_RD_VEC / 4; i++) acc |= w[i];
  s.v = GA_RD_COMBINE(s.v, (GA_RD_ACC_T)(acc != 0));
#else
  unsigned int zero = 0;
#pragma unroll
  for (int i = 0; i < GA_RD_VEC / 4; i++) zero |= (w[i] - 0x01010101u) & ~w[i] & 0x80808080u;
  s.v = GA_RD_COMBINE(s.v, (GA_RD_ACC_T)(zero == 0));
#endif
}
#endif

/* element j of a vector into state j (the states are merged at the end) */
static __device__ __forceinline__ void ga__fold_lanes(ga__state *st,
                                                      const ga__rd_pack<GA_RD_VEC> &t,
                                                      const GA_RD_IDX_T f0,
                                                      const GA_RD_IDX_T imul) {
#if GA_RD_FAST8
  ga__fold_words(st[0], t);
#else
#pragma unroll
  for (int j = 0; j < GA_RD_VEC; j++) ga__take_raw(st[j], t.v[j], f0 + (GA_RD_IDX_T)j * imul);
#endif
}

/* every element of a vector into one state */
static __device__ __forceinline__ void ga__fold_one(ga__state &s,
                                                    const ga__rd_pack<GA_RD_VEC> &t,
                                                    const GA_RD_IDX_T f0,
                                                    const GA_RD_IDX_T imul) {
#if GA_RD_FAST8
  ga__fold_words(s, t);
#else
#pragma unroll
  for (int j = 0; j < GA_RD_VEC; j++) ga__take_raw(s, t.v[j], f0 + (GA_RD_IDX_T)j * imul);
#endif
}

/* ------------------------------------------------------------------ rows */
#if defined(GA_RD_BUILD_ROWS)
/* byte offset and flat-index base of reduced "row" r (all reduced dims but the
 * contiguous one), nro = number of those dims */
static __device__ __forceinline__ void ga__row_decode(const ga__rd_layout &L, const int nro,
                                                      ga__u64 r, ga__i64 &roff,
                                                      GA_RD_IDX_T &fbase) {
  if (nro == 1) {
    roff = (ga__i64)r * L.rsrc[0];
    fbase = (GA_RD_IDX_T)r * (GA_RD_IDX_T)L.rmul[0];
    return;
  }
  roff = 0;
  fbase = 0;
  for (int d = nro - 1; d >= 0; d--) {
    const ga__u64 q = r / L.rdim[d], c = r - q * L.rdim[d];
    r = q;
    roff += (ga__i64)c * L.rsrc[d];
    fbase += (GA_RD_IDX_T)c * (GA_RD_IDX_T)L.rmul[d];
  }
}

/* GA_RD_GROUP threads (a warp, 2 or 4 warps, or the whole CTA) share one work item, i.e. one
 * (output, split) pair, and walk its units (a unit = one contiguous run, or
 * one segment of a long run) one after the other; inside a unit each thread
 * strides 128-bit loads, so the inner loop is a pointer, a counter and the
 * operator. The host picks the group so that a thread sees several vectors
 * per unit: a CTA for long runs, a warp for runs of a few KiB. With
 * GA_RD_FLAT (very short runs) the (run, vector) pairs of the whole share are
 * flattened into one index space instead, so that consecutive iterations of
 * a thread touch different runs and their loads overlap.
 *
 * Runs of a few hundred elements leave a thread with one or two loads per run,
 * too few to cover DRAM latency. Two remedies, both chosen by the host:
 * GA_RD_MU > 1 makes a group load from GA_RD_MU runs of its output at once;
 * GA_RD_ONERUN (each output is a single short run, nothing split) lets groups
 * be part of a warp (GA_RD_GROUP = 1..32 lanes, sized so that a lane still
 * sees about two vectors of the run) and has each group work on GA_RD_MU
 * outputs at once, one accumulator per output. */
#if GA_RD_MINB > 0
#define GA__RD_ROWS_BOUNDS __launch_bounds__(GA_RD_THREADS, GA_RD_MINB)
#elif GA_RD_MU > 1
#define GA__RD_ROWS_BOUNDS __launch_bounds__(GA_RD_THREADS, 3) /* room for the extra loads in flight */
#else
#define GA__RD_ROWS_BOUNDS __launch_bounds__(GA_RD_THREADS)
#endif
extern "C" __global__ void GA__RD_ROWS_BOUNDS
ga_rd_rows(const __grid_constant__ ga__rd_layout L, const char *src, char *d0, char *d1,
           GA_RD_ACC_T *pval, GA_RD_IDX_T *pidx, unsigned int *tickets) {
#if GA_RD_SIMPLE && GA_RD_ROWS_EARLY > 0
  /* The head of this warp's first run, asked into L2 before the wait for the previous kernel
   * of the stream: the first DRAM reads overlap its tail (see ga__prefetch_l2; the same is
   * done in the column walk). Only with full 16-byte vectors: then the run starts on a
   * 16-byte boundary. */
  if (GA_RD_VEC * sizeof(GA_RD_SRC_T) == 16) {
    const unsigned int o = blockIdx.x * (GA_RD_THREADS / 32) + (threadIdx.x >> 5);
    const unsigned int at = (threadIdx.x & 31u) * GA_RD_ROWS_EARLY;
    if (o < (unsigned int)L.nf_total &&
        (ga__u64)at + GA_RD_ROWS_EARLY <= (L.inner / GA_RD_VEC) * 16ULL)
      ga__prefetch_l2(src + ga__foff(L, L.fsrc, o) + at, GA_RD_ROWS_EARLY);
  }
#endif
  ga__grid_dependency_sync();
#if GA_RD_GROUP > 32
  __shared__ ga__state sm[32];
  __shared__ int sm_last[GA_RD_THREADS / GA_RD_GROUP]; /* one slot per group of the CTA */
#endif
  const ga__u64 nwork = L.nf_total * L.splits;
  const int nro = (int)L.nr - 1; /* reduced dims outside the contiguous run */
  const GA_RD_IDX_T imul = (GA_RD_IDX_T)L.rmul[nro];
  const unsigned lane = threadIdx.x % GA_RD_GROUP;
  const ga__u64 group = ((ga__u64)blockIdx.x * GA_RD_THREADS + threadIdx.x) / GA_RD_GROUP;
  const ga__u64 ngroups = (ga__u64)gridDim.x * (GA_RD_THREADS / GA_RD_GROUP);
  const ga__u64 rounds = (nwork + ngroups - 1) / ngroups;

#if GA_RD_TINY
  /* Runs of at most 128 bytes, back to back in memory. A thread per run (the mapping the
   * short-run path below would choose) makes every load instruction of a warp touch 32
   * runs a fragment each - the L1 becomes the limiter (64-73 % of its throughput for rows of
   * 16 floats) - and lanes sharing a run there repeat the per-run work (output offset
   * decoding, first-element check, emit) in every lane. Here consecutive threads take
   * consecutive VECTORS of the whole source, four in flight per thread, so every load
   * instruction is one contiguous 512 bytes; the GA_RD_GROUP lanes holding a run combine
   * with shuffles and the first of them, which holds the run's first element, writes. */
  {
    const unsigned int nvec = (unsigned int)L.nf_total * GA_RD_GROUP; /* host: below 2^31 */
    const unsigned int step = gridDim.x * GA_RD_THREADS;
    const unsigned int sub = threadIdx.x % GA_RD_GROUP;
    const ga__rd_pack<GA_RD_VEC> *pv = reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(src);
    const GA_RD_IDX_T f0 = (GA_RD_IDX_T)(sub * GA_RD_VEC) * imul;
    /* the loop bound is the WARP's first vector, so that whole warps iterate (the shuffles
     * below name all 32 lanes); lanes past the end load vector 0 and drop the result */
    const unsigned int lane32 = threadIdx.x & 31u;
    for (unsigned int q0 = blockIdx.x * GA_RD_THREADS + threadIdx.x; q0 - lane32 < nvec;
         q0 += 4u * step) {
      ga__rd_pack<GA_RD_VEC> t[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const unsigned int q = q0 + (unsigned int)u * step;
        t[u] = pv[q < nvec ? q : 0u];
      }
#if GA_RD_KIND == 1 && GA_RD_WRITE_VAL && !GA_RD_WRITE_IDX && defined(GA_RD_PICK)
      /* MIN / MAX without an index: values only - one instruction per element and per
       * shuffle step instead of compare-and-select on (value, index) pairs. fmax / fmin skip
       * NaNs as the pair rule does. The one thing the pair rule decides that values cannot
       * is the sign of a zero result (the FIRST zero of the run wins): when any lane of the
       * warp sees a zero result, the lanes find the position and sign of their first zero
       * and the lowest position of the group supplies the sign. */
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const unsigned int q = q0 + (unsigned int)u * step;
        GA_RD_X_T m = (GA_RD_X_T)(GA_RD_IDENT);
#pragma unroll
        for (int j = 0; j < GA_RD_VEC; j++) {
          const GA_RD_X_T x = GA_RD_LOAD(t[u].v[j]);
          m = GA_RD_PICK(m, x);
        }
#pragma unroll
        for (int d = GA_RD_GROUP / 2; d > 0; d >>= 1) {
          const GA_RD_X_T other = ga__shfl_down(m, d); /* once: the macro may name it twice */
          m = GA_RD_PICK(m, other);
        }
#if GA_RD_ISFLOAT
        if (__any_sync(0xffffffffu, m == (GA_RD_X_T)0)) {
          unsigned int key = 0xffffffffu;
#pragma unroll
          for (int j = GA_RD_VEC - 1; j >= 0; j--) {
            unsigned char raw[sizeof(GA_RD_SRC_T)];
            memcpy(raw, &t[u].v[j], sizeof(raw));
            if (GA_RD_LOAD(t[u].v[j]) == (GA_RD_X_T)0)
              key = ((sub * GA_RD_VEC + (unsigned int)j) << 1) | (unsigned int)(raw[sizeof(raw) - 1] >> 7);
          }
#pragma unroll
          for (int d = GA_RD_GROUP / 2; d > 0; d >>= 1) {
            const unsigned int other = ga__shfl_down(key, d);
            key = other < key ? other : key;
          }
          if (m == (GA_RD_X_T)0 && key != 0xffffffffu) m = (key & 1u) ? -(GA_RD_X_T)0 : (GA_RD_X_T)0;
        }
#endif
        if (sub == 0 && q < nvec) {
#if GA_RD_ISFLOAT
          const GA_RD_X_T first = GA_RD_LOAD(t[u].v[0]);
          if (L.nan_first != 0 && first != first) m = first;
#endif
          *reinterpret_cast<GA_RD_DST_T *>(d0 + (ga__i64)(q / GA_RD_GROUP) * L.fdst0[0]) = GA_RD_STORE(m);
        }
      }
#else
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const unsigned int q = q0 + (unsigned int)u * step;
        ga__state st = ga__init();
        ga__fold_one(st, t[u], f0, imul);
        st = ga__lanes_reduce<GA_RD_GROUP>(st); /* q < nvec holds for all lanes of a group or
                                                   for none: nvec is a multiple of the group */
        if (sub == 0 && q < nvec) {
          const unsigned int o = q / GA_RD_GROUP;
#if GA_RD_KIND == 1 && GA_RD_ISFLOAT
          const GA_RD_X_T first = GA_RD_LOAD(t[u].v[0]);
          if (L.nan_first != 0 && first != first) {
            st.v = first;
            st.i = 0;
          }
#endif
#if GA_RD_WRITE_VAL
          *reinterpret_cast<GA_RD_DST_T *>(d0 + (ga__i64)o * L.fdst0[0]) = GA_RD_STORE(st.v);
#endif
#if GA_RD_KIND == 1 && GA_RD_WRITE_IDX
          *reinterpret_cast<ga__u64 *>(d1 + (ga__i64)o * L.fdst1[0]) =
              (st.i == GA__IDX_NONE) ? ~(ga__u64)0 : (ga__u64)st.i + L.ioff;
#endif
        }
      }
#endif
    }
  }
#elif GA_RD_SIMPLE
  /* A warp per output, one contiguous run each, nothing split. Few live values besides
   * the vectors in flight: the kernel needs about half the registers of the general
   * loop below, so the CTAs of the NEXT launch of the stream find room to become
   * resident while this grid still runs (they wait in ga__grid_dependency_sync) and
   * start the moment it completes. */
  {
    /* SIGNED loop counters on purpose (the host keeps every extent below 2^31): signed
     * overflow being undefined lets the compiler derive the trip count of a strided loop
     * and batch the loads of the unrolled body; with unsigned counters it must allow for
     * wrap-around and does not (measured in the column walk, fp32 4096 x 4096:
     * 14.9 -> 14.45 us). */
    const unsigned int nout = (unsigned int)L.nf_total;
    const int len = (int)L.inner, nv = len / GA_RD_VEC;
    const int wl = (int)(threadIdx.x & 31u);
    const unsigned int nwarps = gridDim.x * (GA_RD_THREADS / 32);
    for (unsigned int o = blockIdx.x * (GA_RD_THREADS / 32) + (threadIdx.x >> 5); o < nout;
         o += nwarps) {
      const char *base = src + ga__foff(L, L.fsrc, o);
      const ga__rd_pack<GA_RD_VEC> *pv = reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(base);
      ga__state st[GA_RD_VEC];
#pragma unroll
      for (int j = 0; j < GA_RD_VEC; j++) st[j] = ga__init();
#pragma unroll ga__rd_unroll
      for (int i = wl; i < nv; i += 32) {
        const ga__rd_pack<GA_RD_VEC> t = pv[i];
        ga__fold_lanes(st, t, (GA_RD_IDX_T)(i * GA_RD_VEC) * imul, imul);
      }
      for (int i = nv * GA_RD_VEC + wl; i < len; i += 32)
        ga__take(st[0], GA_RD_LOAD(reinterpret_cast<const GA_RD_SRC_T *>(base)[i]),
                 (GA_RD_IDX_T)i * imul);
#pragma unroll
      for (int j = 1; j < GA_RD_VEC; j++) ga__merge(st[0], st[j]);
      const ga__state tot = ga__warp_reduce(st[0]);
      if (wl == 0) ga__emit(L, src, d0, d1, o, tot);
    }
  }
#elif GA_RD_ONERUN
  {
    const unsigned int len = (unsigned int)L.inner, nv = len / GA_RD_VEC;
    for (ga__u64 it = 0; it < rounds; it += GA_RD_MU) {
      ga__state st[GA_RD_MU];
      const char *base[GA_RD_MU];
      ga__u64 w[GA_RD_MU];
      bool live[GA_RD_MU];
#pragma unroll
      for (int k = 0; k < GA_RD_MU; k++) {
        /* neighbouring groups take neighbouring outputs; a slot past the end
         * re-reads the last output and drops the result */
        w[k] = group + (it + (ga__u64)k) * ngroups;
        live[k] = w[k] < nwork;
        if (!live[k]) w[k] = nwork - 1;
        st[k] = ga__init();
        base[k] = src + ga__foff(L, L.fsrc, w[k]);
      }
      /* the run's first element, for the NaN-first rule when the output is written: asked for
       * now, together with the run's vectors, instead of at the end of every output where the
       * wait for it would be exposed (rows of 64 floats: MAX 53.3 -> 48.5 us, ARGMAX 55.0 -> 49.2 us,
       * MAX AND ARGMAX 60.7 -> 55.1 us; rows of 1024: 51.5 / 51.7 / 53.4 -> 49.0 / 50.0 / 51.5 us) */
      GA_RD_SRC_T first_raw[GA_RD_MU];
#pragma unroll
      for (int k = 0; k < GA_RD_MU; k++) first_raw[k] = *reinterpret_cast<const GA_RD_SRC_T *>(base[k]);
#if GA_RD_LAZY
      /* (value, index) operators: scan values only, keeping per output the best value and
       * the first vector that reached it; the element, its bit pattern and its index are
       * recovered from that vector afterwards (same two-step rule as the long-run scan
       * further down, same result as comparing pairs element by element) */
      {
        GA_RD_X_T bv[GA_RD_MU];
        unsigned int bi[GA_RD_MU];
#pragma unroll
        for (int k = 0; k < GA_RD_MU; k++) {
          bv[k] = (GA_RD_X_T)(GA_RD_IDENT);
          bi[k] = lane;
        }
#pragma unroll 2
        for (unsigned int i = lane; i < nv; i += GA_RD_GROUP) {
          ga__rd_pack<GA_RD_VEC> t[GA_RD_MU];
#pragma unroll
          for (int k = 0; k < GA_RD_MU; k++)
            t[k] = reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(base[k])[i];
#pragma unroll
          for (int k = 0; k < GA_RD_MU; k++) {
            GA_RD_X_T m = GA_RD_LOAD(t[k].v[0]);
#pragma unroll
            for (int j = 1; j < GA_RD_VEC; j++) m = GA_RD_PICK(m, GA_RD_LOAD(t[k].v[j]));
            if (GA_RD_BETTER(m, bv[k])) {
              bv[k] = m;
              bi[k] = i;
            }
          }
        }
#pragma unroll
        for (int k = 0; k < GA_RD_MU; k++) {
          if (bi[k] < nv) {
            const ga__rd_pack<GA_RD_VEC> t = reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(base[k])[bi[k]];
            ga__state loc = ga__init();
#pragma unroll
            for (int j = GA_RD_VEC - 1; j >= 0; j--) {
              const GA_RD_X_T x = GA_RD_LOAD(t.v[j]);
              if (x == bv[k]) { /* first match last: it keeps its own bit pattern (+-0) */
                loc.v = x;
                loc.i = (GA_RD_IDX_T)(bi[k] * GA_RD_VEC + (unsigned)j) * imul;
              }
            }
            if (loc.i == GA__IDX_NONE) {
              /* nothing beat the identity and the first vector does not hold it (NaNs):
               * the long way over this lane's vectors */
              for (unsigned int i = lane; i < nv; i += GA_RD_GROUP) {
                const ga__rd_pack<GA_RD_VEC> u = reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(base[k])[i];
                ga__fold_one(loc, u, (GA_RD_IDX_T)(i * GA_RD_VEC) * imul, imul);
              }
            }
            ga__merge(st[k], loc);
          }
        }
      }
#else
#pragma unroll 2
      for (unsigned int i = lane; i < nv; i += GA_RD_GROUP) {
        ga__rd_pack<GA_RD_VEC> t[GA_RD_MU];
#pragma unroll
        for (int k = 0; k < GA_RD_MU; k++)
          t[k] = reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(base[k])[i];
#pragma unroll
        for (int k = 0; k < GA_RD_MU; k++)
          ga__fold_one(st[k], t[k], (GA_RD_IDX_T)(i * GA_RD_VEC) * imul, imul);
      }
#endif
      for (unsigned int i = nv * GA_RD_VEC + lane; i < len; i += GA_RD_GROUP) {
#pragma unroll
        for (int k = 0; k < GA_RD_MU; k++)
          ga__take(st[k], GA_RD_LOAD(reinterpret_cast<const GA_RD_SRC_T *>(base[k])[i]),
                   (GA_RD_IDX_T)i * imul);
      }
#pragma unroll
      for (int k = 0; k < GA_RD_MU; k++) st[k] = ga__lanes_reduce<GA_RD_GROUP>(st[k]);
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < GA_RD_MU; k++) {
          if (live[k]) ga__emit_with_first(L, d0, d1, w[k], st[k], first_raw[k]);
        }
      }
    }
  }
#else
  for (ga__u64 it = 0; it < rounds; it++) {
    const ga__u64 w = group + it * ngroups;
    const bool live = w < nwork;
    ga__u64 o = live ? w : 0, split = 0;
    if (L.splits > 1) {
      const ga__u64 ww = o;
      o = ww / L.splits;
      split = ww - o * L.splits;
    }
    ga__state st[GA_RD_VEC];
#pragma unroll
    for (int j = 0; j < GA_RD_VEC; j++) st[j] = ga__init();

    if (live) {
      const ga__u64 ub = split * L.units / L.splits, ue = (split + 1) * L.units / L.splits;
      const char *obase = src + ga__foff(L, L.fsrc, o);
#if !GA_RD_FLAT
      ga__u64 u = ub;
#if GA_RD_MU > 1
      if (L.nseg == 1) {
        const unsigned int len = (unsigned int)L.inner, nv = len / GA_RD_VEC;
        for (; u + GA_RD_MU <= ue; u += GA_RD_MU) {
          const char *rp[GA_RD_MU];
          GA_RD_IDX_T fb[GA_RD_MU];
#pragma unroll
          for (int k = 0; k < GA_RD_MU; k++) {
            ga__i64 roff;
            ga__row_decode(L, nro, u + (ga__u64)k, roff, fb[k]);
            rp[k] = obase + roff;
          }
#pragma unroll 2
          for (unsigned int i = lane; i < nv; i += GA_RD_GROUP) {
            ga__rd_pack<GA_RD_VEC> t[GA_RD_MU];
#pragma unroll
            for (int k = 0; k < GA_RD_MU; k++)
              t[k] = reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(rp[k])[i];
#pragma unroll
            for (int k = 0; k < GA_RD_MU; k++)
              ga__fold_lanes(st, t[k], fb[k] + (GA_RD_IDX_T)(i * GA_RD_VEC) * imul, imul);
          }
          for (unsigned int i = nv * GA_RD_VEC + lane; i < len; i += GA_RD_GROUP) {
#pragma unroll
            for (int k = 0; k < GA_RD_MU; k++)
              ga__take(st[0], GA_RD_LOAD(reinterpret_cast<const GA_RD_SRC_T *>(rp[k])[i]),
                       fb[k] + (GA_RD_IDX_T)i * imul);
          }
        }
      }
#endif
      for (; u < ue; u++) {
        ga__u64 r = u, g = 0;
        if (L.nseg > 1) {
          r = u / L.nseg;
          g = u - r * L.nseg;
        }
        ga__i64 roff;
        GA_RD_IDX_T fbase;
        ga__row_decode(L, nro, r, roff, fbase);
        const ga__u64 e0 = g * L.seg;
        const unsigned int len = (unsigned int)((L.inner - e0 < L.seg) ? (L.inner - e0) : L.seg);
        const GA_RD_SRC_T *p = reinterpret_cast<const GA_RD_SRC_T *>(obase + roff) + e0;
        fbase += (GA_RD_IDX_T)e0 * imul;
        const unsigned int nv = len / GA_RD_VEC;
        const ga__rd_pack<GA_RD_VEC> *pv = reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(p);
#if GA_RD_MU > 1
        /* leftover runs of a multi-run variant: short by construction */
#pragma unroll 4
        for (unsigned int i = lane; i < nv; i += GA_RD_GROUP) {
          const ga__rd_pack<GA_RD_VEC> t = pv[i];
          ga__fold_lanes(st, t, fbase + (GA_RD_IDX_T)(i * GA_RD_VEC) * imul, imul);
        }
#elif GA_RD_LAZY
        /* (value, index) operators over a long run: the scan keeps only the
         * best value and the vector it came from (strictly better only, so the
         * earliest vector wins ties); the element and its index are recovered
         * from that one vector afterwards. A third of the instructions of
         * comparing and selecting (value, index) pairs per element. */
        {
          GA_RD_X_T bv = (GA_RD_X_T)(GA_RD_IDENT);
          unsigned int bi = lane; /* where to look if nothing beats the identity */
#pragma unroll ga__rd_unroll
          for (unsigned int i = lane; i < nv; i += GA_RD_GROUP) {
            const ga__rd_pack<GA_RD_VEC> t = pv[i];
            GA_RD_X_T m = GA_RD_LOAD(t.v[0]);
#pragma unroll
            for (int j = 1; j < GA_RD_VEC; j++) m = GA_RD_PICK(m, GA_RD_LOAD(t.v[j]));
            if (GA_RD_BETTER(m, bv)) {
              bv = m;
              bi = i;
            }
          }
          if (bi < nv) {
            const ga__rd_pack<GA_RD_VEC> t = pv[bi];
            ga__state loc = ga__init();
#pragma unroll
            for (int j = GA_RD_VEC - 1; j >= 0; j--) {
              const GA_RD_X_T x = GA_RD_LOAD(t.v[j]);
              if (x == bv) { /* first match last: it keeps its own bit pattern (+-0) */
                loc.v = x;
                loc.i = fbase + (GA_RD_IDX_T)(bi * GA_RD_VEC + (unsigned)j) * imul;
              }
            }
            if (loc.i == GA__IDX_NONE) {
              /* nothing beat the identity and the first vector does not hold it
               * (NaNs): find the first element equal to it, if any, the long way */
              for (unsigned int i = lane; i < nv; i += GA_RD_GROUP) {
                const ga__rd_pack<GA_RD_VEC> u = pv[i];
                ga__fold_one(loc, u, fbase + (GA_RD_IDX_T)(i * GA_RD_VEC) * imul, imul);
              }
            }
            ga__merge(st[0], loc);
          }
        }
#else
#pragma unroll ga__rd_unroll
        for (unsigned int i = lane; i < nv; i += GA_RD_GROUP) {
          const ga__rd_pack<GA_RD_VEC> t = pv[i];
          ga__fold_lanes(st, t, fbase + (GA_RD_IDX_T)(i * GA_RD_VEC) * imul, imul);
        }
#endif
        for (unsigned int i = nv * GA_RD_VEC + lane; i < len; i += GA_RD_GROUP)
          ga__take(st[0], GA_RD_LOAD(p[i]), fbase + (GA_RD_IDX_T)i * imul);
      }
#else
      {
        const unsigned int nvrow = (unsigned int)(L.inner / GA_RD_VEC);
        const unsigned int tail = (unsigned int)(L.inner - (ga__u64)nvrow * GA_RD_VEC);
        const unsigned int nrows = (unsigned int)(ue - ub);
        const unsigned int share = nrows * nvrow;
#pragma unroll 4
        for (unsigned int idx = lane; idx < share; idx += GA_RD_GROUP) {
          const unsigned int ru = ga__rd_divide(idx, L.dv);
          const unsigned int pv = idx - ru * nvrow;
          ga__i64 roff;
          GA_RD_IDX_T fbase;
          ga__row_decode(L, nro, ub + ru, roff, fbase);
          const ga__rd_pack<GA_RD_VEC> t = *reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(
              obase + roff + (ga__i64)pv * (ga__i64)(GA_RD_VEC * sizeof(GA_RD_SRC_T)));
          ga__fold_lanes(st, t, fbase + (GA_RD_IDX_T)(pv * GA_RD_VEC) * imul, imul);
        }
        if (tail != 0) {
          for (unsigned int idx = lane; idx < nrows * tail; idx += GA_RD_GROUP) {
            const unsigned int ru = idx / tail;
            const unsigned int e = nvrow * GA_RD_VEC + (idx - ru * tail);
            ga__i64 roff;
            GA_RD_IDX_T fbase;
            ga__row_decode(L, nro, ub + ru, roff, fbase);
            const GA_RD_SRC_T *p = reinterpret_cast<const GA_RD_SRC_T *>(obase + roff);
            ga__take(st[0], GA_RD_LOAD(p[e]), fbase + (GA_RD_IDX_T)e * imul);
          }
        }
      }
#endif
    }
#pragma unroll
    for (int j = 1; j < GA_RD_VEC; j++) ga__merge(st[0], st[j]);
#if GA_RD_GROUP > 32
    const ga__state tot = ga__group_reduce<GA_RD_GROUP / 32>(st[0], sm, threadIdx.x);
#else
    const ga__state tot = ga__warp_reduce(st[0]);
#endif
    if (L.splits == 1) {
      if (live && lane == 0) ga__emit(L, src, d0, d1, o, tot);
#if GA_RD_GROUP > 32
      __syncthreads();
#endif
    } else {
      /* publish, take a ticket, and let the last group of this output finish */
      int last = 0;
      if (live && lane == 0) {
        ga__put_partial(L, pval, pidx, split, o, tot);
        last = ga__take_ticket(&tickets[o], (unsigned int)L.splits) ? 1 : 0;
      }
#if GA_RD_GROUP > 32
      if (lane == 0) sm_last[threadIdx.x / GA_RD_GROUP] = last;
      __syncthreads();
      last = sm_last[threadIdx.x / GA_RD_GROUP];
#else
      last = __shfl_sync(0xffffffffu, last, 0);
#endif
      ga__state fin = ga__init();
      if (last) {
#pragma unroll 4
        for (ga__u64 sp = lane; sp < L.splits; sp += GA_RD_GROUP)
          ga__merge(fin, ga__get_partial(L, pval, pidx, sp, o));
      }
#if GA_RD_GROUP > 32
      fin = ga__group_reduce<GA_RD_GROUP / 32>(fin, sm, threadIdx.x);
      __syncthreads();
#else
      fin = ga__warp_reduce(fin);
#endif
      if (last && lane == 0) ga__emit(L, src, d0, d1, o, fin);
    }
  }
#endif /* !GA_RD_ONERUN */
}
#endif

/* ------------------------------------------------------------------ cols */
#if defined(GA_RD_BUILD_COLS)
#if GA_RD_MINB > 0
#define GA__RD_COLS_BOUNDS __launch_bounds__(32 * GA_RD_BY, GA_RD_MINB)
#elif GA_RD_SIMPLE && GA_RD_KIND == 0
/* the lean walk fits 32 registers: a full complement of resident threads per SM */
#define GA__RD_COLS_BOUNDS __launch_bounds__(32 * GA_RD_BY, 2048 / (32 * GA_RD_BY))
#else
#define GA__RD_COLS_BOUNDS __launch_bounds__(32 * GA_RD_BY)
#endif
extern "C" __global__ void GA__RD_COLS_BOUNDS
ga_rd_cols(const __grid_constant__ ga__rd_layout L, const char *src, char *d0, char *d1,
           GA_RD_ACC_T *pval, GA_RD_IDX_T *pidx, unsigned int *tickets) {
  if (L.early != 0 && threadIdx.x == 0 && blockIdx.x < L.tiles) {
    /* The first rows this row lane will walk, for the CTA's first column tile (only when
     * there is one reduced dimension and no outer kept position: the host sets `early`).
     * An L2 hint, issued before the wait so that the first DRAM reads overlap the
     * previous kernel's tail (see ga__prefetch_l2). */
    const ga__u64 c0 = (ga__u64)blockIdx.x * 32 * GA_RD_VEC;
    const ga__u64 left = L.inner - c0;
    const unsigned int nb = (unsigned int)((left < 32 * GA_RD_VEC ? left : 32 * GA_RD_VEC) *
                                           sizeof(GA_RD_SRC_T)) & ~15u;
    const ga__u64 step = L.splits * GA_RD_BY;
    ga__u64 j = (ga__u64)blockIdx.y * GA_RD_BY + threadIdx.y;
    for (ga__u64 n = 0; n < L.early && j < L.nr_total && nb != 0; n++, j += step)
      ga__prefetch_l2(src + (ga__i64)j * L.rsrc[0] + (ga__i64)(c0 * sizeof(GA_RD_SRC_T)), nb);
  }
  ga__grid_dependency_sync();
  __shared__ ga__state sm[GA_RD_BY][GA_RD_VEC][32];
  __shared__ int sm_last;
  const unsigned tx = threadIdx.x, ty = threadIdx.y;
#if GA_RD_SIMPLE
  /* One reduced dimension, one contiguous kept run and nothing else (the host checks):
   * a pointer walking down the rows with 32-bit counters. Half the registers of the
   * general loop below, so all CTAs of the grid are resident at once and the next
   * launch of the stream finds room beside them. */
  {
    const unsigned int tile = blockIdx.x, split = blockIdx.y, S = (unsigned int)L.splits;
    const unsigned int kc = (unsigned int)L.inner, nrows = (unsigned int)L.nr_total;
    const unsigned int col0 = (tile * 32 + tx) * GA_RD_VEC;
    const bool live = col0 < kc;
    ga__state st[GA_RD_VEC];
#pragma unroll
    for (int j = 0; j < GA_RD_VEC; j++) st[j] = ga__init();
    if (live) {
      /* signed counters: see the note in ga_rd_rows */
      const int jstep = (int)(S * GA_RD_BY), jend = (int)nrows;
      int j = (int)(split * GA_RD_BY + ty);
      const char *p = src + (ga__i64)j * L.rsrc[0] + (ga__i64)col0 * (ga__i64)sizeof(GA_RD_SRC_T);
      const ga__i64 step = (ga__i64)jstep * L.rsrc[0];
      const GA_RD_IDX_T rm = (GA_RD_IDX_T)L.rmul[0];
#pragma unroll ga__rd_unroll
      for (; j < jend; j += jstep) {
        const ga__rd_pack<GA_RD_VEC> t = *reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(p);
#pragma unroll
        for (int k = 0; k < GA_RD_VEC; k++) ga__take_raw(st[k], t.v[k], (GA_RD_IDX_T)j * rm);
        p += step;
      }
    }
#pragma unroll
    for (int k = 0; k < GA_RD_VEC; k++) sm[ty][k][tx] = st[k];
    __syncthreads();
    if (ty < GA_RD_VEC && live) {
      ga__state tot = sm[0][ty][tx];
#pragma unroll
      for (int y = 1; y < GA_RD_BY; y++) ga__merge(tot, sm[y][ty][tx]);
      if (S == 1) {
        ga__emit_lean(L, src, d0, d1, col0 + ty, tot);
      } else {
        pval[(ga__u64)split * L.nf_total + col0 + ty] = tot.v;
#if GA_RD_KIND == 1
        pidx[(ga__u64)split * L.nf_total + col0 + ty] = tot.i;
#endif
      }
    }
    if (S > 1) {
      __syncthreads();
      if (tx == 0 && ty == 0) sm_last = ga__take_ticket(&tickets[tile], S) ? 1 : 0;
      __syncthreads();
      if (sm_last) {
        ga__state fin[GA_RD_VEC];
#pragma unroll
        for (int k = 0; k < GA_RD_VEC; k++) fin[k] = ga__init();
        if (live) {
          for (unsigned int sp = ty; sp < S; sp += GA_RD_BY) {
            GA_RD_ACC_T pv[GA_RD_VEC];
            ga__ldcg_block<(int)(GA_RD_VEC * sizeof(GA_RD_ACC_T))>(pv, &pval[(ga__u64)sp * L.nf_total + col0]);
#if GA_RD_KIND == 1
            GA_RD_IDX_T pi[GA_RD_VEC];
            ga__ldcg_block<(int)(GA_RD_VEC * sizeof(GA_RD_IDX_T))>(pi, &pidx[(ga__u64)sp * L.nf_total + col0]);
#endif
#pragma unroll
            for (int k = 0; k < GA_RD_VEC; k++) {
              ga__state t;
              t.v = pv[k];
#if GA_RD_KIND == 1
              t.i = pi[k];
#endif
              ga__merge(fin[k], t);
            }
          }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GA_RD_VEC; k++) sm[ty][k][tx] = fin[k];
        __syncthreads();
        if (ty < GA_RD_VEC && live) {
          ga__state tot = sm[0][ty][tx];
#pragma unroll
          for (int y = 1; y < GA_RD_BY; y++) ga__merge(tot, sm[y][ty][tx]);
          ga__emit_lean(L, src, d0, d1, col0 + ty, tot);
        }
      }
    }
  }
#else
  const ga__u64 kc = L.inner;                 /* contiguous kept run */
  const ga__u64 ko_total = L.nf_total / kc;   /* outer kept positions */
  const ga__u64 nwork = ko_total * L.tiles;
  /* The splits interleave: split s takes the row blocks s, s + S, s + 2S, ...
   * (a block = GA_RD_BY consecutive reduced positions), so the CTAs running
   * at any moment read one moving window of adjacent rows - sequential DRAM
   * pages - instead of S windows that are far apart. */
  const ga__u64 split = blockIdx.y;
  const ga__u64 nblk = (L.nr_total + GA_RD_BY - 1) / GA_RD_BY;

  for (ga__u64 w = blockIdx.x; w < nwork; w += gridDim.x) {
    ga__u64 ko = 0, tile = w;
    if (ko_total > 1) {
      ko = w / L.tiles;
      tile = w - ko * L.tiles;
    }
    const ga__u64 col0 = (tile * 32 + tx) * GA_RD_VEC;
    const bool live = col0 < kc;
    const ga__u64 o0 = ko * kc + col0; /* first output of this thread */
    ga__state st[GA_RD_VEC];
#pragma unroll
    for (int j = 0; j < GA_RD_VEC; j++) st[j] = ga__init();

    if (live) {
      /* kept offset: the innermost kept dim is the contiguous one */
      ga__i64 koff = (ga__i64)col0 * (ga__i64)sizeof(GA_RD_SRC_T);
      {
        ga__u64 q = ko;
        for (int d = (int)L.nf - 2; d >= 0; d--) {
          const ga__u64 qq = q / L.fdim[d];
          koff += (ga__i64)(q - qq * L.fdim[d]) * L.fsrc[d];
          q = qq;
        }
      }
      const char *base = src + koff;
      const unsigned int cnt =
          (nblk > split) ? (unsigned int)((nblk - split + L.splits - 1) / L.splits) : 0u;
      if (L.nr == 1) {
        /* one reduced dimension: a pointer walking down with a fixed step */
        const ga__u64 j0 = split * GA_RD_BY + ty;
        const ga__u64 jstep = L.splits * GA_RD_BY;
        const ga__i64 step = (ga__i64)jstep * L.rsrc[0];
        const GA_RD_IDX_T fstep = (GA_RD_IDX_T)jstep * (GA_RD_IDX_T)L.rmul[0];
        const char *p = base + (ga__i64)j0 * L.rsrc[0];
        GA_RD_IDX_T f = (GA_RD_IDX_T)j0 * (GA_RD_IDX_T)L.rmul[0];
        /* only the last block can be ragged */
        const unsigned int full = (cnt > 0 && j0 + (ga__u64)(cnt - 1) * jstep >= L.nr_total) ? cnt - 1 : cnt;
#pragma unroll ga__rd_unroll
        for (unsigned int n = 0; n < full; n++) {
          const ga__rd_pack<GA_RD_VEC> t = *reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(p);
#pragma unroll
          for (int k = 0; k < GA_RD_VEC; k++) ga__take_raw(st[k], t.v[k], f);
          p += step;
          f += fstep;
        }
      } else {
        for (unsigned int n = 0; n < cnt; n++) {
          const ga__u64 j = ((ga__u64)n * L.splits + split) * GA_RD_BY + ty;
          if (j >= L.nr_total) break;
          ga__u64 r = j;
          ga__i64 roff = 0;
          GA_RD_IDX_T f = 0;
          for (int d = (int)L.nr - 1; d >= 0; d--) {
            const ga__u64 q = r / L.rdim[d], c = r - q * L.rdim[d];
            r = q;
            roff += (ga__i64)c * L.rsrc[d];
            f += (GA_RD_IDX_T)c * (GA_RD_IDX_T)L.rmul[d];
          }
          const ga__rd_pack<GA_RD_VEC> t =
              *reinterpret_cast<const ga__rd_pack<GA_RD_VEC> *>(base + roff);
#pragma unroll
          for (int k = 0; k < GA_RD_VEC; k++) ga__take_raw(st[k], t.v[k], f);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < GA_RD_VEC; k++) sm[ty][k][tx] = st[k];
    __syncthreads();
    /* row-lane ty finishes vector lane k == ty (fixed order over the row lanes) */
    if (ty < GA_RD_VEC && live) {
      ga__state tot = sm[0][ty][tx];
#pragma unroll
      for (int y = 1; y < GA_RD_BY; y++) ga__merge(tot, sm[y][ty][tx]);
      if (L.splits == 1) {
        ga__emit(L, src, d0, d1, o0 + ty, tot);
      } else { /* partials as [split][output]: neighbouring threads, neighbouring cells */
        pval[split * L.nf_total + o0 + ty] = tot.v;
#if GA_RD_KIND == 1
        pidx[split * L.nf_total + o0 + ty] = tot.i;
#endif
      }
    }
    if (L.splits > 1) {
      /* all partials of this tile are stored: one ticket per tile */
      __syncthreads();
      if (tx == 0 && ty == 0) sm_last = ga__take_ticket(&tickets[w], (unsigned int)L.splits) ? 1 : 0;
      __syncthreads();
      if (sm_last) {
        /* the row lanes share the splits, then combine as above */
        ga__state fin[GA_RD_VEC];
#pragma unroll
        for (int k = 0; k < GA_RD_VEC; k++) fin[k] = ga__init();
        if (live) {
#pragma unroll 4
          for (ga__u64 sp = ty; sp < L.splits; sp += GA_RD_BY) {
            /* the thread's GA_RD_VEC outputs are adjacent cells: one wide load */
            GA_RD_ACC_T pv[GA_RD_VEC];
            ga__ldcg_block<(int)(GA_RD_VEC * sizeof(GA_RD_ACC_T))>(pv, &pval[sp * L.nf_total + o0]);
#if GA_RD_KIND == 1
            GA_RD_IDX_T pi[GA_RD_VEC];
            ga__ldcg_block<(int)(GA_RD_VEC * sizeof(GA_RD_IDX_T))>(pi, &pidx[sp * L.nf_total + o0]);
#endif
#pragma unroll
            for (int k = 0; k < GA_RD_VEC; k++) {
              ga__state t;
              t.v = pv[k];
#if GA_RD_KIND == 1
              t.i = pi[k];
#endif
              ga__merge(fin[k], t);
            }
          }
        }
        __syncthreads(); /* sm still holds this tile's first-stage states */
#pragma unroll
        for (int k = 0; k < GA_RD_VEC; k++) sm[ty][k][tx] = fin[k];
        __syncthreads();
        if (ty < GA_RD_VEC && live) {
          ga__state tot = sm[0][ty][tx];
#pragma unroll
          for (int y = 1; y < GA_RD_BY; y++) ga__merge(tot, sm[y][ty][tx]);
          ga__emit(L, src, d0, d1, o0 + ty, tot);
        }
      }
    }
    __syncthreads();
  }
#endif /* !GA_RD_SIMPLE */
}
#endif

/* --------------------------------------------------------------- general */
#if defined(GA_RD_BUILD_GENERAL)
/* GA_RD_TPO threads per output (1, 32 or GA_RD_THREADS). */
extern "C" __global__ void __launch_bounds__(GA_RD_THREADS)
ga_rd_general(const __grid_constant__ ga__rd_layout L, const char *src, char *d0, char *d1,
              GA_RD_ACC_T *pval, GA_RD_IDX_T *pidx, unsigned int *tickets) {
  ga__grid_dependency_sync();
#if GA_RD_TPO > 32
  __shared__ ga__state sm[32];
#endif
  const unsigned lane = threadIdx.x % GA_RD_TPO;
  const ga__u64 group = ((ga__u64)blockIdx.x * GA_RD_THREADS + threadIdx.x) / GA_RD_TPO;
  const ga__u64 ngroups = (ga__u64)gridDim.x * (GA_RD_THREADS / GA_RD_TPO);
  /* every group runs the same number of rounds so that CTA-wide barriers match */
  const ga__u64 rounds = (L.nf_total + ngroups - 1) / ngroups;

  for (ga__u64 it = 0; it < rounds; it++) {
    const ga__u64 o = group + it * ngroups;
    const bool live = o < L.nf_total;
    ga__state st = ga__init();
    if (live) {
      const char *obase = src + ga__foff(L, L.fsrc, o);
      for (ga__u64 j = lane; j < L.nr_total; j += GA_RD_TPO) {
        ga__u64 r = j;
        ga__i64 roff = 0;
        GA_RD_IDX_T f = 0;
        for (int d = (int)L.nr - 1; d >= 0; d--) {
          const ga__u64 q = r / L.rdim[d], c = r - q * L.rdim[d];
          r = q;
          roff += (ga__i64)c * L.rsrc[d];
          f += (GA_RD_IDX_T)c * (GA_RD_IDX_T)L.rmul[d];
        }
        const GA_RD_SRC_T raw = *reinterpret_cast<const GA_RD_SRC_T *>(obase + roff);
        ga__take(st, GA_RD_LOAD(raw), f);
      }
    }
#if GA_RD_TPO == 32
    st = ga__warp_reduce(st);
#elif GA_RD_TPO > 32
    st = ga__block_reduce(st, sm, threadIdx.x, GA_RD_THREADS);
    __syncthreads();
#endif
    if (live && lane == 0) ga__emit(L, src, d0, d1, o, st);
  }
}
#endif
