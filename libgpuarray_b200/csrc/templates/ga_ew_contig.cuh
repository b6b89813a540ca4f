/* Contiguous elementwise kernel: every array argument is one linear run of n
 * elements (all C- or all F-contiguous with identical shapes).
 *
 * Replaces the kernel built by the reference's gen_elemwise_contig_kernel
 * (src/gpuarray_elemwise.c:444-545), a grid-stride loop of scalar loads.
 * Here each thread moves GA_EW_EPT consecutive elements of every argument
 * with 128-bit accesses and keeps GA_EW_UNROLL such groups in flight, so a
 * warp reads whole 512-byte spans and enough bytes are outstanding to cover
 * HBM latency. The host picks GA_EW_EPT so that the narrowest argument still
 * moves 16 bytes per access; it selects the GA_EW_EPT == 1 build when a base
 * address is not 16-byte aligned.
 *
 * The including translation unit must define:
 *   GA_EW_ARRAYS(X)   X(k, name, storage_t, compute_t, is_read, is_write, mode) per array
 *                     (k = ordinal among arrays; mode is unused here)
 *   GA_EW_SCALARS(X)  X(name, type) per scalar argument
 *   GA_EW_EPT, GA_EW_UNROLL, GA_EW_THREADS, GA_EW_IDX (unsigned int or size_t)
 *   ga_ew_apply(compute_t &arrays..., scalars..., int)  the user's expression
 */
#include "ga_ew_common.cuh"

#define GA__P_ARR(k, n, S, C, R, W, M) , S *n##_p
#define GA__P_SC(n, T) , T n##_s
#define GA__DECL(k, n, S, C, R, W, M) C n##_c[GA_EW_UNROLL * GA_EW_EPT];
#define GA__LOAD(k, n, S, C, R, W, M) \
  if (R) ga__load_run<C, S, GA_EW_EPT>(n##_p + (size_t)v * GA_EW_EPT, &n##_c[u * GA_EW_EPT]);
#define GA__STORE(k, n, S, C, R, W, M) \
  if (W) ga__store_run<C, S, GA_EW_EPT>(n##_p + (size_t)v * GA_EW_EPT, &n##_c[u * GA_EW_EPT]);
#define GA__ARG_ARR(k, n, S, C, R, W, M) n##_c[e],
#define GA__ARG_SC(n, T) n##_s,
#define GA__TDECL(k, n, S, C, R, W, M) C n##_t;
#define GA__TLOAD(k, n, S, C, R, W, M) if (R) n##_t = ga__conv<C, S>::in(n##_p[i]);
#define GA__TSTORE(k, n, S, C, R, W, M) if (W) n##_p[i] = ga__conv<C, S>::out(n##_t);
#define GA__TARG(k, n, S, C, R, W, M) n##_t,

#ifndef GA_EW_EARLY
#define GA_EW_EARLY 1 /* 1: a warp asks the first 32 vectors of every input into L2 before the wait
                         for the previous kernel of the stream (see ga__prefetch_l2). Measured on
                         B200, o = a * b + 0.5f over 2^24 fp32, launches back to back on rotating
                         buffers: 31.0 -> 30.3 us; float16 2^25: 19.8 -> 19.4 us; uint8: no change */
#endif
#define GA__EARLY(k, n, S, C, R, W, M)                                                        \
  if (R) ga__prefetch_l2(n##_p + (size_t)ga__w0 * GA_EW_EPT, 32u * GA_EW_EPT * (unsigned int)sizeof(S));

extern "C" __global__ void __launch_bounds__(GA_EW_THREADS)
ga_ew_contig(const size_t n GA_EW_ARRAYS(GA__P_ARR) GA_EW_SCALARS(GA__P_SC)) {
#if GA_EW_EARLY && GA_EW_EPT > 1
  {
    /* vector builds only: their bases are 16-byte aligned */
    const size_t ga__w0 = (size_t)blockIdx.x * GA_EW_THREADS + (threadIdx.x & ~31u);
    if ((threadIdx.x & 31u) == 0 && (ga__w0 + 32) * GA_EW_EPT <= n) { GA_EW_ARRAYS(GA__EARLY) }
  }
#endif
  ga__grid_dependency_sync();
  const GA_EW_IDX nvec = (GA_EW_IDX)(n / GA_EW_EPT);
  const GA_EW_IDX nthr = (GA_EW_IDX)gridDim.x * GA_EW_THREADS;
  const GA_EW_IDX tid = (GA_EW_IDX)blockIdx.x * GA_EW_THREADS + threadIdx.x;

  for (GA_EW_IDX v0 = tid; v0 < nvec; v0 += nthr * GA_EW_UNROLL) {
    GA_EW_ARRAYS(GA__DECL)
#pragma unroll
    for (int u = 0; u < GA_EW_UNROLL; u++) {
      const GA_EW_IDX v = v0 + (GA_EW_IDX)u * nthr;
      if (v < nvec) { GA_EW_ARRAYS(GA__LOAD) }
    }
#pragma unroll
    for (int e = 0; e < GA_EW_UNROLL * GA_EW_EPT; e++)
      ga_ew_apply(GA_EW_ARRAYS(GA__ARG_ARR) GA_EW_SCALARS(GA__ARG_SC) 0);
#pragma unroll
    for (int u = 0; u < GA_EW_UNROLL; u++) {
      const GA_EW_IDX v = v0 + (GA_EW_IDX)u * nthr;
      if (v < nvec) { GA_EW_ARRAYS(GA__STORE) }
    }
  }

#if GA_EW_EPT > 1
  /* fewer than GA_EW_EPT trailing elements */
  {
    const size_t i = (size_t)nvec * GA_EW_EPT + tid;
    if (i < n) {
      GA_EW_ARRAYS(GA__TDECL)
      GA_EW_ARRAYS(GA__TLOAD)
      ga_ew_apply(GA_EW_ARRAYS(GA__TARG) GA_EW_SCALARS(GA__ARG_SC) 0);
      GA_EW_ARRAYS(GA__TSTORE)
    }
  }
#endif
}
