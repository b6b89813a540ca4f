/* Helpers shared by the elementwise kernel templates: 128-bit packs,
 * storage<->compute conversion, exact 32-bit division by invariant divisors. */
#ifndef GA_EW_COMMON_CUH
#define GA_EW_COMMON_CUH

#include "cluda.h"

template <typename T, int N>
struct alignas((sizeof(T) * N >= 16) ? 16 : sizeof(T) * N) ga__pack {
  T v[N];
};

/* Storage type S <-> type C seen by the expression. Identity except for
 * ga_half computed as float (GE_CONVERT_F16). */
template <typename C, typename S>
struct ga__conv {
  static __device__ __forceinline__ C in(const S &s) { return s; }
  static __device__ __forceinline__ S out(const C &c) { return c; }
};
template <>
struct ga__conv<float, ga_half> {
  static __device__ __forceinline__ float in(const ga_half &s) { return ga_half2float(s); }
  static __device__ __forceinline__ ga_half out(const float &c) { return ga_float2half(c); }
};

/* N consecutive elements starting at p (aligned to min(16, N*sizeof(S))
 * bytes) as the widest loads available, converted into c[0..N). */
template <typename C, typename S, int N>
static __device__ __forceinline__ void ga__load_run(const S *p, C *c) {
  constexpr int PER = (sizeof(S) * N >= 16) ? (16 / sizeof(S)) : N;
#pragma unroll
  for (int k = 0; k < N / PER; k++) {
    const ga__pack<S, PER> t = *reinterpret_cast<const ga__pack<S, PER> *>(p + k * PER);
#pragma unroll
    for (int j = 0; j < PER; j++) c[k * PER + j] = ga__conv<C, S>::in(t.v[j]);
  }
}

template <typename C, typename S, int N>
static __device__ __forceinline__ void ga__store_run(S *p, const C *c) {
  constexpr int PER = (sizeof(S) * N >= 16) ? (16 / sizeof(S)) : N;
#pragma unroll
  for (int k = 0; k < N / PER; k++) {
    ga__pack<S, PER> t;
#pragma unroll
    for (int j = 0; j < PER; j++) t.v[j] = ga__conv<C, S>::out(c[k * PER + j]);
    *reinterpret_cast<ga__pack<S, PER> *>(p + k * PER) = t;
  }
}

/* Division of any 32-bit n by a fixed d >= 1 with one multiply-high:
 * q = (t + ((n - t) >> s1)) >> s2, t = mulhi(m, n). The host derives
 * (m, s1, s2) from d; exact for every n. */
struct ga__div32 {
  unsigned int d, m, s1, s2;
};
static __device__ __forceinline__ unsigned int ga__divide(unsigned int n, const ga__div32 &k) {
  const unsigned int t = __umulhi(k.m, n);
  return (t + ((n - t) >> k.s1)) >> k.s2;
}

#endif
