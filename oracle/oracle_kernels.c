/* CPU oracle for the elementwise/reduction engine. TEST INFRASTRUCTURE ONLY:
 * nothing in the product links or calls this file; only tests/, the smoke
 * check and the cpu_baseline/reference legs of bench.py may use it.
 *
 * Each function restates, in plain C loops, what a kernel of the reference
 * computes:
 *   oracle_minmaxarg   the generated maxandargmax kernel
 *                      (src/gpuarray_reduction.c:557-606: first reduced element
 *                      initialises, reduced axes looped in reduxList order with
 *                      the last listed axis fastest, strict comparison, flat
 *                      index per src/gpuarray/array.h:620-636) and its mirror
 *                      image for min;
 *   oracle_collapse    gpuarray_elemwise_collapse (src/gpuarray_util.c:153-188);
 *   oracle_float2half  device store conversion cvt.rn.f16.f32
 *                      (src/cluda_cuda.h:72-77), i.e. IEEE round-to-nearest-even;
 *   oracle_half2float  cvt.f32.f16 (src/cluda_cuda.h:68-71);
 *   oracle_fma_f32     a*b+c as NVRTC contracts it by default (single rounding;
 *                      the reference passes no -fmad option,
 *                      src/gpuarray_buffer_cuda.c:1113-1121).
 * Pinned by tests/test_oracle.py against the known answers of the reference's
 * tests/check_util.c:41-148 and tests/check_reduction.c, and by
 * tests/test_golden.py against outputs of the reference's own compiled util
 * code (tests/golden/).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include <sys/types.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* typecodes of include/gpuarray/types.h */
enum { T_BOOL = 0, T_BYTE, T_UBYTE, T_SHORT, T_USHORT, T_INT, T_UINT, T_LONG, T_ULONG,
       T_FLOAT = 11, T_DOUBLE = 12, T_HALF = 23 };

float oracle_half2float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
  float f;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      int e = -1;
      do { man <<= 1; e++; } while ((man & 0x400u) == 0);
      bits = sign | ((uint32_t)(112 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
  else bits = sign | ((exp + 112) << 23) | (man << 13);
  memcpy(&f, &bits, 4);
  return f;
}

uint16_t oracle_float2half(float f) {
  uint32_t u, sign, mag, exp, man, half, lost, shift;
  memcpy(&u, &f, 4);
  sign = (u >> 16) & 0x8000u;
  mag = u & 0x7fffffffu;
  if (mag > 0x7f800000u) return (uint16_t)0x7fffu;          /* cvt gives the canonical NaN */
  if (mag == 0x7f800000u) return (uint16_t)(sign | 0x7c00u);
  exp = mag >> 23;
  if (exp >= 113) {
    if (exp >= 143) return (uint16_t)(sign | 0x7c00u);
    man = mag & 0x7fffffu;
    half = ((exp - 112) << 10) | (man >> 13);
    lost = man & 0x1fffu;
    if (lost > 0x1000u || (lost == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
  }
  if (exp < 102) return (uint16_t)sign;
  man = (mag & 0x7fffffu) | 0x800000u;
  shift = 126 - exp;
  half = man >> shift;
  lost = man & ((1u << shift) - 1u);
  if (lost > (1u << (shift - 1)) || (lost == (1u << (shift - 1)) && (half & 1u))) half++;
  return (uint16_t)(sign | half);
}

void oracle_fma_f32(const float *a, const float *b, float c, float *out, size_t n) {
  size_t i;
  for (i = 0; i < n; i++) out[i] = fmaf(a[i], b[i], c);
}

void oracle_collapse(unsigned n, unsigned *pnd, size_t *dims, ssize_t **strs) {
  unsigned nd = *pnd, i, j, k;
  /* size-1 removal, scanning from the last dimension, keeping one dimension */
  for (i = nd; i > 0; i--) {
    if (nd > 1 && dims[i - 1] == 1) {
      for (j = i - 1; j + 1 < nd; j++) {
        dims[j] = dims[j + 1];
        for (k = 0; k < n; k++) if (strs[k]) strs[k][j] = strs[k][j + 1];
      }
      nd--;
    }
  }
  /* merge i into i-1 when contiguous for every argument, from the last pair */
  for (i = nd - 1; i > 0; i--) {
    int ok = 1;
    for (k = 0; k < n; k++)
      ok &= (strs[k] == NULL || strs[k][i - 1] == (ssize_t)dims[i] * strs[k][i]);
    if (!ok) continue;
    dims[i - 1] *= dims[i];
    for (k = 0; k < n; k++) if (strs[k]) strs[k][i - 1] = strs[k][i];
    for (j = i; j + 1 < nd; j++) {
      dims[j] = dims[j + 1];
      for (k = 0; k < n; k++) if (strs[k]) strs[k][j] = strs[k][j + 1];
    }
    nd--;
  }
  *pnd = nd;
}

/* value at byte offset `off` of `p`, as a double-free comparison key is not
 * possible for 64-bit ints, so comparisons are instantiated per type */
#define MINMAX_BODY(T, LOADEXPR)                                                         \
  {                                                                                      \
    T best = LOADEXPR(base + first_off);                                                 \
    int64_t besti = 0, flat = 0;                                                         \
    size_t cnt;                                                                          \
    memset(rc, 0, sizeof(rc));                                                           \
    for (cnt = 0; cnt < nred; cnt++) {                                                   \
      ssize_t off = 0;                                                                   \
      for (k = 0; k < reduxLen; k++) off += (ssize_t)rc[k] * strides[reduxList[k]];      \
      {                                                                                  \
        T v = LOADEXPR(base + off);                                                      \
        if (is_min ? (v < best) : (v > best)) {                                          \
          best = v;                                                                      \
          besti = flat;                                                                  \
          bestoff = off;                                                                 \
        }                                                                                \
      }                                                                                  \
      flat++;                                                                            \
      for (k = reduxLen; k > 0; k--) {                                                   \
        if (++rc[k - 1] < dims[reduxList[k - 1]]) break;                                 \
        rc[k - 1] = 0;                                                                   \
      }                                                                                  \
    }                                                                                    \
    if (dstIdx) dstIdx[o] = besti;                                                       \
  }

#define LD(T) *(const T *)
#define LDH(p) oracle_half2float(*(const uint16_t *)(p))

/* src: element [0..0] pointer with byte strides (may be negative).
 * dstVal: contiguous array of the source type over the free axes in ascending
 * order (raw bytes of the winning element are copied, so -0.0 / NaN payloads
 * survive); dstIdx: contiguous int64. Returns 0, or -1 for bad arguments. */
int oracle_minmaxarg(int typecode, int is_min, const void *src, unsigned nd, const size_t *dims,
                     const ssize_t *strides, unsigned reduxLen, const unsigned *reduxList,
                     void *dstVal, int64_t *dstIdx) {
  unsigned freeax[64], nfree = 0, i, k;
  size_t fc[64], rc[64], nout = 1, nred = 1, o, elsize;
  unsigned char isred[64];
  const char *srcb = (const char *)src;

  if (nd == 0 || nd > 64 || reduxLen == 0 || reduxLen > nd) return -1;
  memset(isred, 0, sizeof(isred));
  for (k = 0; k < reduxLen; k++) {
    if (reduxList[k] >= nd || isred[reduxList[k]]) return -1;
    isred[reduxList[k]] = 1;
    nred *= dims[reduxList[k]];
  }
  for (i = 0; i < nd; i++)
    if (!isred[i]) {
      freeax[nfree++] = i;
      nout *= dims[i];
    }
  switch (typecode) {
  case T_BOOL: case T_BYTE: case T_UBYTE: elsize = 1; break;
  case T_SHORT: case T_USHORT: case T_HALF: elsize = 2; break;
  case T_INT: case T_UINT: case T_FLOAT: elsize = 4; break;
  case T_LONG: case T_ULONG: case T_DOUBLE: elsize = 8; break;
  default: return -1;
  }
  if (nred == 0) return nout == 0 ? 0 : -1;
  memset(fc, 0, sizeof(fc));
  for (o = 0; o < nout; o++) {
    const char *base = srcb;
    ssize_t first_off = 0, bestoff = 0;
    for (i = 0; i < nfree; i++) base += (ssize_t)fc[i] * strides[freeax[i]];
    switch (typecode) {
    case T_BOOL: case T_UBYTE: MINMAX_BODY(uint8_t, LD(uint8_t)) break;
    case T_BYTE: MINMAX_BODY(int8_t, LD(int8_t)) break;
    case T_SHORT: MINMAX_BODY(int16_t, LD(int16_t)) break;
    case T_USHORT: MINMAX_BODY(uint16_t, LD(uint16_t)) break;
    case T_INT: MINMAX_BODY(int32_t, LD(int32_t)) break;
    case T_UINT: MINMAX_BODY(uint32_t, LD(uint32_t)) break;
    case T_LONG: MINMAX_BODY(int64_t, LD(int64_t)) break;
    case T_ULONG: MINMAX_BODY(uint64_t, LD(uint64_t)) break;
    case T_FLOAT: MINMAX_BODY(float, LD(float)) break;
    case T_DOUBLE: MINMAX_BODY(double, LD(double)) break;
    case T_HALF: MINMAX_BODY(float, LDH) break;
    }
    if (dstVal) memcpy((char *)dstVal + o * elsize, base + bestoff, elsize);
    for (i = nfree; i > 0; i--) {
      if (++fc[i - 1] < dims[freeax[i - 1]]) break;
      fc[i - 1] = 0;
    }
  }
  return 0;
}

/* Thread team of the timed CPU baseline. oracle_set_threads(n) fixes the team
 * size whatever OMP_NUM_THREADS says (launchers such as torch.distributed.run
 * export OMP_NUM_THREADS=1); oracle_threads_used() opens a parallel region
 * and returns the team size the runtime really gave. Both return 1 when the
 * file was built without OpenMP. */
int oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) {
    omp_set_dynamic(0);
    omp_set_num_threads(n);
  }
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

int oracle_threads_used(void) {
  int team = 1;
#ifdef _OPENMP
#pragma omp parallel
  {
#pragma omp master
    team = omp_get_num_threads();
  }
#endif
  return team;
}

/* Row-wise max and first argmax of a C-contiguous float matrix: the cfg-3
 * shape, used by the timed CPU baseline (OpenMP over rows when enabled). */
void oracle_rowmaxarg_f32(const float *x, size_t rows, size_t cols, float *vmax, int64_t *imax) {
  ssize_t r;
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
  for (r = 0; r < (ssize_t)rows; r++) {
    const float *p = x + (size_t)r * cols;
    float best = p[0];
    size_t bi = 0, c;
    for (c = 1; c < cols; c++)
      if (p[c] > best) {
        best = p[c];
        bi = c;
      }
    vmax[r] = best;
    imax[r] = (int64_t)bi;
  }
}

/* PCG XSH RR 64/32 as used by the reference's reduction tests to fill their
 * inputs (tests/check_reduction.c:37-63): state starts at the seed, each
 * double takes two 32-bit draws (high word first) scaled by 2^-64. */
void oracle_pcg_fill_f32(uint64_t seed, float *out, size_t n) {
  uint64_t s = seed;
  size_t i;
  int h;
  for (i = 0; i < n; i++) {
    uint64_t w[2];
    for (h = 0; h < 2; h++) {
      uint32_t x, rot;
      s = s * 6364136223846793005ULL + 1442695040888963407ULL;
      x = (uint32_t)((s ^ (s >> 18)) >> 27);
      rot = (uint32_t)(s >> 59) & 31u;
      w[h] = rot ? ((x >> rot) | (x << (32 - rot))) : x;
    }
    out[i] = (float)((double)((w[0] << 32) | w[1]) / 18446744073709551616.0);
  }
}
