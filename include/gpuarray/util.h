/* Type table access, dimension collapsing and host half conversion.
 * Follows src/gpuarray/util.h of the reference (prototypes :33-96,
 * ga_float2half :103-183). */
#ifndef GPUARRAY_UTIL
#define GPUARRAY_UTIL

#include <gpuarray/config.h>
#include <gpuarray/elemwise.h>
#include <gpuarray/types.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Registers a user type; returns its new typecode (>= 512) or -1. */
/* replaces src/gpuarray/util.h:35 */
GPUARRAY_PUBLIC int gpuarray_register_type(gpuarray_type *t, int *ret);
/* Never NULL: unknown codes give a descriptor with typecode -1 and size 0. */
/* replaces src/gpuarray/util.h:46 */
GPUARRAY_PUBLIC const gpuarray_type *gpuarray_get_type(int typecode);
/* replaces src/gpuarray/util.h:57 */
GPUARRAY_PUBLIC size_t gpuarray_get_elsize(int typecode);
/* OR of the GA_USE_* flags needed by a -1 terminated list of typecodes. */
/* replaces src/gpuarray/util.h:74 */
GPUARRAY_PUBLIC int gpuarray_type_flags(int init, ...);
/* replaces src/gpuarray/util.h:76 */
GPUARRAY_PUBLIC int gpuarray_type_flagsa(unsigned int n, gpuelemwise_arg *arg);

/* Removes size-1 dimensions (keeping at least one) and merges neighbouring
 * dimensions that are jointly contiguous for every one of the `n` stride
 * vectors (NULL entries are skipped). Works in place. Same contract as
 * src/gpuarray_util.c:153-188. */
/* replaces src/gpuarray/util.h:97 */
GPUARRAY_PUBLIC void gpuarray_elemwise_collapse(unsigned int n, unsigned int *nd,
                                                size_t *dim, ssize_t **strs);

typedef struct _ga_half_t { uint16_t h; } ga_half_t;

/* float -> IEEE binary16, round to nearest even, NaN payload kept non-zero:
 * the rounding the device applies (cvt.rn.f16.f32) when a kernel stores a
 * GA_HALF result. The reference's host routine (src/gpuarray/util.h:103-183)
 * differs only on exact ties, which it rounds away from zero; the known
 * answers of tests/check_util.c:121-148 hold for both. */
static inline ga_half_t ga_float2half(float f) {
  union { float f; uint32_t u; } in;
  ga_half_t out;
  uint32_t sign, mag, exp, man, shift, lost, half;
  in.f = f;
  sign = (in.u >> 16) & 0x8000u;
  mag = in.u & 0x7fffffffu;
  if (mag >= 0x7f800000u) {          /* inf / nan */
    man = mag & 0x007fffffu;
    out.h = (uint16_t)(sign | 0x7c00u | (man ? ((man >> 13) ? (man >> 13) : 1u) : 0u));
    return out;
  }
  if (mag >= 0x477ff000u) {          /* rounds to or beyond 65520 -> inf */
    out.h = (uint16_t)(sign | 0x7c00u);
    return out;
  }
  exp = mag >> 23;
  if (exp >= 113) {                  /* normal half */
    man = mag & 0x007fffffu;
    half = ((exp - 112) << 10) | (man >> 13);
    lost = man & 0x1fffu;
    if (lost > 0x1000u || (lost == 0x1000u && (half & 1u))) half++;
    out.h = (uint16_t)(sign | half);
    return out;
  }
  if (exp < 102) {                   /* below half of the smallest subnormal */
    out.h = (uint16_t)sign;
    return out;
  }
  man = (mag & 0x007fffffu) | 0x00800000u;
  shift = 126 - exp;                 /* 14..24 */
  half = man >> shift;
  lost = man & ((1u << shift) - 1u);
  if (lost > (1u << (shift - 1)) || (lost == (1u << (shift - 1)) && (half & 1u))) half++;
  out.h = (uint16_t)(sign | half);
  return out;
}

#ifdef __cplusplus
}
#endif
#endif /* GPUARRAY_UTIL */
