/* Host stand-in for the kernel-side header, used only by the SIMT emulator in
 * tests/simt: the kernel templates are compiled for the CPU and their threads
 * run as cooperative fibers (simt_emul.h). Provides the element types, the
 * half conversions (IEEE round-to-nearest-even, like the device instructions)
 * and the few intrinsics the templates use. */
#ifndef CLUDA_H
#define CLUDA_H
#include "simt_emul.h"

typedef unsigned char ga_bool;
typedef signed char ga_byte;
typedef unsigned char ga_ubyte;
typedef short ga_short;
typedef unsigned short ga_ushort;
typedef int ga_int;
typedef unsigned int ga_uint;
typedef long long ga_long;
typedef unsigned long long ga_ulong;
typedef float ga_float;
typedef double ga_double;
typedef size_t ga_size;
typedef ptrdiff_t ga_ssize;

struct ga_half {
  ga_ushort data;
};

static inline float ga_half2float(ga_half h) {
  _Float16 v;
  memcpy(&v, &h.data, 2);
  return (float)v;
}
static inline ga_half ga_float2half(float f) {
  const _Float16 v = (_Float16)f; /* round to nearest even */
  ga_half h;
  memcpy(&h.data, &v, 2);
  return h;
}

static inline float ga__add_f32_f16(float acc, ga_half h) { return acc + ga_half2float(h); }
static inline void ga__grid_dependency_sync() {}
static inline void ga__fence_system() {}
static inline void ga__st_release_sys(unsigned long long *p, unsigned long long v) { *p = v; }
static inline unsigned long long ga__ld_acquire_sys(const unsigned long long *p) { return *p; }
static inline unsigned long long ga__globaltimer_ns() { static unsigned long long t; return t += 1000; }
static inline void ga__nanosleep(unsigned int) {}
template <typename T>
static inline T ga__ld_volatile(const T *p) { return *p; }
static inline void ga__prefetch_l2(const void *, unsigned int) {}
static inline void ga__cp_async16(void *smem, const void *gmem) { memcpy(smem, gmem, 16); }
static inline void ga__cp_async_wait_all() {}
/* ldmatrix.x4.trans: lane 8m + rho publishes the address of row rho of matrix m; lane i
 * reads elements [2*(i%4)][i/4] and [2*(i%4)+1][i/4] of each matrix */
static inline void ga__ldsm_x4_trans(const void *row, unsigned int r[4]) {
  const unsigned lane = simt::cur->linear % 32;
  for (int m = 0; m < 4; m++) {
    unsigned short e[2];
    for (int k = 0; k < 2; k++) {
      const unsigned src = 8 * m + 2 * (lane % 4) + k;
      const unsigned long long a = simt::exchange((unsigned long long)(uintptr_t)row, src);
      memcpy(&e[k], (const char *)(uintptr_t)a + 2 * (lane / 4), 2);
    }
    r[m] = (unsigned int)e[0] | ((unsigned int)e[1] << 16);
  }
}
#endif
