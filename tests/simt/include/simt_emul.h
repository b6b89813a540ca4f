/* A small SIMT emulator: the threads of one CTA run as cooperative fibers
 * (ucontext) on one OS thread, CTAs run one after the other. Barriers and warp
 * shuffles are rendezvous points of the fibers. It executes kernel LOGIC -
 * indexing, tails, splits, arrival tickets, merges - not timing or races. */
#ifndef SIMT_EMUL_H
#define SIMT_EMUL_H
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <ucontext.h>

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __shared__ static
#define __launch_bounds__(...)
#define __grid_constant__
#define warpSize 32

struct simt_dim3 {
  unsigned int x, y, z;
};
struct uint2 {
  unsigned int x, y;
};
struct alignas(16) uint4 {
  unsigned int x, y, z, w;
};

namespace simt {
struct Fiber {
  ucontext_t ctx;
  char *stack;
  simt_dim3 tid;
  unsigned linear;
  int done;
};
extern Fiber *cur;
extern ucontext_t sched;
extern simt_dim3 block_idx, grid_dim, block_dim;
extern unsigned live_threads;
/* rendezvous state */
extern unsigned cta_count, cta_gen;
extern unsigned warp_count[64], warp_gen[64];
extern unsigned long long warp_slot[64][32];
static inline void yield() { swapcontext(&cur->ctx, &sched); }
static inline void cta_barrier() {
  const unsigned g = cta_gen;
  if (++cta_count == live_threads) {
    cta_count = 0;
    cta_gen++;
  } else {
    while (cta_gen == g) yield();
  }
}
static inline void warp_barrier(unsigned w, unsigned lanes) {
  const unsigned g = warp_gen[w];
  if (++warp_count[w] == lanes) {
    warp_count[w] = 0;
    warp_gen[w]++;
  } else {
    while (warp_gen[w] == g) yield();
  }
}
static inline unsigned warp_lanes(unsigned w) {
  const unsigned total = block_dim.x * block_dim.y * block_dim.z;
  const unsigned first = w * 32;
  return total - first < 32 ? total - first : 32;
}
/* every lane publishes, all meet, every lane reads */
static inline unsigned long long exchange(unsigned long long v, unsigned src_lane) {
  const unsigned w = cur->linear / 32, lane = cur->linear % 32, n = warp_lanes(w);
  warp_slot[w][lane] = v;
  warp_barrier(w, n);
  const unsigned long long r = src_lane < n ? warp_slot[w][src_lane] : v;
  warp_barrier(w, n);
  return r;
}
}  // namespace simt

#define threadIdx (simt::cur->tid)
#define blockIdx (simt::block_idx)
#define gridDim (simt::grid_dim)
#define blockDim (simt::block_dim)

static inline void __syncthreads() { simt::cta_barrier(); }
static inline void __syncwarp(unsigned = 0xffffffffu) {
  const unsigned w = simt::cur->linear / 32;
  simt::warp_barrier(w, simt::warp_lanes(w));
}
static inline void __threadfence() {}

template <typename T>
static inline T simt__shfl(T v, unsigned src_lane_in_segment, int width) {
  const unsigned lane = simt::cur->linear % 32;
  const unsigned seg = lane / (unsigned)width * (unsigned)width;
  unsigned long long raw = 0;
  memcpy(&raw, &v, sizeof(T));
  const unsigned src = seg + src_lane_in_segment;
  const unsigned long long got =
      simt::exchange(raw, src_lane_in_segment < (unsigned)width ? src : 0xffffffffu);
  T r;
  memcpy(&r, &got, sizeof(T));
  return src_lane_in_segment < (unsigned)width ? r : v;
}
template <typename T>
static inline T __shfl_down_sync(unsigned, T v, int delta, int width = 32) {
  const unsigned lane = simt::cur->linear % 32;
  return simt__shfl(v, lane % (unsigned)width + (unsigned)delta, width);
}
template <typename T>
static inline T __shfl_sync(unsigned, T v, int src, int width = 32) {
  return simt__shfl(v, (unsigned)src % (unsigned)width, width);
}

static inline int __any_sync(unsigned, int pred) {
  const unsigned w = simt::cur->linear / 32, lane = simt::cur->linear % 32, n = simt::warp_lanes(w);
  simt::warp_slot[w][lane] = pred != 0;
  simt::warp_barrier(w, n);
  int r = 0;
  for (unsigned l = 0; l < n; l++) r |= (int)simt::warp_slot[w][l];
  simt::warp_barrier(w, n);
  return r;
}
static inline unsigned int atomicAdd(unsigned int *p, unsigned int v) {
  const unsigned int old = *p;
  *p = old + v;
  return old;
}
template <typename T>
static inline T __ldcg(const T *p) {
  return *p;
}
static inline unsigned int __umulhi(unsigned int a, unsigned int b) {
  return (unsigned int)(((unsigned long long)a * b) >> 32);
}
static inline int __dp4a(int a, int b, int c) {
  for (int i = 0; i < 4; i++) c += (int)(signed char)(a >> (8 * i)) * (int)(signed char)(b >> (8 * i));
  return c;
}
static inline unsigned int __dp4a(unsigned int a, unsigned int b, unsigned int c) {
  for (int i = 0; i < 4; i++) c += ((a >> (8 * i)) & 0xffu) * ((b >> (8 * i)) & 0xffu);
  return c;
}

/* Runs kernel(args...) over a grid; defined per kernel by SIMT_DEFINE_LAUNCH. */
namespace simt {
typedef void (*Body)(void *);
void run_grid(Body body, void *arg, simt_dim3 grid, simt_dim3 block);
}
#endif
