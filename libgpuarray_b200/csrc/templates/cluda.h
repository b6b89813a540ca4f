/* Kernel-side vocabulary available to every expression, preamble and user
 * kernel: `#include "cluda.h"`.
 *
 * The macro and type names are an API shared with the reference's CUDA
 * flavour of the same header (src/cluda_cuda.h:3-172): user code written for
 * it (pygpu kernels, Theano preambles using WITHIN_KERNEL, GLOBAL_MEM,
 * ga_float, INFINITY, atom_add_fg ...) compiles unchanged. Only sm_100a is
 * targeted, so every atomic maps to a native instruction. */
#ifndef CLUDA_H
#define CLUDA_H

/* ---- qualifiers ---- */
#define KERNEL extern "C" __global__
#define WITHIN_KERNEL extern "C" __device__
#define GLOBAL_MEM
#define LOCAL_MEM __shared__
#define LOCAL_MEM_ARG
#define local_barrier() __syncthreads()
#define GA_DECL_SHARED_PARAM(type, name)
#define GA_DECL_SHARED_BODY(type, name) extern __shared__ type name[];
#define GA_WARP_SIZE warpSize

/* ---- thread geometry: L = local (block), G = global (grid) ---- */
#define LID_0 threadIdx.x
#define LID_1 threadIdx.y
#define LID_2 threadIdx.z
#define LDIM_0 blockDim.x
#define LDIM_1 blockDim.y
#define LDIM_2 blockDim.z
#define GID_0 blockIdx.x
#define GID_1 blockIdx.y
#define GID_2 blockIdx.z
#define GDIM_0 gridDim.x
#define GDIM_1 gridDim.y
#define GDIM_2 gridDim.z

/* ---- element types ---- */
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

/* Storage-only half: arithmetic needs ga_half2float / GE_CONVERT_F16. */
struct ga_half {
  ga_ushort data;
};

static __device__ __forceinline__ float ga_half2float(ga_half h) {
  float f;
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h.data));
  return f;
}
static __device__ __forceinline__ ga_half ga_float2half(float f) {
  ga_half h;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h.data) : "f"(f));
  return h;
}

/* acc + h with h widened exactly and ONE rounding: the same value as
 * acc + ga_half2float(h), in one instruction instead of a conversion and an add */
static __device__ __forceinline__ float ga__add_f32_f16(float acc, ga_half h) {
  float r;
  asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(r) : "h"(h.data), "f"(acc));
  return r;
}

/* ---- constants ---- */
#ifdef NAN
#undef NAN
#endif
#ifdef INFINITY
#undef INFINITY
#endif
#ifdef HUGE_VALF
#undef HUGE_VALF
#endif
#ifdef HUGE_VAL
#undef HUGE_VAL
#endif
#ifdef MAXFLOAT
#undef MAXFLOAT
#endif
#define NAN __int_as_float(0x7fffffff)
#define INFINITY __int_as_float(0x7f800000)
#define HUGE_VALF INFINITY
#define HUGE_VAL __longlong_as_double(0x7ff0000000000000)
#define MAXFLOAT 3.402823466E+38F
#define M_E        2.7182818284590452354
#define M_LOG2E    1.4426950408889634074
#define M_LOG10E   0.43429448190325182765
#define M_LN2      0.69314718055994530942
#define M_LN10     2.30258509299404568402
#define M_PI       3.14159265358979323846
#define M_PI_2     1.57079632679489661923
#define M_PI_4     0.78539816339744830962
#define M_1_PI     0.31830988618379067154
#define M_2_PI     0.63661977236758134308
#define M_2_SQRTPI 1.12837916709551257390
#define M_SQRT2    1.41421356237309504880
#define M_SQRT1_2  0.70710678118654752440

/* ---- atomics: atom_<op>_<type><space>, type i/I/l/L/f/d/e, space g/l ---- */
#define atom_add_ig(a, b) atomicAdd(a, b)
#define atom_add_il(a, b) atomicAdd(a, b)
#define atom_xchg_ig(a, b) atomicExch(a, b)
#define atom_xchg_il(a, b) atomicExch(a, b)
#define atom_add_Ig(a, b) atomicAdd(a, b)
#define atom_add_Il(a, b) atomicAdd(a, b)
#define atom_xchg_Ig(a, b) atomicExch(a, b)
#define atom_xchg_Il(a, b) atomicExch(a, b)
#define atom_add_Lg(a, b) atomicAdd(a, b)
#define atom_add_Ll(a, b) atomicAdd(a, b)
#define atom_xchg_Lg(a, b) atomicExch(a, b)
#define atom_xchg_Ll(a, b) atomicExch(a, b)
#define atom_add_fg(a, b) atomicAdd(a, b)
#define atom_add_fl(a, b) atomicAdd(a, b)
#define atom_xchg_fg(a, b) atomicExch(a, b)
#define atom_xchg_fl(a, b) atomicExch(a, b)
#define atom_add_dg(a, b) atomicAdd(a, b)
#define atom_add_dl(a, b) atomicAdd(a, b)

/* two's complement: a signed 64-bit add is the unsigned one */
static __device__ __forceinline__ ga_long atom_add_lg(ga_long *p, ga_long v) {
  return (ga_long)atomicAdd((unsigned long long *)p, (unsigned long long)v);
}
static __device__ __forceinline__ ga_long atom_xchg_lg(ga_long *p, ga_long v) {
  return (ga_long)atomicExch((unsigned long long *)p, (unsigned long long)v);
}
#define atom_add_ll(a, b) atom_add_lg(a, b)
#define atom_xchg_ll(a, b) atom_xchg_lg(a, b)

static __device__ __forceinline__ ga_double atom_xchg_dg(ga_double *p, ga_double v) {
  return __longlong_as_double(
      (long long)atomicExch((unsigned long long *)p, (unsigned long long)__double_as_longlong(v)));
}
#define atom_xchg_dl(a, b) atom_xchg_dg(a, b)

/* half: compare-and-swap on the containing 32-bit word */
static __device__ __forceinline__ ga_half ga__half_rmw(ga_half *p, ga_half v, int add) {
  ga_uint *word = (ga_uint *)((ga_size)p & ~(ga_size)2);
  const int hi = ((ga_size)p & 2) != 0;
  ga_uint seen = *word, want, prev;
  ga_half cur, upd;
  do {
    prev = seen;
    cur.data = (ga_ushort)(hi ? (prev >> 16) : (prev & 0xffffu));
    upd = add ? ga_float2half(ga_half2float(cur) + ga_half2float(v)) : v;
    want = hi ? ((prev & 0x0000ffffu) | ((ga_uint)upd.data << 16))
              : ((prev & 0xffff0000u) | (ga_uint)upd.data);
    seen = atomicCAS(word, prev, want);
  } while (seen != prev);
  return cur;
}
static __device__ __forceinline__ ga_half atom_add_eg(ga_half *p, ga_half v) {
  return ga__half_rmw(p, v, 1);
}
static __device__ __forceinline__ ga_half atom_xchg_eg(ga_half *p, ga_half v) {
  return ga__half_rmw(p, v, 0);
}
#define atom_add_el(a, b) atom_add_eg(a, b)
#define atom_xchg_el(a, b) atom_xchg_eg(a, b)

/* Programmatic dependent launch (sm_90 and later). A kernel that the library
 * launches with stream serialization relaxed may become resident while its
 * predecessor in the stream is still draining; it must call this before its
 * first access to global memory, which then waits until the predecessor has
 * completed and its writes are visible. Releasing right after lets the
 * successor do the same with us. Both are no-ops under an ordinary launch. */
/* Asks the memory system to bring [p, p + bytes) into L2 (p 16-byte aligned,
 * bytes a multiple of 16). A hint without architectural effect: nothing is
 * loaded into registers or L1, and L2 is the point of coherence, so issuing it
 * BEFORE ga__grid_dependency_sync() is safe even when the previous kernel of
 * the stream is still writing the very same lines - the loads that follow the
 * wait see its data. It lets a kernel's first DRAM reads overlap the tail of
 * its predecessor. */
static __device__ __forceinline__ void ga__prefetch_l2(const void *p, unsigned int bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

/* 16 bytes from global to shared memory without passing through registers
 * (both addresses 16-byte aligned); ga__cp_async_wait_all() waits for the
 * calling thread's copies - a barrier then makes everyone's visible. */
static __device__ __forceinline__ void ga__cp_async16(void *smem, const void *gmem) {
  const unsigned int s = (unsigned int)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
static __device__ __forceinline__ void ga__cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

/* Four 8 x 8 matrices of 16-bit elements from shared memory, TRANSPOSED on the
 * way: lanes 8m .. 8m+7 give the (16-byte aligned) addresses of the eight
 * 16-byte rows of matrix m; lane i receives, in r[m], elements
 * [2*(i%4)][i/4] (low half) and [2*(i%4)+1][i/4] (high half) of matrix m.
 * Every lane of the warp must execute it. */
static __device__ __forceinline__ void ga__ldsm_x4_trans(const void *row, unsigned int r[4]) {
  const unsigned int s = (unsigned int)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s)
               : "memory");
}

static __device__ __forceinline__ void ga__grid_dependency_sync() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

#endif /* CLUDA_H */
