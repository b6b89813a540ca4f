/* Build-time instantiation of the contiguous elementwise template with the
 * "out = a * b + 0.5f" float32 arguments, so that nvcc (-Xptxas -v) reports
 * registers and spills for sm_100a. Not linked into the library: at run time
 * the same template is compiled by NVRTC with the caller's expression. */
#define GA_EW_ARRAYS(X) \
  X(0, a, ga_float, ga_float, 1, 0, 0) X(1, b, ga_float, ga_float, 1, 0, 0) \
  X(2, out, ga_float, ga_float, 0, 1, 0)
#define GA_EW_SCALARS(X)
#define GA_EW_EPT 4
#define GA_EW_UNROLL 4
#define GA_EW_THREADS 256
#define GA_EW_IDX unsigned int
#include "cluda.h"
static __device__ __forceinline__ void ga_ew_apply(ga_float &a, ga_float &b, ga_float &out, int) {
  out = a * b + 0.5f;
}
#include "ga_ew_contig.cuh"
