/* Build-time instantiation of the strided template: fp16 bias + ReLU over 3
 * collapsed dimensions (x gathered, bias broadcast, y vector stores). */
#define GA_EW_ARRAYS(X) \
  X(0, x, ga_half, ga_float, 1, 0, 0) X(1, bias, ga_half, ga_float, 1, 0, 2) \
  X(2, y, ga_half, ga_float, 0, 1, 1)
#define GA_EW_SCALARS(X)
#define GA_EW_EPT 8
#define GA_EW_UNROLL 1
#define GA_EW_THREADS 256
#define GA_EW_IDX unsigned int
#define GA_EW_IDX32 1
#define GA_EW_OFF32 1
#define GA_EW_ND 3
#define GA_EW_NARR 3
#include "cluda.h"
static __device__ __forceinline__ void ga_ew_apply(ga_float &x, ga_float &bias, ga_float &y, int) {
  y = fmaxf(x + bias, 0.0f);
}
#include "ga_ew_strided.cuh"
