/* Row gather r[i0, ...] = v[ind[i0], ...] along axis 0 (GpuArray_take1).
 *
 * Same contract as the kernel the reference generates in
 * src/gpuarray_array.c:325-423: negative indices count from the end, an index
 * out of range sets *err to -1 and leaves the row unwritten. Here threadIdx.x
 * runs along the flattened trailing dimensions, so consecutive threads read
 * and write consecutive elements of a row; blockIdx.y runs over the rows.
 *
 * Defines needed: GA_TK_R_T, GA_TK_V_T, GA_TK_I_T (element, source, index
 * types), GA_TK_ND (rank of v, >= 1). */
#include "cluda.h"

struct ga__tk_layout {
  unsigned long long n0, n1;
  unsigned long long dims[GA_TK_ND];
  long long strs[GA_TK_ND];
};

extern "C" __global__ void __launch_bounds__(256)
ga_take1(const __grid_constant__ ga__tk_layout L, GA_TK_R_T *r, const char *v,
         const GA_TK_I_T *ind, int *err) {
  ga__grid_dependency_sync();
  for (unsigned long long i0 = blockIdx.y; i0 < L.n0; i0 += gridDim.y) {
    long long row = (long long)ind[i0];
    if (row < 0) row += (long long)L.dims[0];
    if (row < 0 || row >= (long long)L.dims[0]) {
      if (threadIdx.x == 0 && blockIdx.x == 0) *err = -1;
      continue;
    }
    const char *base = v + row * L.strs[0];
    for (unsigned long long i1 = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
         i1 < L.n1; i1 += (unsigned long long)gridDim.x * blockDim.x) {
      long long p = 0;
      unsigned long long ii = i1;
#pragma unroll
      for (int d = GA_TK_ND - 1; d >= 1; d--) {
        const unsigned long long q = ii / L.dims[d];
        p += (long long)(ii - q * L.dims[d]) * L.strs[d];
        ii = q;
      }
      r[i0 * L.n1 + i1] = *reinterpret_cast<const GA_TK_V_T *>(base + p);
    }
  }
}
