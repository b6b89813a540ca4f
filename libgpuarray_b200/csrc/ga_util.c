/* Host-side helpers that are part of the exported ABI: feature flags for a
 * set of types and the dimension collapser used by the elementwise engine
 * (reference src/gpuarray_util.c:111-188). */
#include "private.h"

static int flags_for(int typecode) {
  int fl = 0;
  if (typecode == GA_DOUBLE || typecode == GA_CDOUBLE) fl |= GA_USE_DOUBLE;
  if (typecode == GA_HALF) fl |= GA_USE_HALF;
  if (typecode == GA_CFLOAT || typecode == GA_CDOUBLE) fl |= GA_USE_COMPLEX;
  if (gpuarray_get_elsize(typecode) < 4) fl |= GA_USE_SMALL;
  return fl;
}

int gpuarray_type_flags(int init, ...) {
  va_list ap;
  int fl = 0, tc = init;
  va_start(ap, init);
  while (tc != -1) {
    fl |= flags_for(tc);
    tc = va_arg(ap, int);
  }
  va_end(ap);
  return fl;
}

int gpuarray_type_flagsa(unsigned int n, gpuelemwise_arg *args) {
  unsigned int i;
  int fl = 0;
  for (i = 0; i < n; i++) fl |= flags_for(args[i].typecode);
  return fl;
}

/* Deletes entry `at` of every vector (dims and each non-NULL stride list). */
static void drop_dim(unsigned int n, unsigned int nd, unsigned int at, size_t *dims,
                     ssize_t **strs) {
  unsigned int k, j;
  for (j = at; j + 1 < nd; j++) dims[j] = dims[j + 1];
  for (k = 0; k < n; k++)
    if (strs[k] != NULL)
      for (j = at; j + 1 < nd; j++) strs[k][j] = strs[k][j + 1];
}

void gpuarray_elemwise_collapse(unsigned int n, unsigned int *_nd, size_t *dims,
                                ssize_t **strs) {
  unsigned int nd = *_nd, i, k;

  /* Pass 1: extent-1 axes carry no information; keep at least one axis. */
  for (i = nd; i > 0 && nd > 1; i--) {
    if (dims[i - 1] == 1) {
      drop_dim(n, nd, i - 1, dims, strs);
      nd--;
    }
  }
  /* Pass 2, innermost first: axis i folds into i-1 when stepping i-1 once
   * equals stepping i dims[i] times for every argument. */
  for (i = nd - 1; i > 0; i--) {
    int fold = 1;
    for (k = 0; k < n && fold; k++)
      if (strs[k] != NULL && strs[k][i - 1] != (ssize_t)dims[i] * strs[k][i]) fold = 0;
    if (!fold) continue;
    dims[i - 1] *= dims[i];
    for (k = 0; k < n; k++)
      if (strs[k] != NULL) strs[k][i - 1] = strs[k][i];
    drop_dim(n, nd, i, dims, strs);
    nd--;
  }
  *_nd = nd;
}
