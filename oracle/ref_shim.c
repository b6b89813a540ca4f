/* Glue compiled together with the reference's own util sources (see Makefile):
 * exposes its `static inline` half conversion as a symbol so that tests can
 * call the reference's code through ctypes. Contains no reference code. */
#include <gpuarray/util.h>

unsigned short ref_float2half(float f) { return ga_float2half(f).h; }
