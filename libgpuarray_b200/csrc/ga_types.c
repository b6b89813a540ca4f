/* The type table: typecode -> (kernel spelling, size, alignment).
 * Sizes, alignments and spellings are ABI shared with the reference's
 * generated table (src/gpuarray_types.c:107-189). */
#include "private.h"

#define T(name, sz, code) {name, sz, sz, code}
static const gpuarray_type scalar_table[GA_NBASE] = {
    T("ga_bool", 1, GA_BOOL),       T("ga_byte", 1, GA_BYTE),
    T("ga_ubyte", 1, GA_UBYTE),     T("ga_short", 2, GA_SHORT),
    T("ga_ushort", 2, GA_USHORT),   T("ga_int", 4, GA_INT),
    T("ga_uint", 4, GA_UINT),       T("ga_long", 8, GA_LONG),
    T("ga_ulong", 8, GA_ULONG),     T("ga_longlong", 16, GA_LONGLONG),
    T("ga_ulonglong", 16, GA_ULONGLONG), T("ga_float", 4, GA_FLOAT),
    T("ga_double", 8, GA_DOUBLE),   T("ga_quad", 16, GA_QUAD),
    /* complex types align like their component */
    {"ga_cfloat", 8, 4, GA_CFLOAT}, {"ga_cdouble", 16, 8, GA_CDOUBLE},
    {"ga_cquad", 32, 16, GA_CQUAD},
    {NULL, 0, 0, -1}, {NULL, 0, 0, -1}, {NULL, 0, 0, -1},
    {NULL, 0, 0, -1}, {NULL, 0, 0, -1}, {NULL, 0, 0, -1},
    T("ga_half", 2, GA_HALF),
    T("ga_size", sizeof(size_t), GA_SIZE), T("ga_ssize", sizeof(ssize_t), GA_SSIZE),
};
#undef T

/* Vector types are described by (base spelling, base size) x width. */
static const struct { const char *base; size_t sz; int first; int widths; } vec_families[] = {
    {"byte", 1, GA_BYTE2, 5},   {"short", 2, GA_SHORT2, 5}, {"int", 4, GA_INT2, 5},
    {"long", 8, GA_LONG2, 5},
};
static const int vec_width5[5] = {2, 3, 4, 8, 16};
static const int vec_width4[4] = {2, 4, 8, 16};

static gpuarray_type vector_table[GA_NVEC - 256];
static char vector_names[GA_NVEC - 256][16];
static int vector_ready = 0;

static void build_vector_table(void) {
  unsigned f, w;
  int code;
  /* integer families interleave signed/unsigned: byte2, ubyte2, byte3, ... */
  for (f = 0; f < sizeof(vec_families) / sizeof(vec_families[0]); f++) {
    for (w = 0; w < 5; w++) {
      int s;
      for (s = 0; s < 2; s++) {
        code = vec_families[f].first + (int)w * 2 + s;
        snprintf(vector_names[code - 256], 16, "ga_%s%s%d", s ? "u" : "", vec_families[f].base,
                 vec_width5[w]);
        vector_table[code - 256].cluda_name = vector_names[code - 256];
        vector_table[code - 256].size = vec_families[f].sz * (size_t)vec_width5[w];
        vector_table[code - 256].align = 0;
        vector_table[code - 256].typecode = code;
      }
    }
  }
  {
    static const struct { const char *base; size_t sz; int first; } fl[] = {
        {"float", 4, GA_FLOAT2}, {"double", 8, GA_DOUBLE2}, {"half", 2, GA_HALF2}};
    for (f = 0; f < 3; f++)
      for (w = 0; w < 4; w++) {
        code = fl[f].first + (int)w;
        snprintf(vector_names[code - 256], 16, "ga_%s%d", fl[f].base, vec_width4[w]);
        vector_table[code - 256].cluda_name = vector_names[code - 256];
        vector_table[code - 256].size = fl[f].sz * (size_t)vec_width4[w];
        vector_table[code - 256].align = 0;
        vector_table[code - 256].typecode = code;
      }
  }
  vector_ready = 1;
}

static gpuarray_type **user_types = NULL;
static int n_user_types = 0;
static const gpuarray_type unknown_type = {NULL, 0, 0, -1};
static const gpuarray_type buffer_type = {NULL, sizeof(void *), sizeof(void *), GA_BUFFER};

int gpuarray_register_type(gpuarray_type *t, int *ret) {
  gpuarray_type **grown = realloc(user_types, (size_t)(n_user_types + 1) * sizeof(*grown));
  if (grown == NULL) {
    if (ret != NULL) *ret = GA_SYS_ERROR;
    return -1;
  }
  user_types = grown;
  t->typecode = 512 + n_user_types;
  user_types[n_user_types++] = t;
  return t->typecode;
}

const gpuarray_type *gpuarray_get_type(int typecode) {
  if (typecode == GA_BUFFER) return &buffer_type;
  if (typecode >= 0 && typecode < GA_NBASE) return &scalar_table[typecode];
  if (typecode >= 256 && typecode < GA_NVEC) {
    if (!vector_ready) build_vector_table();
    return &vector_table[typecode - 256];
  }
  if (typecode >= 512 && typecode - 512 < n_user_types) return user_types[typecode - 512];
  return &unknown_type;
}

size_t gpuarray_get_elsize(int typecode) { return gpuarray_get_type(typecode)->size; }

const char *ga_ctype(int typecode) { return gpuarray_get_type(typecode)->cluda_name; }

int ga_type_is_computable(int typecode) {
  switch (typecode) {
  case GA_BOOL: case GA_BYTE: case GA_UBYTE: case GA_SHORT: case GA_USHORT:
  case GA_INT: case GA_UINT: case GA_LONG: case GA_ULONG:
  case GA_FLOAT: case GA_DOUBLE: case GA_HALF: case GA_SIZE: case GA_SSIZE:
    return 1;
  default:
    return 0;
  }
}
