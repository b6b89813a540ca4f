/* Build-time instantiation: float32 MAXANDARGMAX, a warp per long run, values
 * scanned alone and the index recovered afterwards (the headline variant). */
#define GA_RD_SRC_T ga_float
#define GA_RD_X_T ga_float
#define GA_RD_ACC_T ga_float
#define GA_RD_DST_T ga_float
#define GA_RD_LOAD(raw) (raw)
#define GA_RD_STORE(a) ((GA_RD_DST_T)(a))
#define GA_RD_MAP(x) ((GA_RD_ACC_T)(x))
#define GA_RD_COMBINE(a, b) ((a) + (b))
#define GA_RD_IDENT (-INFINITY)
#define GA_RD_BETTER(b, a) ((b) > (a))
#define GA_RD_KIND 1
#define GA_RD_ISFLOAT 1
#define GA_RD_WRITE_VAL 1
#define GA_RD_WRITE_IDX 1
#define GA_RD_IDX_T unsigned int
#define GA_RD_VEC 4
#define GA_RD_THREADS 256
#define GA_RD_TPO 32
#define GA_RD_BY 8
#define GA_RD_FLAT 0
#define GA_RD_GROUP 32
#define GA_RD_LAZY 1
#define GA_RD_PICK(a, b) fmaxf((a), (b))
#define GA_RD_BUILD_ROWS
#include "ga_reduce.cuh"
