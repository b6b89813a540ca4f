/* Multi-GPU collectives: gpucomm_* on buffers and GpuArray_* on arrays, over
 * NCCL bound at run time (NVLink 5 / NVSwitch underneath on a B200 node).
 *
 * Same surface and checks as the reference's
 * src/gpuarray_collectives_cuda_nccl.c (type/op mapping :150-185, argument
 * restrictions :192-240, one NCCL call per entry point) and
 * src/gpuarray_array_collectives.c (:29-123). Every call is enqueued on the
 * context's single stream, right behind the kernels that produced its input,
 * so no event bookkeeping (:300-316 there) is needed. The elementwise /
 * reduction engine needs exactly one of them: gpucomm_all_reduce, to combine
 * per-GPU partial results when the reduced extent is sharded. */
#include <dlfcn.h>
#include <limits.h>
#include "private.h"

/* The few NCCL declarations used, so that no NCCL header is needed to build. */
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef enum { ncclSuccess = 0 } ncclResult_t;
typedef enum { ncclSum = 0, ncclProd = 1, ncclMax = 2, ncclMin = 3, ncclNumOps_ = 99 } ncclRedOp_t;
typedef enum { ncclInt8 = 0, ncclUint8 = 1, ncclInt32 = 2, ncclUint32 = 3, ncclInt64 = 4,
               ncclUint64 = 5, ncclFloat16 = 6, ncclFloat32 = 7, ncclFloat64 = 8,
               ncclNumTypes_ = 99 } ncclDataType_t;

static struct {
  ncclResult_t (*GetUniqueId)(ncclUniqueId *);
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*CommCount)(const ncclComm_t, int *);
  ncclResult_t (*CommUserRank)(const ncclComm_t, int *);
  const char *(*GetErrorString)(ncclResult_t);
  ncclResult_t (*Reduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, int,
                         ncclComm_t, CUstream);
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            CUstream);
  ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t,
                                ncclComm_t, CUstream);
  ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, CUstream);
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, CUstream);
} nccl;

static int load_nccl(ga_error_rec *e) {
  static int state = 0;
  static const char *const names[] = {"libnccl.so.2", "libnccl.so", NULL};
  const char *env = getenv("GPUARRAY_NCCL_PATH");
  void *h = NULL;
  int i;
  if (state == 1) return GA_NO_ERROR;
  if (env != NULL && env[0] != '\0') h = dlopen(env, RTLD_LAZY | RTLD_GLOBAL);
  for (i = 0; h == NULL && names[i] != NULL; i++) h = dlopen(names[i], RTLD_LAZY | RTLD_GLOBAL);
  if (h == NULL) return ga_err_fmt(e, GA_LOAD_ERROR, "Could not load \"libnccl.so.2\": %s", dlerror());
#define SYM(field, name)                                                        \
  *(void **)&nccl.field = dlsym(h, name);                                       \
  if (nccl.field == NULL) return ga_err_fmt(e, GA_LOAD_ERROR, "libnccl lacks symbol %s", name);
  SYM(GetUniqueId, "ncclGetUniqueId")
  SYM(CommInitRank, "ncclCommInitRank")
  SYM(CommDestroy, "ncclCommDestroy")
  SYM(CommCount, "ncclCommCount")
  SYM(CommUserRank, "ncclCommUserRank")
  SYM(GetErrorString, "ncclGetErrorString")
  SYM(Reduce, "ncclReduce")
  SYM(AllReduce, "ncclAllReduce")
  SYM(ReduceScatter, "ncclReduceScatter")
  SYM(Broadcast, "ncclBroadcast")
  SYM(AllGather, "ncclAllGather")
#undef SYM
  state = 1;
  return GA_NO_ERROR;
}

struct _gpucomm {
  gpucontext *ctx; /* MUST stay first (reference src/private.h:86-88) */
  ncclComm_t c;
};

static int nccl_fail(gpucontext *ctx, const char *call, ncclResult_t r) {
  return ga_err_fmt(ctx->err, GA_COMM_ERROR, "%s: %s", call, nccl.GetErrorString(r));
}

static int to_nccl_type(int typecode, ncclDataType_t *t) {
  switch (typecode) {
  case GA_BYTE: *t = ncclInt8; return 1;
  case GA_UBYTE: *t = ncclUint8; return 1;
  case GA_INT: *t = ncclInt32; return 1;
  case GA_UINT: *t = ncclUint32; return 1;
  case GA_LONG: case GA_SSIZE: *t = ncclInt64; return 1;
  case GA_ULONG: case GA_SIZE: *t = ncclUint64; return 1;
  case GA_HALF: *t = ncclFloat16; return 1;
  case GA_FLOAT: *t = ncclFloat32; return 1;
  case GA_DOUBLE: *t = ncclFloat64; return 1;
  default: return 0;
  }
}

static int to_nccl_op(int opcode, ncclRedOp_t *op) {
  switch (opcode) {
  case GA_SUM: *op = ncclSum; return 1;
  case GA_PROD: *op = ncclProd; return 1;
  case GA_MAX: *op = ncclMax; return 1;
  case GA_MIN: *op = ncclMin; return 1;
  default: return 0;
  }
}

int gpucomm_gen_clique_id(gpucontext *ctx, gpucommCliqueId *comm_id) {
  ncclUniqueId id;
  ncclResult_t r;
  int err = load_nccl(ctx->err);
  if (err != GA_NO_ERROR) return err;
  r = nccl.GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(ctx, "ncclGetUniqueId", r);
  memcpy(comm_id->internal, id.internal, GA_COMM_ID_BYTES);
  return GA_NO_ERROR;
}

int gpucomm_new(gpucomm **out, gpucontext *ctx, gpucommCliqueId comm_id, int ndev, int rank) {
  gpucomm *comm;
  ncclUniqueId id;
  ncclResult_t r;
  int err = load_nccl(ctx->err);
  *out = NULL;
  if (err != GA_NO_ERROR) return err;
  if (ndev <= 0 || rank < 0 || rank >= ndev)
    return ga_err_fmt(ctx->err, GA_VALUE_ERROR, "Invalid rank %d of %d", rank, ndev);
  comm = calloc(1, sizeof(*comm));
  if (comm == NULL) return ga_err_sys(ctx->err, "calloc");
  comm->ctx = ctx;
  memcpy(id.internal, comm_id.internal, GA_COMM_ID_BYTES);
  ga_ctx_enter(ctx);
  r = nccl.CommInitRank(&comm->c, ndev, id, rank);
  ga_ctx_exit(ctx);
  if (r != ncclSuccess) {
    free(comm);
    return nccl_fail(ctx, "ncclCommInitRank", r);
  }
  ctx->refcnt++;
  *out = comm;
  return GA_NO_ERROR;
}

void gpucomm_free(gpucomm *comm) {
  gpucontext *ctx;
  if (comm == NULL) return;
  ctx = comm->ctx;
  ga_ctx_enter(ctx);
  ga_cu.p_cuStreamSynchronize(ctx->s);
  nccl.CommDestroy(comm->c);
  ga_ctx_exit(ctx);
  free(comm);
  ga_ctx_unref(ctx);
}

const char *gpucomm_error(gpucontext *ctx) { return gpucontext_error(ctx, 0); }

gpucontext *gpucomm_context(gpucomm *comm) { return comm->ctx; }

int gpucomm_get_count(gpucomm *comm, int *devcount) {
  ncclResult_t r = nccl.CommCount(comm->c, devcount);
  return r == ncclSuccess ? GA_NO_ERROR : nccl_fail(comm->ctx, "ncclCommCount", r);
}

int gpucomm_get_rank(gpucomm *comm, int *rank) {
  ncclResult_t r = nccl.CommUserRank(comm->c, rank);
  return r == ncclSuccess ? GA_NO_ERROR : nccl_fail(comm->ctx, "ncclCommUserRank", r);
}

/* Shared argument checks; `times_*` scale `count` for the byte-range test. */
static int check_args(gpucomm *comm, gpudata *src, size_t offsrc, size_t nsrc, gpudata *dest,
                      size_t offdest, size_t ndest, int typecode, const int *opcode,
                      ncclDataType_t *t, ncclRedOp_t *op) {
  gpucontext *ctx = comm->ctx;
  size_t es = gpuarray_get_elsize(typecode);
  if (nsrc > INT_MAX || ndest > INT_MAX)
    return ga_err_set(ctx->err, GA_XLARGE_ERROR, "Count too large for int");
  if (src != NULL && src->ctx != ctx)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "source and comm context differ");
  if (dest != NULL && dest->ctx != ctx)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "destination and comm context differ");
  if (!to_nccl_type(typecode, t)) return ga_err_set(ctx->err, GA_INVALID_ERROR, "Invalid data type");
  if (opcode != NULL && !to_nccl_op(*opcode, op))
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "Invalid reduce op");
  if (src != NULL && (offsrc > src->sz || nsrc * es > src->sz - offsrc))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "source too small for operation");
  if (dest != NULL && (offdest > dest->sz || ndest * es > dest->sz - offdest))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "destination too small for operation");
  return GA_NO_ERROR;
}

#define NCCL_ENQUEUE(name, call)                                   \
  do {                                                             \
    ncclResult_t r_;                                               \
    ga_ctx_enter(ctx);                                             \
    r_ = call;                                                     \
    ga_ctx_exit(ctx);                                              \
    if (r_ != ncclSuccess) return nccl_fail(ctx, name, r_);        \
    return GA_NO_ERROR;                                            \
  } while (0)

int gpucomm_reduce(gpudata *src, size_t offsrc, gpudata *dest, size_t offdest, size_t count,
                   int typecode, int opcode, int root, gpucomm *comm) {
  gpucontext *ctx = comm->ctx;
  ncclDataType_t t;
  ncclRedOp_t op;
  int rank = 0, err;
  err = gpucomm_get_rank(comm, &rank);
  if (err != GA_NO_ERROR) return err;
  err = check_args(comm, src, offsrc, count, rank == root ? dest : NULL, offdest, count, typecode,
                   &opcode, &t, &op);
  if (err != GA_NO_ERROR) return err;
  if (rank == root && dest == NULL)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "root needs a destination");
  NCCL_ENQUEUE("ncclReduce",
               nccl.Reduce((const void *)(src->ptr + offsrc),
                           rank == root ? (void *)(dest->ptr + offdest) : NULL, count, t, op, root,
                           comm->c, ctx->s));
}

int gpucomm_all_reduce(gpudata *src, size_t offsrc, gpudata *dest, size_t offdest, size_t count,
                       int typecode, int opcode, gpucomm *comm) {
  gpucontext *ctx = comm->ctx;
  ncclDataType_t t;
  ncclRedOp_t op;
  int err = check_args(comm, src, offsrc, count, dest, offdest, count, typecode, &opcode, &t, &op);
  if (err != GA_NO_ERROR) return err;
  NCCL_ENQUEUE("ncclAllReduce",
               nccl.AllReduce((const void *)(src->ptr + offsrc), (void *)(dest->ptr + offdest),
                              count, t, op, comm->c, ctx->s));
}

int gpucomm_reduce_scatter(gpudata *src, size_t offsrc, gpudata *dest, size_t offdest,
                           size_t count, int typecode, int opcode, gpucomm *comm) {
  gpucontext *ctx = comm->ctx;
  ncclDataType_t t;
  ncclRedOp_t op;
  int ndev = 0, err;
  err = gpucomm_get_count(comm, &ndev);
  if (err != GA_NO_ERROR) return err;
  err = check_args(comm, src, offsrc, count * (size_t)ndev, dest, offdest, count, typecode, &opcode,
                   &t, &op);
  if (err != GA_NO_ERROR) return err;
  NCCL_ENQUEUE("ncclReduceScatter",
               nccl.ReduceScatter((const void *)(src->ptr + offsrc), (void *)(dest->ptr + offdest),
                                  count, t, op, comm->c, ctx->s));
}

int gpucomm_broadcast(gpudata *array, size_t offset, size_t count, int typecode, int root,
                      gpucomm *comm) {
  gpucontext *ctx = comm->ctx;
  ncclDataType_t t;
  ncclRedOp_t op;
  int err = check_args(comm, array, offset, count, NULL, 0, 0, typecode, NULL, &t, &op);
  if (err != GA_NO_ERROR) return err;
  NCCL_ENQUEUE("ncclBroadcast",
               nccl.Broadcast((const void *)(array->ptr + offset), (void *)(array->ptr + offset),
                              count, t, root, comm->c, ctx->s));
}

int gpucomm_all_gather(gpudata *src, size_t offsrc, gpudata *dest, size_t offdest, size_t count,
                       int typecode, gpucomm *comm) {
  gpucontext *ctx = comm->ctx;
  ncclDataType_t t;
  ncclRedOp_t op;
  int ndev = 0, err;
  err = gpucomm_get_count(comm, &ndev);
  if (err != GA_NO_ERROR) return err;
  err = check_args(comm, src, offsrc, count, dest, offdest, count * (size_t)ndev, typecode, NULL,
                   &t, &op);
  if (err != GA_NO_ERROR) return err;
  NCCL_ENQUEUE("ncclAllGather",
               nccl.AllGather((const void *)(src->ptr + offsrc), (void *)(dest->ptr + offdest),
                              count, t, comm->c, ctx->s));
}

/* ------------------------------------------------------------ on GpuArrays */

static size_t total_elems(const GpuArray *a) {
  size_t n = 1;
  unsigned int i;
  for (i = 0; i < a->nd; i++) n *= a->dimensions[i];
  return n;
}

/* times_src * count(src) must equal times_dest * count(dest); both arrays
 * contiguous in some order, aligned, same type; dest writeable. */
static int check_arrays(int times_src, const GpuArray *src, int times_dest, const GpuArray *dest,
                        size_t *count) {
  gpucontext *ctx = GpuArray_context(src);
  size_t ns = total_elems(src), nd = total_elems(dest);
  if ((size_t)times_src * ns != (size_t)times_dest * nd)
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Size mismatch for transfer");
  if (src->typecode != dest->typecode) return ga_err_set(ctx->err, GA_VALUE_ERROR, "Type mismatch");
  if (!GpuArray_ISALIGNED(src) || !GpuArray_ISALIGNED(dest))
    return ga_err_set(ctx->err, GA_UNALIGNED_ERROR, "Unaligned arrays");
  if (!GpuArray_ISWRITEABLE(dest))
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "Unwritable destination");
  if (!GpuArray_ISONESEGMENT(src) || !GpuArray_ISONESEGMENT(dest))
    return ga_err_set(ctx->err, GA_VALUE_ERROR, "Collectives need contiguous arrays");
  *count = times_src >= times_dest ? ns : nd;
  return GA_NO_ERROR;
}

int GpuArray_reduce_from(const GpuArray *src, int opcode, int root, gpucomm *comm) {
  gpucontext *ctx = GpuArray_context(src);
  if (!GpuArray_ISALIGNED(src)) return ga_err_set(ctx->err, GA_UNALIGNED_ERROR, "Unaligned input");
  return gpucomm_reduce(src->data, src->offset, NULL, 0, total_elems(src), src->typecode, opcode,
                        root, comm);
}

int GpuArray_reduce(const GpuArray *src, GpuArray *dest, int opcode, int root, gpucomm *comm) {
  size_t count = 0;
  int err = check_arrays(1, src, 1, dest, &count);
  if (err != GA_NO_ERROR) return err;
  return gpucomm_reduce(src->data, src->offset, dest->data, dest->offset, count, src->typecode,
                        opcode, root, comm);
}

int GpuArray_all_reduce(const GpuArray *src, GpuArray *dest, int opcode, gpucomm *comm) {
  size_t count = 0;
  int err = check_arrays(1, src, 1, dest, &count);
  if (err != GA_NO_ERROR) return err;
  return gpucomm_all_reduce(src->data, src->offset, dest->data, dest->offset, count,
                            src->typecode, opcode, comm);
}

int GpuArray_reduce_scatter(const GpuArray *src, GpuArray *dest, int opcode, gpucomm *comm) {
  size_t count = 0;
  int ndev = 0, err;
  err = gpucomm_get_count(comm, &ndev);
  if (err != GA_NO_ERROR) return err;
  err = check_arrays(1, src, ndev, dest, &count);
  if (err != GA_NO_ERROR) return err;
  return gpucomm_reduce_scatter(src->data, src->offset, dest->data, dest->offset,
                                total_elems(dest), src->typecode, opcode, comm);
}

int GpuArray_broadcast(GpuArray *array, int root, gpucomm *comm) {
  gpucontext *ctx = GpuArray_context(array);
  int rank = 0, err = gpucomm_get_rank(comm, &rank);
  if (err != GA_NO_ERROR) return err;
  if (!GpuArray_ISALIGNED(array)) return ga_err_set(ctx->err, GA_UNALIGNED_ERROR, "Unaligned input");
  if (rank != root && !GpuArray_ISWRITEABLE(array))
    return ga_err_set(ctx->err, GA_INVALID_ERROR, "Unwritable destination");
  return gpucomm_broadcast(array->data, array->offset, total_elems(array), array->typecode, root,
                           comm);
}

int GpuArray_all_gather(const GpuArray *src, GpuArray *dest, gpucomm *comm) {
  size_t count = 0;
  int ndev = 0, err;
  err = gpucomm_get_count(comm, &ndev);
  if (err != GA_NO_ERROR) return err;
  err = check_arrays(ndev, src, 1, dest, &count);
  if (err != GA_NO_ERROR) return err;
  return gpucomm_all_gather(src->data, src->offset, dest->data, dest->offset, total_elems(src),
                            src->typecode, comm);
}
