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
#include <unistd.h>
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

/* Peer window: see the head of templates/ga_exchange.cuh for the layout and
 * the protocol. The constants mirror the GA_XC_* defines there. */
#define XC_MAX_RANKS 16
#define XC_MAX_CTAS 64
#define XC_DATA_OFF 32768
#define XC_THREADS 256
#define XC_SLOT_BYTES ((size_t)1 << 20)

typedef struct xc_kernel {
  int pair, op, tc;
  ga_function fn;
  struct xc_kernel *next;
} xc_kernel;

typedef struct xc_window { /* a window no communicator uses any more, kept for the next one */
  CUdeviceptr ptr;
  size_t bytes;
  struct xc_window *next;
} xc_window;

struct _gpucomm {
  gpucontext *ctx; /* MUST stay first (reference src/private.h:86-88) */
  ncclComm_t c;
  int ndev, rank;
  int win_state;                 /* 0 not tried yet, 1 in use, -1 unavailable (win_reason) */
  char win_reason[200];
  CUdeviceptr win[XC_MAX_RANKS]; /* [rank]: own allocation; others: imported mappings */
  size_t win_bytes;
  unsigned long long seq;        /* exchanges enqueued so far */
  unsigned long long timeout_ns;
  unsigned int *status_host;     /* pinned, mapped: set by a kernel whose wait ran out */
  CUdeviceptr status_dev;
  xc_kernel *kernels;
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
  comm->ndev = ndev;
  comm->rank = rank;
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

static void peer_window_release(gpucomm *comm);

void gpucomm_free(gpucomm *comm) {
  gpucontext *ctx;
  if (comm == NULL) return;
  ctx = comm->ctx;
  ga_ctx_enter(ctx);
  ga_cu.p_cuStreamSynchronize(ctx->s);
  peer_window_release(comm);
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

/* ------------------------------------------------------------ peer window */

/* What the ranks tell one another while the windows are set up (one
 * all-gather of 128 bytes per rank over the communicator itself). */
typedef union xc_hello {
  struct {
    CUipcMemHandle handle;
    int ok;                      /* this rank allocated and exported its window */
    int pid;
    unsigned long long host;     /* hash of the host name: IPC handles stay on one node */
    char pci[16];                /* two ranks on one GPU cannot wait for each other */
  } f;
  char bytes[128];
} xc_hello;

static int env_off(const char *name) {
  const char *v = getenv(name);
  return v != NULL && v[0] != '\0' && v[0] != '0';
}

/* Frees the windows parked on a context (context teardown). */
void ga_peer_windows_free(gpucontext *ctx) {
  xc_window *w = (xc_window *)ctx->peer_windows, *n;
  ctx->peer_windows = NULL;
  for (; w != NULL; w = n) {
    n = w->next;
    ga_cu.p_cuMemFree(w->ptr);
    free(w);
  }
}

/* Un-maps the peers' windows and parks the own one on the context: a peer may
 * still have it mapped (it closes its mapping in its own gpucomm_free, at a
 * time of its choosing), and freeing exported memory under a live mapping is
 * undefined; the next communicator of the context takes it over instead. */
static void peer_window_release(gpucomm *comm) {
  gpucontext *ctx = comm->ctx;
  xc_kernel *k, *kn;
  int p;
  if (comm->win_state == 1) {
    for (p = 0; p < comm->ndev; p++)
      if (p != comm->rank && comm->win[p] != 0) ga_cu.p_cuIpcCloseMemHandle(comm->win[p]);
  }
  if (comm->win[comm->rank] != 0) {
    xc_window *w = malloc(sizeof(*w));
    if (w != NULL) {
      w->ptr = comm->win[comm->rank];
      w->bytes = comm->win_bytes;
      w->next = (xc_window *)ctx->peer_windows;
      ctx->peer_windows = w;
    } /* else: leaked rather than freed under a peer's mapping */
  }
  memset(comm->win, 0, sizeof(comm->win));
  if (comm->status_host != NULL) ga_cu.p_cuMemFreeHost(comm->status_host);
  comm->status_host = NULL;
  for (k = comm->kernels; k != NULL; k = kn) {
    kn = k->next;
    free(k);
  }
  comm->kernels = NULL;
  comm->win_state = -1;
}

static void peer_window_refuse(gpucomm *comm, const char *fmt, const char *a, int b) {
  snprintf(comm->win_reason, sizeof(comm->win_reason), fmt, a, b);
}

/* COLLECTIVE over the communicator (every rank reaches it in its first sharded
 * reduction): allocates this rank's window, exchanges IPC handles through the
 * communicator, maps the peers' windows, and agrees with all ranks on the
 * outcome, so that either every rank uses the windows or none does. */
static int peer_window_setup(gpucomm *comm) {
  gpucontext *ctx = comm->ctx;
  const int n = comm->ndev, me = comm->rank;
  const size_t bytes = XC_DATA_OFF + 2 * (size_t)n * XC_SLOT_BYTES;
  xc_hello mine, *all = NULL;
  CUdeviceptr stage = 0;
  CUresult cr;
  ncclResult_t nr;
  char host[256];
  int p, q, agreed = 1, opened = 1, err = GA_NO_ERROR;
  const char *t;

  comm->win_state = -1;
  comm->win_reason[0] = '\0';
  memset(&mine, 0, sizeof(mine));
  mine.f.pid = (int)getpid();
  memset(host, 0, sizeof(host));
  gethostname(host, sizeof(host) - 1);
  mine.f.host = ga_hash64(host, strlen(host), 17);
  memcpy(mine.f.pci, ctx->pci_id, sizeof(mine.f.pci));
  t = getenv("GPUARRAY_B200_PEER_TIMEOUT_MS");
  comm->timeout_ns = (t != NULL && atoll(t) > 0 ? (unsigned long long)atoll(t) : 10000ULL) * 1000000ULL;

  ga_ctx_enter(ctx);
  if (n < 2 || n > XC_MAX_RANKS) {
    peer_window_refuse(comm, "%s%d ranks", "", n);
  } else if (env_off("GPUARRAY_B200_NO_PEER_WINDOW")) {
    peer_window_refuse(comm, "%s (rank %d)", "switched off by GPUARRAY_B200_NO_PEER_WINDOW", me);
  } else {
    xc_window **pw = (xc_window **)&ctx->peer_windows, *w;
    for (; (w = *pw) != NULL; pw = &w->next)
      if (w->bytes == bytes) break;
    if (w != NULL) {
      *pw = w->next;
      comm->win[me] = w->ptr;
      free(w);
      cr = CUDA_SUCCESS;
    } else {
      cr = ga_cu.p_cuMemAlloc(&comm->win[me], bytes);
    }
    if (cr == CUDA_SUCCESS) {
      comm->win_bytes = bytes;
      cr = ga_cu.p_cuMemsetD8Async(comm->win[me], 0, XC_DATA_OFF, ctx->s);
    }
    if (cr == CUDA_SUCCESS) cr = ga_cu.p_cuIpcGetMemHandle(&mine.f.handle, comm->win[me]);
    if (cr == CUDA_SUCCESS)
      cr = ga_cu.p_cuMemHostAlloc((void **)&comm->status_host, 64, CU_MEMHOSTALLOC_DEVICEMAP);
    if (cr == CUDA_SUCCESS) {
      memset(comm->status_host, 0, 64);
      cr = ga_cu.p_cuMemHostGetDevicePointer(&comm->status_dev, comm->status_host, 0);
    }
    if (cr == CUDA_SUCCESS) mine.f.ok = 1;
    else peer_window_refuse(comm, "%s: CUDA error %d", "window allocation or export", (int)cr);
  }

  /* first exchange: everyone's hello */
  all = calloc((size_t)n, sizeof(*all));
  if (all == NULL) { err = ga_err_sys(ctx->err, "calloc"); goto out; }
  cr = ga_cu.p_cuMemAlloc(&stage, sizeof(xc_hello) * (size_t)(n + 1));
  if (cr != CUDA_SUCCESS) { err = ga_err_cuda(ctx->err, "cuMemAlloc", cr); goto out; }
  cr = ga_cu.p_cuMemcpyHtoDAsync(stage, &mine, sizeof(mine), ctx->s);
  if (cr != CUDA_SUCCESS) { err = ga_err_cuda(ctx->err, "cuMemcpyHtoDAsync", cr); goto out; }
  nr = nccl.AllGather((const void *)stage, (void *)(stage + sizeof(xc_hello)), sizeof(xc_hello),
                      ncclUint8, comm->c, ctx->s);
  if (nr != ncclSuccess) { err = nccl_fail(ctx, "ncclAllGather", nr); goto out; }
  cr = ga_cu.p_cuMemcpyDtoHAsync(all, stage + sizeof(xc_hello), sizeof(xc_hello) * (size_t)n, ctx->s);
  if (cr == CUDA_SUCCESS) cr = ga_cu.p_cuStreamSynchronize(ctx->s);
  if (cr != CUDA_SUCCESS) { err = ga_err_cuda(ctx->err, "peer window hello", cr); goto out; }
  for (p = 0; p < n; p++) {
    if (!all[p].f.ok) {
      agreed = 0;
      if (comm->win_reason[0] == '\0') peer_window_refuse(comm, "%srank %d has no window", "", p);
    }
    if (all[p].f.host != mine.f.host) {
      agreed = 0;
      if (comm->win_reason[0] == '\0') peer_window_refuse(comm, "%srank %d is on another host", "", p);
    }
    for (q = 0; q < p; q++)
      if (memcmp(all[p].f.pci, all[q].f.pci, sizeof(mine.f.pci)) == 0 || all[p].f.pid == all[q].f.pid) {
        agreed = 0;
        if (comm->win_reason[0] == '\0')
          peer_window_refuse(comm, "%srank %d shares a GPU or a process with another rank", "", p);
      }
  }
  /* second exchange: map the peers; then agree on whether everyone could */
  if (agreed) {
    for (p = 0; p < n && opened; p++) {
      if (p == me) continue;
      cr = ga_cu.p_cuIpcOpenMemHandle(&comm->win[p], all[p].f.handle, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS);
      if (cr != CUDA_SUCCESS) {
        comm->win[p] = 0;
        opened = 0;
        peer_window_refuse(comm, "%s of rank %d failed", "cuIpcOpenMemHandle", p);
      }
    }
  } else {
    opened = 0;
  }
  {
    int flag = opened;
    cr = ga_cu.p_cuMemcpyHtoDAsync(stage, &flag, sizeof(flag), ctx->s);
    if (cr != CUDA_SUCCESS) { err = ga_err_cuda(ctx->err, "cuMemcpyHtoDAsync", cr); goto out; }
    nr = nccl.AllReduce((const void *)stage, (void *)stage, 1, ncclInt32, ncclMin, comm->c, ctx->s);
    if (nr != ncclSuccess) { err = nccl_fail(ctx, "ncclAllReduce", nr); goto out; }
    cr = ga_cu.p_cuMemcpyDtoHAsync(&flag, stage, sizeof(flag), ctx->s);
    if (cr == CUDA_SUCCESS) cr = ga_cu.p_cuStreamSynchronize(ctx->s);
    if (cr != CUDA_SUCCESS) { err = ga_err_cuda(ctx->err, "peer window agreement", cr); goto out; }
    if (flag == 1) {
      comm->win_state = 1;
    } else {
      if (comm->win_reason[0] == '\0') peer_window_refuse(comm, "%sanother rank could not map its peers (%d)", "", flag);
      comm->win_state = 1; /* so that the release below un-maps what was mapped */
      {
        char keep[sizeof(comm->win_reason)];
        memcpy(keep, comm->win_reason, sizeof(keep));
        peer_window_release(comm);
        memcpy(comm->win_reason, keep, sizeof(keep));
      }
    }
  }
out:
  if (stage != 0) ga_cu.p_cuMemFree(stage);
  free(all);
  ga_ctx_exit(ctx);
  return err;
}

/* 1 when results of `bytes_per_rank` bytes can be combined through the peer
 * windows of `comm`; the first call sets them up (collective). */
int ga_comm_peer_ready(gpucomm *comm, size_t bytes_per_rank) {
  if (comm == NULL) return 0;
  if (comm->win_state == 0 && peer_window_setup(comm) != GA_NO_ERROR) return 0;
  return comm->win_state == 1 && bytes_per_rank <= XC_SLOT_BYTES;
}

static void xc_type_defines(ga_strb *sb, int tc, int pair) {
  const char *ct = ga_ctype(tc);
  ga_strb_printf(sb, "#define GA_XC_T %s\n", ct);
  if (tc == GA_HALF) {
    ga_strb_puts(sb, "#define GA_XC_W_T float\n#define GA_XC_LOAD(x) ga_half2float(x)\n"
                     "#define GA_XC_STORE(w) ga_float2half(w)\n");
  } else {
    ga_strb_printf(sb, "#define GA_XC_W_T %s\n#define GA_XC_LOAD(x) (x)\n#define GA_XC_STORE(w) (w)\n", ct);
  }
  ga_strb_printf(sb, "#define GA_XC_PAIR %d\n", pair);
}

/* Enqueues the exchange of `n` partial results held in val (and idx for pair
 * operators; both dense, written in place) on the context's stream.
 *  pair  0: accumulating, op one of GA_SUM / GA_PROD / GA_MIN / GA_MAX or, for integer
 *           types, GA_XC_AND / GA_XC_OR / GA_XC_XOR (folds the collectives do not offer)
 *        1: (value, index), op GA_MIN or GA_MAX
 *        2: value only, op GA_MIN or GA_MAX, equal values (+0.0, -0.0) go to the
 *           rank with the lowest `key`; idx is not used */
int ga_comm_exchange(gpucomm *comm, int pair, int op, int tc, CUdeviceptr val, CUdeviceptr idx,
                     size_t n, unsigned long long key) {
  gpucontext *ctx = comm->ctx;
  xc_kernel *k;
  struct {
    unsigned long long n, seq, slot_bytes, idx_off, timeout_ns, key, win[XC_MAX_RANKS];
    unsigned int nranks, rank, chunk, phases;
  } L;
  const size_t es = gpuarray_get_elsize(tc);
  unsigned int grid[3] = {1, 1, 1}, block[3] = {XC_THREADS, 1, 1};
  void *params[4];
  size_t ctas;
  int p, err;

  if (comm->win_state != 1) return ga_err_set(ctx->err, GA_COMM_ERROR, "No peer windows");
  if (*(volatile unsigned int *)comm->status_host != 0)
    return ga_err_set(ctx->err, GA_COMM_ERROR,
                      "An earlier exchange over peer memory gave up waiting for a rank; the "
                      "communicator cannot be used any more");
  if (n == 0) return GA_NO_ERROR;
  {
    /* what one rank puts into a slot: the values, then (16-byte aligned) the indices or the key */
    const size_t idx_off = (n * es + 15) & ~(size_t)15;
    const size_t need = pair == 1 ? idx_off + n * 8 : pair == 2 ? idx_off + 8 : n * es;
    if (need > XC_SLOT_BYTES)
      return ga_err_set(ctx->err, GA_VALUE_ERROR, "Result too large for the peer windows");
  }
  {
    /* every exchange carries its own sequence number: a captured launch replayed from a
     * CUDA graph would present an old one, find its flags already set and read stale slots */
    CUstreamCaptureStatus cap = CU_STREAM_CAPTURE_STATUS_NONE;
    ga_ctx_enter(ctx);
    ga_cu.p_cuStreamIsCapturing(ctx->s, &cap);
    ga_ctx_exit(ctx);
    if (cap != CU_STREAM_CAPTURE_STATUS_NONE)
      return ga_err_set(ctx->err, GA_UNSUPPORTED_ERROR,
                        "Sharded reductions cannot be captured into a CUDA graph: each exchange over "
                        "peer memory is numbered");
  }
  for (k = comm->kernels; k != NULL; k = k->next)
    if (k->pair == pair && k->op == op && k->tc == tc) break;
  if (k == NULL) {
    ga_strb sb;
    ga_function fn;
    ga_strb_init(&sb);
    xc_type_defines(&sb, tc, pair);
    if (pair) {
      ga_strb_printf(&sb, "#define GA_XC_MIN %d\n", op == GA_MIN);
    } else {
      ga_strb_printf(&sb, "#define GA_XC_OP(a, b) %s\n",
                     op == GA_SUM    ? "((a) + (b))"
                     : op == GA_PROD ? "((a) * (b))"
                     : op == GA_MIN  ? "((b) < (a) ? (b) : (a))"
                     : op == GA_MAX  ? "((b) > (a) ? (b) : (a))"
                     : op == GA_XC_AND ? "((a) & (b))"
                     : op == GA_XC_OR  ? "((a) | (b))"
                                       : "((a) ^ (b))");
    }
    ga_strb_puts(&sb, "#include \"ga_exchange.cuh\"\n");
    if (sb.failed) {
      ga_strb_free(&sb);
      return ga_err_sys(ctx->err, "malloc");
    }
    err = ga_compile(ctx, ga_strb_cstr(&sb), "ga_exchange", NULL, &fn, NULL);
    ga_strb_free(&sb);
    if (err != GA_NO_ERROR) return err;
    fn.dependent_ok = 1;
    k = calloc(1, sizeof(*k));
    if (k == NULL) return ga_err_sys(ctx->err, "calloc");
    k->pair = pair; k->op = op; k->tc = tc; k->fn = fn;
    k->next = comm->kernels;
    comm->kernels = k;
  }
  memset(&L, 0, sizeof(L));
  L.n = n;
  L.seq = ++comm->seq;
  L.slot_bytes = XC_SLOT_BYTES;
  L.idx_off = (n * es + 15) & ~(size_t)15;
  L.timeout_ns = comm->timeout_ns;
  L.key = key;
  for (p = 0; p < comm->ndev; p++) L.win[p] = (unsigned long long)comm->win[p];
  L.nranks = (unsigned int)comm->ndev;
  L.rank = (unsigned int)comm->rank;
  ctas = (n + XC_THREADS - 1) / XC_THREADS;
  if (ctas > XC_MAX_CTAS) ctas = XC_MAX_CTAS;
  L.chunk = (unsigned int)((((n + ctas - 1) / ctas) + 15) & ~(size_t)15);
  grid[0] = (unsigned int)((n + L.chunk - 1) / L.chunk);
  L.phases = 3;
  params[0] = &L;
  params[1] = &val;
  params[2] = &idx;
  params[3] = &comm->status_dev;
  return ga_launch(ctx, &k->fn, grid, block, 0, params);
}

/* State of the peer windows of a communicator, for tests and benchmarks:
 * 0 not set up yet, 1 in use, -1 unavailable (reason, if asked for, is a
 * pointer into the communicator). *timed_out is non-zero once a kernel gave
 * up waiting for a peer. */
GPUARRAY_PUBLIC int gpuarray_b200_comm_peer_state(gpucomm *comm, const char **reason,
                                                  unsigned int *timed_out) {
  if (reason != NULL) *reason = comm->win_reason;
  if (timed_out != NULL)
    *timed_out = comm->status_host != NULL ? *(volatile unsigned int *)comm->status_host : 0;
  return comm->win_state;
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
