/* Entry points that exist only in the B200 engine (no counterpart in the
 * reference): introspection and tooling hooks used by the tests, the
 * benchmark and build-time kernel checks. None of them computes anything. */
#ifndef GPUARRAY_B200_H
#define GPUARRAY_B200_H

#include <gpuarray/buffer.h>
#include <gpuarray/elemwise.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Code of the last error recorded on `ctx` (NULL: the process-global record);
 * gpucontext_error() gives the matching text. */
GPUARRAY_PUBLIC int gpuarray_b200_error_code(gpucontext *ctx);

/* Kernels launched by this library in the process so far (all contexts). */
GPUARRAY_PUBLIC unsigned long long gpuarray_b200_launch_count(void);

/* Compiles CUDA C++ `src` for sm_100a with the library's in-memory headers
 * ("cluda.h", the kernel templates) and NVRTC; needs no GPU. `defines` is a
 * NULL-terminated list of "-DNAME=VALUE" options or NULL; `cache_dir` (may be
 * NULL) is a directory of cubin files reused across runs. On failure *log
 * (malloc'ed, may be NULL) holds the numbered source and the compiler log. */
GPUARRAY_PUBLIC int gpuarray_b200_compile_check(const char *src, const char *const *defines,
                                                const char *cache_dir, size_t *cubin_size,
                                                char **log);

/* The kernel source GpuElemwise would compile for one variant: kind 0
 * contiguous, 1 strided, 2 tiled transpose; `ept` elements per thread chunk;
 * `modes` packs two bits per array argument (0 scalar access, 1 vector,
 * 2 broadcast). malloc'ed; the caller frees. */
GPUARRAY_PUBLIC char *gpuarray_b200_elemwise_source(const char *preamble, const char *expr,
                                                    unsigned int n, gpuelemwise_arg *args,
                                                    int flags, int kind, int ept, int unroll,
                                                    unsigned int nd, int idx32,
                                                    unsigned long long modes, int tp, int tq);

/* The kernel source GpuReduction would compile for one variant: `shape`
 * 0 rows, 1 cols, 2 general; `vec` elements per load; `tpo` threads per
 * output (general); `group` threads sharing a work item (rows: 32 or 256,
 * 0 = default). malloc'ed; the caller frees. */
GPUARRAY_PUBLIC char *gpuarray_b200_reduction_source(int op, int src_tc, int dst_tc, int shape,
                                                     int vec, int idx64, int tpo, int group);

/* Version of the NVRTC the library bound, as major * 1000 + minor * 10 (12090 for
 * 12.9); 0 when none could be loaded. The toolkit's copy under /usr/local/cuda
 * is preferred over one the process may have loaded already. */
GPUARRAY_PUBLIC int gpuarray_b200_nvrtc_version(void);

/* The shape work of GpuElemwise_call on plain shape / byte-stride lists, with no
 * device: contiguous-fast-path test (reference check_contig,
 * src/gpuarray_elemwise.c:547-576), rank padding, broadcast, output-defines-
 * shape and dimension collapsing (check_basic, :272-383). args[i] gives the
 * typecode and GE_* flags of argument i; nds/dims/strides describe the array
 * arguments (entries of GE_SCALAR arguments are ignored). Returns the GA_* code
 * the call would return up to that point; out[0] = 0 contiguous kernel / 1
 * strided kernels, out[1] = element count, out[2] = rank after collapsing,
 * then the collapsed extents, then per array argument its collapsed byte
 * strides (strided path only). out must hold 3 + 8 + 8 * n words. */
GPUARRAY_PUBLIC int gpuarray_b200_elemwise_shapes(unsigned int n, const gpuelemwise_arg *args,
                                                  const unsigned int *nds,
                                                  const size_t *const *dims,
                                                  const ssize_t *const *strides, int call_flags,
                                                  long long *out);

/* Everything GpuElemwise_call decides for a call (kernel, widths, access modes,
 * tile, launch geometry), computed on the host alone for arrays given by rank,
 * extents, byte strides and the address of their first element (alignment only).
 * obj_flags as for GpuElemwise_new, call_flags as for GpuElemwise_call.
 * out[0..15] = kernel (0 contiguous, 1 strided, 2 tiled transpose), elements per
 * thread chunk, chunks in flight (tiled transpose: 2 marks the build that stages
 * with 16-byte asynchronous copies and reads back with transposing matrix
 * loads, 1 the word-staged build), rank after collapsing, index width bits, access
 * modes (2 bits per array argument: 0 gather, 1 vector, 2 broadcast, 3 staged
 * through shared memory), tile P, tile Q, P positions per thread, grid x/y/z,
 * block x/y/z, element count. blob_out (may be NULL) receives the layout
 * parameter block of the strided / transposing kernels (blob_cap words
 * available, *blob_words its length). Reference counterpart of the decisions:
 * src/gpuarray_elemwise.c:385-442,578-602 and src/gpuarray_kernel.c:38-89. */
GPUARRAY_PUBLIC int gpuarray_b200_elemwise_plan(unsigned int n, const gpuelemwise_arg *args,
                                                const unsigned int *nds,
                                                const size_t *const *dims,
                                                const ssize_t *const *strides,
                                                const unsigned long long *bases, int obj_flags,
                                                int call_flags, unsigned int num_sms,
                                                unsigned long long *out,
                                                unsigned long long *blob_out, size_t blob_cap,
                                                size_t *blob_words);

/* The plan GpuReduction_call would make (kernel variant, split of the reduced
 * extent, launch geometry) for a source of the given shape and byte strides on a
 * device with num_sms multiprocessors, computed on the host alone. `base` stands
 * for the address of the source's first element (its alignment decides the
 * vector width); destinations are taken as C-contiguous. out[0..23] = kernel
 * shape (0 rows, 1 cols, 2 general), vector width, group size, flattened runs,
 * runs at once, one-run mode, lazy index, byte folding, threads per output
 * (general kernel), 64-bit index, splits, seg, nseg, units, grid x, grid y,
 * block x, block y (cols: row lanes per CTA), outputs, reduced elements per
 * output, lean rows loop, three spare words. No reference
 * counterpart (its scheduler is src/gpuarray_reduction.c:673-776). */
GPUARRAY_PUBLIC int gpuarray_b200_reduction_plan(int op, int src_tc, int dst_tc, unsigned int nd,
                                                 const size_t *dims, const ssize_t *strides,
                                                 unsigned int reduxLen, const int *reduxList,
                                                 unsigned long long base, unsigned int num_sms,
                                                 unsigned long long *out);

/* gpuarray_b200_reduction_plan plus the parameter block the kernel would
 * receive (struct ga__rd_layout of the reduction template), copied into
 * `layout` (cap bytes available, *used = its size): for tools that run the
 * kernel templates outside the library. */
GPUARRAY_PUBLIC int gpuarray_b200_reduction_layout(int op, int src_tc, int dst_tc, unsigned int nd,
                                                   const size_t *dims, const ssize_t *strides,
                                                   unsigned int reduxLen, const int *reduxList,
                                                   unsigned long long base, unsigned int num_sms,
                                                   unsigned long long *out, void *layout,
                                                   size_t cap, size_t *used);

/* As gpuarray_b200_reduction_source / _layout, for GpuMapReduction: the source
 * of one kernel variant (malloc'ed; the caller frees), and what a call would
 * decide for array arguments given by rank, extents, byte strides and the
 * address of their first element (alignment only), with the destination taken
 * as C-contiguous. out[0..13] = kernel shape (0 rows, 1 cols, 2 general),
 * vector width, group, threads per output, access modes (2 bits per array:
 * 0 gather, 1 vector, 2 broadcast), splits, seg, nseg, units, grid x, grid y,
 * block x, block y, outputs. No reference counterpart (the reference renders
 * one kernel per rank in Python, pygpu/reduction.py:217-239). */
GPUARRAY_PUBLIC char *gpuarray_b200_mapreduction_source(const char *preamble, const char *map_expr,
                                                        const char *reduce_expr,
                                                        const char *neutral, int out_tc,
                                                        unsigned int n, gpuelemwise_arg *args,
                                                        int flags, int shape, int vec, int group,
                                                        int tpo, unsigned long long modes);
GPUARRAY_PUBLIC int gpuarray_b200_mapreduction_plan(int out_tc, unsigned int n,
                                                    const gpuelemwise_arg *args,
                                                    const unsigned int *nds,
                                                    const size_t *const *dims,
                                                    const ssize_t *const *strides,
                                                    const unsigned long long *bases,
                                                    unsigned int reduxLen, const int *reduxList,
                                                    int call_flags, unsigned int num_sms,
                                                    unsigned long long *out, void *layout,
                                                    size_t cap, size_t *used);

/* Tooling hook: the split count a split row reduction is trimmed to so that its grid ends on
 * a full or nearly full wave of resident CTAs (outputs x splits work items of `group` threads,
 * 256 threads per CTA, `slots` CTAs resident at once); *ctas receives the grid size. */
GPUARRAY_PUBLIC unsigned long long gpuarray_b200_reduction_fit_waves(unsigned long long outputs,
                                                                     unsigned long long splits,
                                                                     int group,
                                                                     unsigned long long slots,
                                                                     unsigned int *ctas);

/* State of a communicator's peer-memory windows, through which
 * GpuReduction_call_sharded combines the ranks' partial results with one
 * kernel per GPU (every rank stores its partials into all peers' windows over
 * NVLink and folds what arrives). Returns 0 before the first sharded
 * reduction, 1 when the windows are in use, -1 when they could not be set up
 * on every rank (*reason, if not NULL, then points to a text inside the
 * communicator) and gpucomm_all_reduce is used instead. *timed_out, if not
 * NULL, is non-zero once a kernel gave up waiting for a rank
 * (GPUARRAY_B200_PEER_TIMEOUT_MS, default 10000); sharded calls on that
 * communicator then return GA_COMM_ERROR. GPUARRAY_B200_NO_PEER_WINDOW=1
 * keeps the windows off. No counterpart in the reference. */
struct _gpucomm;
GPUARRAY_PUBLIC int gpuarray_b200_comm_peer_state(struct _gpucomm *comm, const char **reason,
                                                  unsigned int *timed_out);

/* Sum of n contiguous float32 values on the current device WITHOUT allocating
 * anything: no cudaMalloc / cudaFree, no library workspace. (No counterpart in
 * the reference, whose reductions allocate per call.) It is for callers that
 * are not allowed to allocate when they need the result - code living inside
 * another framework's memory pool, latency-critical loops, hosts that must not
 * touch the driver's allocator between stream-ordered work. The partial sums
 * and the arrival ticket of the split reduction live in a 64 KiB block that is
 * part of the library image on every GPU that loads it.
 *   src, dst     device pointers (src 16-byte aligned); dst receives one float
 *   n            at most GPUARRAY_B200_NOALLOC_MAX_ELEMS, else GA_XLARGE_ERROR
 *   cuda_stream  a CUstream / cudaStream_t (NULL: the default stream)
 * The first call on a device resolves the block's device address (threads
 * racing to make it are serialised); make it before any stream capture. The
 * address is cached for the life of the process: a cudaDeviceReset() or a
 * reset of the primary context invalidates it, do not call this entry point
 * after one. src and dst must be device memory of the CURRENT device, or
 * GA_VALUE_ERROR is returned before anything is queued. Calls share the
 * block: do not let two of them overlap on the GPU. Returns a GA_* code; text
 * via gpucontext_error(NULL, 0). */
#define GPUARRAY_B200_NOALLOC_MAX_ELEMS (1ULL << 32)
GPUARRAY_PUBLIC int gpuarray_b200_sum_f32_noalloc(const float *src, size_t n, float *dst,
                                                  void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
