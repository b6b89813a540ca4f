/* Kernel source -> sm_100a machine code -> CUfunction.
 *
 * Replaces the compile half of the reference's CUDA backend
 * (src/gpuarray_buffer_cuda.c:1073-1482): there, source goes NVRTC -> PTX for
 * "compute_XY" -> cuLink -> cubin, the architecture string is derived from the
 * device (and comes out truncated for compute capability 10.0), and a 2Q cache
 * is keyed by the full source text. Here NVRTC is asked for sm_100a SASS
 * directly (nvrtcGetCUBIN), the only option besides the architecture is the
 * language level, so floating-point contraction stays at NVRTC's default
 * (fused multiply-add on), like the reference which passes only -arch.
 *
 * Caches: per context, a list of loaded modules keyed by a 128-bit hash of
 * (library tag, options, NVRTC version, in-library headers, source); optionally a directory of cubin files with
 * the same key (GPUARRAY_CACHE_PATH or gpucontext_props_kernel_cache), which
 * can be filled on a machine without a GPU. */
#include <sys/stat.h>
#include <unistd.h>
#include "private.h"

#define GA_KERNEL_ABI_TAG "ga-b200-k1"
#define GA_ARCH_OPT "--gpu-architecture=sm_100a"

struct ga_module {
  uint64_t key[2];
  CUmodule mod;
  struct ga_module *next;
};

#define GA_STD_OPT "--std=c++17"

/* Everything besides the program text and the headers it includes that
 * decides what machine code comes out: the library's kernel ABI tag, the
 * compiler options and the version of the NVRTC that is bound (two toolkits
 * give different code for the same text). Computed once per process. */
static const char *key_prefix(size_t *len) {
  static char prefix[160];
  static size_t prefix_len = 0;
  if (prefix_len == 0) {
    int major = 0, minor = 0;
    ga_error_rec scratch;
    memset(&scratch, 0, sizeof(scratch));
    if (ga_load_nvrtc(&scratch) == GA_NO_ERROR) ga_rtc.p_nvrtcVersion(&major, &minor);
    prefix_len = (size_t)snprintf(prefix, sizeof(prefix),
                                  GA_KERNEL_ABI_TAG "\n" GA_ARCH_OPT "\n" GA_STD_OPT "\nnvrtc %d.%d\n",
                                  major, minor);
  }
  *len = prefix_len;
  return prefix;
}

#define GA_MAX_TEMPLATES 32

/* bit j of the result: in-library header j is named by an #include "..." of `text` */
static unsigned int includes_of(const char *text) {
  unsigned int mask = 0, j;
  const char *p = text;
  while ((p = strstr(p, "#include \"")) != NULL) {
    const char *name = p + 10, *end = strchr(name, '"');
    if (end == NULL) break;
    for (j = 0; j < ga_template_count && j < GA_MAX_TEMPLATES; j++)
      if (strlen(ga_template_names[j]) == (size_t)(end - name) &&
          strncmp(ga_template_names[j], name, (size_t)(end - name)) == 0)
        mask |= 1u << j;
    p = end;
  }
  return mask;
}

/* The in-library headers a program pulls in are part of its text: the key
 * holds a hash of every header reachable from the program's #include lines
 * (and of no other, so that editing one template leaves the cached kernels of
 * the others valid). Header hashes and their include sets are computed once. */
static void append_header_hashes(ga_strb *sb, const char *src) {
  static int ready = 0;
  static uint64_t hash[GA_MAX_TEMPLATES];
  static unsigned int direct[GA_MAX_TEMPLATES];
  unsigned int reach, frontier, j;
  if (!ready) {
    for (j = 0; j < ga_template_count && j < GA_MAX_TEMPLATES; j++) {
      hash[j] = ga_hash64(ga_template_sources[j], strlen(ga_template_sources[j]), 7);
      direct[j] = includes_of(ga_template_sources[j]);
    }
    ready = 1;
  }
  reach = 0;
  frontier = includes_of(src);
  while (frontier != 0) {
    unsigned int next = 0;
    reach |= frontier;
    for (j = 0; j < ga_template_count && j < GA_MAX_TEMPLATES; j++)
      if (frontier & (1u << j)) next |= direct[j];
    frontier = next & ~reach;
  }
  for (j = 0; j < ga_template_count && j < GA_MAX_TEMPLATES; j++)
    if (reach & (1u << j))
      ga_strb_printf(sb, "%s:%016llx\n", ga_template_names[j], (unsigned long long)hash[j]);
}

static void make_key(const char *src, const char *const *defines, uint64_t key[2]) {
  ga_strb sb;
  size_t plen;
  const char *prefix = key_prefix(&plen);
  ga_strb_init(&sb);
  ga_strb_putn(&sb, prefix, plen);
  if (defines != NULL)
    for (; *defines != NULL; defines++) {
      ga_strb_puts(&sb, *defines);
      ga_strb_puts(&sb, "\n");
    }
  append_header_hashes(&sb, src);
  ga_strb_puts(&sb, src);
  key[0] = ga_hash64(ga_strb_cstr(&sb), sb.len, 0);
  key[1] = ga_hash64(ga_strb_cstr(&sb), sb.len, 0x9e3779b97f4a7c15ULL);
  ga_strb_free(&sb);
}

/* "0001\t<line>\n..." followed by the compiler log, like the reference's
 * gpukernel_source_with_line_numbers (src/gpuarray_util.c:85-109). */
static char *numbered_listing(const char *src, const char *log) {
  ga_strb sb;
  unsigned line = 1;
  const char *p = src, *nl;
  ga_strb_init(&sb);
  while (*p != '\0') {
    nl = strchr(p, '\n');
    ga_strb_printf(&sb, "%04u\t", line++);
    if (nl == NULL) {
      ga_strb_puts(&sb, p);
      ga_strb_puts(&sb, "\n");
      break;
    }
    ga_strb_putn(&sb, p, (size_t)(nl - p) + 1);
    p = nl + 1;
  }
  if (log != NULL) {
    ga_strb_puts(&sb, "\nCompiler log:\n");
    ga_strb_puts(&sb, log);
  }
  return sb.s; /* ownership moves to the caller */
}

static int disk_get(const char *dir, const uint64_t key[2], char **bin, size_t *sz) {
  char path[4096];
  FILE *f;
  long n;
  if (dir == NULL) return -1;
  snprintf(path, sizeof(path), "%s/%016llx%016llx.cubin", dir, (unsigned long long)key[0],
           (unsigned long long)key[1]);
  f = fopen(path, "rb");
  if (f == NULL) return -1;
  if (fseek(f, 0, SEEK_END) != 0 || (n = ftell(f)) <= 0 || fseek(f, 0, SEEK_SET) != 0) {
    fclose(f);
    return -1;
  }
  *bin = malloc((size_t)n);
  if (*bin == NULL || fread(*bin, 1, (size_t)n, f) != (size_t)n) {
    free(*bin);
    *bin = NULL;
    fclose(f);
    return -1;
  }
  fclose(f);
  *sz = (size_t)n;
  return 0;
}

static void disk_put(const char *dir, const uint64_t key[2], const char *bin, size_t sz) {
  char path[4096], tmp[4200];
  FILE *f;
  if (dir == NULL) return;
  mkdir(dir, 0777);
  snprintf(path, sizeof(path), "%s/%016llx%016llx.cubin", dir, (unsigned long long)key[0],
           (unsigned long long)key[1]);
  snprintf(tmp, sizeof(tmp), "%s.%ld.tmp", path, (long)getpid());
  f = fopen(tmp, "wb");
  if (f == NULL) return;
  {
    const int written = fwrite(bin, 1, sz, f) == sz;
    const int closed = fclose(f) == 0; /* always close, even after a short write */
    if (written && closed) rename(tmp, path);
    else unlink(tmp);
  }
}

static int nvrtc_build(ga_error_rec *e, const char *src, const char *const *defines, char **bin,
                       size_t *bin_sz, char **err_str) {
  nvrtcProgram prog = NULL;
  nvrtcResult r;
  const char *opts[64];
  int nopts = 0, err;
  size_t logsz = 0;
  char *log = NULL;

  err = ga_load_nvrtc(e);
  if (err != GA_NO_ERROR) return err;

  opts[nopts++] = GA_ARCH_OPT;
  opts[nopts++] = GA_STD_OPT;
  if (defines != NULL)
    for (; *defines != NULL && nopts < 63; defines++) opts[nopts++] = *defines;

  r = ga_rtc.p_nvrtcCreateProgram(&prog, src, "ga_kernel.cu", (int)ga_template_count,
                                  (const char *const *)ga_template_sources,
                                  (const char *const *)ga_template_names);
  if (r != NVRTC_SUCCESS)
    return ga_err_fmt(e, GA_IMPL_ERROR, "nvrtcCreateProgram: %s", ga_rtc.p_nvrtcGetErrorString(r));

  r = ga_rtc.p_nvrtcCompileProgram(prog, nopts, opts);
  if (r != NVRTC_SUCCESS) {
    if (ga_rtc.p_nvrtcGetProgramLogSize(prog, &logsz) == NVRTC_SUCCESS && logsz > 1) {
      log = malloc(logsz);
      if (log != NULL && ga_rtc.p_nvrtcGetProgramLog(prog, log) != NVRTC_SUCCESS) {
        free(log);
        log = NULL;
      }
    }
    if (err_str != NULL) *err_str = numbered_listing(src, log);
    /* keep the head of the log in the error message: it usually names the
     * offending token of the user's expression */
    err = ga_err_fmt(e, GA_IMPL_ERROR, "nvrtcCompileProgram: %s%s%.800s",
                     ga_rtc.p_nvrtcGetErrorString(r), log ? ": " : "", log ? log : "");
    free(log);
    ga_rtc.p_nvrtcDestroyProgram(&prog);
    return err;
  }
  r = ga_rtc.p_nvrtcGetCUBINSize(prog, bin_sz);
  if (r == NVRTC_SUCCESS) {
    *bin = malloc(*bin_sz);
    if (*bin == NULL) {
      ga_rtc.p_nvrtcDestroyProgram(&prog);
      return ga_err_sys(e, "malloc");
    }
    r = ga_rtc.p_nvrtcGetCUBIN(prog, *bin);
  }
  ga_rtc.p_nvrtcDestroyProgram(&prog);
  if (r != NVRTC_SUCCESS) {
    free(*bin);
    *bin = NULL;
    return ga_err_fmt(e, GA_IMPL_ERROR, "nvrtcGetCUBIN: %s", ga_rtc.p_nvrtcGetErrorString(r));
  }
  return GA_NO_ERROR;
}

int ga_compile_cubin(ga_error_rec *e, const char *src, const char *const *defines,
                     const char *cache_dir, char **bin, size_t *bin_sz, char **err_str) {
  uint64_t key[2];
  int err;
  if (err_str != NULL) *err_str = NULL;
  make_key(src, defines, key);
  if (disk_get(cache_dir, key, bin, bin_sz) == 0) return GA_NO_ERROR;
  err = nvrtc_build(e, src, defines, bin, bin_sz, err_str);
  if (err == GA_NO_ERROR) disk_put(cache_dir, key, *bin, *bin_sz);
  return err;
}

/* GPUARRAY_B200_SOURCE_LOG=<dir>: every kernel source this process builds or
 * loads is also written to <dir>/<hash of the text>.src. The collected texts
 * let `python -m libgpuarray_b200.warm_cache` rebuild the cubin cache on a
 * machine without a GPU (NVRTC needs none), e.g. after the kernel templates
 * changed or before a deployment that must not compile at start-up. */
static void log_source(const char *src) {
  const char *dir = getenv("GPUARRAY_B200_SOURCE_LOG");
  char path[4096];
  FILE *f;
  size_t len;
  if (dir == NULL || dir[0] == '\0') return;
  len = strlen(src);
  mkdir(dir, 0777);
  snprintf(path, sizeof(path), "%s/%016llx%016llx.src", dir,
           (unsigned long long)ga_hash64(src, len, 0),
           (unsigned long long)ga_hash64(src, len, 0x9e3779b97f4a7c15ULL));
  f = fopen(path, "rb");
  if (f != NULL) { /* already there */
    fclose(f);
    return;
  }
  f = fopen(path, "wb");
  if (f == NULL) return;
  fwrite(src, 1, len, f);
  fclose(f);
}

int ga_compile(gpucontext *ctx, const char *src, const char *fname, const char *const *defines,
               ga_function *out, char **err_str) {
  uint64_t key[2];
  struct ga_module *m;
  CUresult r;
  int err = GA_NO_ERROR;

  if (err_str != NULL) *err_str = NULL;
  make_key(src, defines, key);
  for (m = ctx->modules; m != NULL; m = m->next)
    if (m->key[0] == key[0] && m->key[1] == key[1]) break;

  if (m == NULL) {
    char *bin = NULL;
    size_t bin_sz = 0;
    if (defines == NULL) log_source(src);
    if (disk_get(ctx->kernel_cache_path, key, &bin, &bin_sz) != 0) {
      err = nvrtc_build(ctx->err, src, defines, &bin, &bin_sz, err_str);
      if (err != GA_NO_ERROR) return err;
      disk_put(ctx->kernel_cache_path, key, bin, bin_sz);
    }
    m = calloc(1, sizeof(*m));
    if (m == NULL) {
      free(bin);
      return ga_err_sys(ctx->err, "calloc");
    }
    ga_ctx_enter(ctx);
    r = ga_cu.p_cuModuleLoadData(&m->mod, bin);
    ga_ctx_exit(ctx);
    free(bin);
    if (r != CUDA_SUCCESS) {
      free(m);
      return ga_err_cuda(ctx->err, "cuModuleLoadData", r);
    }
    m->key[0] = key[0];
    m->key[1] = key[1];
    m->next = ctx->modules;
    ctx->modules = m;
  }

  out->dependent_ok = 0;
  ga_ctx_enter(ctx);
  r = ga_cu.p_cuModuleGetFunction(&out->f, m->mod, fname);
  if (r != CUDA_SUCCESS) err = ga_err_cuda(ctx->err, "cuModuleGetFunction", r);
  else {
    ga_cu.p_cuFuncGetAttribute(&out->max_threads, CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, out->f);
    ga_cu.p_cuFuncGetAttribute(&out->num_regs, CU_FUNC_ATTRIBUTE_NUM_REGS, out->f);
    ga_cu.p_cuFuncGetAttribute(&out->static_smem, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, out->f);
  }
  ga_ctx_exit(ctx);
  return err;
}

void ga_modules_free(gpucontext *ctx) {
  struct ga_module *m, *n;
  for (m = ctx->modules; m != NULL; m = n) {
    n = m->next;
    ga_cu.p_cuModuleUnload(m->mod);
    free(m);
  }
  ctx->modules = NULL;
}

static unsigned long long launch_counter = 0;

/* Number of kernels this library has launched in the process so far. */
GPUARRAY_PUBLIC unsigned long long gpuarray_b200_launch_count(void) { return launch_counter; }

/* GPUARRAY_B200_NO_PDL=1 falls back to fully serialized launches. */
static int dependent_launch_enabled(void) {
  static int state = -1;
  if (state < 0) {
    const char *env = getenv("GPUARRAY_B200_NO_PDL");
    state = !(env != NULL && env[0] != '\0' && env[0] != '0');
  }
  return state;
}

int ga_launch(gpucontext *ctx, const ga_function *fn, const unsigned grid[3],
              const unsigned block[3], size_t shared, void **params) {
  CUresult r;
  ga_ctx_enter(ctx);
  if (shared + (size_t)fn->static_smem > ctx->smem_block) {
    r = ga_cu.p_cuFuncSetAttribute(fn->f, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                   (int)shared);
    if (r != CUDA_SUCCESS) {
      ga_ctx_exit(ctx);
      return ga_err_cuda(ctx->err, "cuFuncSetAttribute", r);
    }
  }
  if (fn->dependent_ok && dependent_launch_enabled()) {
    /* programmatic dependent launch: the kernel may become resident while the
     * previous kernel of the stream drains; it waits for it before touching
     * memory (ga__grid_dependency_sync in the templates) */
    CUlaunchConfig cfg;
    CUlaunchAttribute attr;
    memset(&cfg, 0, sizeof(cfg));
    memset(&attr, 0, sizeof(attr));
    attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    attr.value.programmaticStreamSerializationAllowed = 1;
    cfg.gridDimX = grid[0]; cfg.gridDimY = grid[1]; cfg.gridDimZ = grid[2];
    cfg.blockDimX = block[0]; cfg.blockDimY = block[1]; cfg.blockDimZ = block[2];
    cfg.sharedMemBytes = (unsigned)shared;
    cfg.hStream = ctx->s;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    r = ga_cu.p_cuLaunchKernelEx(&cfg, fn->f, params, NULL);
  } else {
    r = ga_cu.p_cuLaunchKernel(fn->f, grid[0], grid[1], grid[2], block[0], block[1], block[2],
                               (unsigned)shared, ctx->s, params, NULL);
  }
  ga_ctx_exit(ctx);
  if (r != CUDA_SUCCESS) return ga_err_cuda(ctx->err, "cuLaunchKernel", r);
  launch_counter++;
  return GA_NO_ERROR;
}

/* Version of the NVRTC the library bound (major * 1000 + minor * 10), 0 when it
 * cannot be loaded. */
GPUARRAY_PUBLIC int gpuarray_b200_nvrtc_version(void) {
  int major = 0, minor = 0;
  if (ga_load_nvrtc(ga_global_err) != GA_NO_ERROR) return 0;
  if (ga_rtc.p_nvrtcVersion(&major, &minor) != NVRTC_SUCCESS) return 0;
  return major * 1000 + minor * 10;
}

/* Test and tooling hook: compile a program for sm_100a without any device.
 * Returns GA_NO_ERROR and the cubin size, or an error with *log (malloc'ed,
 * may be NULL) holding the numbered source and compiler output. */
GPUARRAY_PUBLIC int gpuarray_b200_compile_check(const char *src, const char *const *defines,
                                               const char *cache_dir, size_t *cubin_size,
                                               char **log) {
  char *bin = NULL;
  size_t sz = 0;
  int err = ga_compile_cubin(ga_global_err, src, defines, cache_dir, &bin, &sz, log);
  free(bin);
  if (cubin_size != NULL) *cubin_size = sz;
  return err;
}
