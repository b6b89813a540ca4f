/* Run-time binding to the CUDA driver and NVRTC.
 *
 * The library never links libcuda directly, so it loads (and its host-only
 * entry points work) on machines without a driver; anything that needs the
 * device fails with GA_LOAD_ERROR instead. Plays the part of the reference's
 * src/loaders/libcuda.c and libnvrtc.c; unlike those it also binds
 * nvrtcGetCUBIN, because kernels are compiled straight to sm_100a machine
 * code without a PTX/link step. */
#include <dlfcn.h>
#include "private.h"

struct ga_cuda_api ga_cu;
struct ga_nvrtc_api ga_rtc;

#define GA_STR_(x) #x
#define GA_STR(x) GA_STR_(x)

static void *open_first(const char *const *names, char *tried, size_t triedsz) {
  void *h = NULL;
  tried[0] = '\0';
  for (; *names != NULL; names++) {
    h = dlopen(*names, RTLD_LAZY | RTLD_LOCAL);
    if (h != NULL) return h;
    strncat(tried, *names, triedsz - strlen(tried) - 1);
    strncat(tried, " ", triedsz - strlen(tried) - 1);
  }
  return NULL;
}

int ga_load_cuda(ga_error_rec *e) {
  static int state = 0; /* 0 untried, 1 ok, -1 failed */
  static const char *const names[] = {"libcuda.so.1", "libcuda.so", NULL};
  char tried[256];
  void *h;
  if (state == 1) return GA_NO_ERROR;
  h = open_first(names, tried, sizeof(tried));
  if (h == NULL) {
    state = -1;
    return ga_err_fmt(e, GA_LOAD_ERROR, "Could not load \"libcuda.so\" (tried: %s): %s",
                      tried, dlerror());
  }
#define X(n)                                                                        \
  ga_cu.p_##n = (__typeof__(&n))dlsym(h, GA_STR(n));                                \
  if (ga_cu.p_##n == NULL) {                                                        \
    state = -1;                                                                     \
    return ga_err_fmt(e, GA_LOAD_ERROR, "libcuda.so lacks symbol %s", GA_STR(n));   \
  }
  GA_CU_FUNCS(X)
#undef X
  {
    CUresult r = ga_cu.p_cuInit(0);
    if (r != CUDA_SUCCESS) {
      state = -1;
      return ga_err_cuda(e, "cuInit", r);
    }
  }
  state = 1;
  return GA_NO_ERROR;
}

int ga_load_nvrtc(ga_error_rec *e) {
  static int state = 0;
  /* The toolkit's own NVRTC first, by path: a bare soname would resolve to
   * whatever copy the process has loaded already (PyTorch bundles an older
   * one), and which compiler built a kernel would then depend on import order. */
  static const char *const names[] = {
      "/usr/local/cuda/lib64/libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so",
      "libnvrtc.so.12", "libnvrtc.so", NULL};
  char tried[512];
  void *h = NULL;
  const char *env;
  if (state == 1) return GA_NO_ERROR;
  env = getenv("GPUARRAY_NVRTC_PATH");
  if (env != NULL && env[0] != '\0') h = dlopen(env, RTLD_LAZY | RTLD_LOCAL);
  if (h == NULL) h = open_first(names, tried, sizeof(tried));
  if (h == NULL) {
    state = -1;
    return ga_err_fmt(e, GA_LOAD_ERROR, "Could not load \"libnvrtc.so\" (tried: %s): %s",
                      tried, dlerror());
  }
#define X(n)                                                                        \
  ga_rtc.p_##n = (__typeof__(&n))dlsym(h, GA_STR(n));                               \
  if (ga_rtc.p_##n == NULL) {                                                       \
    state = -1;                                                                     \
    return ga_err_fmt(e, GA_LOAD_ERROR, "libnvrtc.so lacks symbol %s", GA_STR(n));  \
  }
  GA_NVRTC_FUNCS(X)
#undef X
  state = 1;
  return GA_NO_ERROR;
}
