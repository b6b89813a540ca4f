/* Error records, the growable string used for code generation, and a hash.
 * Replaces the reference's src/util/error.c, src/util/strb.c and the use it
 * makes of xxhash for kernel-cache keys. */
#include "private.h"

static ga_error_rec global_err_storage;
ga_error_rec *ga_global_err = &global_err_storage;

const char *gpuarray_error_str(int err) {
  static const char *const text[] = {
      "No error",
      "Out of memory",
      "Value invalid or out of range",
      "Unknown device error",
      "Invalid value or operation",
      "Unsupported operation",
      NULL, /* GA_SYS_ERROR: strerror(errno) */
      "Could not execute helper program",
      "Device does not support operation",
      "Buffer is read-only",
      "Buffer is write-only",
      "Error in BLAS call",
      "Unaligned array",
      "Copy is needed but disallowed by parameters",
      "No devices are available",
      "Undeterminate error",
      "Error in collectives call",
      "Input size too large for operation",
      "Error loading library",
  };
  if (err == GA_SYS_ERROR) return strerror(errno);
  if (err < 0 || err >= (int)(sizeof(text) / sizeof(text[0]))) return "Unknown GA error";
  return text[err];
}

int ga_err_set(ga_error_rec *e, int code, const char *msg) {
  if (e == NULL) e = ga_global_err;
  e->code = code;
  snprintf(e->msg, GA_ERR_MSGLEN, "%s", msg);
  return code;
}

int ga_err_fmt(ga_error_rec *e, int code, const char *fmt, ...) {
  va_list ap;
  if (e == NULL) e = ga_global_err;
  e->code = code;
  va_start(ap, fmt);
  vsnprintf(e->msg, GA_ERR_MSGLEN, fmt, ap);
  va_end(ap);
  return code;
}

int ga_err_sys(ga_error_rec *e, const char *what) {
  return ga_err_fmt(e, GA_SYS_ERROR, "%s: %s", what, strerror(errno));
}

int ga_err_cuda(ga_error_rec *e, const char *call, CUresult r) {
  const char *name = NULL, *descr = NULL;
  if (ga_cu.p_cuGetErrorName != NULL) ga_cu.p_cuGetErrorName(r, &name);
  if (ga_cu.p_cuGetErrorString != NULL) ga_cu.p_cuGetErrorString(r, &descr);
  return ga_err_fmt(e, r == CUDA_ERROR_OUT_OF_MEMORY ? GA_MEMORY_ERROR : GA_IMPL_ERROR,
                    "%s: %s: %s", call, name ? name : "CUDA_ERROR", descr ? descr : "?");
}

/* ---------------------------------------------------------------- strings */

void ga_strb_init(ga_strb *sb) { memset(sb, 0, sizeof(*sb)); }

void ga_strb_free(ga_strb *sb) {
  free(sb->s);
  memset(sb, 0, sizeof(*sb));
}

static int strb_reserve(ga_strb *sb, size_t extra) {
  size_t need = sb->len + extra + 1, cap;
  char *p;
  if (sb->failed) return -1;
  if (need <= sb->cap) return 0;
  cap = sb->cap ? sb->cap : 1024;
  while (cap < need) cap *= 2;
  p = realloc(sb->s, cap);
  if (p == NULL) {
    sb->failed = 1;
    return -1;
  }
  sb->s = p;
  sb->cap = cap;
  return 0;
}

void ga_strb_putn(ga_strb *sb, const char *s, size_t n) {
  if (strb_reserve(sb, n) != 0) return;
  memcpy(sb->s + sb->len, s, n);
  sb->len += n;
  sb->s[sb->len] = '\0';
}

void ga_strb_puts(ga_strb *sb, const char *s) { ga_strb_putn(sb, s, strlen(s)); }

void ga_strb_printf(ga_strb *sb, const char *fmt, ...) {
  va_list ap;
  int n;
  va_start(ap, fmt);
  n = vsnprintf(NULL, 0, fmt, ap);
  va_end(ap);
  if (n < 0) {
    sb->failed = 1;
    return;
  }
  if (strb_reserve(sb, (size_t)n) != 0) return;
  va_start(ap, fmt);
  vsnprintf(sb->s + sb->len, (size_t)n + 1, fmt, ap);
  va_end(ap);
  sb->len += (size_t)n;
}

const char *ga_strb_cstr(ga_strb *sb) { return sb->s ? sb->s : ""; }

/* FNV-1a with a final avalanche; keys the kernel caches. */
uint64_t ga_hash64(const void *data, size_t len, uint64_t seed) {
  const unsigned char *p = (const unsigned char *)data;
  uint64_t h = 0xcbf29ce484222325ULL ^ seed;
  size_t i;
  for (i = 0; i < len; i++) {
    h ^= p[i];
    h *= 0x100000001b3ULL;
  }
  h ^= h >> 33;
  h *= 0xff51afd7ed558ccdULL;
  h ^= h >> 33;
  return h;
}
