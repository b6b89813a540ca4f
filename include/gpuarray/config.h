/* Build configuration shared by every public header of the B200 engine.
 *
 * Mirrors the role of the reference's src/gpuarray/config.h:1-46: it fixes the
 * API version number that clients compile against and the export attribute.
 * Only Linux/GCC-style visibility is provided; this library targets sm_100a
 * hosts exclusively. */
#ifndef GPUARRAY_CONFIG
#define GPUARRAY_CONFIG

#include <stddef.h>
#include <stdint.h>
#include <sys/types.h>

/* Same API level the reference announces (src/gpuarray/config.h:6). */
#define GPUARRAY_API_VERSION 2
/* Shared-library ABI the reference ships (src/CMakeLists.txt:111). */
#define GPUARRAY_ABI_VERSION 3

#if defined(__GNUC__) && __GNUC__ >= 4
#define GPUARRAY_PUBLIC __attribute__((visibility("default")))
#else
#define GPUARRAY_PUBLIC
#endif

#endif /* GPUARRAY_CONFIG */
