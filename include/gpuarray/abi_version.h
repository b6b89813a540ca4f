/* The reference generates this file with CMake; clients only include it
 * through config.h. Kept so that `#include <gpuarray/abi_version.h>` works. */
#ifndef GPUARRAY_ABI_VERSION_H
#define GPUARRAY_ABI_VERSION_H
#include <gpuarray/config.h>
#endif
