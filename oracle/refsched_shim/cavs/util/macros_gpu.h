// Stand-in for cavs/util/macros_gpu.h: the scheduler's only CUDA call is one
// cudaMalloc of an index buffer, served from the host heap here.  TEST INFRASTRUCTURE.
#ifndef ORACLE_SHIM_CAVS_UTIL_MACROS_GPU_H_
#define ORACLE_SHIM_CAVS_UTIL_MACROS_GPU_H_
#include <cstddef>
#include <cstdlib>
#include "cavs/util/logging.h"
static inline int cudaMalloc(void** out, std::size_t bytes) { *out = std::malloc(bytes ? bytes : 1); return 0; }
#define checkCudaError(call) do { (void)(call); } while (0)
#endif
