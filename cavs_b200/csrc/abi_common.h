// Shared by every translation unit behind the C ABI: status codes, the
// thread-local error message, and CUDA error capture.
#ifndef CAVS_B200_ABI_COMMON_H_
#define CAVS_B200_ABI_COMMON_H_

#include <string>

#include "cavs_b200.h"

namespace cavs_b200 {
// Records msg as the calling thread's last error and returns code.
int Fail(int code, const std::string& msg);
// Process-wide count of kernels this library has launched (see cavs_launch_count).
void CountLaunch();
}  // namespace cavs_b200

#define CAVS_REQUIRE(cond, code, msg) \
  do { if (!(cond)) return ::cavs_b200::Fail((code), (msg)); } while (0)

#ifdef __CUDACC__
#include <cuda_runtime.h>
#define CAVS_CUDA(call)                                                                                  \
  do {                                                                                                   \
    cudaError_t _e = (call);                                                                             \
    if (_e != cudaSuccess)                                                                               \
      return ::cavs_b200::Fail(CAVS_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(_e));       \
  } while (0)
#define CAVS_LAUNCH_CHECK(name)                                                                          \
  do {                                                                                                   \
    cudaError_t _e = cudaGetLastError();                                                                 \
    if (_e != cudaSuccess)                                                                               \
      return ::cavs_b200::Fail(CAVS_ERR_CUDA, std::string(name) + " launch: " + cudaGetErrorString(_e)); \
    ::cavs_b200::CountLaunch();                                                                          \
  } while (0)
#endif

#endif
