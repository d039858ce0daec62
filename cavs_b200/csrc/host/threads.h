// How many host threads one engine's per-batch work (level scheduling, table packing) may use.
#ifndef CAVS_B200_HOST_THREADS_H_
#define CAVS_B200_HOST_THREADS_H_

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <thread>

namespace cavs_b200 {

// CAVS_HOST_THREADS overrides.  Otherwise the machine's hardware threads are shared out among the GPUs it shows (one
// process per GPU is the expected use: eight ranks on one host must not each start a thread per core), up to `cap`.
inline int HostThreadBudget(int cap) {
  if (const char* env = std::getenv("CAVS_HOST_THREADS")) return std::max(1, std::min(64, std::atoi(env)));
  const int hw = static_cast<int>(std::max(1u, std::thread::hardware_concurrency()));
  int gpus = 0;
  if (cudaGetDeviceCount(&gpus) != cudaSuccess || gpus < 1) {
    gpus = 1;
    (void)cudaGetLastError();   // no device is not an error of the caller's
  }
  return std::max(1, std::min(cap, hw / gpus));
}

}  // namespace cavs_b200
#endif
