// Grid sizing shared by the HBM-bound kernels: a launch never exceeds
// (SM count x resident CTAs per SM), and kernels stride over their work.
#ifndef CAVS_B200_KERNELS_LAUNCH_H_
#define CAVS_B200_KERNELS_LAUNCH_H_

#include <cuda_runtime.h>

#include <algorithm>
#include <cstddef>

namespace cavs_b200 {

// SMs of the current device (148 on B200); queried once per process.
inline int SmCount() {
  static int cached = 0;
  if (cached == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      cached = n;
    else
      cached = 148;
  }
  return cached;
}

// CTAs of `threads` threads that fit on one SM by thread count (2048 threads per SM).
inline int ResidentCtas(int threads) { return std::max(1, 2048 / threads); }

// Grid for a kernel where one warp handles one row and strides over rows.
inline int GridForWarps(long long n_rows, int warps_per_cta) {
  const long long want = (n_rows + warps_per_cta - 1) / warps_per_cta;
  const long long cap = static_cast<long long>(SmCount()) * ResidentCtas(warps_per_cta * 32);
  return static_cast<int>(std::max(1LL, std::min(want, cap)));
}

// Grid for a kernel where one thread handles one element (or vector) and strides.
inline int GridForElems(size_t n_elems, int threads) {
  const size_t want = (n_elems + threads - 1) / threads;
  const size_t cap = static_cast<size_t>(SmCount()) * ResidentCtas(threads);
  return static_cast<int>(std::max<size_t>(1, std::min(want, cap)));
}

}  // namespace cavs_b200
#endif
