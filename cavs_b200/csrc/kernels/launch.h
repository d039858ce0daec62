// Grid sizing shared by the HBM-bound kernels: a launch never exceeds
// (SM count x resident CTAs per SM), and kernels stride over their work.
#ifndef CAVS_B200_KERNELS_LAUNCH_H_
#define CAVS_B200_KERNELS_LAUNCH_H_

#include <cuda_runtime.h>

#include <algorithm>
#include <cstddef>
#include <cstdlib>

namespace cavs_b200 {

// Most devices one process is expected to drive; per-device caches are arrays of this size.
constexpr int kMaxDevices = 64;

// Ordinal of the calling thread's current device, clamped into the per-device cache arrays.
inline int CurrentDevice() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
  return dev < kMaxDevices ? dev : kMaxDevices - 1;
}

// SMs of the current device (148 on B200); queried once per device.
inline int SmCount() {
  static int cached[kMaxDevices] = {};
  const int dev = CurrentDevice();
  if (cached[dev] == 0) {
    int n = 0;
    cached[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
  }
  return cached[dev];
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

// Chained launches (programmatic dependent launch).  A level is a fixed sequence of short kernels, each
// consuming the previous one's output; launched this way, the next kernel's CTAs are placed on the SMs and
// run their prologue (barrier setup, TMEM allocation, descriptor prefetch) while the previous kernel is
// still draining, instead of after it.  Protocol for every kernel launched through LaunchChained:
//   ChainRelease()  first instruction: lets the following kernel start being placed once all CTAs of
//                   this one are resident;
//   ChainAcquire()  before the first access to global memory that another kernel writes or reads:
//                   returns when the preceding kernel has completed and its writes are visible.
// Both are no-ops for a kernel launched the ordinary way.  CAVS_PDL=0 in the environment turns the
// launch attribute off (ordinary stream order).
// An early release is only a gain when the following kernel places one CTA per SM (the GEMM) or is
// tiny: a wide grid-stride kernel whose CTAs are placed while the previous kernel still holds part of
// the SMs ends up unevenly spread, and its slowest SM sets its duration.  The caller says which case
// applies with ChainHint before the launch; kernels take the hint as an argument.
inline bool ChainedLaunchEnabled() {
  static int cached = -1;
  if (cached < 0) {
    const char* v = std::getenv("CAVS_PDL");
    cached = (v != nullptr && v[0] == '0') ? 0 : 1;
  }
  return cached == 1;
}

// Hint for the next launches issued by this host thread: may the kernel release its successor early?
inline thread_local int g_chain_early = 0;
inline void ChainHint(bool release_early) { g_chain_early = release_early ? 1 : 0; }
inline int ChainEarly() { return g_chain_early; }

template <typename... KArgs, typename... Args>
inline cudaError_t LaunchChained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = ChainedLaunchEnabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void ChainRelease(int early) {
  if (early) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void ChainAcquire() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

}  // namespace cavs_b200
#endif
