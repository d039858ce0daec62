// Run-time compilation of generated CUDA source for sm_100a and launching of the result.
//
// Stands where the reference's RTC::CudaRTCWrapper does (cavs/backend/cudaRTC_wrapper.h:16-95: nvrtcCompileProgram
// to PTX for compute_52, cuModuleLoadDataEx, cuLaunchKernel).  Here the program is compiled straight to a cubin for
// sm_100a; NVRTC and the driver API are bound on first use (dlopen), so the host library loads -- and kernels can
// be compiled -- on machines without a GPU driver.
#ifndef CAVS_BACKEND_CUDARTC_WRAPPER_H_
#define CAVS_BACKEND_CUDARTC_WRAPPER_H_

#include <string>
#include <vector>

namespace RTC {

class CudaRTCWrapper {
 public:
  CudaRTCWrapper() = default;
  ~CudaRTCWrapper();
  CudaRTCWrapper(const CudaRTCWrapper&) = delete;
  CudaRTCWrapper& operator=(const CudaRTCWrapper&) = delete;

  // Compiles `source` (which must define extern "C" __global__ `kernel_name`).  Fatal with the compiler log on error.
  void Compile(const std::string& kernel_name, const std::string& source);
  bool compiled() const { return !cubin_.empty(); }
  size_t cubin_bytes() const { return cubin_.size(); }
  // Loads the module into the current context on first use and launches a 1-D grid.  args: addresses of the
  // kernel's arguments, in order.
  void Launch(std::vector<void*>& args, unsigned int grid, unsigned int block, void* stream);

 private:
  std::string name_;
  std::vector<char> cubin_;
  void* module_ = nullptr;
  void* function_ = nullptr;
};

}  // namespace RTC
#endif
