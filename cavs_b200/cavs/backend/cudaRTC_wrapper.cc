#include "cavs/backend/cudaRTC_wrapper.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdlib>
#include <mutex>

#include "cavs/util/logging.h"

namespace RTC {
namespace {

// The slices of NVRTC and of the driver API used here, bound at run time.
struct Nvrtc {
  int (*CreateProgram)(void**, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  int (*CompileProgram)(void*, int, const char* const*) = nullptr;
  int (*GetCUBINSize)(void*, size_t*) = nullptr;
  int (*GetCUBIN)(void*, char*) = nullptr;
  int (*GetProgramLogSize)(void*, size_t*) = nullptr;
  int (*GetProgramLog)(void*, char*) = nullptr;
  int (*DestroyProgram)(void**) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  std::string why;
};
struct Driver {
  int (*ModuleLoadData)(void**, const void*) = nullptr;
  int (*ModuleGetFunction)(void**, void*, const char*) = nullptr;
  int (*ModuleUnload)(void*) = nullptr;
  int (*LaunchKernel)(void*, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, void*, void**, void**) = nullptr;
  int (*GetErrorString)(int, const char**) = nullptr;
  std::string why;
};

void* OpenFirst(std::initializer_list<std::string> names, std::string* why) {
  for (const auto& n : names) {
    if (void* h = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL)) return h;
  }
  *why = std::string("could not load ") + *names.begin() + ": " + dlerror();
  return nullptr;
}
template <typename F>
void Bind(void* h, const char* name, F* fn, std::string* why) {
  *fn = reinterpret_cast<F>(dlsym(h, name));
  if (*fn == nullptr && why->empty()) *why = std::string("missing symbol ") + name;
}

Nvrtc& GetNvrtc() {
  static Nvrtc api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* home = std::getenv("CUDA_HOME");
    const std::string root = home ? home : "/usr/local/cuda";
    void* h = OpenFirst({"libnvrtc.so.12", "libnvrtc.so", root + "/lib64/libnvrtc.so.12", root + "/lib64/libnvrtc.so"}, &api.why);
    if (!h) return;
    Bind(h, "nvrtcCreateProgram", &api.CreateProgram, &api.why);
    Bind(h, "nvrtcCompileProgram", &api.CompileProgram, &api.why);
    Bind(h, "nvrtcGetCUBINSize", &api.GetCUBINSize, &api.why);
    Bind(h, "nvrtcGetCUBIN", &api.GetCUBIN, &api.why);
    Bind(h, "nvrtcGetProgramLogSize", &api.GetProgramLogSize, &api.why);
    Bind(h, "nvrtcGetProgramLog", &api.GetProgramLog, &api.why);
    Bind(h, "nvrtcDestroyProgram", &api.DestroyProgram, &api.why);
    Bind(h, "nvrtcGetErrorString", &api.GetErrorString, &api.why);
  });
  return api;
}
Driver& GetDriver() {
  static Driver api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = OpenFirst({"libcuda.so.1", "libcuda.so"}, &api.why);
    if (!h) return;
    Bind(h, "cuModuleLoadData", &api.ModuleLoadData, &api.why);
    Bind(h, "cuModuleGetFunction", &api.ModuleGetFunction, &api.why);
    Bind(h, "cuModuleUnload", &api.ModuleUnload, &api.why);
    Bind(h, "cuLaunchKernel", &api.LaunchKernel, &api.why);
    Bind(h, "cuGetErrorString", &api.GetErrorString, &api.why);
  });
  return api;
}
std::string DriverError(int rc) {
  const char* s = nullptr;
  if (GetDriver().GetErrorString) GetDriver().GetErrorString(rc, &s);
  return std::string(s ? s : "CUDA driver error") + " (" + std::to_string(rc) + ")";
}

}  // namespace

CudaRTCWrapper::~CudaRTCWrapper() {
  if (module_ && GetDriver().ModuleUnload) GetDriver().ModuleUnload(module_);
}

void CudaRTCWrapper::Compile(const std::string& kernel_name, const std::string& source) {
  Nvrtc& rtc = GetNvrtc();
  CHECK(rtc.why.empty()) << "run-time compilation is unavailable: " << rtc.why;
  name_ = kernel_name;
  void* prog = nullptr;
  int rc = rtc.CreateProgram(&prog, source.c_str(), (kernel_name + ".cu").c_str(), 0, nullptr, nullptr);
  CHECK(rc == 0) << "nvrtcCreateProgram: " << rtc.GetErrorString(rc);
  // --fmad=false as the reference's generated kernels (cavs/backend/cudaRTC_wrapper.h:49): the fused groups must
  // round like the separate elementwise operators they replace.
  const char* opts[] = {"--gpu-architecture=sm_100a", "--fmad=false", "--std=c++17"};
  rc = rtc.CompileProgram(prog, 3, opts);
  if (rc != 0) {
    size_t n = 0;
    rtc.GetProgramLogSize(prog, &n);
    std::string log(n, '\0');
    if (n) rtc.GetProgramLog(prog, &log[0]);
    LOG(FATAL) << "run-time compilation of " << kernel_name << " failed: " << rtc.GetErrorString(rc) << "\n" << log << "\n" << source;
  }
  size_t bytes = 0;
  rc = rtc.GetCUBINSize(prog, &bytes);
  CHECK(rc == 0 && bytes > 0) << "nvrtcGetCUBINSize: " << rtc.GetErrorString(rc);
  cubin_.resize(bytes);
  rc = rtc.GetCUBIN(prog, cubin_.data());
  CHECK(rc == 0) << "nvrtcGetCUBIN: " << rtc.GetErrorString(rc);
  rtc.DestroyProgram(&prog);
}

void CudaRTCWrapper::Launch(std::vector<void*>& args, unsigned int grid, unsigned int block, void* stream) {
  CHECK(compiled()) << "kernel " << name_ << " was never compiled";
  Driver& drv = GetDriver();
  CHECK(drv.why.empty()) << "the CUDA driver is unavailable: " << drv.why;
  if (function_ == nullptr) {
    CHECK(cudaFree(nullptr) == cudaSuccess) << "no CUDA context";   // makes the runtime's primary context current
    int rc = drv.ModuleLoadData(&module_, cubin_.data());
    CHECK(rc == 0) << "cuModuleLoadData(" << name_ << "): " << DriverError(rc);
    rc = drv.ModuleGetFunction(&function_, module_, name_.c_str());
    CHECK(rc == 0) << "cuModuleGetFunction(" << name_ << "): " << DriverError(rc);
  }
  const int rc = drv.LaunchKernel(function_, grid, 1, 1, block, 1, 1, 0, stream, args.data(), nullptr);
  CHECK(rc == 0) << "cuLaunchKernel(" << name_ << "): " << DriverError(rc);
}

}  // namespace RTC
