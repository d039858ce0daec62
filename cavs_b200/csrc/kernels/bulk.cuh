// Asynchronous row staging for the HBM-bound kernels: untiled bulk copies (global -> shared memory)
// that complete on an mbarrier, so a CTA keeps several stages of rows in flight while it computes.
// Every wait is bounded; a wait that expires returns false and the caller raises a status word.
#ifndef CAVS_B200_KERNELS_BULK_CUH_
#define CAVS_B200_KERNELS_BULK_CUH_

#include <cstdint>

namespace cavs_b200 {
namespace bulk {

constexpr uint32_t kSpinLimit = 1u << 21;

__device__ __forceinline__ uint32_t SmemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void FenceMbarInit() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void MbarExpectTx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Polls a phase parity; sleeps between polls once the wait is clearly not a pipeline hiccup.
// false: the limit expired (about a third of a second).
__device__ __forceinline__ bool MbarWait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if (it > 4096) __nanosleep(128);
  }
  return false;
}
// dst (shared), src (global) 16-byte aligned, bytes a multiple of 16.  The copy reads this GPU's memory only.
__device__ __forceinline__ void Load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

}  // namespace bulk
}  // namespace cavs_b200
#endif
