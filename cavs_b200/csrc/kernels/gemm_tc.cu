// Host side of the tcgen05 GEMM: tensor-map encoding, tile-shape choice, optional
// deterministic split-K, and the C ABI entry point.
#include "kernels/gemm_tc.cuh"

#include <mutex>

#include "abi_common.h"
#include "kernels/gemm.h"
#include "kernels/launch.h"

namespace cavs_b200 {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver entry point; it is fetched through the runtime so
// the library carries no link-time dependency on libcuda.
EncodeFn GetEncodeFn(std::string* err) {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  static std::string once_err;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || sym == nullptr)
      once_err = std::string("cuTensorMapEncodeTiled unavailable: ") + cudaGetErrorString(e);
    else
      fn = reinterpret_cast<EncodeFn>(sym);
  });
  if (!fn) *err = once_err;
  return fn;
}

// 2-D bf16 tensor map over a row-major matrix [outer, inner] with row pitch ld elements,
// 128-byte swizzle, zero fill outside the extents.
int EncodeBf16(CUtensorMap* map, const void* base, long long inner, long long outer, long long ld, int box_inner,
               int box_outer) {
  std::string err;
  EncodeFn fn = GetEncodeFn(&err);
  if (!fn) return Fail(CAVS_ERR_CUDA, err);
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Fail(CAVS_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(r));
  return CAVS_OK;
}

__global__ void __launch_bounds__(256) SplitKReduce(float* __restrict__ c, long long ldc, const float* __restrict__ part,
                                                    int m, int n, int splits, int accumulate) {
  const long long total = static_cast<long long>(m) * n;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    float acc = 0.0f;
    for (int z = 0; z < splits; ++z) acc += part[z * total + i];   // fixed order: deterministic
    float* dst = c + (i / n) * ldc + (i % n);
    *dst = accumulate ? *dst + acc : acc;
  }
}

template <int kBN, int kAMajor, int kBMajor>
int Launch(const CUtensorMap& ma, const CUtensorMap& mb, const tc::Params& p, dim3 grid, cudaStream_t stream) {
  using S = tc::Smem<kBN>;
  auto kern = tc::GemmBf16Kernel<kBN, kAMajor, kBMajor>;
  static bool configured = false;   // per instantiation
  if (!configured) {
    CAVS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes));
    configured = true;
  }
  kern<<<grid, tc::kThreads, S::kBytes, stream>>>(ma, mb, p);
  CAVS_LAUNCH_CHECK("gemm_bf16");
  return CAVS_OK;
}

template <int kBN>
int Dispatch(int a_major, int b_major, const CUtensorMap& ma, const CUtensorMap& mb, const tc::Params& p, dim3 grid,
             cudaStream_t stream) {
  if (a_major == tc::kMajorK && b_major == tc::kMajorK) return Launch<kBN, 0, 0>(ma, mb, p, grid, stream);
  if (a_major == tc::kMajorK && b_major == tc::kMajorMN) return Launch<kBN, 0, 1>(ma, mb, p, grid, stream);
  if (a_major == tc::kMajorMN && b_major == tc::kMajorK) return Launch<kBN, 1, 0>(ma, mb, p, grid, stream);
  return Launch<kBN, 1, 1>(ma, mb, p, grid, stream);
}

bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

size_t GemmBf16ScratchBytes(int m, int n, int splits) {
  return splits > 1 ? static_cast<size_t>(splits) * m * n * sizeof(float) : 0;
}

int GemmBf16SplitsFor(int m, int n, int k) {
  // The kernel is persistent over (tile, split) work items; pick the smallest split count whose
  // work-item count fills whole waves of SMs noticeably better, keeping each split >= 32 K blocks.
  const int bn = n > 128 ? 256 : 128;
  const long long tiles = static_cast<long long>((m + tc::kBM - 1) / tc::kBM) * ((n + bn - 1) / bn);
  const int nkb = (k + tc::kBK - 1) / tc::kBK;
  const int sms = SmCount();
  auto fill = [&](long long items) { return static_cast<double>(items) / (((items + sms - 1) / sms) * sms); };
  int best = 1;
  double best_fill = fill(tiles);
  for (int s = 2; s <= 32 && nkb / s >= 32; ++s) {
    const double f = fill(tiles * s);
    if (f > best_fill + 0.04) { best = s; best_fill = f; }
    if (best_fill > 0.95) break;
  }
  return best;
}

int GemmBf16(const GemmBf16Args& g, cudaStream_t stream) {
  CAVS_REQUIRE(g.m >= 0 && g.n >= 0 && g.k >= 0, CAVS_ERR_BAD_ARG, "gemm_bf16: negative dimension");
  if (g.m == 0 || g.n == 0) return CAVS_OK;
  CAVS_REQUIRE(g.k > 0, CAVS_ERR_BAD_ARG, "gemm_bf16: k must be positive");
  CAVS_REQUIRE(g.a && g.b && g.c, CAVS_ERR_BAD_ARG, "gemm_bf16: null pointer");
  CAVS_REQUIRE(g.a_major == 0 || g.a_major == 1, CAVS_ERR_BAD_ARG, "gemm_bf16: a_major must be 0 (K) or 1 (MN)");
  CAVS_REQUIRE(g.b_major == 0 || g.b_major == 1, CAVS_ERR_BAD_ARG, "gemm_bf16: b_major must be 0 (K) or 1 (MN)");
  CAVS_REQUIRE(g.out_mode >= 0 && g.out_mode <= 2, CAVS_ERR_BAD_ARG, "gemm_bf16: bad out_mode");
  // TMA: 16-byte aligned bases and row pitches (8 bf16 elements).
  CAVS_REQUIRE(Aligned16(g.a) && Aligned16(g.b) && g.lda % 8 == 0 && g.ldb % 8 == 0, CAVS_ERR_BAD_ARG,
               "gemm_bf16: operands need 16-byte aligned bases and row pitches that are multiples of 8 elements");
  CAVS_REQUIRE(g.ldc >= g.n, CAVS_ERR_BAD_ARG, "gemm_bf16: ldc < n");
  const int splits = std::max(1, g.splits);
  CAVS_REQUIRE(splits == 1 || g.out_mode != tc::kStoreBf16, CAVS_ERR_BAD_ARG, "gemm_bf16: split-K needs an fp32 output");
  CAVS_REQUIRE(splits == 1 || (g.scratch && g.scratch_bytes >= GemmBf16ScratchBytes(g.m, g.n, splits)), CAVS_ERR_CAPACITY,
               "gemm_bf16: split-K scratch too small");

  const bool wide = g.n > 128;
  const int bn = wide ? 256 : 128;
  CUtensorMap ma, mb;
  int rc;
  if (g.a_major == tc::kMajorK) rc = EncodeBf16(&ma, g.a, g.k, g.m, g.lda, tc::kBK, tc::kBM);   // [m, k]
  else                          rc = EncodeBf16(&ma, g.a, g.m, g.k, g.lda, 64, tc::kBK);         // [k, m]
  if (rc) return rc;
  if (g.b_major == tc::kMajorK) rc = EncodeBf16(&mb, g.b, g.k, g.n, g.ldb, tc::kBK, bn);         // [n, k]
  else                          rc = EncodeBf16(&mb, g.b, g.n, g.k, g.ldb, 64, tc::kBK);         // [k, n]
  if (rc) return rc;

  const int nkb = (g.k + tc::kBK - 1) / tc::kBK;
  const int kb_per = (nkb + splits - 1) / splits;
  const int eff_splits = (nkb + kb_per - 1) / kb_per;
  tc::Params p{};
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.kb_per_split = kb_per;
  p.status = g.status;
  if (eff_splits > 1) {
    p.c = g.scratch; p.ldc = g.n; p.split_stride = static_cast<long long>(g.m) * g.n; p.out_mode = tc::kStoreF32;
  } else {
    p.c = g.c; p.ldc = g.ldc; p.split_stride = 0; p.out_mode = g.out_mode;
  }
  p.n_splits = eff_splits;
  const long long n_work = static_cast<long long>((g.n + bn - 1) / bn) * ((g.m + tc::kBM - 1) / tc::kBM) * eff_splits;
  dim3 grid(static_cast<unsigned>(std::min<long long>(n_work, SmCount())));
  rc = wide ? Dispatch<256>(g.a_major, g.b_major, ma, mb, p, grid, stream)
            : Dispatch<128>(g.a_major, g.b_major, ma, mb, p, grid, stream);
  if (rc) return rc;
  if (eff_splits > 1) {
    const size_t total = static_cast<size_t>(g.m) * g.n;
    SplitKReduce<<<GridForElems(total, 256), 256, 0, stream>>>(static_cast<float*>(g.c), g.ldc,
                                                               static_cast<const float*>(g.scratch), g.m, g.n, eff_splits,
                                                               g.out_mode == tc::kAccumF32 ? 1 : 0);
    CAVS_LAUNCH_CHECK("gemm_bf16 split-K reduce");
  }
  return CAVS_OK;
}

}  // namespace cavs_b200

extern "C" int cavs_gemm_bf16(void* c, long long ldc, int out_mode, const void* a, long long lda, int a_major,
                              const void* b, long long ldb, int b_major, int m, int n, int k, int splits, void* scratch,
                              size_t scratch_bytes, int* status, void* stream) {
  cavs_b200::GemmBf16Args g{};
  g.c = c; g.ldc = ldc; g.out_mode = out_mode;
  g.a = a; g.lda = lda; g.a_major = a_major;
  g.b = b; g.ldb = ldb; g.b_major = b_major;
  g.m = m; g.n = n; g.k = k;
  g.splits = splits; g.scratch = scratch; g.scratch_bytes = scratch_bytes; g.status = status;
  return cavs_b200::GemmBf16(g, static_cast<cudaStream_t>(stream));
}

extern "C" size_t cavs_gemm_bf16_scratch_bytes(int m, int n, int splits) {
  return cavs_b200::GemmBf16ScratchBytes(m, n, splits);
}
