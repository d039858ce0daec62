// fp32 GEMM on the CUDA cores (FFMA), used by the fp32 configurations whose results
// must stay within 1e-5 relative of the reference's cublasSgemm calls
// (cavs/backend/cublas_wrapper.cc:13-28): tcgen05 has no fp32-input MMA and TF32 keeps
// only 10 mantissa bits.  These configurations are small and latency-bound, so a
// straightforward 64x64x16 register-tiled kernel with element strides (any transpose
// without a copy) is sufficient; the sum over k runs in ascending order within a thread.
#include <cstdint>

#include "abi_common.h"
#include "kernels/gemm.h"

namespace cavs_b200 {
namespace {

constexpr int kTM = 64, kTN = 64, kTK = 16;

__global__ void __launch_bounds__(256) GemmF32Kernel(GemmF32Args g) {
  __shared__ float sa[kTK][kTM + 4];
  __shared__ float sb[kTK][kTN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < g.k; k0 += kTK) {
    // A tile: 64 x 16, B tile: 16 x 64; 1024 elements each, 4 per thread.
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * 256;
      // Walk the fastest-varying global dimension with consecutive threads.
      int ai, ak;
      if (g.a_cs == 1) { ak = idx & 15; ai = idx >> 4; } else { ai = idx & 63; ak = idx >> 6; }
      const int gi = m0 + ai, gk = k0 + ak;
      sa[ak][ai] = (gi < g.m && gk < g.k) ? g.a[gi * g.a_rs + gk * g.a_cs] : 0.0f;
      int bk, bj;
      if (g.b_cs == 1) { bj = idx & 63; bk = idx >> 6; } else { bk = idx & 15; bj = idx >> 4; }
      const int gj = n0 + bj, gk2 = k0 + bk;
      sb[bk][bj] = (gj < g.n && gk2 < g.k) ? g.b[gk2 * g.b_rs + gj * g.b_cs] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gi = m0 + ty * 4 + i;
    if (gi >= g.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gj = n0 + tx * 4 + j;
      if (gj >= g.n) continue;
      float* dst = g.c + gi * g.ldc + gj;
      *dst = g.accumulate ? *dst + acc[i][j] : acc[i][j];
    }
  }
}

}  // namespace

int GemmF32(const GemmF32Args& g, cudaStream_t stream) {
  CAVS_REQUIRE(g.m >= 0 && g.n >= 0 && g.k >= 0, CAVS_ERR_BAD_ARG, "gemm_f32: negative dimension");
  if (g.m == 0 || g.n == 0) return CAVS_OK;
  CAVS_REQUIRE(g.a && g.b && g.c, CAVS_ERR_BAD_ARG, "gemm_f32: null pointer");
  dim3 grid((g.n + kTN - 1) / kTN, (g.m + kTM - 1) / kTM);
  GemmF32Kernel<<<grid, 256, 0, stream>>>(g);
  CAVS_LAUNCH_CHECK("gemm_f32");
  return CAVS_OK;
}

}  // namespace cavs_b200

extern "C" int cavs_gemm_f32(float* c, long long ldc, int accumulate, const float* a, long long a_row_stride,
                             long long a_col_stride, const float* b, long long b_row_stride, long long b_col_stride, int m,
                             int n, int k, void* stream) {
  cavs_b200::GemmF32Args g;
  g.c = c; g.ldc = ldc; g.accumulate = accumulate;
  g.a = a; g.a_rs = a_row_stride; g.a_cs = a_col_stride;
  g.b = b; g.b_rs = b_row_stride; g.b_cs = b_col_stride;
  g.m = m; g.n = n; g.k = k;
  return cavs_b200::GemmF32(g, static_cast<cudaStream_t>(stream));
}
