// fp32 GEMM on the CUDA cores (FFMA), used by the fp32 configurations whose results
// must stay within 1e-5 relative of the reference's cublasSgemm calls
// (cavs/backend/cublas_wrapper.cc:13-28): tcgen05 has no fp32-input MMA and TF32 keeps
// only 10 mantissa bits.  These configurations are small and latency-bound: a 64x64x16
// register-tiled kernel with element strides (any transpose without a copy) and a
// software-pipelined k loop; the sum over k runs in ascending order within a thread.
#include <cstdint>

#include "abi_common.h"
#include "kernels/gemm.h"

namespace cavs_b200 {
namespace {

constexpr int kTM = 64, kTN = 64, kTK = 16;

// One k-step's share of the A and B tiles for this thread: 4 elements each (tiles are 64 x 16 and 16 x 64).
struct TileRegs { float a[4], b[4]; };

__device__ __forceinline__ void LoadTile(const GemmF32Args& g, int m0, int n0, int k0, TileRegs& r) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int idx = threadIdx.x + e * 256;
    // Walk the fastest-varying global dimension with consecutive threads.
    int ai, ak;
    if (g.a_cs == 1) { ak = idx & 15; ai = idx >> 4; } else { ai = idx & 63; ak = idx >> 6; }
    const int gi = m0 + ai, gk = k0 + ak;
    r.a[e] = (gi < g.m && gk < g.k) ? g.a[gi * g.a_rs + gk * g.a_cs] : 0.0f;
    int bk, bj;
    if (g.b_cs == 1) { bj = idx & 63; bk = idx >> 6; } else { bk = idx & 15; bj = idx >> 4; }
    const int gj = n0 + bj, gk2 = k0 + bk;
    r.b[e] = (gj < g.n && gk2 < g.k) ? g.b[gk2 * g.b_rs + gj * g.b_cs] : 0.0f;
  }
}
__device__ __forceinline__ void StoreTile(const GemmF32Args& g, float (*sa)[kTM + 4], float (*sb)[kTN + 4], const TileRegs& r) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int idx = threadIdx.x + e * 256;
    int ai, ak;
    if (g.a_cs == 1) { ak = idx & 15; ai = idx >> 4; } else { ai = idx & 63; ak = idx >> 6; }
    sa[ak][ai] = r.a[e];
    int bk, bj;
    if (g.b_cs == 1) { bj = idx & 63; bk = idx >> 6; } else { bk = idx & 15; bj = idx >> 4; }
    sb[bk][bj] = r.b[e];
  }
}

// The k loop is software-pipelined: the next step's operands travel from global memory to registers while the
// current step's tiles (in shared memory, double-buffered) are multiplied, so a step costs its arithmetic and one
// barrier instead of a global-memory round trip -- these GEMMs have few tiles and long k loops (a level of a few
// hundred rows against [H, 4H] weights), i.e. their duration is the k loop's latency.
__global__ void __launch_bounds__(256) GemmF32Kernel(GemmF32Args g) {
  __shared__ float sa[2][kTK][kTM + 4];
  __shared__ float sb[2][kTK][kTN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
  float acc[4][4] = {};
  TileRegs regs;
  LoadTile(g, m0, n0, 0, regs);
  StoreTile(g, sa[0], sb[0], regs);
  __syncthreads();
  int cur = 0;
  for (int k0 = 0; k0 < g.k; k0 += kTK) {
    const bool more = k0 + kTK < g.k;
    if (more) LoadTile(g, m0, n0, k0 + kTK, regs);
#pragma unroll
    for (int kk = 0; kk < kTK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[cur][kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[cur][kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (more) StoreTile(g, sa[cur ^ 1], sb[cur ^ 1], regs);   // the other buffer: last read before the previous barrier
    __syncthreads();
    cur ^= 1;
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
