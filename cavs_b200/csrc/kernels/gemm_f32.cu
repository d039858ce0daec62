// fp32 GEMM on the CUDA cores (FFMA), used by the fp32 configurations whose results
// must stay within 1e-5 relative of the reference's cublasSgemm calls
// (cavs/backend/cublas_wrapper.cc:13-28): tcgen05 has no fp32-input MMA and TF32 keeps
// only 10 mantissa bits.  These configurations are small and latency-bound: a 64x64x16
// register-tiled kernel with element strides (any transpose without a copy) and a
// software-pipelined k loop; the sum over k runs in ascending order within a thread.
#include <cstdint>

#include "abi_common.h"
#include "kernels/gemm.h"
#include "kernels/launch.h"

#include <algorithm>

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
  // k split: CTA z multiplies the k range [z * k_per_split, ...) and stores its partial product into slab z of the scratch
  const int k_begin = g.k_per_split > 0 ? blockIdx.z * g.k_per_split : 0;
  const int k_end = g.k_per_split > 0 ? min(g.k, k_begin + g.k_per_split) : g.k;
  if (g.k_per_split > 0) { g.c = g.scratch + static_cast<size_t>(blockIdx.z) * g.m * g.n; g.ldc = g.n; g.accumulate = 0; }
  g.k = k_end;   // the tile loaders guard against k
  float acc[4][4] = {};
  TileRegs regs;
  LoadTile(g, m0, n0, k_begin, regs);
  StoreTile(g, sa[0], sb[0], regs);
  __syncthreads();
  int cur = 0;
  for (int k0 = k_begin; k0 < k_end; k0 += kTK) {
    const bool more = k0 + kTK < k_end;
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

// C[i,j] (+)= sum over splits, in split order
__global__ void __launch_bounds__(256) GemmF32Reduce(float* __restrict__ c, long long ldc, const float* __restrict__ part, int m, int n,
                                                     int splits, int accumulate) {
  const long long total = static_cast<long long>(m) * n;
  for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * 256) {
    float acc = 0.0f;
    for (int z = 0; z < splits; ++z) acc += part[z * total + i];
    float* dst = c + (i / n) * ldc + (i % n);
    *dst = accumulate ? *dst + acc : acc;
  }
}

}  // namespace

int GemmF32(const GemmF32Args& g_in, cudaStream_t stream) {
  GemmF32Args g = g_in;
  CAVS_REQUIRE(g.m >= 0 && g.n >= 0 && g.k >= 0, CAVS_ERR_BAD_ARG, "gemm_f32: negative dimension");
  if (g.m == 0 || g.n == 0) return CAVS_OK;
  CAVS_REQUIRE(g.a && g.b && g.c, CAVS_ERR_BAD_ARG, "gemm_f32: null pointer");
  dim3 grid((g.n + kTN - 1) / kTN, (g.m + kTM - 1) / kTM);
  // Few tiles and a long k loop: split k over enough CTAs to fill the machine once (at least 64 k per split).
  const long long tiles = static_cast<long long>(grid.x) * grid.y;
  int splits = 1;
  if (g.scratch != nullptr && tiles < SmCount() && g.k >= 256) {
    splits = static_cast<int>(std::min<long long>(std::min<long long>(16, g.k / 64), (2LL * SmCount()) / tiles));
    while (splits > 1 && static_cast<size_t>(splits) * g.m * g.n * sizeof(float) > g.scratch_bytes) --splits;
  }
  g.k_per_split = 0;
  if (splits > 1) {
    g.k_per_split = ((g.k + splits - 1) / splits + kTK - 1) / kTK * kTK;
    splits = (g.k + g.k_per_split - 1) / g.k_per_split;
    grid.z = splits;
  }
  GemmF32Kernel<<<grid, 256, 0, stream>>>(g);
  CAVS_LAUNCH_CHECK("gemm_f32");
  if (splits > 1) {
    GemmF32Reduce<<<GridForElems(static_cast<size_t>(g.m) * g.n, 256), 256, 0, stream>>>(g_in.c, g_in.ldc, g.scratch, g.m, g.n, splits,
                                                                                          g_in.accumulate ? 1 : 0);
    CAVS_LAUNCH_CHECK("gemm_f32 split reduce");
  }
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
