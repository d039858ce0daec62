// The fused child-sum Tree-LSTM cell in operator form: every input is a dense level-local tensor, as the
// reference's op-by-op dataflow produces them (Gather outputs for the children's h|c, MatMul outputs for the
// three products), so one operator replaces the ~20 elementwise / slice / concat launches of a level in
// apps/paper/tree-lstm-cavs.cc:138-171 (forward) and the ~40 of its gradient.  Same arithmetic, in the same
// order, as the indexed kernels the engine uses (kernels/cell.cu); fp32 only, like the reference's ops.
// HBM-bound; one thread per 4 (or 1) hidden units of a row, grid capped at SMs x resident CTAs.
#include <cstdint>

#include "abi_common.h"
#include "kernels/launch.h"

namespace cavs_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxSlotsDense = 4;

struct Ptrs { const float* p[kMaxSlotsDense]; };
struct MutPtrs { float* p[kMaxSlotsDense]; };

__device__ __forceinline__ float Sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

template <int K>
__global__ void __launch_bounds__(kThreads)
CellDenseFwd(float* __restrict__ hc, float* __restrict__ gates, const float* __restrict__ A, const float* __restrict__ P,
             Ptrs Q, Ptrs child_hc, const float* __restrict__ bias, int rows, int H) {
  const long long total = static_cast<long long>(rows) * H;
  const long long stride = static_cast<long long>(gridDim.x) * kThreads;
  const int G = (3 + K) * H;
  for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
    const int b = static_cast<int>(i / H), j = static_cast<int>(i % H);
    const float* a = A + static_cast<size_t>(b) * 4 * H + j;
    const float* p = P + static_cast<size_t>(b) * 3 * H + j;
    // add order (xW + hU) + b; bias blocks i,f,u,o; W columns i,o,u,f (tree-lstm-cavs.cc:120-123,143-148,160-165)
    const float gi = Sigmoid((a[0] + p[0]) + bias[j]);
    const float go = Sigmoid((a[H] + p[H]) + bias[3 * H + j]);
    const float gu = tanhf((a[2 * H] + p[2 * H]) + bias[2 * H + j]);
    float cc = gi * gu;
    float* g = gates + static_cast<size_t>(b) * G + j;
#pragma unroll
    for (int c = 0; c < K; ++c) {
      const float q = Q.p[c] ? Q.p[c][static_cast<size_t>(b) * H + j] : 0.0f;
      const float cch = child_hc.p[c] ? child_hc.p[c][static_cast<size_t>(b) * 2 * H + H + j] : 0.0f;
      const float gf = Sigmoid((a[3 * H] + q) + bias[H + j]);
      cc = cc + gf * cch;
      g[(3 + c) * H] = gf;
    }
    g[0] = gi; g[H] = go; g[2 * H] = gu;
    hc[static_cast<size_t>(b) * 2 * H + j] = go * tanhf(cc);
    hc[static_cast<size_t>(b) * 2 * H + H + j] = cc;
  }
}

template <int K>
__global__ void __launch_bounds__(kThreads)
CellDenseBwd(float* __restrict__ dA, MutPtrs ZF, MutPtrs d_child_c, const float* __restrict__ d_hc, const float* __restrict__ dOut,
             const float* __restrict__ gates, const float* __restrict__ hc, Ptrs child_hc, int rows, int H) {
  const long long total = static_cast<long long>(rows) * H;
  const long long stride = static_cast<long long>(gridDim.x) * kThreads;
  const int G = (3 + K) * H;
  for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
    const int b = static_cast<int>(i / H), j = static_cast<int>(i % H);
    const float mh = d_hc ? d_hc[static_cast<size_t>(b) * 2 * H + j] : 0.0f;
    const float mc = d_hc ? d_hc[static_cast<size_t>(b) * 2 * H + H + j] : 0.0f;
    const float dh = (dOut ? dOut[static_cast<size_t>(b) * H + j] : 0.0f) + mh;
    const float* g = gates + static_cast<size_t>(b) * G + j;
    const float gi = g[0], go = g[H], gu = g[2 * H];
    const float th = tanhf(hc[static_cast<size_t>(b) * 2 * H + H + j]);
    const float d_o = dh * th;
    const float dc = mc + (dh * go) * (1.0f - th * th);
    const float zi = (dc * gu) * gi * (1.0f - gi);
    const float zo = d_o * go * (1.0f - go);
    const float zu = (dc * gi) * (1.0f - gu * gu);
    float zfs = 0.0f;
#pragma unroll
    for (int c = 0; c < K; ++c) {
      const float gf = g[(3 + c) * H];
      const float cch = child_hc.p[c] ? child_hc.p[c][static_cast<size_t>(b) * 2 * H + H + j] : 0.0f;
      const float z = (dc * cch) * gf * (1.0f - gf);
      zfs += z;
      if (ZF.p[c]) ZF.p[c][static_cast<size_t>(b) * H + j] = z;
      if (d_child_c.p[c]) d_child_c.p[c][static_cast<size_t>(b) * H + j] = dc * gf;
    }
    float* d = dA + static_cast<size_t>(b) * 4 * H + j;
    d[0] = zi; d[H] = zo; d[2 * H] = zu; d[3 * H] = zfs;
  }
}

#define DENSE_K(K_, ...)                                   \
  switch (K_) {                                            \
    case 1: { constexpr int K = 1; __VA_ARGS__; break; }   \
    case 2: { constexpr int K = 2; __VA_ARGS__; break; }   \
    case 3: { constexpr int K = 3; __VA_ARGS__; break; }   \
    default: { constexpr int K = 4; __VA_ARGS__; break; }  \
  }

}  // namespace
}  // namespace cavs_b200

using namespace cavs_b200;

extern "C" int cavs_treelstm_cell_dense_fwd(float* hc, float* gates, const float* A, const float* P, const float* const* Q,
                                            const float* const* child_hc, const float* bias, int rows, int hidden, int n_slots,
                                            void* stream) {
  CAVS_REQUIRE(rows >= 0 && hidden > 0 && n_slots >= 1 && n_slots <= kMaxSlotsDense, CAVS_ERR_BAD_ARG,
               "treelstm_cell_dense_fwd: bad shape (child slots 1..4)");
  if (rows == 0) return CAVS_OK;
  CAVS_REQUIRE(hc && gates && A && P && Q && child_hc && bias, CAVS_ERR_BAD_ARG, "treelstm_cell_dense_fwd: null pointer");
  Ptrs q{}, ch{};
  for (int c = 0; c < n_slots; ++c) { q.p[c] = Q[c]; ch.p[c] = child_hc[c]; }
  const int grid = GridForElems(static_cast<size_t>(rows) * hidden, kThreads);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DENSE_K(n_slots, CellDenseFwd<K><<<grid, kThreads, 0, st>>>(hc, gates, A, P, q, ch, bias, rows, hidden));
  CAVS_LAUNCH_CHECK("treelstm_cell_dense_fwd");
  return CAVS_OK;
}

extern "C" int cavs_treelstm_cell_dense_bwd(float* dA, float* const* ZF, float* const* d_child_c, const float* d_hc,
                                            const float* dOut, const float* gates, const float* hc, const float* const* child_hc,
                                            int rows, int hidden, int n_slots, void* stream) {
  CAVS_REQUIRE(rows >= 0 && hidden > 0 && n_slots >= 1 && n_slots <= kMaxSlotsDense, CAVS_ERR_BAD_ARG,
               "treelstm_cell_dense_bwd: bad shape (child slots 1..4)");
  if (rows == 0) return CAVS_OK;
  CAVS_REQUIRE(dA && ZF && d_child_c && gates && hc && child_hc, CAVS_ERR_BAD_ARG, "treelstm_cell_dense_bwd: null pointer");
  MutPtrs zf{}, dcc{};
  Ptrs ch{};
  for (int c = 0; c < n_slots; ++c) { zf.p[c] = ZF[c]; dcc.p[c] = d_child_c[c]; ch.p[c] = child_hc[c]; }
  const int grid = GridForElems(static_cast<size_t>(rows) * hidden, kThreads);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DENSE_K(n_slots, CellDenseBwd<K><<<grid, kThreads, 0, st>>>(dA, zf, dcc, d_hc, dOut, gates, hc, ch, rows, hidden));
  CAVS_LAUNCH_CHECK("treelstm_cell_dense_bwd");
  return CAVS_OK;
}
