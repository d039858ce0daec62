// Parameter update, bf16 shadow copies and column reductions.
//
// SGD replaces SGDKernel (cavs/backend/op_impl_sgd.cu:15-47): w <- w - lr * g.
// Adagrad has no counterpart in the reference (it registers only SGD); it is defined as
// acc += g^2; w <- w - lr * g / (sqrt(acc) + eps).
// ColumnSum replaces the serial-per-thread column reduction the reference uses for bias
// gradients (cavs/backend/op_impl_elementwise.cuh:31-37) with a two-stage, fixed-order
// reduction.
#include <cuda_bf16.h>

#include <cstdint>

#include "abi_common.h"
#include "kernels/cell.h"
#include "kernels/launch.h"

namespace cavs_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kColChunks = 64;   // row chunks of the first column-sum stage

__global__ void __launch_bounds__(kThreads) SgdKernel(float* __restrict__ w, const float* __restrict__ g, size_t n, float lr) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  const size_t n4 = n / 4;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n4; i += stride) {
    float4 wv = reinterpret_cast<float4*>(w)[i];
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    wv.x -= lr * gv.x; wv.y -= lr * gv.y; wv.z -= lr * gv.z; wv.w -= lr * gv.w;
    reinterpret_cast<float4*>(w)[i] = wv;
  }
  for (size_t i = n4 * 4 + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) w[i] -= lr * g[i];
}

__global__ void __launch_bounds__(kThreads)
AdagradKernel(float* __restrict__ w, float* __restrict__ acc, const float* __restrict__ g, size_t n, float lr, float eps) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  const size_t n4 = n / 4;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n4; i += stride) {
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    // Zero gradient: neither the accumulator nor the weight changes (w - lr * 0 / (sqrt(acc) + eps) == w), so the
    // rows of an embedding table that the batch did not touch cost one read instead of three reads and two writes.
    if (gv.x == 0.0f && gv.y == 0.0f && gv.z == 0.0f && gv.w == 0.0f) continue;
    float4 wv = reinterpret_cast<float4*>(w)[i];
    float4 av = reinterpret_cast<float4*>(acc)[i];
    av.x += gv.x * gv.x; av.y += gv.y * gv.y; av.z += gv.z * gv.z; av.w += gv.w * gv.w;
    wv.x -= lr * gv.x / (sqrtf(av.x) + eps); wv.y -= lr * gv.y / (sqrtf(av.y) + eps);
    wv.z -= lr * gv.z / (sqrtf(av.z) + eps); wv.w -= lr * gv.w / (sqrtf(av.w) + eps);
    reinterpret_cast<float4*>(acc)[i] = av;
    reinterpret_cast<float4*>(w)[i] = wv;
  }
  for (size_t i = n4 * 4 + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    const float a = acc[i] + g[i] * g[i];
    acc[i] = a;
    w[i] -= lr * g[i] / (sqrtf(a) + eps);
  }
}

// The update of listed rows of a table: w[rows[i], :] takes gradient row g[i, :] (SGD, or Adagrad when acc is given),
// the same arithmetic per element as the dense kernels above.  width is a multiple of 4.
template <bool kAdagrad>
__global__ void __launch_bounds__(kThreads)
UpdateRowsKernel(float* __restrict__ w, float* __restrict__ acc, const float* __restrict__ g, const int32_t* __restrict__ rows,
                 int n_rows, int width, float lr, float eps) {
  const int w4 = width / 4;
  const size_t total = static_cast<size_t>(n_rows) * w4;
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
    const int r = static_cast<int>(i / w4), c = static_cast<int>(i % w4);
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    if (kAdagrad && gv.x == 0.0f && gv.y == 0.0f && gv.z == 0.0f && gv.w == 0.0f) continue;
    const size_t at = static_cast<size_t>(__ldg(rows + r)) * w4 + c;
    float4 wv = reinterpret_cast<float4*>(w)[at];
    if (kAdagrad) {
      float4 av = reinterpret_cast<float4*>(acc)[at];
      av.x += gv.x * gv.x; av.y += gv.y * gv.y; av.z += gv.z * gv.z; av.w += gv.w * gv.w;
      wv.x -= lr * gv.x / (sqrtf(av.x) + eps); wv.y -= lr * gv.y / (sqrtf(av.y) + eps);
      wv.z -= lr * gv.z / (sqrtf(av.z) + eps); wv.w -= lr * gv.w / (sqrtf(av.w) + eps);
      reinterpret_cast<float4*>(acc)[at] = av;
    } else {
      wv.x -= lr * gv.x; wv.y -= lr * gv.y; wv.z -= lr * gv.z; wv.w -= lr * gv.w;
    }
    reinterpret_cast<float4*>(w)[at] = wv;
  }
}

__global__ void __launch_bounds__(kThreads) CastBf16Kernel(__nv_bfloat16* __restrict__ dst, const float* __restrict__ src, size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
}

__global__ void __launch_bounds__(kThreads)
CastRowsBf16Kernel(__nv_bfloat16* __restrict__ dst, const float* __restrict__ src, long long rows, int cols, long long src_pitch) {
  const long long total = rows * cols;
  const long long stride = static_cast<long long>(gridDim.x) * kThreads;
  for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride)
    dst[i] = __float2bfloat16_rn(src[(i / cols) * src_pitch + (i % cols)]);
}

// Stage 1: CTA (x = column tile of kThreads, y = row chunk) sums its rows in order.
template <typename T>
__global__ void __launch_bounds__(kThreads)
ColumnSumStage1(float* __restrict__ partial, const T* __restrict__ x, long long pitch, int rows, int cols, int rows_per_chunk) {
  const int col = blockIdx.x * kThreads + threadIdx.x;
  if (col >= cols) return;
  const int r0 = blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
  float acc = 0.0f;
  for (int r = r0; r < r1; ++r) acc += static_cast<float>(x[static_cast<long long>(r) * pitch + col]);
  partial[static_cast<size_t>(blockIdx.y) * cols + col] = acc;
}
// Stage 2 optionally permutes column blocks of width `block`: source block b lands in
// destination block map[b] (used to turn gate order i,o,u,f into bias order i,f,u,o).
__global__ void __launch_bounds__(kThreads)
ColumnSumStage2(float* __restrict__ out, const float* __restrict__ partial, int cols, int chunks, int block, int4 map) {
  const int col = blockIdx.x * kThreads + threadIdx.x;
  if (col >= cols) return;
  float acc = 0.0f;
  for (int c = 0; c < chunks; ++c) acc += partial[static_cast<size_t>(c) * cols + col];
  int dst = col;
  if (block > 0) {
    const int b = col / block;
    const int nb = b == 0 ? map.x : b == 1 ? map.y : b == 2 ? map.z : map.w;
    dst = nb * block + col % block;
  }
  out[dst] = acc;
}

}  // namespace

int LaunchSgd(float* w, const float* g, size_t n, float lr, cudaStream_t st) {
  if (n == 0) return CAVS_OK;
  CAVS_REQUIRE(w && g, CAVS_ERR_BAD_ARG, "sgd: null pointer");
  CAVS_REQUIRE(((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(g)) & 15u) == 0, CAVS_ERR_BAD_ARG, "sgd: buffers must be 16-byte aligned");
  SgdKernel<<<GridForElems(n / 4 + 1, kThreads), kThreads, 0, st>>>(w, g, n, lr);
  CAVS_LAUNCH_CHECK("sgd");
  return CAVS_OK;
}

int LaunchUpdateRows(float* w, float* acc, const float* g, const int32_t* rows, int n_rows, int width, float lr, float eps,
                     cudaStream_t st) {
  if (n_rows == 0 || width == 0) return CAVS_OK;
  CAVS_REQUIRE(w && g && rows && n_rows > 0, CAVS_ERR_BAD_ARG, "update_rows: null pointer");
  CAVS_REQUIRE(width % 4 == 0 && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(acc)) & 15u) == 0,
               CAVS_ERR_BAD_ARG, "update_rows: rows must be 16-byte aligned and a multiple of 4 floats wide");
  const int grid = GridForElems(static_cast<size_t>(n_rows) * (width / 4), kThreads);
  if (acc) UpdateRowsKernel<true><<<grid, kThreads, 0, st>>>(w, acc, g, rows, n_rows, width, lr, eps);
  else UpdateRowsKernel<false><<<grid, kThreads, 0, st>>>(w, nullptr, g, rows, n_rows, width, lr, eps);
  CAVS_LAUNCH_CHECK("update_rows");
  return CAVS_OK;
}

int LaunchAdagrad(float* w, float* acc, const float* g, size_t n, float lr, float eps, cudaStream_t st) {
  if (n == 0) return CAVS_OK;
  CAVS_REQUIRE(w && acc && g, CAVS_ERR_BAD_ARG, "adagrad: null pointer");
  CAVS_REQUIRE(((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(acc)) & 15u) == 0,
               CAVS_ERR_BAD_ARG, "adagrad: buffers must be 16-byte aligned");
  AdagradKernel<<<GridForElems(n / 4 + 1, kThreads), kThreads, 0, st>>>(w, acc, g, n, lr, eps);
  CAVS_LAUNCH_CHECK("adagrad");
  return CAVS_OK;
}

int LaunchCastBf16(void* dst, const float* src, size_t n, cudaStream_t st) {
  if (n == 0) return CAVS_OK;
  CAVS_REQUIRE(dst && src, CAVS_ERR_BAD_ARG, "cast_bf16: null pointer");
  CastBf16Kernel<<<GridForElems(n, kThreads), kThreads, 0, st>>>(static_cast<__nv_bfloat16*>(dst), src, n);
  CAVS_LAUNCH_CHECK("cast_bf16");
  return CAVS_OK;
}

int LaunchCastRowsBf16(void* dst, const float* src, long long rows, int cols, long long src_pitch, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return CAVS_OK;
  CAVS_REQUIRE(dst && src, CAVS_ERR_BAD_ARG, "cast_rows_bf16: null pointer");
  CastRowsBf16Kernel<<<GridForElems(static_cast<size_t>(rows) * cols, kThreads), kThreads, 0, st>>>(static_cast<__nv_bfloat16*>(dst), src, rows, cols, src_pitch);
  CAVS_LAUNCH_CHECK("cast_rows_bf16");
  return CAVS_OK;
}

size_t ColumnSumScratchBytes(int cols) { return static_cast<size_t>(kColChunks) * cols * sizeof(float); }

int LaunchColumnSum(float* out, const void* x, bool bf16, long long pitch, int rows, int cols, float* scratch, cudaStream_t st,
                    int block, int m0, int m1, int m2, int m3) {
  CAVS_REQUIRE(rows >= 0 && cols > 0, CAVS_ERR_BAD_ARG, "column_sum: bad shape");
  CAVS_REQUIRE(out && scratch && (x || rows == 0), CAVS_ERR_BAD_ARG, "column_sum: null pointer");
  const int rows_per_chunk = std::max(1, (rows + kColChunks - 1) / kColChunks);
  const int chunks = std::max(1, (rows + rows_per_chunk - 1) / rows_per_chunk);
  dim3 grid((cols + kThreads - 1) / kThreads, chunks);
  if (bf16) ColumnSumStage1<__nv_bfloat16><<<grid, kThreads, 0, st>>>(scratch, static_cast<const __nv_bfloat16*>(x), pitch, rows, cols, rows_per_chunk);
  else ColumnSumStage1<float><<<grid, kThreads, 0, st>>>(scratch, static_cast<const float*>(x), pitch, rows, cols, rows_per_chunk);
  CAVS_LAUNCH_CHECK("column_sum stage 1");
  CAVS_REQUIRE(block == 0 || cols == 4 * block, CAVS_ERR_BAD_ARG, "column_sum: block permutation needs cols == 4 * block");
  ColumnSumStage2<<<(cols + kThreads - 1) / kThreads, kThreads, 0, st>>>(out, scratch, cols, chunks, block, make_int4(m0, m1, m2, m3));
  CAVS_LAUNCH_CHECK("column_sum stage 2");
  return CAVS_OK;
}


namespace {
constexpr int kSumParts = 1024;
// out[blockIdx.x] = sum of |x| over the CTA's strided share, folded in a fixed tree: deterministic.
__global__ void __launch_bounds__(kThreads) AbsSumStage1(float* __restrict__ partial, const float* __restrict__ x, size_t n) {
  __shared__ float sm[kThreads];
  float acc = 0.0f;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * kThreads)
    acc += fabsf(x[i]);
  sm[threadIdx.x] = acc;
  __syncthreads();
  for (int o = kThreads / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) sm[threadIdx.x] += sm[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[blockIdx.x] = sm[0];
}
__global__ void AbsSumStage2(float* __restrict__ out, const float* __restrict__ partial, int parts) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    float acc = 0.0f;
    for (int i = 0; i < parts; ++i) acc += partial[i];
    *out = acc;
  }
}
__global__ void __launch_bounds__(kThreads) FillKernel(float* __restrict__ x, size_t n, float v) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * kThreads) x[i] = v;
}
__global__ void __launch_bounds__(kThreads) AxpyKernel(float* __restrict__ y, const float* __restrict__ x, size_t n, float a) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * kThreads)
    y[i] = y[i] + a * x[i];
}
// norms[b] = ||g[off_b : off_b + len_b]||_2, one CTA per block, fixed reduction order.
__global__ void __launch_bounds__(kThreads) BlockNormKernel(float* __restrict__ norms, const float* __restrict__ g,
                                                           const unsigned long long* __restrict__ offs, int n_blocks) {
  __shared__ float sm[kThreads];
  const int b = blockIdx.x;
  const size_t lo = offs[b], hi = offs[b + 1];
  float acc = 0.0f;
  for (size_t i = lo + threadIdx.x; i < hi; i += kThreads) acc += g[i] * g[i];
  sm[threadIdx.x] = acc;
  __syncthreads();
  for (int o = kThreads / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) sm[threadIdx.x] += sm[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) norms[b] = sqrtf(sm[0]);
}
// g *= clip / max(sum of the block norms, clip)
__global__ void __launch_bounds__(kThreads) ClipScaleKernel(float* __restrict__ g, size_t n, const float* __restrict__ norms, int n_blocks,
                                                           float clip) {
  float sum = 0.0f;
  for (int b = 0; b < n_blocks; ++b) sum += norms[b];
  const float scale = clip / fmaxf(sum, clip);
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * kThreads) g[i] *= scale;
}
}  // namespace

}  // namespace cavs_b200

using namespace cavs_b200;

extern "C" int cavs_abs_sum(float* out, const float* x, size_t count, float* scratch, void* stream) {
  CAVS_REQUIRE(out && scratch && (x || count == 0), CAVS_ERR_BAD_ARG, "abs_sum: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int parts = static_cast<int>(std::min<size_t>(kSumParts, std::max<size_t>(1, (count + kThreads - 1) / kThreads)));
  AbsSumStage1<<<parts, kThreads, 0, st>>>(scratch, x, count);
  CAVS_LAUNCH_CHECK("abs_sum stage 1");
  AbsSumStage2<<<1, 32, 0, st>>>(out, scratch, parts);
  CAVS_LAUNCH_CHECK("abs_sum stage 2");
  return CAVS_OK;
}

extern "C" int cavs_fill(float* x, size_t count, float value, void* stream) {
  if (count == 0) return CAVS_OK;
  CAVS_REQUIRE(x, CAVS_ERR_BAD_ARG, "fill: null pointer");
  FillKernel<<<GridForElems(count, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, count, value);
  CAVS_LAUNCH_CHECK("fill");
  return CAVS_OK;
}

extern "C" int cavs_axpy(float* y, const float* x, size_t count, float alpha, void* stream) {
  if (count == 0) return CAVS_OK;
  CAVS_REQUIRE(x && y, CAVS_ERR_BAD_ARG, "axpy: null pointer");
  AxpyKernel<<<GridForElems(count, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(y, x, count, alpha);
  CAVS_LAUNCH_CHECK("axpy");
  return CAVS_OK;
}

extern "C" int cavs_clip_gradients(float* g, const unsigned long long* block_offsets, int n_blocks, float clip, float* scratch,
                                   void* stream) {
  CAVS_REQUIRE(g && block_offsets && scratch && n_blocks >= 1 && n_blocks <= 256, CAVS_ERR_BAD_ARG, "clip_gradients: bad argument");
  CAVS_REQUIRE(clip > 0.0f, CAVS_ERR_BAD_ARG, "clip_gradients: the threshold must be positive");
  CAVS_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 7u) == 0, CAVS_ERR_BAD_ARG, "clip_gradients: scratch must be 8-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // block_offsets is a host array; it travels as the head of the scratch buffer
  unsigned long long* d_offs = reinterpret_cast<unsigned long long*>(scratch);
  float* norms = scratch + 2 * (n_blocks + 1);
  CAVS_CUDA(cudaMemcpyAsync(d_offs, block_offsets, sizeof(unsigned long long) * (n_blocks + 1), cudaMemcpyHostToDevice, st));
  BlockNormKernel<<<n_blocks, kThreads, 0, st>>>(norms, g, d_offs, n_blocks);
  CAVS_LAUNCH_CHECK("clip_gradients norms");
  const size_t n = block_offsets[n_blocks];
  ClipScaleKernel<<<GridForElems(n, kThreads), kThreads, 0, st>>>(g, n, norms, n_blocks, clip);
  CAVS_LAUNCH_CHECK("clip_gradients scale");
  return CAVS_OK;
}

extern "C" size_t cavs_clip_gradients_scratch_bytes(int n_blocks) {
  return sizeof(float) * (2 * (static_cast<size_t>(n_blocks) + 1) + n_blocks + 8);
}
