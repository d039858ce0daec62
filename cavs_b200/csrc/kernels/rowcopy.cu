// Row gather / scatter / zero: the data movement behind the Gather, Scatter, Pull,
// Push and FunctionPopRet graph ops.
//
// Replaces the reference's one-CTA-per-row, 4-byte-per-thread copy kernels
// (cavs/backend/functor_batched_memcpy.cuh:19-75) and their per-launch pageable
// index upload (cavs/backend/op_impl_graphop.cu:68,80,149,241,308).  Here the index
// list already lives in device memory, rows move as 128-bit words, one warp streams a
// row with four independent loads in flight per lane, and the grid is a fixed
// multiple of the SM count that strides over rows, so a launch of any size fills the
// machine without tail quantisation.
//
// HBM-bound: algorithmic bytes per row = 2 * row_bytes + 4 (gather / scatter),
// row_bytes (zero).
#include <cstdint>

#include "abi_common.h"
#include "kernels/launch.h"

namespace cavs_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerCta = kThreads / 32;

enum class Dir { kGather, kScatter };

// One warp per row; lanes stride over 16-byte words, 4 words in flight per lane.
template <Dir kDir>
__global__ void __launch_bounds__(kThreads) RowCopyVec16(uint4* __restrict__ out, const uint4* __restrict__ inp,
                                                         const int32_t* __restrict__ ids, int n_ids, int words) {
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const int n_warps = gridDim.x * kWarpsPerCta;
  for (int b = warp0; b < n_ids; b += n_warps) {
    const int id = __ldg(ids + b);
    const size_t src_row = kDir == Dir::kGather ? static_cast<size_t>(id) : static_cast<size_t>(b);
    const size_t dst_row = kDir == Dir::kGather ? static_cast<size_t>(b) : static_cast<size_t>(id);
    if (id < 0) {
      // Negative id: a gather writes a zero row, a scatter skips the row.
      if (kDir == Dir::kGather) {
        uint4* d = out + dst_row * words;
        for (int w = lane; w < words; w += 32) d[w] = make_uint4(0, 0, 0, 0);
      }
      continue;
    }
    const uint4* s = inp + src_row * words;
    uint4* d = out + dst_row * words;
    int w = lane;
    for (; w + 96 < words; w += 128) {
      const uint4 v0 = __ldcs(s + w), v1 = __ldcs(s + w + 32), v2 = __ldcs(s + w + 64), v3 = __ldcs(s + w + 96);
      d[w] = v0; d[w + 32] = v1; d[w + 64] = v2; d[w + 96] = v3;
    }
    for (; w < words; w += 32) d[w] = __ldcs(s + w);
  }
}

// Fallback for rows that are not a multiple of 16 bytes or buffers that are not
// 16-byte aligned: 4-byte words (row_bytes must be a multiple of 4).
template <Dir kDir>
__global__ void __launch_bounds__(kThreads) RowCopyWord(uint32_t* __restrict__ out, const uint32_t* __restrict__ inp,
                                                        const int32_t* __restrict__ ids, int n_ids, int words) {
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const int n_warps = gridDim.x * kWarpsPerCta;
  for (int b = warp0; b < n_ids; b += n_warps) {
    const int id = __ldg(ids + b);
    const size_t src_row = kDir == Dir::kGather ? static_cast<size_t>(id) : static_cast<size_t>(b);
    const size_t dst_row = kDir == Dir::kGather ? static_cast<size_t>(b) : static_cast<size_t>(id);
    if (id < 0) {
      if (kDir == Dir::kGather)
        for (int w = lane; w < words; w += 32) out[dst_row * words + w] = 0u;
      continue;
    }
    for (int w = lane; w < words; w += 32) out[dst_row * words + w] = inp[src_row * words + w];
  }
}

__global__ void __launch_bounds__(kThreads) ZeroWords16(uint4* __restrict__ out, size_t words) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < words; i += stride)
    out[i] = make_uint4(0, 0, 0, 0);
}
__global__ void __launch_bounds__(kThreads) ZeroWords4(uint32_t* __restrict__ out, size_t words) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < words; i += stride) out[i] = 0u;
}

bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Strided form: rows of `width` floats inside wider rows (pitches in floats), optional row indices on either
// side, optional accumulation.  One warp per row.
__global__ void __launch_bounds__(kThreads) RowCopy2d(float* __restrict__ dst, long long dst_pitch,
                                                      const int32_t* __restrict__ dst_ids, const float* __restrict__ src,
                                                      long long src_pitch, const int32_t* __restrict__ src_ids, int rows,
                                                      int width, int accumulate) {
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const int n_warps = gridDim.x * kWarpsPerCta;
  for (int b = warp0; b < rows; b += n_warps) {
    const int dr = dst_ids ? __ldg(dst_ids + b) : b;
    const int sr = src_ids ? __ldg(src_ids + b) : b;
    if (dr < 0) continue;
    float* d = dst + static_cast<long long>(dr) * dst_pitch;
    const float* s = sr >= 0 ? src + static_cast<long long>(sr) * src_pitch : nullptr;
    for (int c = lane; c < width; c += 32) {
      const float v = s ? s[c] : 0.0f;
      d[c] = accumulate ? d[c] + v : v;
    }
  }
}

template <Dir kDir>
int RowCopy(void* out, const void* inp, const int32_t* ids, int n_ids, size_t row_bytes, cudaStream_t stream,
            const char* name) {
  CAVS_REQUIRE(n_ids >= 0, CAVS_ERR_BAD_ARG, std::string(name) + ": negative row count");
  if (n_ids == 0 || row_bytes == 0) return CAVS_OK;
  CAVS_REQUIRE(out && inp && ids, CAVS_ERR_BAD_ARG, std::string(name) + ": null pointer");
  CAVS_REQUIRE(row_bytes % 4 == 0 && row_bytes / 4 <= 0x7fffffff, CAVS_ERR_BAD_ARG,
               std::string(name) + ": row_bytes must be a multiple of 4");
  const int grid = GridForWarps(n_ids, kWarpsPerCta);
  if (row_bytes % 16 == 0 && Aligned16(out) && Aligned16(inp)) {
    RowCopyVec16<kDir><<<grid, kThreads, 0, stream>>>(static_cast<uint4*>(out), static_cast<const uint4*>(inp), ids,
                                                       n_ids, static_cast<int>(row_bytes / 16));
  } else {
    RowCopyWord<kDir><<<grid, kThreads, 0, stream>>>(static_cast<uint32_t*>(out), static_cast<const uint32_t*>(inp), ids,
                                                      n_ids, static_cast<int>(row_bytes / 4));
  }
  CAVS_LAUNCH_CHECK(name);
  return CAVS_OK;
}

}  // namespace
}  // namespace cavs_b200

using namespace cavs_b200;

extern "C" int cavs_gather_rows(void* out, const void* inp, const int32_t* ids, int n_ids, size_t row_bytes,
                                void* stream) {
  return RowCopy<Dir::kGather>(out, inp, ids, n_ids, row_bytes, static_cast<cudaStream_t>(stream), "gather_rows");
}

extern "C" int cavs_scatter_rows(void* out, const int32_t* ids, const void* inp, int n_ids, size_t row_bytes,
                                 void* stream) {
  return RowCopy<Dir::kScatter>(out, inp, ids, n_ids, row_bytes, static_cast<cudaStream_t>(stream), "scatter_rows");
}

extern "C" int cavs_copy_rows_2d(float* dst, long long dst_pitch, const int32_t* dst_ids, const float* src, long long src_pitch,
                                 const int32_t* src_ids, int rows, int width, int accumulate, void* stream) {
  CAVS_REQUIRE(rows >= 0 && width >= 0 && dst_pitch >= width && src_pitch >= 0, CAVS_ERR_BAD_ARG, "copy_rows_2d: bad shape");
  if (rows == 0 || width == 0) return CAVS_OK;
  CAVS_REQUIRE(dst && src, CAVS_ERR_BAD_ARG, "copy_rows_2d: null pointer");
  RowCopy2d<<<GridForWarps(rows, kWarpsPerCta), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      dst, dst_pitch, dst_ids, src, src_pitch, src_ids, rows, width, accumulate ? 1 : 0);
  CAVS_LAUNCH_CHECK("copy_rows_2d");
  return CAVS_OK;
}

extern "C" int cavs_zero_rows(void* out, int n_rows, size_t row_bytes, void* stream) {
  CAVS_REQUIRE(n_rows >= 0, CAVS_ERR_BAD_ARG, "zero_rows: negative row count");
  const size_t bytes = static_cast<size_t>(n_rows) * row_bytes;
  if (bytes == 0) return CAVS_OK;
  CAVS_REQUIRE(out, CAVS_ERR_BAD_ARG, "zero_rows: null pointer");
  CAVS_REQUIRE(bytes % 4 == 0, CAVS_ERR_BAD_ARG, "zero_rows: byte count must be a multiple of 4");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (bytes % 16 == 0 && Aligned16(out)) {
    const size_t words = bytes / 16;
    ZeroWords16<<<GridForElems(words, kThreads), kThreads, 0, st>>>(static_cast<uint4*>(out), words);
  } else {
    const size_t words = bytes / 4;
    ZeroWords4<<<GridForElems(words, kThreads), kThreads, 0, st>>>(static_cast<uint32_t*>(out), words);
  }
  CAVS_LAUNCH_CHECK("zero_rows");
  return CAVS_OK;
}
