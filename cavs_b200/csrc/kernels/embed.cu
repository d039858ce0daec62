// Embedding lookup and its deterministic segmented gradient.
//
// Forward replaces BatchedCopy (cavs/backend/op_impl_embedding_lookup.cu:23-35,64-72);
// token ids are int32 here (the reference carries them as floats and casts on device).
// Backward replaces BatchedSparseUpdate's atomicAdd accumulation (:91-103), whose result
// depends on the order in which duplicate tokens arrive.  Here rows are grouped by token
// on the host once per batch (stable counting sort), every group is cut into chunks of at
// most kEmbedChunk rows, each chunk is summed in row order by one CTA, and the chunks of a
// group are summed in chunk order: the same bits on every run.
#include <cuda_bf16.h>

#include <cstdint>

#include "abi_common.h"
#include "kernels/cell.h"
#include "kernels/launch.h"

namespace cavs_b200 {
namespace {

constexpr int kThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads)
EmbedFwd(T* __restrict__ out, const float* __restrict__ table, const int32_t* __restrict__ tok, int rows, int E, int vocab) {
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int n_warps = gridDim.x * (kThreads / 32);
  for (int t = warp0; t < rows; t += n_warps) {
    int id = __ldg(tok + t);
    if (id < 0 || id >= vocab) id = 0;
    const float* src = table + static_cast<size_t>(id) * E;
    T* dst = out + static_cast<size_t>(t) * E;
    if ((E & 3) == 0) {
      for (int e = lane * 4; e < E; e += 128) {
        const float4 v = *reinterpret_cast<const float4*>(src + e);
        if constexpr (sizeof(T) == 4) {
          *reinterpret_cast<float4*>(dst + e) = v;
        } else {
          __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
          uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
          *reinterpret_cast<uint2*>(dst + e) = u;
        }
      }
    } else {
      for (int e = lane; e < E; e += 32) dst[e] = static_cast<T>(src[e]);
    }
  }
}

// One CTA per chunk: partial[chunk,:] = sum over the chunk's rows.  Four interleaved running sums
// per column (rows r, r+1, r+2, r+3 mod 4) combined as ((s0+s1)+(s2+s3)): a fixed order.
template <int kVec>
__global__ void __launch_bounds__(kThreads)
EmbedBwdChunks(float* __restrict__ partial, const float* __restrict__ dX, const int32_t* __restrict__ order,
               const int32_t* __restrict__ chunk_off, int E) {
  __shared__ int32_t rows_sm[kEmbedChunk];
  const int chunk = blockIdx.x;
  const int begin = chunk_off[chunk], cnt = chunk_off[chunk + 1] - begin;
  for (int r = threadIdx.x; r < cnt; r += kThreads) rows_sm[r] = order[begin + r];
  __syncthreads();
  for (int e = threadIdx.x * kVec; e < E; e += kThreads * kVec) {
    float acc[4][kVec];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int v = 0; v < kVec; ++v) acc[u][v] = 0.0f;
    int r = 0;
    for (; r + 4 <= cnt; r += 4) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float* src = dX + static_cast<size_t>(rows_sm[r + u]) * E + e;
        if (kVec == 4) {
          const float4 t = *reinterpret_cast<const float4*>(src);
          acc[u][0] += t.x; acc[u][1 % kVec] += t.y; acc[u][2 % kVec] += t.z; acc[u][3 % kVec] += t.w;
        } else {
          acc[u][0] += *src;
        }
      }
    }
    for (int u = 0; r < cnt; ++r, ++u) {
      const float* src = dX + static_cast<size_t>(rows_sm[r]) * E + e;
      if (kVec == 4) {
        const float4 t = *reinterpret_cast<const float4*>(src);
        acc[u][0] += t.x; acc[u][1 % kVec] += t.y; acc[u][2 % kVec] += t.z; acc[u][3 % kVec] += t.w;
      } else {
        acc[u][0] += *src;
      }
    }
    float* dst = partial + static_cast<size_t>(chunk) * E + e;
#pragma unroll
    for (int v = 0; v < kVec; ++v) dst[v] = (acc[0][v] + acc[1][v]) + (acc[2][v] + acc[3][v]);
  }
}
// One CTA per segment: dtable[tok,:] = sum of its chunks' partials.  The loads of eight chunks
// are issued together; the adds keep chunk order, so the result is the plain left-to-right sum.
template <int kVec>
__global__ void __launch_bounds__(kThreads)
EmbedBwdSegments(float* __restrict__ dtable, const float* __restrict__ partial, const int32_t* __restrict__ seg_first_chunk,
                 const int32_t* __restrict__ seg_tok, int E) {
  const int seg = blockIdx.x;
  const int c0 = seg_first_chunk[seg], c1 = seg_first_chunk[seg + 1];
  float* dst = dtable + static_cast<size_t>(seg_tok[seg]) * E;
  for (int e = threadIdx.x * kVec; e < E; e += kThreads * kVec) {
    float acc[kVec];
#pragma unroll
    for (int v = 0; v < kVec; ++v) acc[v] = 0.0f;
    int c = c0;
    for (; c + 8 <= c1; c += 8) {
      float t[8][kVec];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float* src = partial + static_cast<size_t>(c + u) * E + e;
        if (kVec == 4) {
          const float4 q = *reinterpret_cast<const float4*>(src);
          t[u][0] = q.x; t[u][1 % kVec] = q.y; t[u][2 % kVec] = q.z; t[u][3 % kVec] = q.w;
        } else {
          t[u][0] = *src;
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int v = 0; v < kVec; ++v) acc[v] += t[u][v];
    }
    for (; c < c1; ++c)
#pragma unroll
      for (int v = 0; v < kVec; ++v) acc[v] += partial[static_cast<size_t>(c) * E + e + v];
#pragma unroll
    for (int v = 0; v < kVec; ++v) dst[e + v] = acc[v];
  }
}

// ---- Segmented row sums (rows grouped by token), any input precision ----
// The input projection x.W and its gradients depend on a vertex only through its token, so the
// engine sums d(pre-activation) rows per distinct token before the weight-gradient and
// embedding-gradient GEMMs.  Same fixed-order two-level scheme as above: chunks of at most
// kEmbedChunk rows, then the chunks of a segment in order.
template <typename TIn>
__device__ __forceinline__ void Load4(const TIn* p, float (&v)[4]) {
  if constexpr (sizeof(TIn) == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
}
// One CTA per chunk; width must be a multiple of 4.  partial[chunk,:] in fp32 -- except for a chunk that is its
// segment's only one (chunk_out[chunk] = segment index, else -1; optional table): its sums are final and go
// straight to out[segment,:], skipping the partial round trip (most tokens of a batch occur a few times).
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(kThreads)
SegSumChunks(float* __restrict__ partial, TOut* __restrict__ out, const int32_t* __restrict__ chunk_out,
             const TIn* __restrict__ x, long long pitch, const int32_t* __restrict__ order,
             const int32_t* __restrict__ chunk_off, int width) {
  __shared__ int32_t rows_sm[kEmbedChunk];
  const int chunk = blockIdx.x;
  const int direct = chunk_out != nullptr ? chunk_out[chunk] : -1;
  const int begin = chunk_off[chunk], cnt = chunk_off[chunk + 1] - begin;
  for (int r = threadIdx.x; r < cnt; r += kThreads) rows_sm[r] = order[begin + r];
  __syncthreads();
  for (int e = threadIdx.x * 4; e < width; e += kThreads * 4) {
    float acc[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int v = 0; v < 4; ++v) acc[u][v] = 0.0f;
    int r = 0;
    // Eight row loads in flight per thread; accumulator u still takes rows u, u + 4, u + 8, ... in order.
    for (; r + 8 <= cnt; r += 8) {
      float t[8][4];
#pragma unroll
      for (int u = 0; u < 8; ++u) Load4(x + static_cast<long long>(rows_sm[r + u]) * pitch + e, t[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] += t[u][v];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] += t[u + 4][v];
    }
    for (; r + 4 <= cnt; r += 4) {
      float t[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) Load4(x + static_cast<long long>(rows_sm[r + u]) * pitch + e, t[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] += t[u][v];
    }
    for (int u = 0; r < cnt; ++r, ++u) {
      float t[4];
      Load4(x + static_cast<long long>(rows_sm[r]) * pitch + e, t);
#pragma unroll
      for (int v = 0; v < 4; ++v) acc[u][v] += t[v];
    }
    const float4 sum =
        make_float4((acc[0][0] + acc[1][0]) + (acc[2][0] + acc[3][0]), (acc[0][1] + acc[1][1]) + (acc[2][1] + acc[3][1]),
                    (acc[0][2] + acc[1][2]) + (acc[2][2] + acc[3][2]), (acc[0][3] + acc[1][3]) + (acc[2][3] + acc[3][3]));
    if (direct < 0) {
      *reinterpret_cast<float4*>(partial + static_cast<size_t>(chunk) * width + e) = sum;
    } else {
      // 0 + sum, as the second pass would compute it for a single chunk
      TOut* dst = out + static_cast<size_t>(direct) * width + e;
      if constexpr (sizeof(TOut) == 4) {
        *reinterpret_cast<float4*>(dst) = sum;
      } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(sum.x, sum.y), b = __floats2bfloat162_rn(sum.z, sum.w);
        uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(dst) = u;
      }
    }
  }
}
// Scalar forms of the two passes for widths or pitches that are not multiples of 4 (same summation order
// per column: rows of a chunk in order, then chunks in order).
template <typename TIn>
__global__ void __launch_bounds__(kThreads)
SegSumChunksScalar(float* __restrict__ partial, const TIn* __restrict__ x, long long pitch, const int32_t* __restrict__ order,
                   const int32_t* __restrict__ chunk_off, int width) {
  const int chunk = blockIdx.x;
  const int begin = chunk_off[chunk], cnt = chunk_off[chunk + 1] - begin;
  for (int e = threadIdx.x; e < width; e += kThreads) {
    float acc = 0.0f;
    for (int r = 0; r < cnt; ++r) acc += static_cast<float>(x[static_cast<long long>(order[begin + r]) * pitch + e]);
    partial[static_cast<size_t>(chunk) * width + e] = acc;
  }
}
template <typename TOut>
__global__ void __launch_bounds__(kThreads)
SegSumFinalScalar(TOut* __restrict__ out, const float* __restrict__ partial, const int32_t* __restrict__ seg_first_chunk, int width) {
  const int seg = blockIdx.x;
  const int c0 = seg_first_chunk[seg], c1 = seg_first_chunk[seg + 1];
  for (int e = threadIdx.x; e < width; e += kThreads) {
    float acc = 0.0f;
    for (int c = c0; c < c1; ++c) acc += partial[static_cast<size_t>(c) * width + e];
    out[static_cast<size_t>(seg) * width + e] = static_cast<TOut>(acc);
  }
}
// One CTA per segment: out[seg,:] = sum of its chunks' partials in chunk order (fp32 or bf16 output).
template <typename TOut>
__global__ void __launch_bounds__(kThreads)
SegSumFinal(TOut* __restrict__ out, const float* __restrict__ partial, const int32_t* __restrict__ seg_first_chunk, int width,
            int skip_single) {
  const int seg = blockIdx.x;
  const int c0 = seg_first_chunk[seg], c1 = seg_first_chunk[seg + 1];
  if (skip_single && c1 - c0 == 1) return;   // written by the first pass
  for (int e = threadIdx.x * 4; e < width; e += kThreads * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int c = c0;
    for (; c + 8 <= c1; c += 8) {
      float4 t[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) t[u] = *reinterpret_cast<const float4*>(partial + static_cast<size_t>(c + u) * width + e);
#pragma unroll
      for (int u = 0; u < 8; ++u) { acc[0] += t[u].x; acc[1] += t[u].y; acc[2] += t[u].z; acc[3] += t[u].w; }
    }
    for (; c < c1; ++c) {
      const float4 t = *reinterpret_cast<const float4*>(partial + static_cast<size_t>(c) * width + e);
      acc[0] += t.x; acc[1] += t.y; acc[2] += t.z; acc[3] += t.w;
    }
    TOut* dst = out + static_cast<size_t>(seg) * width + e;
    if constexpr (sizeof(TOut) == 4) {
      *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else {
      __nv_bfloat162 a = __floats2bfloat162_rn(acc[0], acc[1]), b = __floats2bfloat162_rn(acc[2], acc[3]);
      uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(dst) = u;
    }
  }
}

// Second pass for the segments that have more than one chunk (listed in multi_seg).  A CTA takes one such
// segment and 128 columns: its eight groups of 32 lanes each sum every eighth chunk partial (group g: chunks
// c0 + g, c0 + g + 8, ...), four loads in flight, and the eight group sums are folded in group order -- a fixed
// tree, so the result is deterministic, and the longest segment of a batch (the token shared by all internal
// vertices has ~1000 chunks) is no longer one serial chain.
template <typename TOut>
__global__ void __launch_bounds__(kThreads)
SegSumFinalMulti(TOut* __restrict__ out, const float* __restrict__ partial, const int32_t* __restrict__ seg_first_chunk,
                 const int32_t* __restrict__ multi_seg, int width) {
  __shared__ float4 fold[kThreads];
  const int seg = multi_seg[blockIdx.x];
  const int c0 = seg_first_chunk[seg], c1 = seg_first_chunk[seg + 1];
  const int g = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.y * 128 + lane * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (e < width) {
    int c = c0 + g;
    for (; c + 24 < c1; c += 32) {
      float4 t[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) t[u] = *reinterpret_cast<const float4*>(partial + static_cast<size_t>(c + 8 * u) * width + e);
#pragma unroll
      for (int u = 0; u < 4; ++u) { acc.x += t[u].x; acc.y += t[u].y; acc.z += t[u].z; acc.w += t[u].w; }
    }
    for (; c < c1; c += 8) {
      const float4 t = *reinterpret_cast<const float4*>(partial + static_cast<size_t>(c) * width + e);
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
  }
  fold[threadIdx.x] = acc;
  __syncthreads();
  if (g == 0 && e < width) {
    float4 s = fold[lane];
#pragma unroll
    for (int k = 1; k < kThreads / 32; ++k) {
      const float4 t = fold[k * 32 + lane];
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    TOut* dst = out + static_cast<size_t>(seg) * width + e;
    if constexpr (sizeof(TOut) == 4) {
      *reinterpret_cast<float4*>(dst) = s;
    } else {
      __nv_bfloat162 a = __floats2bfloat162_rn(s.x, s.y), b = __floats2bfloat162_rn(s.z, s.w);
      uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(dst) = u;
    }
  }
}

}  // namespace

int LaunchSegmentedRowSum(void* out, bool out_bf16, const void* x, bool in_bf16, long long pitch, int width, const int32_t* order,
                          const int32_t* chunk_off, int n_chunks, const int32_t* seg_first_chunk, int n_seg, float* scratch,
                          cudaStream_t st, const int32_t* chunk_out, const int32_t* multi_seg, int n_multi) {
  CAVS_REQUIRE(n_chunks >= 0 && n_seg >= 0 && width > 0 && pitch >= width, CAVS_ERR_BAD_ARG,
               "segmented_row_sum: width must be positive and pitch >= width");
  if (n_chunks == 0 || n_seg == 0) return CAVS_OK;
  CAVS_REQUIRE(out && x && order && chunk_off && seg_first_chunk && scratch, CAVS_ERR_BAD_ARG, "segmented_row_sum: null pointer");
  using bf = __nv_bfloat16;
  const bool vec = width % 4 == 0 && pitch % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(scratch)) & 15u) == 0;
  if (!vec) {
    if (in_bf16) SegSumChunksScalar<bf><<<n_chunks, kThreads, 0, st>>>(scratch, static_cast<const bf*>(x), pitch, order, chunk_off, width);
    else SegSumChunksScalar<float><<<n_chunks, kThreads, 0, st>>>(scratch, static_cast<const float*>(x), pitch, order, chunk_off, width);
    CAVS_LAUNCH_CHECK("segmented_row_sum chunks");
    if (out_bf16) SegSumFinalScalar<bf><<<n_seg, kThreads, 0, st>>>(static_cast<bf*>(out), scratch, seg_first_chunk, width);
    else SegSumFinalScalar<float><<<n_seg, kThreads, 0, st>>>(static_cast<float*>(out), scratch, seg_first_chunk, width);
    CAVS_LAUNCH_CHECK("segmented_row_sum final");
    return CAVS_OK;
  }
  const int skip = chunk_out != nullptr ? 1 : 0;
  if (in_bf16 && out_bf16) SegSumChunks<bf, bf><<<n_chunks, kThreads, 0, st>>>(scratch, static_cast<bf*>(out), chunk_out, static_cast<const bf*>(x), pitch, order, chunk_off, width);
  else if (in_bf16) SegSumChunks<bf, float><<<n_chunks, kThreads, 0, st>>>(scratch, static_cast<float*>(out), chunk_out, static_cast<const bf*>(x), pitch, order, chunk_off, width);
  else if (out_bf16) SegSumChunks<float, bf><<<n_chunks, kThreads, 0, st>>>(scratch, static_cast<bf*>(out), chunk_out, static_cast<const float*>(x), pitch, order, chunk_off, width);
  else SegSumChunks<float, float><<<n_chunks, kThreads, 0, st>>>(scratch, static_cast<float*>(out), chunk_out, static_cast<const float*>(x), pitch, order, chunk_off, width);
  CAVS_LAUNCH_CHECK("segmented_row_sum chunks");
  if (skip && multi_seg != nullptr) {
    // every single-chunk segment is done; only the listed multi-chunk ones need the second pass
    if (n_multi > 0) {
      const dim3 grid(n_multi, (width + 127) / 128);
      if (out_bf16) SegSumFinalMulti<bf><<<grid, kThreads, 0, st>>>(static_cast<bf*>(out), scratch, seg_first_chunk, multi_seg, width);
      else SegSumFinalMulti<float><<<grid, kThreads, 0, st>>>(static_cast<float*>(out), scratch, seg_first_chunk, multi_seg, width);
    }
  } else if (out_bf16) {
    SegSumFinal<__nv_bfloat16><<<n_seg, kThreads, 0, st>>>(static_cast<__nv_bfloat16*>(out), scratch, seg_first_chunk, width, skip);
  } else {
    SegSumFinal<float><<<n_seg, kThreads, 0, st>>>(static_cast<float*>(out), scratch, seg_first_chunk, width, skip);
  }
  CAVS_LAUNCH_CHECK("segmented_row_sum final");
  return CAVS_OK;
}

int LaunchSegmentedRowSumFinal(void* out, bool out_bf16, const float* partial, const int32_t* seg_first_chunk,
                               const int32_t* multi_seg, int n_multi, int width, cudaStream_t st) {
  CAVS_REQUIRE(n_multi >= 0 && width > 0 && width % 4 == 0, CAVS_ERR_BAD_ARG, "segmented_row_sum_final: width must be a positive multiple of 4");
  if (n_multi == 0) return CAVS_OK;
  CAVS_REQUIRE(out && partial && seg_first_chunk && multi_seg, CAVS_ERR_BAD_ARG, "segmented_row_sum_final: null pointer");
  using bf = __nv_bfloat16;
  const dim3 grid(n_multi, (width + 127) / 128);
  if (out_bf16) SegSumFinalMulti<bf><<<grid, kThreads, 0, st>>>(static_cast<bf*>(out), partial, seg_first_chunk, multi_seg, width);
  else SegSumFinalMulti<float><<<grid, kThreads, 0, st>>>(static_cast<float*>(out), partial, seg_first_chunk, multi_seg, width);
  CAVS_LAUNCH_CHECK("segmented_row_sum_final");
  return CAVS_OK;
}

int LaunchEmbedFwd(void* out, bool bf16, const float* table, const int32_t* tok, int rows, int E, int vocab, cudaStream_t st) {
  CAVS_REQUIRE(rows >= 0 && E > 0 && vocab > 0, CAVS_ERR_BAD_ARG, "embed_fwd: bad shape");
  if (rows == 0) return CAVS_OK;
  CAVS_REQUIRE(out && table && tok, CAVS_ERR_BAD_ARG, "embed_fwd: null pointer");
  const int grid = GridForWarps(rows, kThreads / 32);
  if (bf16) EmbedFwd<__nv_bfloat16><<<grid, kThreads, 0, st>>>(static_cast<__nv_bfloat16*>(out), table, tok, rows, E, vocab);
  else EmbedFwd<float><<<grid, kThreads, 0, st>>>(static_cast<float*>(out), table, tok, rows, E, vocab);
  CAVS_LAUNCH_CHECK("embed_fwd");
  return CAVS_OK;
}

int LaunchEmbedBwd(float* dtable, const float* dX, const int32_t* order, const int32_t* /*chunk_seg*/, const int32_t* chunk_off,
                   int n_chunks, const int32_t* seg_first_chunk, const int32_t* seg_tok, int n_seg, float* scratch, int E,
                   cudaStream_t st) {
  CAVS_REQUIRE(n_chunks >= 0 && n_seg >= 0 && E > 0, CAVS_ERR_BAD_ARG, "embed_bwd: bad shape");
  if (n_chunks == 0 || n_seg == 0) return CAVS_OK;
  CAVS_REQUIRE(dtable && dX && order && chunk_off && seg_first_chunk && seg_tok && scratch, CAVS_ERR_BAD_ARG, "embed_bwd: null pointer");
  if (E % 4 == 0 && ((reinterpret_cast<uintptr_t>(dX) | reinterpret_cast<uintptr_t>(scratch)) & 15u) == 0)
    EmbedBwdChunks<4><<<n_chunks, kThreads, 0, st>>>(scratch, dX, order, chunk_off, E);
  else
    EmbedBwdChunks<1><<<n_chunks, kThreads, 0, st>>>(scratch, dX, order, chunk_off, E);
  CAVS_LAUNCH_CHECK("embed_bwd chunks");
  if (E % 4 == 0 && ((reinterpret_cast<uintptr_t>(dtable) | reinterpret_cast<uintptr_t>(scratch)) & 15u) == 0)
    EmbedBwdSegments<4><<<n_seg, kThreads, 0, st>>>(dtable, scratch, seg_first_chunk, seg_tok, E);
  else
    EmbedBwdSegments<1><<<n_seg, kThreads, 0, st>>>(dtable, scratch, seg_first_chunk, seg_tok, E);
  CAVS_LAUNCH_CHECK("embed_bwd segments");
  return CAVS_OK;
}

}  // namespace cavs_b200
