// Loss head: classifier + softmax cross-entropy, forward and backward in one pass over
// the pushed hidden rows, for small class counts.
//
// Replaces FullyConnected (two cublasSgemm, cavs/backend/op_impl_fullyconnected_cublas.cc:33-85),
// cudnnSoftmaxForward + SoftmaxEntropyLossForwardKernel
// (cavs/backend/op_impl_softmax_entropy_logits_loss.cu:106-140), their gradients
// (:213-250 and op_impl_fullyconnected_cublas.cc:104-176: three more cublasSgemm) and the
// two device-wide synchronisations in between.  HBM-bound: reads each hidden row once
// from DRAM (the second use hits L2), writes d(hidden) once.
//
// Determinism: dWc / dbc / the loss sum are accumulated per CTA in a fixed row order,
// written to scratch, and reduced across CTAs in index order by a second kernel.
#include <cuda_bf16.h>

#include <cstdint>
#include <mutex>

#include "abi_common.h"
#include "kernels/bulk.cuh"
#include "kernels/cell.h"
#include "kernels/launch.h"

namespace cavs_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kRowsPerBlock = 32;     // rows per CTA iteration (4 per warp)
constexpr int kMaxC = 8;
constexpr int kCtasPerSm = 2;
// Floats per per-CTA partial record ([C*H] dWc, [C] dbc, [1] loss sum), padded to 16 bytes so the
// 128-bit stores of every CTA's record stay aligned.
__host__ __device__ constexpr int PartialStride(int C, int H) { return (C * H + C + 1 + 3) & ~3; }
constexpr int kMaxColsPerThread = 8;  // H <= kThreads * kMaxColsPerThread

__device__ __forceinline__ float WarpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// kVec = 4 when H is a multiple of 4 (128-bit accesses), else 1.
// kIters > 0: H == 128 * kIters, so a lane's whole share of a row (kIters 128-bit words) is loaded
// up front and every loop unrolls; kIters == 0: generic loops.
template <int C, int kVec, int kIters>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
LossHeadKernel(float* __restrict__ loss, float* __restrict__ dOut, float* __restrict__ dz_out, float* __restrict__ partial,
               const float* __restrict__ h, long long h_pitch, const int32_t* __restrict__ label,
               const float* __restrict__ Wc, const float* __restrict__ bc, int rows, int H, float inv_rows) {
  extern __shared__ float sm[];
  float* sW = sm;                          // [C][H]
  float* sdz = sm + C * H;                 // [kRowsPerBlock][C]
  float* sloss = sdz + kRowsPerBlock * C;  // [kWarps]
  for (int i = threadIdx.x; i < C * H; i += kThreads) sW[i] = Wc[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float accW[kMaxColsPerThread][C];        // columns (threadIdx.x + q * kThreads) * kVec + e, q-major
#pragma unroll
  for (int q = 0; q < kMaxColsPerThread; ++q)
#pragma unroll
    for (int c = 0; c < C; ++c) accW[q][c] = 0.0f;
  float accb = 0.0f;        // thread c < C owns class c of the bias gradient
  float loss_acc = 0.0f;    // per warp (lane 0)
  constexpr int kQ = kMaxColsPerThread / kVec;   // vector slots per thread

  const int n_blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  for (int blk = blockIdx.x; blk < n_blocks; blk += gridDim.x) {
    const int r0 = blk * kRowsPerBlock;
    // Phase 1: each warp handles rows r0 + warp, r0 + warp + kWarps, ...
    for (int rr = warp; rr < kRowsPerBlock; rr += kWarps) {
      const int t = r0 + rr;
      float dz[C];
      if (t < rows) {
        const float* hr = h + static_cast<long long>(t) * h_pitch;
        float z[C];
#pragma unroll
        for (int c = 0; c < C; ++c) z[c] = 0.0f;
        if (kIters > 0) {
          float4 hv[kIters > 0 ? kIters : 1];
#pragma unroll
          for (int it = 0; it < kIters; ++it) hv[it] = *reinterpret_cast<const float4*>(hr + lane * 4 + it * 128);
#pragma unroll
          for (int it = 0; it < kIters; ++it) {
#pragma unroll
            for (int c = 0; c < C; ++c) {
              const float4 w = *reinterpret_cast<const float4*>(sW + c * H + lane * 4 + it * 128);
              z[c] = fmaf(hv[it].x, w.x, fmaf(hv[it].y, w.y, fmaf(hv[it].z, w.z, fmaf(hv[it].w, w.w, z[c]))));
            }
          }
        } else if (kVec == 4) {
          for (int j = lane * 4; j < H; j += 128) {
            const float4 hv = *reinterpret_cast<const float4*>(hr + j);
#pragma unroll
            for (int c = 0; c < C; ++c) {
              const float4 w = *reinterpret_cast<const float4*>(sW + c * H + j);
              z[c] = fmaf(hv.x, w.x, fmaf(hv.y, w.y, fmaf(hv.z, w.z, fmaf(hv.w, w.w, z[c]))));
            }
          }
        } else {
          for (int j = lane; j < H; j += 32) {
            const float hv = hr[j];
#pragma unroll
            for (int c = 0; c < C; ++c) z[c] = fmaf(hv, sW[c * H + j], z[c]);
          }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < C; ++c) { z[c] = WarpSum(z[c]) + bc[c]; mx = fmaxf(mx, z[c]); }
        float den = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c) { z[c] = expf(z[c] - mx); den += z[c]; }
        const int y = label[t];
        float lrow = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const float pc = z[c] / den;
          dz[c] = (y >= 0) ? (pc - (c == y ? 1.0f : 0.0f)) * inv_rows : 0.0f;
          if (c == y) lrow = -logf(pc);
        }
        if (lane == 0) { loss[t] = lrow; loss_acc += lrow; }
        if (dz_out != nullptr && lane == 0) {
          // d(logits) row, zero-padded to kMaxC floats: the consumer rebuilds d(hidden) = dz Wc itself.
          float pad[kMaxC];
#pragma unroll
          for (int c = 0; c < kMaxC; ++c) pad[c] = c < C ? dz[c < C ? c : 0] : 0.0f;
          float4* dst = reinterpret_cast<float4*>(dz_out + static_cast<long long>(t) * kMaxC);
          dst[0] = make_float4(pad[0], pad[1], pad[2], pad[3]);
          dst[1] = make_float4(pad[4], pad[5], pad[6], pad[7]);
        }
        float* dr = dOut + static_cast<long long>(t) * H;
        if (dOut == nullptr) {
          // d(hidden) is not materialised
        } else if (kVec == 4) {
#pragma unroll 4
          for (int j = lane * 4; j < H; j += 128) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int c = 0; c < C; ++c) {
              const float4 w = *reinterpret_cast<const float4*>(sW + c * H + j);
              a.x = fmaf(dz[c], w.x, a.x); a.y = fmaf(dz[c], w.y, a.y); a.z = fmaf(dz[c], w.z, a.z); a.w = fmaf(dz[c], w.w, a.w);
            }
            __stcs(reinterpret_cast<float4*>(dr + j), a);
          }
        } else {
          for (int j = lane; j < H; j += 32) {
            float a = 0.0f;
#pragma unroll
            for (int c = 0; c < C; ++c) a = fmaf(dz[c], sW[c * H + j], a);
            dr[j] = a;
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < C; ++c) dz[c] = 0.0f;
      }
      if (lane == 0) {
#pragma unroll
        for (int c = 0; c < C; ++c) sdz[rr * C + c] = dz[c];
      }
    }
    __syncthreads();
    // Phase 2: dWc += dz^T h with each thread owning fixed columns; rows in ascending order.
    const int r_end = min(kRowsPerBlock, rows - r0);
#pragma unroll 8
    for (int rr = 0; rr < r_end; ++rr) {
      const float* hr = h + static_cast<long long>(r0 + rr) * h_pitch;
      if (kVec == 4) {
#pragma unroll
        for (int q = 0; q < kQ; ++q) {
          const int j = (threadIdx.x + q * kThreads) * 4;
          if (j < H) {
            const float4 hv = *reinterpret_cast<const float4*>(hr + j);
#pragma unroll
            for (int c = 0; c < C; ++c) {
              const float d = sdz[rr * C + c];
              accW[q * 4 + 0][c] = fmaf(d, hv.x, accW[q * 4 + 0][c]);
              accW[q * 4 + 1][c] = fmaf(d, hv.y, accW[q * 4 + 1][c]);
              accW[q * 4 + 2][c] = fmaf(d, hv.z, accW[q * 4 + 2][c]);
              accW[q * 4 + 3][c] = fmaf(d, hv.w, accW[q * 4 + 3][c]);
            }
          }
        }
      } else {
#pragma unroll
        for (int q = 0; q < kMaxColsPerThread; ++q) {
          const int j = threadIdx.x + q * kThreads;
          if (j < H) {
            const float hv = hr[j];
#pragma unroll
            for (int c = 0; c < C; ++c) accW[q][c] = fmaf(sdz[rr * C + c], hv, accW[q][c]);
          }
        }
      }
      if (threadIdx.x < C) accb += sdz[rr * C + threadIdx.x];
    }
    __syncthreads();
  }
  // Per-CTA partial: [C*H] dWc, [C] dbc, [1] loss sum.
  float* mine = partial + static_cast<size_t>(blockIdx.x) * PartialStride(C, H);
  if (kVec == 4) {
#pragma unroll
    for (int q = 0; q < kQ; ++q) {
      const int j = (threadIdx.x + q * kThreads) * 4;
      if (j < H) {
#pragma unroll
        for (int c = 0; c < C; ++c)
          *reinterpret_cast<float4*>(mine + c * H + j) =
              make_float4(accW[q * 4 + 0][c], accW[q * 4 + 1][c], accW[q * 4 + 2][c], accW[q * 4 + 3][c]);
      }
    }
  } else {
#pragma unroll
    for (int q = 0; q < kMaxColsPerThread; ++q) {
      const int j = threadIdx.x + q * kThreads;
      if (j < H) {
#pragma unroll
        for (int c = 0; c < C; ++c) mine[c * H + j] = accW[q][c];
      }
    }
  }
  if (threadIdx.x < C) mine[C * H + threadIdx.x] = accb;
  if (lane == 0) sloss[warp] = loss_acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.0f;
    for (int w = 0; w < kWarps; ++w) s += sloss[w];
    mine[C * H + C] = s;
  }
}

// Streaming form for H <= 1024 (H a multiple of 4): rows arrive in shared memory through bulk copies that
// complete on an mbarrier, kStreamStages batches of kStreamRows rows in flight per CTA, so DRAM latency is
// hidden without occupancy.  Each thread owns four columns for the CTA's whole life: its slice of the
// classifier and its dWc accumulators live in registers, every row is read from DRAM exactly once and
// from shared memory once.  Per batch: partial logits per thread -> transpose-reduce inside the warp
// (lane l ends up with row l/4) -> shared memory across the 8 warps -> one barrier -> every warp finishes
// the softmax of the 8 rows -> every thread adds dz^T h for its columns from registers.  Same per-CTA partial record as
// LossHeadKernel.  A bulk copy that does not land within the wait limit raises *status (if given),
// poisons the CTA's loss sum with NaN and ends the CTA's loop.
constexpr int kStreamRows = 8;
constexpr int kStreamStages = 3;

template <int C>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
LossHeadStream(float* __restrict__ loss, float* __restrict__ dOut, float* __restrict__ dz_out, float* __restrict__ partial,
               const float* __restrict__ h, long long h_pitch, const int32_t* __restrict__ label,
               const float* __restrict__ Wc, const float* __restrict__ bc, int rows, int H, float inv_rows,
               int* __restrict__ status, const int32_t* __restrict__ row_index, LossTokenRows tr) {
  extern __shared__ __align__(16) float sm[];
  float* stage = sm;                                                  // [kStreamStages][kStreamRows][H]
  float* red = sm + kStreamStages * kStreamRows * H;                  // [2][kWarps][kStreamRows][C], by batch parity
  __shared__ __align__(8) unsigned long long bars[kStreamStages];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int j = tid * 4;
  const bool col_ok = j < H;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * 4u;
  const int n_batches = (rows + kStreamRows - 1) / kStreamRows;
  const int my_batches = blockIdx.x < n_batches ? (n_batches - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  auto issue = [&](int k) {   // thread 0: start the copies of this CTA's k-th batch
    const int s = k % kStreamStages;
    const int r0 = (blockIdx.x + k * gridDim.x) * kStreamRows;
    const int cnt = min(kStreamRows, rows - r0);
    const uint32_t bar = bulk::SmemAddr(&bars[s]);
    bulk::MbarExpectTx(bar, row_bytes * cnt);
    for (int r = 0; r < cnt; ++r) {
      // row_index (optional): the hidden row of loss row t lives at h[row_index[t]] (rows shared between vertices)
      const long long src = row_index != nullptr ? row_index[r0 + r] : r0 + r;
      bulk::Load(bulk::SmemAddr(stage + (s * kStreamRows + r) * H), h + src * h_pitch, row_bytes, bar);
    }
  };
  if (tid == 0) {
    for (int s = 0; s < kStreamStages; ++s) bulk::MbarInit(bulk::SmemAddr(&bars[s]), 1);
    bulk::FenceMbarInit();
  }
  __syncthreads();
  if (tid == 0)
    for (int k = 0; k < kStreamStages && k < my_batches; ++k) issue(k);

  float wc[C][4], accW[C][4];
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const float4 w = col_ok ? *reinterpret_cast<const float4*>(Wc + c * H + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    wc[c][0] = w.x; wc[c][1] = w.y; wc[c][2] = w.z; wc[c][3] = w.w;
#pragma unroll
    for (int e = 0; e < 4; ++e) accW[c][e] = 0.0f;
  }
  float accb = 0.0f;       // thread c < C: bias gradient of class c
  float loss_acc = 0.0f;   // thread r < kStreamRows: loss of the rows it finished
  bool aborted = false;    // uniform across the CTA (decided at the batch barrier)

  for (int k = 0; k < my_batches; ++k) {
    const int s = k % kStreamStages;
    const int r0 = (blockIdx.x + k * gridDim.x) * kStreamRows;
    const int cnt = min(kStreamRows, rows - r0);
    const bool landed = bulk::MbarWait(bulk::SmemAddr(&bars[s]), (k / kStreamStages) & 1);
    float hr[kStreamRows][4];
#pragma unroll
    for (int r = 0; r < kStreamRows; ++r) {
      const float4 v = (col_ok && r < cnt) ? *reinterpret_cast<const float4*>(stage + (s * kStreamRows + r) * H + j)
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
      hr[r][0] = v.x; hr[r][1] = v.y; hr[r][2] = v.z; hr[r][3] = v.w;
    }
    // Partial logits of the thread's columns, then the warp's transpose-reduce: 8 rows -> 4 -> 2 -> 1 value
    // per lane while the lane distance halves, then the last two butterfly steps.
#pragma unroll
    for (int c = 0; c < C; ++c) {
      float v[kStreamRows];
#pragma unroll
      for (int r = 0; r < kStreamRows; ++r)
        v[r] = fmaf(hr[r][0], wc[c][0], fmaf(hr[r][1], wc[c][1], fmaf(hr[r][2], wc[c][2], hr[r][3] * wc[c][3])));
      const bool b16 = lane & 16, b8 = lane & 8, b4 = lane & 4;
      float w4[4], w2[2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float recv = __shfl_xor_sync(0xffffffffu, b16 ? v[i] : v[i + 4], 16);
        w4[i] = (b16 ? v[i + 4] : v[i]) + recv;
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float recv = __shfl_xor_sync(0xffffffffu, b8 ? w4[i] : w4[i + 2], 8);
        w2[i] = (b8 ? w4[i + 2] : w4[i]) + recv;
      }
      float y = (b4 ? w2[1] : w2[0]) + __shfl_xor_sync(0xffffffffu, b4 ? w2[0] : w2[1], 4);
      y += __shfl_xor_sync(0xffffffffu, y, 2);
      y += __shfl_xor_sync(0xffffffffu, y, 1);
      // lane l now holds the warp's sum for row ((l>>2)&1) + 2*((l>>3)&1) + 4*((l>>4)&1) = l >> 2
      if ((lane & 3) == 0) red[(((k & 1) * kWarps + warp) * kStreamRows + (lane >> 2)) * C + c] = y;
    }
    // The barrier: the stage has been read by everyone and the partial logits are visible.  It also carries
    // every thread's wait result, so all threads agree on whether to go on.
    aborted = __syncthreads_or(landed ? 0 : 1) != 0;
    if (aborted) break;
    if (tid == 0 && k + kStreamStages < my_batches) issue(k + kStreamStages);
    // Every warp finishes the softmax of all eight rows itself (lane l takes row l & 7; the four copies per
    // row are identical), so there is no second barrier and no phase in which eight threads work while the
    // rest wait; the d(logits) values then travel by shuffle.  red is double-buffered by batch parity: a
    // warp may already write the next batch's partials while a slower one still reads these.
    const int rr = lane & (kStreamRows - 1);
    const int t = r0 + rr;
    float dz[C];
    float lrow = 0.0f;
    {
      float z[C], mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < C; ++c) {
        float a = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) a += red[(((k & 1) * kWarps + w) * kStreamRows + rr) * C + c];
        z[c] = a + bc[c];
        mx = fmaxf(mx, z[c]);
      }
      float den = 0.0f;
#pragma unroll
      for (int c = 0; c < C; ++c) { z[c] = expf(z[c] - mx); den += z[c]; }
      const float inv_den = 1.0f / den;
      const bool token_row = tr.hist != nullptr && t >= tr.rows_v;
      if (!token_row) {
        const int y = rr < cnt ? label[t] : -1;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const float pc = z[c] * inv_den;
          dz[c] = (y >= 0) ? (pc - (c == y ? 1.0f : 0.0f)) * inv_rows : 0.0f;
          if (c == y) lrow = -logf(pc);
          z[c] = pc;
        }
      } else {
        // A token row stands for all leaves that carry the token (they share the hidden row): hist[c] of them have
        // label c, so d(logits) = (count * p - hist) / rows and the loss is -sum_c hist[c] log p[c].
        float hist[C], count = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          hist[c] = rr < cnt ? static_cast<float>(tr.hist[static_cast<long long>(t - tr.rows_v) * kMaxC + c]) : 0.0f;
          count += hist[c];
        }
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const float pc = z[c] * inv_den;
          dz[c] = (count * pc - hist[c]) * inv_rows;
          if (hist[c] > 0.0f) lrow -= hist[c] * logf(pc);
          z[c] = pc;
        }
      }
      if (tid < kStreamRows && tid < cnt) {   // warp 0, one lane per row, publishes the row's results
        loss_acc += lrow;
        float pad[kMaxC];
        if (!token_row) {
          loss[t] = lrow;
          if (dz_out != nullptr) {
#pragma unroll
            for (int c = 0; c < kMaxC; ++c) pad[c] = c < C ? dz[c < C ? c : 0] : 0.0f;
            float4* dst = reinterpret_cast<float4*>(dz_out + static_cast<long long>(t) * kMaxC);
            dst[0] = make_float4(pad[0], pad[1], pad[2], pad[3]);
            dst[1] = make_float4(pad[4], pad[5], pad[6], pad[7]);
          }
        } else {
          // the token's class probabilities: each of its leaves derives its own d(logits) and loss from them
#pragma unroll
          for (int c = 0; c < kMaxC; ++c) pad[c] = c < C ? z[c < C ? c : 0] : 0.0f;
          float4* dst = reinterpret_cast<float4*>(tr.ptok + static_cast<long long>(t - tr.rows_v) * kMaxC);
          dst[0] = make_float4(pad[0], pad[1], pad[2], pad[3]);
          dst[1] = make_float4(pad[4], pad[5], pad[6], pad[7]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kStreamRows; ++r) {
      float d[C];
#pragma unroll
      for (int c = 0; c < C; ++c) d[c] = __shfl_sync(0xffffffffu, dz[c], r);
#pragma unroll
      for (int c = 0; c < C; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) accW[c][e] = fmaf(d[c], hr[r][e], accW[c][e]);
      if (dOut != nullptr && col_ok && r < cnt) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
          for (int e = 0; e < 4; ++e) a[e] = fmaf(d[c], wc[c][e], a[e]);
        __stcs(reinterpret_cast<float4*>(dOut + static_cast<long long>(r0 + r) * H + j), make_float4(a[0], a[1], a[2], a[3]));
      }
      // bias gradient: thread c < C of warp 0 adds d(logits)[r][c], rows in order
#pragma unroll
      for (int c = 0; c < C; ++c)
        if (tid == c) accb += d[c];
    }
  }
  float* mine = partial + static_cast<size_t>(blockIdx.x) * PartialStride(C, H);
  if (col_ok) {
#pragma unroll
    for (int c = 0; c < C; ++c)
      *reinterpret_cast<float4*>(mine + c * H + j) = make_float4(accW[c][0], accW[c][1], accW[c][2], accW[c][3]);
  }
  if (tid < C) mine[C * H + tid] = accb;
  __shared__ float sloss[kStreamRows];
  if (tid < kStreamRows) sloss[tid] = loss_acc;
  __syncthreads();
  if (tid == 0) {
    float sum = 0.0f;
    for (int r = 0; r < kStreamRows; ++r) sum += sloss[r];
    if (aborted) {
      sum = NAN;
      if (status != nullptr) atomicExch(status, 1);
    }
    mine[C * H + C] = sum;
  }
}

// Eight lanes share one output element: lane q sums the partials p = q, q + 8, ... in order, then the eight
// sub-sums are folded in a fixed butterfly, so the result does not depend on the launch shape.
constexpr int kReduceLanes = 8;
__global__ void __launch_bounds__(kThreads)
LossHeadReduce(float* __restrict__ dWc, float* __restrict__ dbc, float* __restrict__ loss_sum,
               const float* __restrict__ partial, int n_parts, int CH, int C, int stride, int accumulate) {
  const int width = CH + C + 1;
  const int q = threadIdx.x % kReduceLanes;
  const int per_cta = kThreads / kReduceLanes;
  const int padded = (width + per_cta - 1) / per_cta * per_cta;   // whole groups stay in the loop together
  for (int i = blockIdx.x * per_cta + threadIdx.x / kReduceLanes; i < padded; i += gridDim.x * per_cta) {
    float s = 0.0f;
    if (i < width)
      for (int p = q; p < n_parts; p += kReduceLanes) s += partial[static_cast<size_t>(p) * stride + i];
#pragma unroll
    for (int o = kReduceLanes / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (q == 0 && i < width) {
      float* dst = i < CH ? dWc + i : (i < CH + C ? dbc + (i - CH) : loss_sum);
      if (dst) *dst = accumulate ? *dst + s : s;
    }
  }
}

int LossGrid(int rows) {
  const int n_blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  return std::max(1, std::min(n_blocks, SmCount() * kCtasPerSm));
}

}  // namespace

namespace {
__global__ void __launch_bounds__(kThreads)
LeafLossFill(float* __restrict__ loss, const float* __restrict__ ptok, const int32_t* __restrict__ tok_slot,
             const int32_t* __restrict__ label, int n_leaf, int C) {
  for (int t = blockIdx.x * kThreads + threadIdx.x; t < n_leaf; t += gridDim.x * kThreads) {
    const int y = label[t];
    loss[t] = (y >= 0 && y < C) ? -logf(ptok[static_cast<size_t>(tok_slot[t]) * kMaxC + y]) : 0.0f;
  }
}
}  // namespace

int LaunchLeafLossFill(float* loss, const float* ptok, const int32_t* tok_slot, const int32_t* label, int n_leaf, int C,
                       cudaStream_t st) {
  if (n_leaf <= 0) return CAVS_OK;
  CAVS_REQUIRE(loss && ptok && tok_slot && label, CAVS_ERR_BAD_ARG, "leaf_loss_fill: null pointer");
  LeafLossFill<<<GridForElems(static_cast<size_t>(n_leaf), kThreads), kThreads, 0, st>>>(loss, ptok, tok_slot, label, n_leaf, C);
  CAVS_LAUNCH_CHECK("leaf_loss_fill");
  return CAVS_OK;
}

bool LossHeadStreams(const float* h, long long h_pitch, int H) {
  return H % 4 == 0 && H <= kThreads * 4 && h_pitch % 4 == 0 && (reinterpret_cast<uintptr_t>(h) & 15u) == 0;
}

size_t LossHeadScratchBytes(int H, int C) {
  return static_cast<size_t>(SmCount()) * kCtasPerSm * PartialStride(C, H) * sizeof(float);
}

int LaunchLossHead(float* loss, float* loss_sum, float* dOut, float* dWc, float* dbc, const float* h, long long h_pitch,
                   const int32_t* label, const float* Wc, const float* bc, int rows, int H, int C, float inv_rows,
                   float* scratch, cudaStream_t st, bool accumulate, float* dz_out, int* status, const int32_t* row_index,
                   LossTokenRows token_rows) {
  CAVS_REQUIRE(rows >= 0 && H > 0 && C > 0, CAVS_ERR_BAD_ARG, "loss_head: bad shape");
  CAVS_REQUIRE(C <= kMaxC, CAVS_ERR_UNSUPPORTED, "loss_head: fused path supports at most 8 classes");
  CAVS_REQUIRE(H <= kThreads * kMaxColsPerThread, CAVS_ERR_UNSUPPORTED, "loss_head: hidden size above 2048");
  CAVS_REQUIRE(loss && (dOut || dz_out) && dWc && dbc && h && label && Wc && bc && scratch, CAVS_ERR_BAD_ARG, "loss_head: null pointer");
  CAVS_REQUIRE((reinterpret_cast<uintptr_t>(dz_out) & 15u) == 0, CAVS_ERR_BAD_ARG, "loss_head: dz rows must be 16-byte aligned");
  // Streaming form: 16-byte aligned rows of at most 1024 floats.
  const bool stream_ok = H % 4 == 0 && H <= kThreads * 4 && h_pitch % 4 == 0 &&
                         ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(dOut) | reinterpret_cast<uintptr_t>(scratch) |
                           reinterpret_cast<uintptr_t>(Wc)) & 15u) == 0;
  CAVS_REQUIRE(token_rows.hist == nullptr || (stream_ok && token_rows.ptok != nullptr && row_index != nullptr), CAVS_ERR_UNSUPPORTED,
               "loss_head: token rows need the streaming form, indexed hidden rows and a probability table");
  CAVS_REQUIRE(row_index == nullptr || stream_ok, CAVS_ERR_UNSUPPORTED,
               "loss_head: indexed hidden rows need the streaming form (hidden a multiple of 4, at most 1024, 16-byte aligned rows)");
  if (stream_ok && rows > 0) {
    const int n_batches = (rows + kStreamRows - 1) / kStreamRows;
    const int sgrid = std::max(1, std::min(n_batches, SmCount() * kCtasPerSm));
    const size_t ssmem = (static_cast<size_t>(kStreamStages) * kStreamRows * H + 2 * kWarps * kStreamRows * C) * sizeof(float);
#define STREAM_CASE(CC)                                                                                              \
  case CC:                                                                                                           \
    if (ssmem > 48 * 1024)                                                                                           \
      CAVS_CUDA(cudaFuncSetAttribute(LossHeadStream<CC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ssmem));  \
    LossHeadStream<CC><<<sgrid, kThreads, ssmem, st>>>(loss, dOut, dz_out, scratch, h, h_pitch, label, Wc, bc, rows, H, inv_rows, status, row_index, token_rows); \
    break;
    switch (C) {
      STREAM_CASE(1) STREAM_CASE(2) STREAM_CASE(3) STREAM_CASE(4) STREAM_CASE(5) STREAM_CASE(6) STREAM_CASE(7) STREAM_CASE(8)
      default: return Fail(CAVS_ERR_UNSUPPORTED, "loss_head: class count");
    }
#undef STREAM_CASE
    CAVS_LAUNCH_CHECK("loss_head stream");
    const int swidth = C * H + C + 1;
    LossHeadReduce<<<std::min((swidth * kReduceLanes + kThreads - 1) / kThreads, 4 * SmCount()), kThreads, 0, st>>>(dWc, dbc, loss_sum, scratch, sgrid, C * H, C, PartialStride(C, H), accumulate ? 1 : 0);
    CAVS_LAUNCH_CHECK("loss_head reduce");
    return CAVS_OK;
  }
  const int grid = rows > 0 ? LossGrid(rows) : 1;
  const size_t smem = (static_cast<size_t>(C) * H + kRowsPerBlock * C + kWarps) * sizeof(float);
  const bool vec4 = H % 4 == 0 && h_pitch % 4 == 0 && ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(dOut) | reinterpret_cast<uintptr_t>(scratch)) & 15u) == 0;
  CAVS_REQUIRE(smem <= 200 * 1024, CAVS_ERR_UNSUPPORTED, "loss_head: classifier does not fit in shared memory");
#define LOSS_LAUNCH(CC, VV, II)                                                                                      \
  do {                                                                                                               \
    if (smem > 48 * 1024)                                                                                            \
      CAVS_CUDA(cudaFuncSetAttribute(LossHeadKernel<CC, VV, II>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    LossHeadKernel<CC, VV, II><<<grid, kThreads, smem, st>>>(loss, dOut, dz_out, scratch, h, h_pitch, label, Wc, bc, rows, H, inv_rows); \
  } while (0)
#define LOSS_CASE(CC)                                                        \
  case CC: {                                                                 \
    if (vec4 && H == 1024) LOSS_LAUNCH(CC, 4, 8);                            \
    else if (vec4 && H == 512) LOSS_LAUNCH(CC, 4, 4);                        \
    else if (vec4 && H == 256) LOSS_LAUNCH(CC, 4, 2);                        \
    else if (vec4) LOSS_LAUNCH(CC, 4, 0);                                    \
    else LOSS_LAUNCH(CC, 1, 0);                                              \
    break;                                                                   \
  }
  switch (C) {
    LOSS_CASE(1) LOSS_CASE(2) LOSS_CASE(3) LOSS_CASE(4) LOSS_CASE(5) LOSS_CASE(6) LOSS_CASE(7) LOSS_CASE(8)
    default: return Fail(CAVS_ERR_UNSUPPORTED, "loss_head: class count");
  }
#undef LOSS_LAUNCH
#undef LOSS_CASE
  CAVS_LAUNCH_CHECK("loss_head");
  const int width = C * H + C + 1;
  LossHeadReduce<<<std::min((width * kReduceLanes + kThreads - 1) / kThreads, 4 * SmCount()), kThreads, 0, st>>>(dWc, dbc, loss_sum, scratch, grid, C * H, C, PartialStride(C, H), accumulate ? 1 : 0);
  CAVS_LAUNCH_CHECK("loss_head reduce");
  return CAVS_OK;
}

}  // namespace cavs_b200

// ---------------------------------------------------------------------------------------------
// Softmax cross-entropy over wide logit rows (language-model heads: classes = vocabulary).
// One CTA per row, three passes over the row held in registers where it fits: max, sum of
// exponentials, then dz = (softmax - onehot) * inv_rows written in place of the logits (and
// optionally as bf16 for the gradient GEMMs).  Replaces cudnnSoftmaxForward + the two
// elementwise kernels + cublasSscal (op_impl_softmax_entropy_logits_loss.cu:106-140,213-250).
// The classifier products around it (logits, dH, dWc) are ordinary GEMMs.
// ---------------------------------------------------------------------------------------------
namespace cavs_b200 {
namespace {

__device__ __forceinline__ float BlockReduce(float v, bool is_max, float* sm) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  __syncthreads();               // sm may still be read by the previous reduction
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  float r = sm[0];
  for (int w = 1; w < kWarps; ++w) r = is_max ? fmaxf(r, sm[w]) : r + sm[w];   // fixed order
  return r;
}

__global__ void __launch_bounds__(kThreads)
SoftmaxXentRows(float* __restrict__ loss, float* __restrict__ z, __nv_bfloat16* __restrict__ dz_bf16, long long ldz,
                const float* __restrict__ bias, const int32_t* __restrict__ label, int rows, int C, float inv_rows) {
  __shared__ float sm[kWarps];
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    float* zr = z + static_cast<long long>(r) * ldz;
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < C; c += kThreads) {
      const float v = zr[c] + (bias ? bias[c] : 0.0f);
      zr[c] = v;
      mx = fmaxf(mx, v);
    }
    mx = BlockReduce(mx, true, sm);
    float den = 0.0f;
    for (int c = threadIdx.x; c < C; c += kThreads) den += expf(zr[c] - mx);
    den = BlockReduce(den, false, sm);
    const int y = label[r];
    const float scale = (y >= 0) ? inv_rows : 0.0f;
    if (threadIdx.x == 0) loss[r] = (y >= 0 && y < C) ? -(zr[y] - mx - logf(den)) : 0.0f;
    __syncthreads();               // loss read zr[y] before it is overwritten below
    for (int c = threadIdx.x; c < C; c += kThreads) {
      const float d = (expf(zr[c] - mx) / den - (c == y ? 1.0f : 0.0f)) * scale;
      zr[c] = d;
      if (dz_bf16) dz_bf16[static_cast<long long>(r) * ldz + c] = __float2bfloat16_rn(d);
    }
  }
}

}  // namespace

int LaunchSoftmaxXentRows(float* loss, float* z, void* dz_bf16, long long ldz, const float* bias, const int32_t* label, int rows,
                          int C, float inv_rows, cudaStream_t st) {
  CAVS_REQUIRE(rows >= 0 && C > 0 && ldz >= C, CAVS_ERR_BAD_ARG, "softmax_xent_rows: bad shape");
  if (rows == 0) return CAVS_OK;
  CAVS_REQUIRE(loss && z && label, CAVS_ERR_BAD_ARG, "softmax_xent_rows: null pointer");
  const int grid = std::min(rows, SmCount() * 8);
  SoftmaxXentRows<<<grid, kThreads, 0, st>>>(loss, z, static_cast<__nv_bfloat16*>(dz_bf16), ldz, bias, label, rows, C, inv_rows);
  CAVS_LAUNCH_CHECK("softmax_xent_rows");
  return CAVS_OK;
}

}  // namespace cavs_b200

// ---------------------------------------------------------------------------------------------
// Loss head for callers that cannot allocate device memory.
//
// Some hosts of this library own the GPU's memory outright: an embedding application that hands
// the whole device to its own pool at start-up, or a step loop that forbids cudaMalloc / cudaFree
// once it is running because both stall the device.  Such a caller can still pass inputs and
// outputs it already owns, but it has nowhere to get the per-CTA partial buffer the loss head
// reduces through.  cavs_fc_softmax_xent_static therefore keeps that buffer inside the library, in
// a fixed-size __device__ array, and calls no allocating routine at all.
//
// The array is per device (every GPU that loads the library holds its kStaticScratchFloats * 4
// bytes until the process exits) and is shared by every call on that device:
//   * calls that may overlap on the GPU (different streams, different threads) race on it;
//     issue them on one stream or order them yourself;
//   * nothing in it has to start at zero -- each launch first overwrites every record the
//     reduction then reads -- so the previous call's leftovers are harmless;
//   * shapes whose partial records do not fit are rejected with CAVS_ERR_CAPACITY.
// The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
// device current) and caches it; make that first call before starting any stream capture.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int kStaticMaxCtas = 296;                  // 148 SMs x 2 resident CTAs on B200
constexpr int kStaticMaxStride = 10240;              // floats per CTA record: classes*hidden + classes + 1, padded
constexpr size_t kStaticScratchFloats = static_cast<size_t>(kStaticMaxCtas) * kStaticMaxStride;   // 12.1 MB

static __device__ __align__(256) float g_loss_head_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
float* g_static_ptr[kMaxDevices] = {};
std::mutex g_static_mu;

// Device address of g_loss_head_scratch on the current device (the host-side symbol is only a
// handle; a kernel must be given this address, never &g_loss_head_scratch).
int StaticScratch(float** out) {
  int dev = 0;
  CAVS_CUDA(cudaGetDevice(&dev));
  CAVS_REQUIRE(dev >= 0 && dev < kMaxDevices, CAVS_ERR_UNSUPPORTED, "fc_softmax_xent_static: device ordinal above 63");
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    CAVS_CUDA(cudaGetSymbolAddress(&p, g_loss_head_scratch));
    g_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_ptr[dev];
  return CAVS_OK;
}

}  // namespace

extern "C" int cavs_fc_softmax_xent_static(float* loss, float* loss_sum, float* dH, float* dWc, float* dbc, const float* h,
                                           long long h_pitch, const int32_t* label, const float* Wc, const float* bc, int rows,
                                           int hidden, int classes, float inv_rows, void* stream) {
  using namespace cavs_b200;
  CAVS_REQUIRE(hidden > 0 && classes > 0, CAVS_ERR_BAD_ARG, "fc_softmax_xent_static: bad shape");
  CAVS_REQUIRE(LossHeadScratchBytes(hidden, classes) <= kStaticScratchFloats * sizeof(float) &&
                   PartialStride(classes, hidden) <= kStaticMaxStride,
               CAVS_ERR_CAPACITY,
               "fc_softmax_xent_static: classes*hidden + classes + 1 = " + std::to_string(classes * hidden + classes + 1) +
                   " floats per partial record exceeds the built-in scratch (" + std::to_string(kStaticMaxStride) +
                   " floats x " + std::to_string(kStaticMaxCtas) + " CTAs); use cavs_fc_softmax_xent with caller scratch");
  float* scratch = nullptr;
  if (int rc = StaticScratch(&scratch)) return rc;
  return LaunchLossHead(loss, loss_sum, dH, dWc, dbc, h, h_pitch, label, Wc, bc, rows, hidden, classes, inv_rows, scratch,
                        static_cast<cudaStream_t>(stream));
}
