// Fused child-sum Tree-GRU cell kernels (an extension: the reference has no GRU vertex function;
// the definition is the CPU oracle's, oracle/cavs_oracle.c).  Per vertex, with children h_k:
//   ht = sum_k h_k                         r_k = sigmoid((a_r + h_k U_r) + b_r)
//   z  = sigmoid((a_z + ht U_z) + b_z)     m   = sum_k r_k o h_k
//   n  = tanh((a_n + m U_n) + b_n)         h   = (1 - z) o ht + z o n
// a = x.W comes from the per-token input projection (one row per distinct token, read through
// a_row); the three recurrent products are GEMMs between these kernels.  The state row is h only.
// Same structure as the Tree-LSTM kernels (kernels/cell.cu): HBM-bound, one thread per kVec hidden
// units of one vertex, grids capped at SMs x resident CTAs.
#include <cuda_bf16.h>

#include <cstdint>

#include "abi_common.h"
#include "kernels/gru.h"
#include "kernels/launch.h"

namespace cavs_b200 {
namespace {

constexpr int kThreads = 256;

template <typename T> __device__ __forceinline__ float Ld(const T* p);
template <> __device__ __forceinline__ float Ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float Ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void St(T* p, float v);
template <> __device__ __forceinline__ void St<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void St<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float Sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

#define GRU_LOOP(rows, H)                                                                        \
  const long long total = static_cast<long long>(rows) * (H);                                    \
  const long long stride = static_cast<long long>(gridDim.x) * kThreads;                         \
  for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride)

// r_k and m = sum_k r_k o h_k for the level's rows.  R [n_total,K,H] fp32 (saved), M [n_total,H] (GEMM operand).
template <typename T, int K>
__global__ void __launch_bounds__(kThreads)
GruGateR(float* __restrict__ R, T* __restrict__ M, const T* __restrict__ A, const T* __restrict__ PR,
         const float* __restrict__ bias, const float* __restrict__ state, const int32_t* __restrict__ child,
         const int32_t* __restrict__ a_row, int n_total, int off, int rows, int H) {
  GRU_LOOP(rows, H) {
    const int b = static_cast<int>(i / H), j = static_cast<int>(i % H);
    const size_t t = static_cast<size_t>(off) + b;
    const float ar = Ld(A + static_cast<size_t>(a_row ? a_row[t] : t) * 3 * H + j) , br = bias[j];
    float m = 0.0f;
#pragma unroll
    for (int c = 0; c < K; ++c) {
      const int ch = child[static_cast<size_t>(c) * n_total + t];
      const float hc = ch >= 0 ? state[static_cast<size_t>(ch) * H + j] : 0.0f;
      const float r = Sigmoid((ar + Ld(PR + (static_cast<size_t>(b) * K + c) * H + j)) + br);
      R[(t * K + c) * H + j] = r;
      m += r * hc;
    }
    St(M + t * H + j, m);
  }
}

// z, n and the new state.  ZN [n_total,2H] fp32 (saved).  kLeaf: no children (pz = pn = 0, ht = 0).
template <typename T, int K, bool kLeaf>
__global__ void __launch_bounds__(kThreads)
GruOut(float* __restrict__ state, float* __restrict__ ZN, const T* __restrict__ A, const T* __restrict__ PZ,
       const T* __restrict__ PN, const float* __restrict__ bias, const int32_t* __restrict__ child,
       const int32_t* __restrict__ a_row, int n_total, int off, int rows, int H) {
  GRU_LOOP(rows, H) {
    const int b = static_cast<int>(i / H), j = static_cast<int>(i % H);
    const size_t t = static_cast<size_t>(off) + b;
    const T* a = A + static_cast<size_t>(a_row ? a_row[t] : t) * 3 * H + j;
    float ht = 0.0f, pz = 0.0f, pn = 0.0f;
    if (!kLeaf) {
#pragma unroll
      for (int c = 0; c < K; ++c) {
        const int ch = child[static_cast<size_t>(c) * n_total + t];
        const float hc = ch >= 0 ? state[static_cast<size_t>(ch) * H + j] : 0.0f;
        ht = (c == 0) ? hc : ht + hc;
      }
      pz = Ld(PZ + static_cast<size_t>(b) * H + j);
      pn = Ld(PN + static_cast<size_t>(b) * H + j);
    }
    const float z = Sigmoid((Ld(a + H) + pz) + bias[H + j]);
    const float n = tanhf((Ld(a + 2 * H) + pn) + bias[2 * H + j]);
    ZN[t * 2 * H + j] = z;
    ZN[t * 2 * H + H + j] = n;
    state[t * H + j] = (1.0f - z) * ht + z * n;
  }
}

// First backward stage: dh = dOut + parent's message; writes the z / n pre-activation gradients into
// dA's blocks 1, 2 and d(ht) into the level-local dHt; leaves also zero dA's r block.
template <typename T, int K, bool kLeaf>
__global__ void __launch_bounds__(kThreads)
GruBwdA(T* __restrict__ dA, float* __restrict__ dHt, const float* __restrict__ mailbox, const float* __restrict__ dOut,
        const float* __restrict__ ZN, const float* __restrict__ state, const int32_t* __restrict__ child,
        const int32_t* __restrict__ parent, int n_total, int off, int rows, int H) {
  GRU_LOOP(rows, H) {
    const int b = static_cast<int>(i / H), j = static_cast<int>(i % H);
    const size_t t = static_cast<size_t>(off) + b;
    const float dh = dOut[t * H + j] + (parent[t] >= 0 ? mailbox[t * H + j] : 0.0f);
    const float z = ZN[t * 2 * H + j], n = ZN[t * 2 * H + H + j];
    float ht = 0.0f;
    if (!kLeaf) {
#pragma unroll
      for (int c = 0; c < K; ++c) {
        const int ch = child[static_cast<size_t>(c) * n_total + t];
        const float hc = ch >= 0 ? state[static_cast<size_t>(ch) * H + j] : 0.0f;
        ht = (c == 0) ? hc : ht + hc;
      }
    }
    const float zz = (dh * (n - ht)) * z * (1.0f - z);
    const float zn = (dh * z) * (1.0f - n * n);
    St(dA + t * 3 * H + H + j, zz);
    St(dA + t * 3 * H + 2 * H + j, zn);
    if (kLeaf) St(dA + t * 3 * H + j, 0.0f);
    else dHt[static_cast<size_t>(b) * H + j] = dh * (1.0f - z);
  }
}

// Second stage: zr_k = (dm o h_k) r_k (1 - r_k) -> ZR [n_total,K,H] (GEMM operand), dA block 0 = sum_k zr_k.
template <typename T, int K>
__global__ void __launch_bounds__(kThreads)
GruBwdB1(T* __restrict__ dA, T* __restrict__ ZR, const float* __restrict__ dm, const float* __restrict__ R,
         const float* __restrict__ state, const int32_t* __restrict__ child, int n_total, int off, int rows, int H) {
  GRU_LOOP(rows, H) {
    const int b = static_cast<int>(i / H), j = static_cast<int>(i % H);
    const size_t t = static_cast<size_t>(off) + b;
    const float d = dm[static_cast<size_t>(b) * H + j];
    float acc = 0.0f;
#pragma unroll
    for (int c = 0; c < K; ++c) {
      const int ch = child[static_cast<size_t>(c) * n_total + t];
      const float hc = ch >= 0 ? state[static_cast<size_t>(ch) * H + j] : 0.0f;
      const float r = R[(t * K + c) * H + j];
      const float zr = (d * hc) * r * (1.0f - r);
      St(ZR + (t * K + c) * H + j, zr);
      acc += zr;
    }
    St(dA + t * 3 * H + j, acc);
  }
}

// Third stage: mailbox[child_k] = ((d(ht) + dsz) + dm o r_k) + dqr_k.
template <int K>
__global__ void __launch_bounds__(kThreads)
GruBwdB2(float* __restrict__ mailbox, const float* __restrict__ dHt, const float* __restrict__ dsz,
         const float* __restrict__ dm, const float* __restrict__ dqr, const float* __restrict__ R,
         const int32_t* __restrict__ child, int n_total, int off, int rows, int H) {
  GRU_LOOP(rows, H) {
    const int b = static_cast<int>(i / H), j = static_cast<int>(i % H);
    const size_t t = static_cast<size_t>(off) + b;
    const float base = dHt[static_cast<size_t>(b) * H + j] + dsz[static_cast<size_t>(b) * H + j];
    const float d = dm[static_cast<size_t>(b) * H + j];
#pragma unroll
    for (int c = 0; c < K; ++c) {
      const int ch = child[static_cast<size_t>(c) * n_total + t];
      if (ch < 0) continue;
      mailbox[static_cast<size_t>(ch) * H + j] = (base + d * R[(t * K + c) * H + j]) + dqr[(static_cast<size_t>(b) * K + c) * H + j];
    }
  }
}

#define DISPATCH_K(K_, ...)                                \
  do {                                                     \
    switch (K_) {                                          \
      case 1: { constexpr int K = 1; __VA_ARGS__; break; } \
      case 2: { constexpr int K = 2; __VA_ARGS__; break; } \
      case 3: { constexpr int K = 3; __VA_ARGS__; break; } \
      default: { constexpr int K = 4; __VA_ARGS__; break; } \
    }                                                      \
  } while (0)

int Check(const char* name, int rows, int H, int K) {
  CAVS_REQUIRE(rows >= 0 && H > 0 && K >= 1 && K <= 4, CAVS_ERR_BAD_ARG, std::string(name) + ": bad shape");
  return CAVS_OK;
}

}  // namespace

using bf = __nv_bfloat16;

int LaunchGruGateR(float* R, void* M, bool bf16, const void* A, const void* PR, const float* bias, const float* state,
                   const int32_t* child, const int32_t* a_row, int n_total, int off, int rows, int H, int K, cudaStream_t st) {
  if (int rc = Check("gru_gate_r", rows, H, K)) return rc;
  if (rows == 0) return CAVS_OK;
  const int grid = GridForElems(static_cast<size_t>(rows) * H, kThreads);
  DISPATCH_K(K, {
    if (bf16) GruGateR<bf, K><<<grid, kThreads, 0, st>>>(R, static_cast<bf*>(M), static_cast<const bf*>(A), static_cast<const bf*>(PR), bias, state, child, a_row, n_total, off, rows, H);
    else GruGateR<float, K><<<grid, kThreads, 0, st>>>(R, static_cast<float*>(M), static_cast<const float*>(A), static_cast<const float*>(PR), bias, state, child, a_row, n_total, off, rows, H);
  });
  CAVS_LAUNCH_CHECK("gru_gate_r");
  return CAVS_OK;
}

int LaunchGruOut(float* state, float* ZN, bool bf16, const void* A, const void* PZ, const void* PN, const float* bias,
                 const int32_t* child, const int32_t* a_row, int n_total, int off, int rows, int H, int K, bool leaf,
                 cudaStream_t st) {
  if (int rc = Check("gru_out", rows, H, K)) return rc;
  if (rows == 0) return CAVS_OK;
  const int grid = GridForElems(static_cast<size_t>(rows) * H, kThreads);
  DISPATCH_K(K, {
    if (bf16) {
      auto a = static_cast<const bf*>(A); auto pz = static_cast<const bf*>(PZ); auto pn = static_cast<const bf*>(PN);
      if (leaf) GruOut<bf, K, true><<<grid, kThreads, 0, st>>>(state, ZN, a, pz, pn, bias, child, a_row, n_total, off, rows, H);
      else GruOut<bf, K, false><<<grid, kThreads, 0, st>>>(state, ZN, a, pz, pn, bias, child, a_row, n_total, off, rows, H);
    } else {
      auto a = static_cast<const float*>(A); auto pz = static_cast<const float*>(PZ); auto pn = static_cast<const float*>(PN);
      if (leaf) GruOut<float, K, true><<<grid, kThreads, 0, st>>>(state, ZN, a, pz, pn, bias, child, a_row, n_total, off, rows, H);
      else GruOut<float, K, false><<<grid, kThreads, 0, st>>>(state, ZN, a, pz, pn, bias, child, a_row, n_total, off, rows, H);
    }
  });
  CAVS_LAUNCH_CHECK("gru_out");
  return CAVS_OK;
}

int LaunchGruBwdA(void* dA, float* dHt, bool bf16, const float* mailbox, const float* dOut, const float* ZN, const float* state,
                  const int32_t* child, const int32_t* parent, int n_total, int off, int rows, int H, int K, bool leaf,
                  cudaStream_t st) {
  if (int rc = Check("gru_bwd_a", rows, H, K)) return rc;
  if (rows == 0) return CAVS_OK;
  const int grid = GridForElems(static_cast<size_t>(rows) * H, kThreads);
  DISPATCH_K(K, {
    if (bf16) {
      if (leaf) GruBwdA<bf, K, true><<<grid, kThreads, 0, st>>>(static_cast<bf*>(dA), dHt, mailbox, dOut, ZN, state, child, parent, n_total, off, rows, H);
      else GruBwdA<bf, K, false><<<grid, kThreads, 0, st>>>(static_cast<bf*>(dA), dHt, mailbox, dOut, ZN, state, child, parent, n_total, off, rows, H);
    } else {
      if (leaf) GruBwdA<float, K, true><<<grid, kThreads, 0, st>>>(static_cast<float*>(dA), dHt, mailbox, dOut, ZN, state, child, parent, n_total, off, rows, H);
      else GruBwdA<float, K, false><<<grid, kThreads, 0, st>>>(static_cast<float*>(dA), dHt, mailbox, dOut, ZN, state, child, parent, n_total, off, rows, H);
    }
  });
  CAVS_LAUNCH_CHECK("gru_bwd_a");
  return CAVS_OK;
}

int LaunchGruBwdB1(void* dA, void* ZR, bool bf16, const float* dm, const float* R, const float* state, const int32_t* child,
                   int n_total, int off, int rows, int H, int K, cudaStream_t st) {
  if (int rc = Check("gru_bwd_b1", rows, H, K)) return rc;
  if (rows == 0) return CAVS_OK;
  const int grid = GridForElems(static_cast<size_t>(rows) * H, kThreads);
  DISPATCH_K(K, {
    if (bf16) GruBwdB1<bf, K><<<grid, kThreads, 0, st>>>(static_cast<bf*>(dA), static_cast<bf*>(ZR), dm, R, state, child, n_total, off, rows, H);
    else GruBwdB1<float, K><<<grid, kThreads, 0, st>>>(static_cast<float*>(dA), static_cast<float*>(ZR), dm, R, state, child, n_total, off, rows, H);
  });
  CAVS_LAUNCH_CHECK("gru_bwd_b1");
  return CAVS_OK;
}

int LaunchGruBwdB2(float* mailbox, const float* dHt, const float* dsz, const float* dm, const float* dqr, const float* R,
                   const int32_t* child, int n_total, int off, int rows, int H, int K, cudaStream_t st) {
  if (int rc = Check("gru_bwd_b2", rows, H, K)) return rc;
  if (rows == 0) return CAVS_OK;
  const int grid = GridForElems(static_cast<size_t>(rows) * H, kThreads);
  DISPATCH_K(K, { GruBwdB2<K><<<grid, kThreads, 0, st>>>(mailbox, dHt, dsz, dm, dqr, R, child, n_total, off, rows, H); });
  CAVS_LAUNCH_CHECK("gru_bwd_b2");
  return CAVS_OK;
}

}  // namespace cavs_b200
