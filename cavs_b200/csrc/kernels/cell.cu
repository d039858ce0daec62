// Fused child-sum Tree-LSTM cell, forward and gate-gradient backward, plus the two
// index kernels that feed / drain the per-level gate GEMMs.
//
// Replaces the ~40 per-level launches the reference's vertex function expands to --
// Slice / Add / Sigmoid / Tanh / Mul / Concat / Mirror / Accumulate statements or their
// NVRTC-fused groups (apps/paper/tree-lstm-cavs.cc:129-172,
// cavs/midend/runtime_compiler/code_generator.cc:20-185,
// cavs/backend/op_impl_fused_kernel.cu:62-64) -- by one kernel per direction per level.
// The forward Scatter (op_impl_graphop.cu:108-161) is fused away: the cell writes h|c
// straight into the tensor-id-ordered state array the next level gathers from.  The
// backward Scatter(Child=c) of d(c_child) is fused into the backward cell; d(h_child)
// needs the dgrad GEMM first and is written by ScatterChildGrad.
//
// All kernels are HBM-bound streaming kernels: each thread owns kVec consecutive hidden
// units of one vertex, grids are capped at SMs x resident CTAs and stride over the level.
//
// Gate order in memory: pre-activations from the input projection A are i,o,u,f
// (W's column blocks, tree-lstm-cavs.cc:143-148); the bias is i,f,u,o (:120-123);
// saved gates are i,o,u,f_0..f_{K-1}.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <cstdlib>

#include "abi_common.h"
#include "kernels/bulk.cuh"
#include "kernels/cell.h"
#include "kernels/launch.h"

namespace cavs_b200 {
namespace {

constexpr int kThreads = 256;

template <int V> struct Vec { float v[V]; };

template <int V>
__device__ __forceinline__ Vec<V> LoadF(const float* p) {
  Vec<V> r;
  if constexpr (V == 4) { const float4 t = *reinterpret_cast<const float4*>(p); r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; }
  else if constexpr (V == 2) { const float2 t = *reinterpret_cast<const float2*>(p); r.v[0] = t.x; r.v[1] = t.y; }
  else { r.v[0] = *p; }
  return r;
}
template <int V>
__device__ __forceinline__ Vec<V> LoadF(const __nv_bfloat16* p) {
  Vec<V> r;
  if constexpr (V == 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y;
  } else if constexpr (V == 2) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    r.v[0] = a.x; r.v[1] = a.y;
  } else {
    r.v[0] = __bfloat162float(*p);
  }
  return r;
}
template <int V>
__device__ __forceinline__ Vec<V> LoadF(const __half* p) {
  Vec<V> r;
  if constexpr (V == 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y;
  } else if constexpr (V == 2) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(p));
    r.v[0] = a.x; r.v[1] = a.y;
  } else {
    r.v[0] = __half2float(*p);
  }
  return r;
}
template <int V>
__device__ __forceinline__ Vec<V> Zero() { Vec<V> r; for (int i = 0; i < V; ++i) r.v[i] = 0.0f; return r; }

template <int V>
__device__ __forceinline__ void Store(float* p, const Vec<V>& r) {
  if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  else if constexpr (V == 2) *reinterpret_cast<float2*>(p) = make_float2(r.v[0], r.v[1]);
  else *p = r.v[0];
}
template <int V>
__device__ __forceinline__ void Store(__nv_bfloat16* p, const Vec<V>& r) {
  if constexpr (V == 4) {
    __nv_bfloat162 a = __floats2bfloat162_rn(r.v[0], r.v[1]), b = __floats2bfloat162_rn(r.v[2], r.v[3]);
    uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
  } else if constexpr (V == 2) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(r.v[0], r.v[1]);
  } else {
    *p = __float2bfloat16_rn(r.v[0]);
  }
}

template <int V>
__device__ __forceinline__ void Store(__half* p, const Vec<V>& r) {
  if constexpr (V == 4) {
    __half2 a = __floats2half2_rn(r.v[0], r.v[1]), b = __floats2half2_rn(r.v[2], r.v[3]);
    uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
  } else if constexpr (V == 2) {
    *reinterpret_cast<__half2*>(p) = __floats2half2_rn(r.v[0], r.v[1]);
  } else {
    *p = __float2half_rn(r.v[0]);
  }
}

// Store of a value that is next read much later (the saved gates: written forward, read backward): marked
// evict-first so that it does not push the rows other CTAs re-read (hot token rows, the next level's children)
// out of L2.
template <int V, typename T>
__device__ __forceinline__ void StoreStream(T* p, const Vec<V>& r) { Store<V>(p, r); }
template <>
__device__ __forceinline__ void StoreStream<4, __half>(__half* p, const Vec<4>& r) {
  __half2 a = __floats2half2_rn(r.v[0], r.v[1]), b = __floats2half2_rn(r.v[2], r.v[3]);
  uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
  __stcs(reinterpret_cast<uint2*>(p), u);
}

// Saved gates (values in [-1, 1]) are kept in fp16 in the bf16-GEMM configurations: 11 mantissa
// bits cost ~5e-4 relative in the backward products and halve the largest forward-to-backward
// tensor; the fp32 configurations keep fp32 gates.
template <typename TP> struct GateType { using type = float; };
template <> struct GateType<__nv_bfloat16> { using type = __half; };

// kFast = false: libm-accurate forms (the fp32 configurations must stay within 1e-5 of the
// reference's 1/(1+expf(-x)) and tanhf, cavs/midend/runtime_compiler/expression.h:40-72).
// kFast = true (bf16-GEMM configurations, 2e-2 contract): exp2-unit forms, ~1e-6 absolute error,
// a fraction of the instructions -- the cell kernels are otherwise issue-bound, not HBM-bound.
template <bool kFast>
__device__ __forceinline__ float SigmoidT(float x) {
  return kFast ? __fdividef(1.0f, 1.0f + __expf(-x)) : 1.0f / (1.0f + expf(-x));
}
template <bool kFast>
__device__ __forceinline__ float TanhT(float x) {
  return kFast ? 1.0f - __fdividef(2.0f, __expf(2.0f * x) + 1.0f) : tanhf(x);
}

// S[t] = sum_c h(child_c(t)), HK[t,c] = h(child_c(t)); missing children contribute zeros.
// Gather(Child=c) + Slice + Add of the reference (tree-lstm-cavs.cc:131-136).
template <typename T, int K, int V>
__global__ void __launch_bounds__(kThreads)
GatherChildH(T* __restrict__ S, T* __restrict__ HK, const float* __restrict__ state, int state_pitch,
             const int32_t* __restrict__ child, int n_total, int off, int rows, int H, int chain_early) {
  ChainRelease(chain_early);
  ChainAcquire();
  const int hv = H / V;
  const long long total = static_cast<long long>(rows) * hv;
  const long long stride = static_cast<long long>(gridDim.x) * kThreads;
  for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
    const int b = static_cast<int>(i / hv), j = static_cast<int>(i % hv) * V;
    const int t = off + b;
    Vec<V> s = Zero<V>();
#pragma unroll
    for (int c = 0; c < K; ++c) {
      const int ch = __ldg(child + static_cast<size_t>(c) * n_total + t);
      const Vec<V> h = ch >= 0 ? LoadF<V>(state + static_cast<size_t>(ch) * state_pitch + j) : Zero<V>();
#pragma unroll
      for (int e = 0; e < V; ++e) s.v[e] = (c == 0) ? h.v[e] : s.v[e] + h.v[e];
      Store<V>(HK + (static_cast<size_t>(t) * K + c) * H + j, h);
    }
    Store<V>(S + static_cast<size_t>(t) * H + j, s);
  }
}

// TP: storage type of the gate pre-activations A, P, Q (fp32, or bf16 written by the GEMM epilogue).
template <typename TP, int K, int V, bool kLeaf>
__global__ void __launch_bounds__(kThreads)
CellFwd(float* __restrict__ state, typename GateType<TP>::type* __restrict__ gates, const TP* __restrict__ A, const TP* __restrict__ P,
        const TP* __restrict__ Q, const float* __restrict__ bias, const int32_t* __restrict__ child,
        const int32_t* __restrict__ a_row, int n_total, int off, int rows, int H, int chain_early, int store_leaf_gates,
        int tok_base, typename GateType<TP>::type* __restrict__ gates_f, long long pitch3, long long pitch_f) {
  ChainRelease(chain_early);
  ChainAcquire();
  constexpr bool kFast = sizeof(TP) == 2;
  const int hv = H / V;
  const long long total = static_cast<long long>(rows) * hv;
  const long long stride = static_cast<long long>(gridDim.x) * kThreads;
  for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
    const int b = static_cast<int>(i / hv), j = static_cast<int>(i % hv) * V;
    const size_t t = static_cast<size_t>(off) + b;
    // The input projection depends on the vertex only through its token: with a_row, A holds one row
    // per distinct token and a_row[t] selects it (hot rows stay in L2); without, one row per vertex.
    const size_t ar = a_row ? static_cast<size_t>(__ldg(a_row + t)) : t;
    const TP* a = A + ar * 4 * H + j;
    const Vec<V> ai = LoadF<V>(a), ao = LoadF<V>(a + H), au = LoadF<V>(a + 2 * H), af = kLeaf ? Zero<V>() : LoadF<V>(a + 3 * H);
    const Vec<V> bi = LoadF<V>(bias + j), bf = LoadF<V>(bias + H + j), bu = LoadF<V>(bias + 2 * H + j), bo = LoadF<V>(bias + 3 * H + j);
    Vec<V> pi = Zero<V>(), po = Zero<V>(), pu = Zero<V>();
    if (!kLeaf) {
      if (tok_base >= 0) {
        // A level whose children are all leaves with per-token states (child index = tok_base + token row): the
        // products h_child.U depend on the child's token only, so P holds them once per token, [tokens, 4H] =
        // h_tok.U_iou | h_tok.U_f, and the row's pre-activation is the sum over its children.
#pragma unroll
        for (int c = 0; c < K; ++c) {
          const int ch = __ldg(child + static_cast<size_t>(c) * n_total + t);
          if (ch >= 0) {
            const TP* p = P + static_cast<size_t>(ch - tok_base) * 4 * H + j;
            const Vec<V> xi = LoadF<V>(p), xo = LoadF<V>(p + H), xu = LoadF<V>(p + 2 * H);
#pragma unroll
            for (int e = 0; e < V; ++e) { pi.v[e] += xi.v[e]; po.v[e] += xo.v[e]; pu.v[e] += xu.v[e]; }
          }
        }
      } else {
        const TP* p = P + static_cast<size_t>(b) * 3 * H + j;
        pi = LoadF<V>(p); po = LoadF<V>(p + H); pu = LoadF<V>(p + 2 * H);
      }
    }
    Vec<V> gi, go, gu, cc, hh;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      gi.v[e] = SigmoidT<kFast>((ai.v[e] + pi.v[e]) + bi.v[e]);
      go.v[e] = SigmoidT<kFast>((ao.v[e] + po.v[e]) + bo.v[e]);
      gu.v[e] = TanhT<kFast>((au.v[e] + pu.v[e]) + bu.v[e]);
      cc.v[e] = gi.v[e] * gu.v[e];
    }
    typename GateType<TP>::type* g = gates + t * pitch3 + j;           // i | o | u
    typename GateType<TP>::type* gfp = gates_f + t * pitch_f + j;      // f_0 .. f_{K-1}
    // Leaves have no child cell state: their forget gates multiply zeros in the forward pass and
    // receive a zero gradient in the backward pass, so they are neither computed nor stored.
    if (!kLeaf) {
#pragma unroll
      for (int c = 0; c < K; ++c) {
        const int ch = __ldg(child + static_cast<size_t>(c) * n_total + t);
        const Vec<V> q = tok_base >= 0 ? (ch >= 0 ? LoadF<V>(P + static_cast<size_t>(ch - tok_base) * 4 * H + 3 * H + j) : Zero<V>())
                                       : LoadF<V>(Q + (static_cast<size_t>(b) * K + c) * H + j);
        const Vec<V> cch = ch >= 0 ? LoadF<V>(state + static_cast<size_t>(ch) * 2 * H + H + j) : Zero<V>();
        Vec<V> gf;
#pragma unroll
        for (int e = 0; e < V; ++e) {
          gf.v[e] = SigmoidT<kFast>((af.v[e] + q.v[e]) + bf.v[e]);
          cc.v[e] = cc.v[e] + gf.v[e] * cch.v[e];
        }
        StoreStream<V>(gfp + c * H, gf);
      }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) hh.v[e] = go.v[e] * TanhT<kFast>(cc.v[e]);
    // A leaf's gates are a function of its input-projection row alone: when the backward pass recomputes them
    // (LaunchCellBwd with A), they are not stored.
    if (!kLeaf || store_leaf_gates) { StoreStream<V>(g, gi); StoreStream<V>(g + H, go); StoreStream<V>(g + 2 * H, gu); }
    Store<V>(state + t * 2 * H + j, hh);
    Store<V>(state + t * 2 * H + H + j, cc);
  }
}

// The rest of the forward cell when the gate products' epilogue has already finished the gates (bf16 mode, the
// gate epilogue of the tensor-core GEMM): c = i o u + sum_c f_c o c_c, h = o o tanh(c).  Reads the saved gates
// G3 [n_total, 3H] (i|o|u) and GF [n_total, K, H] and the children's cell states, writes h|c.
template <int K, int V>
__global__ void __launch_bounds__(kThreads)
CellFwdGated(float* __restrict__ state, const __half* __restrict__ G3, const __half* __restrict__ GF,
             const int32_t* __restrict__ child, int n_total, int off, int rows, int H, int chain_early) {
  ChainRelease(chain_early);
  ChainAcquire();
  const int hv = H / V;
  const long long total = static_cast<long long>(rows) * hv;
  const long long stride = static_cast<long long>(gridDim.x) * kThreads;
  for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
    const int b = static_cast<int>(i / hv), j = static_cast<int>(i % hv) * V;
    const size_t t = static_cast<size_t>(off) + b;
    const __half* g = G3 + t * 3 * H + j;
    const Vec<V> gi = LoadF<V>(g), go = LoadF<V>(g + H), gu = LoadF<V>(g + 2 * H);
    Vec<V> cc, hh;
#pragma unroll
    for (int e = 0; e < V; ++e) cc.v[e] = gi.v[e] * gu.v[e];
#pragma unroll
    for (int c = 0; c < K; ++c) {
      const int ch = __ldg(child + static_cast<size_t>(c) * n_total + t);
      if (ch >= 0) {
        const Vec<V> gf = LoadF<V>(GF + (t * K + c) * H + j);
        const Vec<V> cch = LoadF<V>(state + static_cast<size_t>(ch) * 2 * H + H + j);
#pragma unroll
        for (int e = 0; e < V; ++e) cc.v[e] = cc.v[e] + gf.v[e] * cch.v[e];
      }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) hh.v[e] = go.v[e] * TanhT<true>(cc.v[e]);
    Store<V>(state + t * 2 * H + j, hh);
    Store<V>(state + t * 2 * H + H + j, cc);
  }
}

// Thread mapping: tpr = H / V threads cover one row, a CTA covers kThreads / tpr rows per iteration
// and strides over the level, so a thread keeps the same hidden units for its whole life.  That lets
// it accumulate the bias gradient (column sums of zi, zo, zu, sum zf) in registers; at the end the
// CTA folds its rows in a fixed order and adds the result to its own row of dB_part
// ([gridDim.x, 4H], zeroed by the caller before the first level), which a final column sum
// reduces in CTA order.  dB_part == nullptr skips this (H / V > kThreads).
//
// kHead: d(pushed h) is not read from dOut but rebuilt as dz[t,:] . Wc[:, j] from the loss head's
// d(logits) rows (dz, [n_total, 8] zero-padded) and the classifier weights (Wc [C, H], C <= 8), whose
// copy in shared memory -- same fused-multiply-add order as the loss head itself.
template <typename T, int K, int V, bool kLeaf, bool kHead>
__global__ void __launch_bounds__(kThreads)
CellBwd(T* __restrict__ dA, T* __restrict__ ZF, float* __restrict__ mailbox, float* __restrict__ dB_part,
        const float* __restrict__ dOut, const typename GateType<T>::type* __restrict__ gates, const float* __restrict__ state,
        const int32_t* __restrict__ child, const int32_t* __restrict__ parent, int n_total, int off, int rows, int H,
        const float* __restrict__ dz, const float* __restrict__ Wc, int C, int chain_early,
        const T* __restrict__ A, const int32_t* __restrict__ a_row, const float* __restrict__ bias,
        const int32_t* __restrict__ child_state, const typename GateType<T>::type* __restrict__ gates_f, long long pitch3,
        long long pitch_f) {
  ChainRelease(chain_early);
  ChainAcquire();
  __shared__ float fold[kThreads * 4 * V];
  extern __shared__ __align__(16) float s_wc[];   // kHead: the classifier [C, H]
  if (kHead) {
    // All of a thread's loads are issued before the first store: one L2 round trip for the whole copy.
    if (V == 4 && C <= kHeadDzPitch && H <= kThreads * 4 && (reinterpret_cast<uintptr_t>(Wc) & 15u) == 0) {
      float4 w[kHeadDzPitch];
      const int n4 = C * H / 4;
#pragma unroll
      for (int c = 0; c < kHeadDzPitch; ++c) {
        const int i = threadIdx.x + c * kThreads;
        if (i < n4) w[c] = __ldg(reinterpret_cast<const float4*>(Wc) + i);
      }
#pragma unroll
      for (int c = 0; c < kHeadDzPitch; ++c) {
        const int i = threadIdx.x + c * kThreads;
        if (i < n4) reinterpret_cast<float4*>(s_wc)[i] = w[c];
      }
    } else {
      for (int i = threadIdx.x; i < C * H; i += kThreads) s_wc[i] = Wc[i];
    }
    __syncthreads();
  }
  const int tpr = H / V;
  const int rows_per_iter = tpr <= kThreads ? kThreads / tpr : 1;
  const int r_in = tpr <= kThreads ? threadIdx.x / tpr : 0;
  const bool active = r_in < rows_per_iter;
  float sb[4][V];
#pragma unroll
  for (int g4 = 0; g4 < 4; ++g4)
#pragma unroll
    for (int e = 0; e < V; ++e) sb[g4][e] = 0.0f;
  for (int cg0 = (tpr <= kThreads ? threadIdx.x % tpr : threadIdx.x); cg0 < tpr; cg0 += kThreads) {
    const int j = cg0 * V;
    for (long long b = static_cast<long long>(blockIdx.x) * rows_per_iter + r_in; active && b < rows;
         b += static_cast<long long>(gridDim.x) * rows_per_iter) {
      const size_t t = static_cast<size_t>(off) + b;
      const bool has_parent = __ldg(parent + t) >= 0;
      // Gather of d(h|c) left by the parent; roots see zeros (op_impl_graphop.cu:77-86).
      const Vec<V> mh = has_parent ? LoadF<V>(mailbox + t * 2 * H + j) : Zero<V>();
      const Vec<V> mc = has_parent ? LoadF<V>(mailbox + t * 2 * H + H + j) : Zero<V>();
      Vec<V> dOutv;
      if (kHead) {
        const float4 d0 = __ldg(reinterpret_cast<const float4*>(dz + t * kHeadDzPitch));
        const float4 d1 = __ldg(reinterpret_cast<const float4*>(dz + t * kHeadDzPitch) + 1);
        const float dzr[kHeadDzPitch] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
        dOutv = Zero<V>();
        // The thread's classifier columns are re-read from shared memory for every row: keeping them in
        // registers costs a third of the occupancy, and reading them through L1 loses to the streaming data.
        const float* wcol = s_wc + j;
        asm volatile("" : "+l"(wcol));   // opaque per row: stops the loads from being hoisted into registers
#pragma unroll
        for (int c = 0; c < kHeadDzPitch; ++c) {
          if (c < C) {
            const Vec<V> w = LoadF<V>(wcol + static_cast<size_t>(c) * H);
#pragma unroll
            for (int e = 0; e < V; ++e) dOutv.v[e] = fmaf(dzr[c], w.v[e], dOutv.v[e]);
          }
        }
      } else {
        dOutv = LoadF<V>(dOut + t * H + j);
      }
      const typename GateType<T>::type* g = gates + t * pitch3 + j;
      const typename GateType<T>::type* gfp = gates_f + t * pitch_f + j;
      Vec<V> gi, go, gu, cown;
      if (kLeaf && A != nullptr) {
        // Leaf with recomputation: i, o, u and c = i o u follow from the input-projection row (shared by every
        // vertex carrying the token, so mostly an L2 hit) exactly as the forward pass computed them; neither the
        // saved gates nor the saved cell state are read.
        const size_t ar = a_row ? static_cast<size_t>(__ldg(a_row + t)) : t;
        const T* a = A + ar * 4 * H + j;
        const Vec<V> ai = LoadF<V>(a), ao = LoadF<V>(a + H), au = LoadF<V>(a + 2 * H);
        const Vec<V> bi = LoadF<V>(bias + j), bu = LoadF<V>(bias + 2 * H + j), bo = LoadF<V>(bias + 3 * H + j);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          gi.v[e] = SigmoidT<sizeof(T) == 2>((ai.v[e] + 0.0f) + bi.v[e]);
          go.v[e] = SigmoidT<sizeof(T) == 2>((ao.v[e] + 0.0f) + bo.v[e]);
          gu.v[e] = TanhT<sizeof(T) == 2>((au.v[e] + 0.0f) + bu.v[e]);
          cown.v[e] = gi.v[e] * gu.v[e];
        }
      } else {
        gi = LoadF<V>(g); go = LoadF<V>(g + H); gu = LoadF<V>(g + 2 * H);
        cown = LoadF<V>(state + t * 2 * H + H + j);
      }
      Vec<V> zi, zo, zu, dc, zfs = Zero<V>();
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float dh = dOutv.v[e] + mh.v[e];
        const float th = TanhT<sizeof(T) == 2>(cown.v[e]);
        const float d_o = dh * th;
        dc.v[e] = mc.v[e] + (dh * go.v[e]) * (1.0f - th * th);
        zi.v[e] = (dc.v[e] * gu.v[e]) * gi.v[e] * (1.0f - gi.v[e]);
        zo.v[e] = d_o * go.v[e] * (1.0f - go.v[e]);
        zu.v[e] = (dc.v[e] * gi.v[e]) * (1.0f - gu.v[e] * gu.v[e]);
      }
      if (!kLeaf) {
#pragma unroll
        for (int c = 0; c < K; ++c) {
          const int ch = __ldg(child + static_cast<size_t>(c) * n_total + t);
          const Vec<V> gf = LoadF<V>(gfp + c * H);
          Vec<V> z = Zero<V>();
          if (ch >= 0) {
            // c of the child is read from the state array, then d(c_child) = dc * f_c goes to the
            // child's mailbox row (a different array; the child's level runs in a later launch).
            const int chs = child_state ? __ldg(child_state + static_cast<size_t>(c) * n_total + t) : ch;
            const Vec<V> cch = LoadF<V>(state + static_cast<size_t>(chs) * 2 * H + H + j);
            Vec<V> dcc;
#pragma unroll
            for (int e = 0; e < V; ++e) {
              z.v[e] = (dc.v[e] * cch.v[e]) * gf.v[e] * (1.0f - gf.v[e]);
              dcc.v[e] = dc.v[e] * gf.v[e];
              zfs.v[e] += z.v[e];
            }
            Store<V>(mailbox + static_cast<size_t>(ch) * 2 * H + H + j, dcc);
          }
          Store<V>(ZF + (t * K + c) * H + j, z);
        }
      }
      T* d = dA + t * 4 * H + j;
      Store<V>(d, zi); Store<V>(d + H, zo); Store<V>(d + 2 * H, zu); Store<V>(d + 3 * H, zfs);
#pragma unroll
      for (int e = 0; e < V; ++e) { sb[0][e] += zi.v[e]; sb[1][e] += zo.v[e]; sb[2][e] += zu.v[e]; sb[3][e] += zfs.v[e]; }
    }
  }
  if (dB_part == nullptr) return;   // uniform across the grid
  // Fold the CTA's row groups in order, then add into this CTA's partial row.
#pragma unroll
  for (int g4 = 0; g4 < 4; ++g4)
#pragma unroll
    for (int e = 0; e < V; ++e) fold[(threadIdx.x * 4 + g4) * V + e] = sb[g4][e];
  __syncthreads();
  if (r_in == 0 && threadIdx.x < tpr) {
    float* mine = dB_part + static_cast<size_t>(blockIdx.x) * 4 * H;
#pragma unroll
    for (int g4 = 0; g4 < 4; ++g4)
#pragma unroll
      for (int e = 0; e < V; ++e) {
        float acc = 0.0f;
        for (int r = 0; r < rows_per_iter; ++r) acc += fold[((r * tpr + threadIdx.x) * 4 + g4) * V + e];
        mine[g4 * H + threadIdx.x * V + e] += acc;
      }
  }
}

// The backward cell of an internal level in the bf16 configuration with the fused loss-head gradient, as a streaming
// kernel: one producer thread per CTA fetches each row's operands -- mailbox row, saved gates, own and children's cell
// states, d(logits) row -- into shared memory with bulk copies that complete on an mbarrier, kBwdStages rows ahead
// (the row's index entries one further), so DRAM latency is hidden by copies in flight rather than by resident warps:
// the register-heavy arithmetic (80 registers, a third of the warp slots) no longer limits the bytes in flight.
// H / 4 consumer threads own four hidden units each, as in CellBwd, and compute the same expressions in the same
// order.  Every wait is bounded; one that expires raises *status and ends the CTA's loop.
constexpr int kBwdStages = 2;
constexpr int kBwdConsumers = 256;
constexpr int kBwdThreads = kBwdConsumers + 32;

template <int K>
struct BwdStageLayout {
  // byte offsets inside one stage; every array starts on a 16-byte boundary (H a multiple of 8)
  int hdr, dz, mail, g3, gf, cown, cch, bytes;
  __host__ __device__ explicit BwdStageLayout(int H) {
    hdr = 0;                       // int32: parent, child rows (targets of d(c)) ...
    dz = 64;                       // kHeadDzPitch floats
    mail = dz + 32;                // 2H floats: d(h) | d(c) left by the parent
    g3 = mail + 8 * H;             // 3H halves: i | o | u
    gf = g3 + 6 * H;               // K x H halves
    cown = gf + 2 * K * H;         // H floats
    cch = cown + 4 * H;            // K x H floats
    bytes = cch + 4 * K * H;
  }
};

__device__ __forceinline__ void MbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int K>
__global__ void __launch_bounds__(kBwdThreads, 2)
CellBwdStream(__nv_bfloat16* __restrict__ dA, __nv_bfloat16* __restrict__ ZF, float* __restrict__ mailbox, float* __restrict__ dB_part,
              const __half* __restrict__ gates, const __half* __restrict__ gates_f, long long pitch3, long long pitch_f,
              const float* __restrict__ state, const int32_t* __restrict__ child, const int32_t* __restrict__ child_state,
              const int32_t* __restrict__ parent, int n_total, int off, int rows, int H, const float* __restrict__ dz,
              const float* __restrict__ Wc, int C, int chain_early, int* __restrict__ status) {
  ChainRelease(chain_early);
  ChainAcquire();
  extern __shared__ __align__(128) unsigned char bwd_smem[];
  __shared__ __align__(8) unsigned long long full_bar[kBwdStages], empty_bar[kBwdStages];
  const BwdStageLayout<K> lay(H);
  float* s_wc = reinterpret_cast<float*>(bwd_smem);                              // [C, H]
  unsigned char* stages = bwd_smem + ((static_cast<size_t>(C) * H * 4 + 127) / 128) * 128;
  const int tid = threadIdx.x;
  const int tpr = H / 4;                     // consumer threads in use
  const bool consumer = tid < tpr;
  const bool producer = tid == kBwdConsumers;
  for (int i = tid; i < C * H; i += kBwdThreads) s_wc[i] = Wc[i];
  if (tid == 0) {
    for (int s = 0; s < kBwdStages; ++s) {
      bulk::MbarInit(bulk::SmemAddr(&full_bar[s]), 1);
      bulk::MbarInit(bulk::SmemAddr(&empty_bar[s]), tpr);
    }
    bulk::FenceMbarInit();
  }
  __syncthreads();
  const int n_my = blockIdx.x < rows ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  float sb[4][4];
#pragma unroll
  for (int g4 = 0; g4 < 4; ++g4)
#pragma unroll
    for (int e = 0; e < 4; ++e) sb[g4][e] = 0.0f;

  if (producer) {
    int par = -1, ch[K], chs[K];
    auto fetch = [&](int i) {
      const size_t t = static_cast<size_t>(off) + blockIdx.x + static_cast<size_t>(i) * gridDim.x;
      par = __ldg(parent + t);
#pragma unroll
      for (int c = 0; c < K; ++c) {
        ch[c] = __ldg(child + static_cast<size_t>(c) * n_total + t);
        chs[c] = child_state ? __ldg(child_state + static_cast<size_t>(c) * n_total + t) : ch[c];
      }
    };
    if (n_my > 0) fetch(0);
    int issued = 0;
    for (int i = 0; i < n_my; ++i) {
      const int s = i % kBwdStages;
      if (i >= kBwdStages && !bulk::MbarWait(bulk::SmemAddr(&empty_bar[s]), ((i / kBwdStages) - 1) & 1)) {
        if (status != nullptr) atomicExch(status, 1);
        break;
      }
      const size_t t = static_cast<size_t>(off) + blockIdx.x + static_cast<size_t>(i) * gridDim.x;
      const int my_par = par;
      int my_ch[K], my_chs[K];
#pragma unroll
      for (int c = 0; c < K; ++c) { my_ch[c] = ch[c]; my_chs[c] = chs[c]; }
      if (i + 1 < n_my) fetch(i + 1);                      // the next row's index entries travel while this row is issued
      unsigned char* st = stages + static_cast<size_t>(s) * lay.bytes;
      int32_t* hdr = reinterpret_cast<int32_t*>(st + lay.hdr);
      hdr[0] = my_par;
#pragma unroll
      for (int c = 0; c < K; ++c) hdr[1 + c] = my_ch[c];
      uint32_t bytes = 32u + 6u * H + 2u * K * H + 4u * H;
      if (my_par >= 0) bytes += 8u * H;
#pragma unroll
      for (int c = 0; c < K; ++c)
        if (my_ch[c] >= 0) bytes += 4u * H;
      const uint32_t bar = bulk::SmemAddr(&full_bar[s]);
      bulk::MbarExpectTx(bar, bytes);                       // release: the header is visible to whoever sees the phase flip
      bulk::Load(bulk::SmemAddr(st + lay.dz), dz + t * kHeadDzPitch, 32u, bar);
      if (my_par >= 0) bulk::Load(bulk::SmemAddr(st + lay.mail), mailbox + t * 2 * H, 8u * H, bar);
      bulk::Load(bulk::SmemAddr(st + lay.g3), gates + t * pitch3, 6u * H, bar);
      bulk::Load(bulk::SmemAddr(st + lay.gf), gates_f + t * pitch_f, 2u * K * H, bar);
      bulk::Load(bulk::SmemAddr(st + lay.cown), state + t * 2 * H + H, 4u * H, bar);
#pragma unroll
      for (int c = 0; c < K; ++c)
        if (my_ch[c] >= 0)
          bulk::Load(bulk::SmemAddr(st + lay.cch + c * 4 * H), state + static_cast<size_t>(my_chs[c]) * 2 * H + H, 4u * H, bar);
      issued = i + 1;
    }
    // Error path only: copies of rows nobody will consume may still be in flight; wait for them (bounded) before the
    // CTA leaves, so that none lands in shared memory that is no longer this CTA's.
    if (issued < n_my || (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0)) {
      for (int i = max(0, issued - kBwdStages); i < issued; ++i)
        bulk::MbarWait(bulk::SmemAddr(&full_bar[i % kBwdStages]), (i / kBwdStages) & 1);
    }
  } else if (consumer) {
    const int j = tid * 4;
    for (int i = 0; i < n_my; ++i) {
      const int s = i % kBwdStages;
      if (!bulk::MbarWait(bulk::SmemAddr(&full_bar[s]), (i / kBwdStages) & 1)) {
        if (status != nullptr) atomicExch(status, 1);
        break;
      }
      const size_t t = static_cast<size_t>(off) + blockIdx.x + static_cast<size_t>(i) * gridDim.x;
      const unsigned char* st = stages + static_cast<size_t>(s) * lay.bytes;
      const int32_t* hdr = reinterpret_cast<const int32_t*>(st + lay.hdr);
      const bool has_parent = hdr[0] >= 0;
      int ch[K];
#pragma unroll
      for (int c = 0; c < K; ++c) ch[c] = hdr[1 + c];
      const float* sdz = reinterpret_cast<const float*>(st + lay.dz);
      const float4 d0 = *reinterpret_cast<const float4*>(sdz), d1 = *reinterpret_cast<const float4*>(sdz + 4);
      const float dzr[kHeadDzPitch] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
      const float* smail = reinterpret_cast<const float*>(st + lay.mail);
      const Vec<4> mh = has_parent ? LoadF<4>(smail + j) : Zero<4>();
      const Vec<4> mc = has_parent ? LoadF<4>(smail + H + j) : Zero<4>();
      const __half* sg = reinterpret_cast<const __half*>(st + lay.g3);
      const Vec<4> gi = LoadF<4>(sg + j), go = LoadF<4>(sg + H + j), gu = LoadF<4>(sg + 2 * H + j);
      const Vec<4> cown = LoadF<4>(reinterpret_cast<const float*>(st + lay.cown) + j);
      Vec<4> gfv[K], cchv[K];
#pragma unroll
      for (int c = 0; c < K; ++c) {
        gfv[c] = LoadF<4>(reinterpret_cast<const __half*>(st + lay.gf) + c * H + j);
        cchv[c] = ch[c] >= 0 ? LoadF<4>(reinterpret_cast<const float*>(st + lay.cch) + c * H + j) : Zero<4>();
      }
      MbarArrive(bulk::SmemAddr(&empty_bar[s]));             // everything of this stage is in registers
      // d(pushed h) = d(logits) . Wc[:, j]: same fused-multiply-add order as the loss head (see CellBwd)
      Vec<4> dOutv = Zero<4>();
#pragma unroll
      for (int c = 0; c < kHeadDzPitch; ++c) {
        if (c < C) {
          const Vec<4> w = LoadF<4>(s_wc + static_cast<size_t>(c) * H + j);
#pragma unroll
          for (int e = 0; e < 4; ++e) dOutv.v[e] = fmaf(dzr[c], w.v[e], dOutv.v[e]);
        }
      }
      Vec<4> zi, zo, zu, dc, zfs = Zero<4>();
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float dh = dOutv.v[e] + mh.v[e];
        const float th = TanhT<true>(cown.v[e]);
        const float d_o = dh * th;
        dc.v[e] = mc.v[e] + (dh * go.v[e]) * (1.0f - th * th);
        zi.v[e] = (dc.v[e] * gu.v[e]) * gi.v[e] * (1.0f - gi.v[e]);
        zo.v[e] = d_o * go.v[e] * (1.0f - go.v[e]);
        zu.v[e] = (dc.v[e] * gi.v[e]) * (1.0f - gu.v[e] * gu.v[e]);
      }
#pragma unroll
      for (int c = 0; c < K; ++c) {
        Vec<4> z = Zero<4>();
        if (ch[c] >= 0) {
          Vec<4> dcc;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            z.v[e] = (dc.v[e] * cchv[c].v[e]) * gfv[c].v[e] * (1.0f - gfv[c].v[e]);
            dcc.v[e] = dc.v[e] * gfv[c].v[e];
            zfs.v[e] += z.v[e];
          }
          Store<4>(mailbox + static_cast<size_t>(ch[c]) * 2 * H + H + j, dcc);
        }
        Store<4>(ZF + (t * K + c) * H + j, z);
      }
      __nv_bfloat16* d = dA + t * 4 * H + j;
      Store<4>(d, zi); Store<4>(d + H, zo); Store<4>(d + 2 * H, zu); Store<4>(d + 3 * H, zfs);
#pragma unroll
      for (int e = 0; e < 4; ++e) { sb[0][e] += zi.v[e]; sb[1][e] += zo.v[e]; sb[2][e] += zu.v[e]; sb[3][e] += zfs.v[e]; }
    }
  }
  __syncthreads();
  if (dB_part != nullptr && consumer) {
    // one row per CTA iteration, so a thread's sums are final: they go straight into this CTA's partial row
    float* mine = dB_part + static_cast<size_t>(blockIdx.x) * 4 * H;
#pragma unroll
    for (int g4 = 0; g4 < 4; ++g4)
#pragma unroll
      for (int e = 0; e < 4; ++e) mine[g4 * H + tid * 4 + e] += sb[g4][e];
  }
}

// The forward cell of a level whose children are all leaves with per-token states (CellFwd with tok_base >= 0), bf16
// configuration, as a streaming kernel on the scheme of CellBwdStream: per row the producer thread fetches the input
// projection row and, per child, the child token's product row and cell state into shared memory, two rows ahead; the
// bias sits in shared memory for the CTA's life.  Same expressions in the same order as CellFwd.
template <int K>
__global__ void __launch_bounds__(kBwdThreads, 2)
CellFwdTokStream(float* __restrict__ state, __half* __restrict__ gates, __half* __restrict__ gates_f, long long pitch3, long long pitch_f,
                 const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ P, const float* __restrict__ bias,
                 const int32_t* __restrict__ child, const int32_t* __restrict__ a_row, int n_total, int off, int rows, int H,
                 int tok_base, int chain_early, int* __restrict__ status) {
  ChainRelease(chain_early);
  ChainAcquire();
  extern __shared__ __align__(128) unsigned char fwd_smem[];
  __shared__ __align__(8) unsigned long long full_bar[kBwdStages], empty_bar[kBwdStages];
  // stage: header (child rows) | A row (4H bf16) | K product rows (4H bf16 each) | K cell-state rows (H floats each)
  const int o_a = 64, o_p = o_a + 8 * H, o_c = o_p + K * 8 * H, stage_bytes = o_c + K * 4 * H;
  float* s_bias = reinterpret_cast<float*>(fwd_smem);                           // [4H]: i | f | u | o
  unsigned char* stages = fwd_smem + static_cast<size_t>(16) * H;
  const int tid = threadIdx.x;
  const int tpr = H / 4;
  const bool consumer = tid < tpr;
  const bool producer = tid == kBwdConsumers;
  for (int i = tid; i < 4 * H; i += kBwdThreads) s_bias[i] = bias[i];
  if (tid == 0) {
    for (int s = 0; s < kBwdStages; ++s) {
      bulk::MbarInit(bulk::SmemAddr(&full_bar[s]), 1);
      bulk::MbarInit(bulk::SmemAddr(&empty_bar[s]), tpr);
    }
    bulk::FenceMbarInit();
  }
  __syncthreads();
  const int n_my = blockIdx.x < rows ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (producer) {
    int ar = 0, ch[K];
    auto fetch = [&](int i) {
      const size_t t = static_cast<size_t>(off) + blockIdx.x + static_cast<size_t>(i) * gridDim.x;
      ar = a_row ? __ldg(a_row + t) : static_cast<int>(t);
#pragma unroll
      for (int c = 0; c < K; ++c) ch[c] = __ldg(child + static_cast<size_t>(c) * n_total + t);
    };
    if (n_my > 0) fetch(0);
    int issued = 0;
    for (int i = 0; i < n_my; ++i) {
      const int s = i % kBwdStages;
      if (i >= kBwdStages && !bulk::MbarWait(bulk::SmemAddr(&empty_bar[s]), ((i / kBwdStages) - 1) & 1)) {
        if (status != nullptr) atomicExch(status, 1);
        break;
      }
      const int my_ar = ar;
      int my_ch[K];
#pragma unroll
      for (int c = 0; c < K; ++c) my_ch[c] = ch[c];
      if (i + 1 < n_my) fetch(i + 1);
      unsigned char* st = stages + static_cast<size_t>(s) * stage_bytes;
      int32_t* hdr = reinterpret_cast<int32_t*>(st);
      uint32_t bytes = 8u * H;
#pragma unroll
      for (int c = 0; c < K; ++c) {
        hdr[c] = my_ch[c];
        if (my_ch[c] >= 0) bytes += 12u * H;
      }
      const uint32_t bar = bulk::SmemAddr(&full_bar[s]);
      bulk::MbarExpectTx(bar, bytes);
      bulk::Load(bulk::SmemAddr(st + o_a), A + static_cast<size_t>(my_ar) * 4 * H, 8u * H, bar);
#pragma unroll
      for (int c = 0; c < K; ++c)
        if (my_ch[c] >= 0) {
          bulk::Load(bulk::SmemAddr(st + o_p + c * 8 * H), P + static_cast<size_t>(my_ch[c] - tok_base) * 4 * H, 8u * H, bar);
          bulk::Load(bulk::SmemAddr(st + o_c + c * 4 * H), state + static_cast<size_t>(my_ch[c]) * 2 * H + H, 4u * H, bar);
        }
      issued = i + 1;
    }
    if (issued < n_my || (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0)) {
      for (int i = max(0, issued - kBwdStages); i < issued; ++i)
        bulk::MbarWait(bulk::SmemAddr(&full_bar[i % kBwdStages]), (i / kBwdStages) & 1);
    }
  } else if (consumer) {
    const int j = tid * 4;
    const Vec<4> bi = LoadF<4>(s_bias + j), bf = LoadF<4>(s_bias + H + j), bu = LoadF<4>(s_bias + 2 * H + j), bo = LoadF<4>(s_bias + 3 * H + j);
    for (int i = 0; i < n_my; ++i) {
      const int s = i % kBwdStages;
      if (!bulk::MbarWait(bulk::SmemAddr(&full_bar[s]), (i / kBwdStages) & 1)) {
        if (status != nullptr) atomicExch(status, 1);
        break;
      }
      const size_t t = static_cast<size_t>(off) + blockIdx.x + static_cast<size_t>(i) * gridDim.x;
      const unsigned char* st = stages + static_cast<size_t>(s) * stage_bytes;
      const int32_t* hdr = reinterpret_cast<const int32_t*>(st);
      const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(st + o_a) + j;
      const Vec<4> ai = LoadF<4>(a), ao = LoadF<4>(a + H), au = LoadF<4>(a + 2 * H), af = LoadF<4>(a + 3 * H);
      Vec<4> pi = Zero<4>(), po = Zero<4>(), pu = Zero<4>(), q[K], cch[K];
#pragma unroll
      for (int c = 0; c < K; ++c) {
        if (hdr[c] >= 0) {
          const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(st + o_p + c * 8 * H) + j;
          const Vec<4> xi = LoadF<4>(p), xo = LoadF<4>(p + H), xu = LoadF<4>(p + 2 * H);
#pragma unroll
          for (int e = 0; e < 4; ++e) { pi.v[e] += xi.v[e]; po.v[e] += xo.v[e]; pu.v[e] += xu.v[e]; }
          q[c] = LoadF<4>(p + 3 * H);
          cch[c] = LoadF<4>(reinterpret_cast<const float*>(st + o_c + c * 4 * H) + j);
        } else {
          q[c] = Zero<4>();
          cch[c] = Zero<4>();
        }
      }
      MbarArrive(bulk::SmemAddr(&empty_bar[s]));
      Vec<4> gi, go, gu, cc, hh;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        gi.v[e] = SigmoidT<true>((ai.v[e] + pi.v[e]) + bi.v[e]);
        go.v[e] = SigmoidT<true>((ao.v[e] + po.v[e]) + bo.v[e]);
        gu.v[e] = TanhT<true>((au.v[e] + pu.v[e]) + bu.v[e]);
        cc.v[e] = gi.v[e] * gu.v[e];
      }
      __half* g = gates + t * pitch3 + j;
      __half* gfp = gates_f + t * pitch_f + j;
#pragma unroll
      for (int c = 0; c < K; ++c) {
        Vec<4> gf;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          gf.v[e] = SigmoidT<true>((af.v[e] + q[c].v[e]) + bf.v[e]);
          cc.v[e] = cc.v[e] + gf.v[e] * cch[c].v[e];
        }
        StoreStream<4>(gfp + c * H, gf);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) hh.v[e] = go.v[e] * TanhT<true>(cc.v[e]);
      StoreStream<4>(g, gi); StoreStream<4>(g + H, go); StoreStream<4>(g + 2 * H, gu);
      Store<4>(state + t * 2 * H + j, hh);
      Store<4>(state + t * 2 * H + H + j, cc);
    }
  }
}

// mailbox[child_c(t)].h = ds[b] + dq[b,c]: Scatter(Child=c) of the child-state gradient
// (cavs/backend/op_decl_graphop.cc:25-41).
template <int K, int V>
__global__ void __launch_bounds__(kThreads)
ScatterChildGrad(float* __restrict__ mailbox, const float* __restrict__ ds, const float* __restrict__ dq,
                 const int32_t* __restrict__ child, int n_total, int off, int rows, int H, int chain_early) {
  ChainRelease(chain_early);
  ChainAcquire();
  const int hv = H / V;
  const long long total = static_cast<long long>(rows) * hv;
  const long long stride = static_cast<long long>(gridDim.x) * kThreads;
  for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
    const int b = static_cast<int>(i / hv), j = static_cast<int>(i % hv) * V;
    const int t = off + b;
    const Vec<V> s = LoadF<V>(ds + static_cast<size_t>(b) * H + j);
#pragma unroll
    for (int c = 0; c < K; ++c) {
      const int ch = __ldg(child + static_cast<size_t>(c) * n_total + t);
      if (ch < 0) continue;
      const Vec<V> q = LoadF<V>(dq + (static_cast<size_t>(b) * K + c) * H + j);
      Vec<V> r;
#pragma unroll
      for (int e = 0; e < V; ++e) r.v[e] = s.v[e] + q.v[e];
      Store<V>(mailbox + static_cast<size_t>(ch) * 2 * H + j, r);
    }
  }
}

// Per-token sums of the gate gradients dA (the first pass of the segmented sums, one CTA per chunk of at most
// kEmbedChunk rows of one token) with the leaf level's backward cell folded in.  Rows are sorted by token and, within
// a token, by tensor id, and a chunk never mixes leaves and internal vertices:
//   * a chunk of internal vertices sums their stored dA rows (accumulator u takes rows u, u+4, ... in order);
//   * a chunk of leaves never had its dA rows stored: each thread owns four hidden units, rebuilds the token's
//     i, o, u gates and cell state from its input-projection row once, then for every leaf of the chunk reads the
//     parent's d(h|c) from the mailbox and d(logits) (or the stored d(h)), forms zi, zo, zu exactly as CellBwd
//     does, and accumulates them in row order.  The forget-gate block of a leaf is zero.
// Every chunk writes its fp32 sums to partial[chunk, 4H] (their column sums are the bias gradient); a chunk that is
// its token's only one also writes the final row out[token, 4H].
struct LeafGradArgs {
  const float* mailbox;      // [n_total, 2H]
  const float* dOut;         // [n_total, H] or NULL when dz is given
  const float* dz;           // [n_total, kHeadDzPitch] or NULL
  const float* Wc;           // [C, H]
  const float* bias;         // [4H] i,f,u,o
  const int32_t* chunk_seg;  // [n_chunks] token row of A for each chunk
  int C, n_leaf, H;
  const float* ptok;         // [tokens, kHeadDzPitch] class probabilities per token, or NULL (then dz / dOut)
  const int32_t* hist;       // [tokens, kHeadDzPitch] with ptok: how many of the token's leaves carry each label
  float inv_rows;
  // Leaves whose parents sit on a level that hands d(h) down per token instead of per leaf: their entries in
  // `order` carry kOrderNoDh (the h half of their mailbox row is not written), and the token's share dh_tok[token row]
  // ([tokens, H]) is added once, by the token's first chunk (seg_first_chunk[token row]).
  const float* dh_tok;
  const int32_t* seg_first_chunk;
};

// kMode: where a leaf's d(h) comes from -- 0 stored d(h) rows, 1 stored d(logits) rows, 2 the token's class
// probabilities and label histogram (one instantiation each, so no path carries the other paths' registers).
template <typename T, int kMode>
__global__ void __launch_bounds__(kThreads)
TokenGradChunks(float* __restrict__ partial, T* __restrict__ out, const int32_t* __restrict__ chunk_out, const T* __restrict__ dA,
                const T* __restrict__ A, const int32_t* __restrict__ order, const int32_t* __restrict__ chunk_off, LeafGradArgs lg) {
  __shared__ int32_t rows_sm[kEmbedChunk];
  constexpr int V = 4;
  constexpr bool kFast = sizeof(T) == 2;
  const int chunk = blockIdx.x, H = lg.H, width = 4 * H;
  const int begin = chunk_off[chunk], cnt = chunk_off[chunk + 1] - begin;
  const int direct = chunk_out[chunk];
  if (cnt == 0) return;   // an empty chunk's partial row is filled by the caller (column sums kept by the backward cell)
  for (int r = threadIdx.x; r < cnt; r += kThreads) rows_sm[r] = order[begin + r];
  __syncthreads();
  float* mine = partial + static_cast<size_t>(chunk) * width;
  T* final_row = direct >= 0 ? out + static_cast<size_t>(direct) * width : nullptr;
  if ((rows_sm[0] & (kOrderNoDh - 1)) >= lg.n_leaf) {
    // internal vertices: sum the stored rows
    for (int e = threadIdx.x * V; e < width; e += kThreads * V) {
      Vec<V> acc[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] = Zero<V>();
      int r = 0;
      for (; r + 8 <= cnt; r += 8) {
        Vec<V> t[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) t[u] = LoadF<V>(dA + static_cast<size_t>(rows_sm[r + u]) * width + e);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int v = 0; v < V; ++v) acc[u].v[v] += t[u].v[v];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int v = 0; v < V; ++v) acc[u].v[v] += t[u + 4].v[v];
      }
      for (int u = 0; r < cnt; ++r, u = (u + 1) & 3) {
        const Vec<V> t = LoadF<V>(dA + static_cast<size_t>(rows_sm[r]) * width + e);
#pragma unroll
        for (int v = 0; v < V; ++v) acc[u].v[v] += t.v[v];
      }
      Vec<V> sum;
#pragma unroll
      for (int v = 0; v < V; ++v) sum.v[v] = (acc[0].v[v] + acc[1].v[v]) + (acc[2].v[v] + acc[3].v[v]);
      Store<V>(mine + e, sum);
      if (final_row) Store<V>(final_row + e, sum);
    }
    return;
  }
  // leaves of one token
  const T* a = A + static_cast<size_t>(lg.chunk_seg[chunk]) * width;
  if constexpr (kMode == 2) {
    // All leaves of a token share their forward values, so the map from (d(h), d(c)) to the gate gradients is ONE linear
    // map per token: the rows' d(h) and d(c) are summed first (fixed order) and the map is applied once.  The loss
    // head's share of the summed d(h) follows from the token's class probabilities and label histogram,
    //   sum over labelled leaves of (p - onehot(y)) . Wc / rows = (sum_c (n_lab p[c] - hist[c]) Wc[c]) / rows,
    // and enters, like the d(h) handed down per token, through the token's first chunk.
    const int seg = lg.chunk_seg[chunk];
    const bool first = __ldg(lg.seg_first_chunk + seg) == chunk;
    for (int j = threadIdx.x * V; j < H; j += kThreads * V) {
      Vec<V> sh[2], sc[2];
      sh[0] = sh[1] = sc[0] = sc[1] = Zero<V>();
      constexpr int kRows = 4;
      for (int r0 = 0; r0 < cnt; r0 += kRows) {
        Vec<V> mh[kRows], mc[kRows];
#pragma unroll
        for (int u = 0; u < kRows; ++u) {
          if (r0 + u < cnt) {
            const int32_t entry = rows_sm[r0 + u];
            const float* m = lg.mailbox + static_cast<size_t>(entry & (kOrderNoDh - 1)) * 2 * H + j;
            mh[u] = (entry & kOrderNoDh) ? Zero<V>() : LoadF<V>(m);
            mc[u] = LoadF<V>(m + H);
          } else {
            mh[u] = mc[u] = Zero<V>();
          }
        }
#pragma unroll
        for (int u = 0; u < kRows; ++u)
#pragma unroll
          for (int e = 0; e < V; ++e) { sh[u & 1].v[e] += mh[u].v[e]; sc[u & 1].v[e] += mc[u].v[e]; }
      }
      Vec<V> dh, dcm;
#pragma unroll
      for (int e = 0; e < V; ++e) { dh.v[e] = sh[0].v[e] + sh[1].v[e]; dcm.v[e] = sc[0].v[e] + sc[1].v[e]; }
      if (first) {
        const float4 p0 = __ldg(reinterpret_cast<const float4*>(lg.ptok + static_cast<size_t>(seg) * kHeadDzPitch));
        const float4 p1 = __ldg(reinterpret_cast<const float4*>(lg.ptok + static_cast<size_t>(seg) * kHeadDzPitch) + 1);
        const float pk[kHeadDzPitch] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        // the histogram lives in the index tables, which are only 4-byte aligned: scalar loads
        int hk[kHeadDzPitch];
        int n_lab = 0;
#pragma unroll
        for (int c = 0; c < kHeadDzPitch; ++c) { hk[c] = __ldg(lg.hist + static_cast<size_t>(seg) * kHeadDzPitch + c); n_lab += hk[c]; }
        Vec<V> head = Zero<V>();
#pragma unroll
        for (int c = 0; c < kHeadDzPitch; ++c) {
          if (c < lg.C) {
            const Vec<V> w = LoadF<V>(lg.Wc + static_cast<size_t>(c) * H + j);
            const float coef = static_cast<float>(n_lab) * pk[c] - static_cast<float>(hk[c]);
#pragma unroll
            for (int e = 0; e < V; ++e) head.v[e] = fmaf(coef, w.v[e], head.v[e]);
          }
        }
#pragma unroll
        for (int e = 0; e < V; ++e) dh.v[e] += head.v[e] * lg.inv_rows;
        if (lg.dh_tok != nullptr) {
          const Vec<V> dt = LoadF<V>(lg.dh_tok + static_cast<size_t>(seg) * H + j);
#pragma unroll
          for (int e = 0; e < V; ++e) dh.v[e] += dt.v[e];
        }
      }
      const Vec<V> ai = LoadF<V>(a + j), ao = LoadF<V>(a + H + j), au = LoadF<V>(a + 2 * H + j);
      const Vec<V> bi = LoadF<V>(lg.bias + j), bu = LoadF<V>(lg.bias + 2 * H + j), bo = LoadF<V>(lg.bias + 3 * H + j);
      Vec<V> si, so, su;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float gi = SigmoidT<kFast>((ai.v[e] + 0.0f) + bi.v[e]);
        const float go = SigmoidT<kFast>((ao.v[e] + 0.0f) + bo.v[e]);
        const float gu = TanhT<kFast>((au.v[e] + 0.0f) + bu.v[e]);
        const float th = TanhT<kFast>(gi * gu);
        const float dc = dcm.v[e] + (dh.v[e] * go) * (1.0f - th * th);
        si.v[e] = (dc * gu) * gi * (1.0f - gi);
        so.v[e] = (dh.v[e] * th) * go * (1.0f - go);
        su.v[e] = (dc * gi) * (1.0f - gu * gu);
      }
      const Vec<V> zero = Zero<V>();
      Store<V>(mine + j, si); Store<V>(mine + H + j, so); Store<V>(mine + 2 * H + j, su); Store<V>(mine + 3 * H + j, zero);
      if (final_row) {
        Store<V>(final_row + j, si); Store<V>(final_row + H + j, so); Store<V>(final_row + 2 * H + j, su);
        Store<V>(final_row + 3 * H + j, zero);
      }
    }
    return;
  }
  for (int j = threadIdx.x * V; j < H; j += kThreads * V) {
    const Vec<V> ai = LoadF<V>(a + j), ao = LoadF<V>(a + H + j), au = LoadF<V>(a + 2 * H + j);
    const Vec<V> bi = LoadF<V>(lg.bias + j), bu = LoadF<V>(lg.bias + 2 * H + j), bo = LoadF<V>(lg.bias + 3 * H + j);
    Vec<V> gi, go, gu, th;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      gi.v[e] = SigmoidT<kFast>((ai.v[e] + 0.0f) + bi.v[e]);
      go.v[e] = SigmoidT<kFast>((ao.v[e] + 0.0f) + bo.v[e]);
      gu.v[e] = TanhT<kFast>((au.v[e] + 0.0f) + bu.v[e]);
      th.v[e] = TanhT<kFast>(gi.v[e] * gu.v[e]);
    }
    // kMode 0 / 1: every leaf has its own d(h) row or d(logits) row, so the rows are mapped one by one.
    constexpr bool by_dz = kMode == 1;
    Vec<V> wc[kHeadDzPitch];
    if (by_dz) {
#pragma unroll
      for (int c = 0; c < kHeadDzPitch; ++c) wc[c] = c < lg.C ? LoadF<V>(lg.Wc + static_cast<size_t>(c) * H + j) : Zero<V>();
    }
    Vec<V> si = Zero<V>(), so = Zero<V>(), su = Zero<V>();
    // Rows in pairs: the loads of a pair are issued together (a chunk of a frequent token is a long
    // serial loop otherwise), the accumulation stays in row order.
    constexpr int kGroup = 2;
    for (int r0 = 0; r0 < cnt; r0 += kGroup) {
      Vec<V> mh[kGroup], mc[kGroup], dOutv[kGroup];
      float4 d0[kGroup], d1[kGroup];
#pragma unroll
      for (int u = 0; u < kGroup; ++u) {
        // A scheduled leaf always has a parent (a single-vertex sample is never scheduled), so its mailbox row is
        // valid and the loads do not wait for a parent lookup.
        const int32_t entry = rows_sm[r0 + u < cnt ? r0 + u : r0];
        const size_t t = static_cast<size_t>(entry & (kOrderNoDh - 1));
        mh[u] = (entry & kOrderNoDh) ? Zero<V>() : LoadF<V>(lg.mailbox + t * 2 * H + j);
        mc[u] = LoadF<V>(lg.mailbox + t * 2 * H + H + j);
        if (by_dz) {
          d0[u] = __ldg(reinterpret_cast<const float4*>(lg.dz + t * kHeadDzPitch));
          d1[u] = __ldg(reinterpret_cast<const float4*>(lg.dz + t * kHeadDzPitch) + 1);
        } else {
          dOutv[u] = LoadF<V>(lg.dOut + t * H + j);
        }
      }
#pragma unroll
      for (int u = 0; u < kGroup; ++u) {
        if (r0 + u >= cnt) break;
        if (by_dz) {
          const float dzr[kHeadDzPitch] = {d0[u].x, d0[u].y, d0[u].z, d0[u].w, d1[u].x, d1[u].y, d1[u].z, d1[u].w};
          dOutv[u] = Zero<V>();
#pragma unroll
          for (int c = 0; c < kHeadDzPitch; ++c)
#pragma unroll
            for (int e = 0; e < V; ++e) dOutv[u].v[e] = fmaf(dzr[c], wc[c].v[e], dOutv[u].v[e]);
        }
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const float dh = dOutv[u].v[e] + mh[u].v[e];
          const float d_o = dh * th.v[e];
          const float dc = mc[u].v[e] + (dh * go.v[e]) * (1.0f - th.v[e] * th.v[e]);
          si.v[e] += (dc * gu.v[e]) * gi.v[e] * (1.0f - gi.v[e]);
          so.v[e] += d_o * go.v[e] * (1.0f - go.v[e]);
          su.v[e] += (dc * gi.v[e]) * (1.0f - gu.v[e] * gu.v[e]);
        }
      }
    }
    if (lg.dh_tok != nullptr && __ldg(lg.seg_first_chunk + lg.chunk_seg[chunk]) == chunk) {
      // d(h) handed down per token: one more term of the same linear map, with no d(c) of its own
      const Vec<V> dt = LoadF<V>(lg.dh_tok + static_cast<size_t>(lg.chunk_seg[chunk]) * H + j);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float dh = dt.v[e];
        const float dc = (dh * go.v[e]) * (1.0f - th.v[e] * th.v[e]);
        si.v[e] += (dc * gu.v[e]) * gi.v[e] * (1.0f - gi.v[e]);
        so.v[e] += (dh * th.v[e]) * go.v[e] * (1.0f - go.v[e]);
        su.v[e] += (dc * gi.v[e]) * (1.0f - gu.v[e] * gu.v[e]);
      }
    }
    const Vec<V> zero = Zero<V>();
    Store<V>(mine + j, si); Store<V>(mine + H + j, so); Store<V>(mine + 2 * H + j, su); Store<V>(mine + 3 * H + j, zero);
    if (final_row) {
      Store<V>(final_row + j, si); Store<V>(final_row + H + j, so); Store<V>(final_row + 2 * H + j, su);
      Store<V>(final_row + 3 * H + j, zero);
    }
  }
}

// Per-token sums over parent-child links.  Link (t, c) = entry t * K + c of `order` contributes the row
// [ dA[t, 0:3H] | ZF[t * K + c, 0:H] ]: the parent's d(pre-activation) of i, o, u and of the forget gate of that child.
// A chunk is at most kEmbedChunk links of one token (the token of the CHILD), summed in list order; a chunk that is its
// token's only one writes the final row out[chunk_out, 4H], every other chunk its partial row partial[chunk, 4H] (fp32).
template <typename T>
__global__ void __launch_bounds__(kThreads)
LinkSumChunks(float* __restrict__ partial, T* __restrict__ out, const int32_t* __restrict__ chunk_out, const T* __restrict__ dA,
              const T* __restrict__ ZF, const int32_t* __restrict__ order, const int32_t* __restrict__ chunk_off, int H, int K) {
  __shared__ int32_t link_sm[kEmbedChunk];
  __shared__ int32_t row_sm[kEmbedChunk];
  constexpr int V = 4;
  const int chunk = blockIdx.x, width = 4 * H;
  const int begin = chunk_off[chunk], cnt = chunk_off[chunk + 1] - begin;
  if (cnt == 0) return;
  for (int r = threadIdx.x; r < cnt; r += kThreads) {
    const int32_t link = order[begin + r];
    link_sm[r] = link;
    row_sm[r] = link / K;
  }
  __syncthreads();
  const int direct = chunk_out[chunk];
  float* mine = partial + static_cast<size_t>(chunk) * width;
  T* final_row = direct >= 0 ? out + static_cast<size_t>(direct) * width : nullptr;
  for (int e = threadIdx.x * V; e < width; e += kThreads * V) {
    const bool own = e >= 3 * H;                       // the forget-gate block comes from the link's own ZF row
    const T* base = own ? ZF + (e - 3 * H) : dA + e;
    const size_t pitch = own ? H : width;
    const int32_t* idx = own ? link_sm : row_sm;
    Vec<V> acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = Zero<V>();
    int r = 0;
    for (; r + 4 <= cnt; r += 4) {
      Vec<V> t[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) t[u] = LoadF<V>(base + static_cast<size_t>(idx[r + u]) * pitch);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < V; ++v) acc[u].v[v] += t[u].v[v];
    }
    for (int u = 0; r < cnt; ++r, ++u) {
      const Vec<V> t = LoadF<V>(base + static_cast<size_t>(idx[r]) * pitch);
#pragma unroll
      for (int v = 0; v < V; ++v) acc[u].v[v] += t.v[v];
    }
    Vec<V> sum;
#pragma unroll
    for (int v = 0; v < V; ++v) sum.v[v] = (acc[0].v[v] + acc[1].v[v]) + (acc[2].v[v] + acc[3].v[v]);
    // only the second pass reads the partial rows, and it runs over multi-chunk tokens alone
    if (final_row) Store<V>(final_row + e, sum);
    else Store<V>(mine + e, sum);
  }
}

int VecWidth(int H) { return H % 4 == 0 ? 4 : (H % 2 == 0 ? 2 : 1); }


#define DISPATCH_KV(K_, V_, ...)                                             \
  do {                                                                        \
    const int _k = (K_), _v = (V_);                                           \
    if (_k == 1 && _v == 4) { constexpr int K = 1, V = 4; __VA_ARGS__; }             \
    else if (_k == 1 && _v == 2) { constexpr int K = 1, V = 2; __VA_ARGS__; }        \
    else if (_k == 1 && _v == 1) { constexpr int K = 1, V = 1; __VA_ARGS__; }        \
    else if (_k == 2 && _v == 4) { constexpr int K = 2, V = 4; __VA_ARGS__; }        \
    else if (_k == 2 && _v == 2) { constexpr int K = 2, V = 2; __VA_ARGS__; }        \
    else if (_k == 2 && _v == 1) { constexpr int K = 2, V = 1; __VA_ARGS__; }        \
    else if (_k == 3 && _v == 4) { constexpr int K = 3, V = 4; __VA_ARGS__; }        \
    else if (_k == 3 && _v == 2) { constexpr int K = 3, V = 2; __VA_ARGS__; }        \
    else if (_k == 3 && _v == 1) { constexpr int K = 3, V = 1; __VA_ARGS__; }        \
    else if (_k == 4 && _v == 4) { constexpr int K = 4, V = 4; __VA_ARGS__; }        \
    else if (_k == 4 && _v == 2) { constexpr int K = 4, V = 2; __VA_ARGS__; }        \
    else { constexpr int K = 4, V = 1; __VA_ARGS__; }                                \
  } while (0)

int CheckCommon(const char* name, int rows, int H, int K) {
  CAVS_REQUIRE(rows >= 0 && H > 0, CAVS_ERR_BAD_ARG, std::string(name) + ": bad shape");
  CAVS_REQUIRE(K >= 1 && K <= 4, CAVS_ERR_BAD_ARG, std::string(name) + ": child slots must be 1..4");
  return CAVS_OK;
}

}  // namespace

int CellBwdMaxGrid() { return SmCount() * ResidentCtas(kThreads); }
bool CellBwdFusesBias(int H) { return H / VecWidth(H) <= kThreads; }

int LaunchGatherChildH(void* S, void* HK, bool bf16, const float* state, const int32_t* child, int n_total, int off,
                       int rows, int H, int K, cudaStream_t st, int state_pitch) {
  if (state_pitch <= 0) state_pitch = 2 * H;
  if (int rc = CheckCommon("gather_child_h", rows, H, K)) return rc;
  if (rows == 0) return CAVS_OK;
  const int v = VecWidth(H);
  const int grid = GridForElems(static_cast<size_t>(rows) * (H / v), kThreads);
  DISPATCH_KV(K, v, {
    if (bf16) LaunchChained(GatherChildH<__nv_bfloat16, K, V>, dim3(grid), dim3(kThreads), 0, st, static_cast<__nv_bfloat16*>(S), static_cast<__nv_bfloat16*>(HK), state, state_pitch, child, n_total, off, rows, H, ChainEarly());
    else LaunchChained(GatherChildH<float, K, V>, dim3(grid), dim3(kThreads), 0, st, static_cast<float*>(S), static_cast<float*>(HK), state, state_pitch, child, n_total, off, rows, H, ChainEarly());
  });
  CAVS_LAUNCH_CHECK("gather_child_h");
  return CAVS_OK;
}

// Where the forget gates live and the row pitches (in gate elements) of the two parts of the saved gates.
template <typename GT>
struct GateView { GT* f; long long pitch3, pitch_f; };
template <typename GT>
GateView<GT> MakeGateView(const void* gates, const void* gates_f, int H, int K) {
  GT* g = static_cast<GT*>(const_cast<void*>(gates));
  if (gates_f != nullptr) return {static_cast<GT*>(const_cast<void*>(gates_f)), 3LL * H, static_cast<long long>(K) * H};
  return {g + 3LL * H, (3LL + K) * H, (3LL + K) * H};
}

int LaunchCellFwd(float* state, void* gates, const void* A, const void* P, const void* Q, bool preact_bf16, const float* bias,
                  const int32_t* child, const int32_t* a_row, int n_total, int off, int rows, int H, int K, bool leaf, cudaStream_t st,
                  bool store_leaf_gates, int tok_base, void* gates_f, int* status) {
  CAVS_REQUIRE(tok_base < 0 || (!leaf && P != nullptr), CAVS_ERR_BAD_ARG, "treelstm_cell_fwd: per-token products apply to an internal level");
  if (int rc = CheckCommon("treelstm_cell_fwd", rows, H, K)) return rc;
  if (rows == 0) return CAVS_OK;
  const int v = VecWidth(H);
  // The by-token level of the bf16 configuration streams its rows through shared memory (CellFwdTokStream).
  static const bool stream_ok = [] { const char* e = std::getenv("CAVS_CELL_FWD_STREAM"); return !(e != nullptr && e[0] == '0'); }();
  if (stream_ok && preact_bf16 && tok_base >= 0 && !leaf && H % 8 == 0 && H / 4 <= kBwdConsumers && H / 4 >= 128) {
    const GateView<__half> gv = MakeGateView<__half>(gates, gates_f, H, K);
    const bool aligned = ((reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(gates) | reinterpret_cast<uintptr_t>(gv.f) |
                           reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(P) | reinterpret_cast<uintptr_t>(bias)) & 15u) == 0;
    const size_t smem = static_cast<size_t>(16) * H + static_cast<size_t>(kBwdStages) * (64 + 8 * H + static_cast<size_t>(K) * 12 * H);
    if (aligned && smem <= 100 * 1024) {
      const int sgrid = static_cast<int>(std::min<long long>(rows, 2LL * SmCount()));
      DISPATCH_KV(K, 4, {
        (void)V;
        static bool configured[kMaxDevices] = {};
        const int dev = CurrentDevice();
        if (!configured[dev]) {
          CAVS_CUDA(cudaFuncSetAttribute(CellFwdTokStream<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
          configured[dev] = true;
        }
        LaunchChained(CellFwdTokStream<K>, dim3(sgrid), dim3(kBwdThreads), smem, st, state, static_cast<__half*>(gates), gv.f, gv.pitch3,
                      gv.pitch_f, static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(P), bias, child, a_row, n_total, off,
                      rows, H, tok_base, ChainEarly(), status);
      });
      CAVS_LAUNCH_CHECK("treelstm_cell_fwd (streaming)");
      return CAVS_OK;
    }
  }
  const int grid = GridForElems(static_cast<size_t>(rows) * (H / v), kThreads);
  DISPATCH_KV(K, v, {
    if (preact_bf16) {
      using TP = __nv_bfloat16;
      auto* a = static_cast<const TP*>(A); auto* p = static_cast<const TP*>(P); auto* q = static_cast<const TP*>(Q);
      const GateView<__half> gv = MakeGateView<__half>(gates, gates_f, H, K);
      if (leaf) LaunchChained(CellFwd<TP, K, V, true>, dim3(grid), dim3(kThreads), 0, st, state, static_cast<__half*>(gates), a, p, q, bias, child, a_row, n_total, off, rows, H, ChainEarly(), store_leaf_gates ? 1 : 0, tok_base, gv.f, gv.pitch3, gv.pitch_f);
      else LaunchChained(CellFwd<TP, K, V, false>, dim3(grid), dim3(kThreads), 0, st, state, static_cast<__half*>(gates), a, p, q, bias, child, a_row, n_total, off, rows, H, ChainEarly(), store_leaf_gates ? 1 : 0, tok_base, gv.f, gv.pitch3, gv.pitch_f);
    } else {
      auto* a = static_cast<const float*>(A); auto* p = static_cast<const float*>(P); auto* q = static_cast<const float*>(Q);
      const GateView<float> gv = MakeGateView<float>(gates, gates_f, H, K);
      if (leaf) LaunchChained(CellFwd<float, K, V, true>, dim3(grid), dim3(kThreads), 0, st, state, static_cast<float*>(gates), a, p, q, bias, child, a_row, n_total, off, rows, H, ChainEarly(), store_leaf_gates ? 1 : 0, tok_base, gv.f, gv.pitch3, gv.pitch_f);
      else LaunchChained(CellFwd<float, K, V, false>, dim3(grid), dim3(kThreads), 0, st, state, static_cast<float*>(gates), a, p, q, bias, child, a_row, n_total, off, rows, H, ChainEarly(), store_leaf_gates ? 1 : 0, tok_base, gv.f, gv.pitch3, gv.pitch_f);
    }
  });
  CAVS_LAUNCH_CHECK("treelstm_cell_fwd");
  return CAVS_OK;
}

int LaunchCellFwdGated(float* state, const void* gates3, const void* gates_f, const int32_t* child, int n_total, int off, int rows,
                       int H, int K, cudaStream_t st) {
  if (int rc = CheckCommon("treelstm_cell_fwd_gated", rows, H, K)) return rc;
  if (rows == 0) return CAVS_OK;
  CAVS_REQUIRE(state && gates3 && gates_f && child, CAVS_ERR_BAD_ARG, "treelstm_cell_fwd_gated: null pointer");
  const int v = VecWidth(H);
  const int grid = GridForElems(static_cast<size_t>(rows) * (H / v), kThreads);
  DISPATCH_KV(K, v, {
    LaunchChained(CellFwdGated<K, V>, dim3(grid), dim3(kThreads), 0, st, state, static_cast<const __half*>(gates3),
                  static_cast<const __half*>(gates_f), child, n_total, off, rows, H, ChainEarly());
  });
  CAVS_LAUNCH_CHECK("treelstm_cell_fwd_gated");
  return CAVS_OK;
}

int CellBwdGrid(int rows, int H) {
  const int v = VecWidth(H), tpr = H / v;
  const int rows_per_iter = tpr <= kThreads ? kThreads / tpr : 1;
  const long long want = (static_cast<long long>(rows) + rows_per_iter - 1) / rows_per_iter;
  return static_cast<int>(std::max(1LL, std::min<long long>(want, CellBwdMaxGrid())));
}

int LaunchCellBwd(void* dA, void* ZF, bool bf16, float* mailbox, float* dB_part, const float* dOut, const void* gates,
                  const float* state, const int32_t* child, const int32_t* parent, int n_total, int off, int rows, int H,
                  int K, bool leaf, cudaStream_t st, const float* dz, const float* Wc, int C, const void* A,
                  const int32_t* a_row, const float* bias, const int32_t* child_state, const void* gates_f, int* status) {
  if (int rc = CheckCommon("treelstm_cell_bwd", rows, H, K)) return rc;
  if (rows == 0) return CAVS_OK;
  const bool head = dz != nullptr;
  CAVS_REQUIRE(A == nullptr || (leaf && bias != nullptr), CAVS_ERR_BAD_ARG,
               "treelstm_cell_bwd: gate recomputation applies to leaf levels and needs the bias");
  CAVS_REQUIRE(head ? (Wc && C >= 1 && C <= kHeadDzPitch && (reinterpret_cast<uintptr_t>(dz) & 15u) == 0) : dOut != nullptr,
               CAVS_ERR_BAD_ARG, "treelstm_cell_bwd: needs dOut, or 16-byte aligned dz rows with Wc and 1..8 classes");
  const int v = VecWidth(H);
  CAVS_REQUIRE(dB_part == nullptr || H / v <= kThreads, CAVS_ERR_UNSUPPORTED,
               "treelstm_cell_bwd: the fused bias gradient needs hidden / vector width <= 256");
  const size_t head_smem = head ? static_cast<size_t>(C) * H * sizeof(float) : 0;
  CAVS_REQUIRE(head_smem <= 32 * 1024, CAVS_ERR_UNSUPPORTED, "treelstm_cell_bwd: classifier above 32 KB (classes * hidden <= 8192)");
  // Internal levels of the bf16 configuration with the fused loss-head gradient stream their rows through shared
  // memory (CellBwdStream) when the rows are wide enough to keep a CTA's consumers busy and 16-byte granular.
  static const bool stream_ok = [] { const char* v = std::getenv("CAVS_CELL_BWD_STREAM"); return !(v != nullptr && v[0] == '0'); }();
  if (stream_ok && bf16 && !leaf && head && A == nullptr && H % 8 == 0 && H / 4 <= kBwdConsumers && H / 4 >= 128 && dB_part != nullptr) {
    const GateView<__half> gv = MakeGateView<__half>(gates, gates_f, H, K);
    const bool aligned = ((reinterpret_cast<uintptr_t>(mailbox) | reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(gates) |
                           reinterpret_cast<uintptr_t>(gv.f) | reinterpret_cast<uintptr_t>(dz) | reinterpret_cast<uintptr_t>(dA) |
                           reinterpret_cast<uintptr_t>(ZF)) & 15u) == 0;
    if (aligned) {
      size_t smem = 0;
      DISPATCH_KV(K, 4, { (void)V; smem = (head_smem + 127) / 128 * 128 + static_cast<size_t>(kBwdStages) * BwdStageLayout<K>(H).bytes; });
      if (smem <= 100 * 1024) {
        const int sgrid = static_cast<int>(std::min<long long>(rows, 2LL * SmCount()));
        DISPATCH_KV(K, 4, {
          (void)V;
          static bool configured[kMaxDevices] = {};
          const int dev = CurrentDevice();
          if (!configured[dev]) {
            CAVS_CUDA(cudaFuncSetAttribute(CellBwdStream<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
            configured[dev] = true;
          }
          LaunchChained(CellBwdStream<K>, dim3(sgrid), dim3(kBwdThreads), smem, st, static_cast<__nv_bfloat16*>(dA),
                        static_cast<__nv_bfloat16*>(ZF), mailbox, dB_part, static_cast<const __half*>(gates),
                        static_cast<const __half*>(gv.f), gv.pitch3, gv.pitch_f, state, child, child_state, parent, n_total, off, rows, H,
                        dz, Wc, C, ChainEarly(), status);
        });
        CAVS_LAUNCH_CHECK("treelstm_cell_bwd (streaming)");
        return CAVS_OK;
      }
    }
  }
  const int grid = CellBwdGrid(rows, H);
#define CELL_BWD(TT, GT, LEAF, HEAD)                                                                                   \
  do {                                                                                                                 \
    const GateView<GT> gv = MakeGateView<GT>(gates, gates_f, H, K);                                                    \
    LaunchChained(CellBwd<TT, K, V, LEAF, HEAD>, dim3(grid), dim3(kThreads), head_smem, st, static_cast<TT*>(dA), static_cast<TT*>(ZF), mailbox, dB_part, dOut, \
                                                           static_cast<const GT*>(gates), state, child, parent, n_total, off,  \
                                                           rows, H, dz, Wc, C, ChainEarly(), static_cast<const TT*>(A), a_row, bias, child_state, \
                                                           static_cast<const GT*>(gv.f), gv.pitch3, gv.pitch_f);       \
  } while (0)
  DISPATCH_KV(K, v, {
    if (bf16) {
      if (leaf) { if (head) CELL_BWD(__nv_bfloat16, __half, true, true); else CELL_BWD(__nv_bfloat16, __half, true, false); }
      else { if (head) CELL_BWD(__nv_bfloat16, __half, false, true); else CELL_BWD(__nv_bfloat16, __half, false, false); }
    } else {
      if (leaf) { if (head) CELL_BWD(float, float, true, true); else CELL_BWD(float, float, true, false); }
      else { if (head) CELL_BWD(float, float, false, true); else CELL_BWD(float, float, false, false); }
    }
  });
#undef CELL_BWD
  CAVS_LAUNCH_CHECK("treelstm_cell_bwd");
  return CAVS_OK;
}

int LaunchTokenGradChunks(float* partial, void* out, bool bf16, const int32_t* chunk_out, const void* dA, const void* A,
                          const int32_t* order, const int32_t* chunk_off, const int32_t* chunk_seg, int n_chunks,
                          const float* mailbox, const float* dOut, const float* dz, const float* Wc, int C, const float* bias,
                          int n_leaf, int H, cudaStream_t st, const float* ptok, const int32_t* hist, float inv_rows,
                          const float* dh_tok, const int32_t* seg_first_chunk) {
  CAVS_REQUIRE(n_chunks >= 0 && H > 0 && H % 4 == 0, CAVS_ERR_BAD_ARG, "token_grad_chunks: hidden must be a positive multiple of 4");
  CAVS_REQUIRE((dh_tok == nullptr && ptok == nullptr) || seg_first_chunk != nullptr, CAVS_ERR_BAD_ARG,
               "token_grad_chunks: per-token terms need the tokens' first chunks");
  if (n_chunks == 0) return CAVS_OK;
  CAVS_REQUIRE(partial && out && chunk_out && dA && A && order && chunk_off && chunk_seg && mailbox && bias &&
                   ((dz || ptok) ? (Wc && C >= 1 && C <= kHeadDzPitch && (!ptok || hist)) : dOut != nullptr),
               CAVS_ERR_BAD_ARG, "token_grad_chunks: null pointer");
  LeafGradArgs lg{mailbox, dOut, dz, Wc, bias, chunk_seg, C, n_leaf, H, ptok, hist, inv_rows, dh_tok, seg_first_chunk};
#define TOKEN_GRAD(TT, MODE)                                                                                              \
  TokenGradChunks<TT, MODE><<<n_chunks, kThreads, 0, st>>>(partial, static_cast<TT*>(out), chunk_out, static_cast<const TT*>(dA), \
                                                           static_cast<const TT*>(A), order, chunk_off, lg)
  const int mode = ptok ? 2 : (dz ? 1 : 0);
  if (bf16) {
    if (mode == 2) TOKEN_GRAD(__nv_bfloat16, 2); else if (mode == 1) TOKEN_GRAD(__nv_bfloat16, 1); else TOKEN_GRAD(__nv_bfloat16, 0);
  } else {
    if (mode == 2) TOKEN_GRAD(float, 2); else if (mode == 1) TOKEN_GRAD(float, 1); else TOKEN_GRAD(float, 0);
  }
#undef TOKEN_GRAD
  CAVS_LAUNCH_CHECK("token_grad_chunks");
  return CAVS_OK;
}

int LaunchLinkSumChunks(float* partial, void* out, bool bf16, const int32_t* chunk_out, const void* dA, const void* ZF,
                        const int32_t* order, const int32_t* chunk_off, int n_chunks, int H, int K, cudaStream_t st) {
  CAVS_REQUIRE(n_chunks >= 0 && H > 0 && H % 4 == 0 && K >= 1 && K <= 4, CAVS_ERR_BAD_ARG, "link_sum_chunks: bad shape");
  if (n_chunks == 0) return CAVS_OK;
  CAVS_REQUIRE(partial && out && chunk_out && dA && ZF && order && chunk_off, CAVS_ERR_BAD_ARG, "link_sum_chunks: null pointer");
  if (bf16)
    LinkSumChunks<__nv_bfloat16><<<n_chunks, kThreads, 0, st>>>(partial, static_cast<__nv_bfloat16*>(out), chunk_out,
                                                                static_cast<const __nv_bfloat16*>(dA),
                                                                static_cast<const __nv_bfloat16*>(ZF), order, chunk_off, H, K);
  else
    LinkSumChunks<float><<<n_chunks, kThreads, 0, st>>>(partial, static_cast<float*>(out), chunk_out, static_cast<const float*>(dA),
                                                        static_cast<const float*>(ZF), order, chunk_off, H, K);
  CAVS_LAUNCH_CHECK("link_sum_chunks");
  return CAVS_OK;
}

int LaunchScatterChildGrad(float* mailbox, const float* ds, const float* dq, const int32_t* child, int n_total, int off,
                           int rows, int H, int K, cudaStream_t st) {
  if (int rc = CheckCommon("scatter_child_grad", rows, H, K)) return rc;
  if (rows == 0) return CAVS_OK;
  const int v = VecWidth(H);
  const int grid = GridForElems(static_cast<size_t>(rows) * (H / v), kThreads);
  DISPATCH_KV(K, v, { LaunchChained(ScatterChildGrad<K, V>, dim3(grid), dim3(kThreads), 0, st, mailbox, ds, dq, child, n_total, off, rows, H, ChainEarly()); });
  CAVS_LAUNCH_CHECK("scatter_child_grad");
  return CAVS_OK;
}

}  // namespace cavs_b200
