// bf16 x bf16 -> fp32 GEMM on the Blackwell tensor cores (tcgen05.mma, accumulator in
// TMEM), operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte
// swizzle), written directly in PTX.
//
// This is the only dense contraction of the vertex-function path: the per-level gate
// products, their data gradients, and the once-per-step weight gradients.  The
// reference issues these as cublasSgemm calls (cavs/backend/cublas_wrapper.cc:13-28,
// cavs/backend/op_impl_blas3_cublas.cc:35-70).
//
// Persistent CTAs (one per SM) walk BM x BN output tiles (optionally K-splits of them):
//   warp 0      TMA producer: one elected lane walks the K blocks, filling a ring of stages
//   warp 1      allocates TMEM, one elected lane issues tcgen05.mma and commits to mbarriers
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one 32-lane quarter each) and store
// Two TMEM accumulators alternate so the epilogue of one tile overlaps the next tile's MMAs.
// Operands may be K-major (row-major [rows, K]) or MN-major (row-major [K, rows]); the
// latter is what the weight gradient dW = X^T dY needs, so no transpose pass exists.
// Every mbarrier wait is bounded; on expiry the CTA raises *status and unwinds.
#ifndef CAVS_B200_KERNELS_GEMM_TC_CUH_
#define CAVS_B200_KERNELS_GEMM_TC_CUH_

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels/launch.h"

namespace cavs_b200 {
namespace tc {

constexpr int kBM = 128;        // rows of C per CTA (UMMA M)
constexpr int kBK = 64;         // K elements per stage: 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;      // K per tcgen05.mma for 16-bit inputs
constexpr int kThreads = 192;
constexpr uint32_t kSpinLimit = 1u << 21;

enum Major : int { kMajorK = 0, kMajorMN = 1 };
enum OutMode : int { kStoreF32 = 0, kAccumF32 = 1, kStoreBf16 = 2, kScatterF32 = 3, kGateActF16 = 4 };

struct Params {
  void* c;            // output, row-major
  long long ldc;      // elements
  long long split_stride;  // elements between K-split partial outputs (0 when splits == 1)
  int m, n, k;
  int kb_per_split;   // K blocks per work item
  int out_mode;
  int n_splits;       // K splits per tile (work items = tiles x splits)
  int a_row_off;      // added to the row coordinate of K-major A tiles (a level's view into an arena map)
  int tma_store;      // 1: the epilogue stages C in shared memory and writes it with TMA (map_c valid)
  int chain_early;    // 1: release the following kernel at once (chained launches, kernels/launch.h)
  // kScatterF32: GEMM row r = t * sc_slots + c goes to output row child[c * sc_n_total + sc_off + t] (skipped when
  // negative) after adding sc_addend[t, col]: the child-gradient scatter of a level done by the epilogue.
  const int32_t* sc_child;
  const float* sc_addend;
  long long sc_addend_ld;
  int sc_n_total, sc_off, sc_slots;
  // kGateActF16: the epilogue finishes the LSTM gates instead of storing pre-activations.  GEMM row r belongs to
  // vertex t = act_t_off + r / act_rpv; column n of this product is column act_col0 + n of the gate order i,o,u,f
  // (hidden size act_h per gate).  value = act((acc + act_a[row(t), act_col0 + n]) + bias), sigmoid for i, o, f and
  // tanh for u, stored as fp16 through the output map at row c_row_off + r.  act_a: bf16 [*, 4 act_h] input
  // projection, one row per vertex or per act_a_row[t]; act_bias: [4 act_h] in the order i,f,u,o.
  const void* act_a;
  const int32_t* act_a_row;
  const float* act_bias;
  int act_col0, act_h, act_rpv, act_t_off;
  int c_row_off;      // added to the output row (an output map / pointer over a whole arena); the last 32-row slab of a
                      // bulk-stored product may spill up to 31 rows past row m - 1 of such an arena
  int* status;        // device word, set non-zero when a bounded wait expires
  uint32_t spin_limit;    // polls per bounded wait; 0 = kSpinLimit
  int withhold_loads;     // wait self-test: the producer issues no operand load, so every consumer wait runs out
};

// kMB: 128-row blocks of C per tile.  kMB = 2 (256 x 256 tiles, long-K weight gradients only): the operand bytes a
// CTA pulls out of L2 per flop drop by a third, which is what bounds those GEMMs; the two accumulators fill all
// 512 TMEM columns, so the epilogue is not overlapped with the next tile's MMAs (irrelevant at thousands of
// k-blocks per tile).
template <int kBN, int kMB = 1>
struct Smem {
  static constexpr int kATile = kMB * kBM * kBK * 2;
  static constexpr int kBTile = kBN * kBK * 2;
  static constexpr int kStage = kATile + kBTile;
  static constexpr int kStages = kMB == 2 ? 3 : ((kBN == 256) ? 4 : (kBN == 128 ? 6 : 7));
  // Epilogue staging: 4 warps x 2 slots x (32 rows x 128 bytes), 128-byte swizzled for the TMA store.
  static constexpr int kCSlot = 32 * 128;
  static constexpr int kCOff = kStages * kStage;
  static constexpr int kBarOff = kCOff + 4 * 2 * kCSlot;
  static constexpr int kBytes = kBarOff + 256 + 1024;  // barriers (<= 17 x 8 bytes + TMEM slot) + slack for 1024-byte alignment
};

__device__ __forceinline__ uint32_t SmemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void MbarExpectTx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait on a phase parity: non-blocking polls with a short sleep once the wait
// is clearly not a pipeline hiccup.  Returns false if the limit expired (~0.3 s).
__device__ __forceinline__ bool MbarWait(uint32_t bar, uint32_t parity, uint32_t limit = kSpinLimit) {
  for (uint32_t it = 0; it < limit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if (it > 4096) __nanosleep(128);
  }
  return false;
}
__device__ __forceinline__ void TmaLoad2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ bool ElectOne() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile whose base is
// 1024-byte aligned.  K-major: rows of 128 bytes, 8-row groups 1024 bytes apart (SBO).
// MN-major: 64-element (128-byte) runs along MN per K index, 8 K-indices per 1024-byte
// group (SBO), next 64-element block along MN one whole 64x64 box (8192 bytes) further (LBO).
__device__ __forceinline__ uint64_t SmemDesc(uint32_t addr, int major) {
  const uint64_t start = (addr & 0x3FFFFu) >> 4;
  const uint64_t lbo = (major == kMajorMN) ? (8192u >> 4) : 1u;
  const uint64_t sbo = 1024u >> 4;
  return start | (lbo << 16) | (sbo << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulate, bf16 A and B, given majors, N and M.
__host__ __device__ constexpr uint32_t InstrDesc(int a_major, int b_major, int n, int m) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_major) << 15) |
         (static_cast<uint32_t>(b_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void UmmaBf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void UmmaCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void TmemLoad32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void MbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Two 32-column accumulator chunks per round trip: both loads are issued before the wait.
__device__ __forceinline__ void TmemLoad64(uint32_t taddr, uint32_t (&r)[64]) {
#define CAVS_TMEM_LD32(BASE, ADDR)                                                                                        \
  asm volatile(                                                                                                           \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                           \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                                          \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"                          \
      : "=r"(r[BASE + 0]), "=r"(r[BASE + 1]), "=r"(r[BASE + 2]), "=r"(r[BASE + 3]), "=r"(r[BASE + 4]), "=r"(r[BASE + 5]), \
        "=r"(r[BASE + 6]), "=r"(r[BASE + 7]), "=r"(r[BASE + 8]), "=r"(r[BASE + 9]), "=r"(r[BASE + 10]),                  \
        "=r"(r[BASE + 11]), "=r"(r[BASE + 12]), "=r"(r[BASE + 13]), "=r"(r[BASE + 14]), "=r"(r[BASE + 15]),              \
        "=r"(r[BASE + 16]), "=r"(r[BASE + 17]), "=r"(r[BASE + 18]), "=r"(r[BASE + 19]), "=r"(r[BASE + 20]),              \
        "=r"(r[BASE + 21]), "=r"(r[BASE + 22]), "=r"(r[BASE + 23]), "=r"(r[BASE + 24]), "=r"(r[BASE + 25]),              \
        "=r"(r[BASE + 26]), "=r"(r[BASE + 27]), "=r"(r[BASE + 28]), "=r"(r[BASE + 29]), "=r"(r[BASE + 30]),              \
        "=r"(r[BASE + 31])                                                                                                \
      : "r"(ADDR))
  CAVS_TMEM_LD32(0, taddr);
  CAVS_TMEM_LD32(32, taddr + 32);
#undef CAVS_TMEM_LD32
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void TmaStore2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
// Writes this lane's 128-byte row of a staging slot: eight 16-byte words at 128-byte-swizzled positions.
template <int kBase, int kKind>   // kKind 0: fp32 (32 columns), 1: bf16, 2: fp16 (64 columns)
__device__ __forceinline__ void StageRow(uint32_t slot, int lane, const uint32_t (&r)[64]) {
  const uint32_t row = slot + lane * 128;
  const uint32_t sw = lane & 7;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    uint32_t v0, v1, v2, v3;
    if (kKind == 2) {   // 8 columns -> 16 bytes of fp16
      __half2 t0 = __floats2half2_rn(__uint_as_float(r[kBase + 8 * w + 0]), __uint_as_float(r[kBase + 8 * w + 1]));
      __half2 t1 = __floats2half2_rn(__uint_as_float(r[kBase + 8 * w + 2]), __uint_as_float(r[kBase + 8 * w + 3]));
      __half2 t2 = __floats2half2_rn(__uint_as_float(r[kBase + 8 * w + 4]), __uint_as_float(r[kBase + 8 * w + 5]));
      __half2 t3 = __floats2half2_rn(__uint_as_float(r[kBase + 8 * w + 6]), __uint_as_float(r[kBase + 8 * w + 7]));
      v0 = *reinterpret_cast<uint32_t*>(&t0); v1 = *reinterpret_cast<uint32_t*>(&t1);
      v2 = *reinterpret_cast<uint32_t*>(&t2); v3 = *reinterpret_cast<uint32_t*>(&t3);
    } else if (kKind == 1) {   // 8 columns -> 16 bytes
      __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(r[kBase + 8 * w + 0]), __uint_as_float(r[kBase + 8 * w + 1]));
      __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(r[kBase + 8 * w + 2]), __uint_as_float(r[kBase + 8 * w + 3]));
      __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(r[kBase + 8 * w + 4]), __uint_as_float(r[kBase + 8 * w + 5]));
      __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(r[kBase + 8 * w + 6]), __uint_as_float(r[kBase + 8 * w + 7]));
      v0 = *reinterpret_cast<uint32_t*>(&t0); v1 = *reinterpret_cast<uint32_t*>(&t1);
      v2 = *reinterpret_cast<uint32_t*>(&t2); v3 = *reinterpret_cast<uint32_t*>(&t3);
    } else {       // 4 columns -> 16 bytes
      v0 = r[kBase + 4 * w + 0]; v1 = r[kBase + 4 * w + 1]; v2 = r[kBase + 4 * w + 2]; v3 = r[kBase + 4 * w + 3];
    }
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row + ((w ^ sw) << 4)), "r"(v0), "r"(v1), "r"(v2), "r"(v3) : "memory");
  }
}

// Stores 32 consecutive accumulator columns of one row (registers r[base..base+32)).
template <int kBase>
__device__ __forceinline__ void StoreChunk(const Params& p, const uint32_t (&r)[64], int row, int col0, long long zoff) {
  if (row >= p.m || col0 >= p.n) return;
  if (p.out_mode == kStoreBf16) {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c) + zoff + static_cast<long long>(row + p.c_row_off) * p.ldc + col0;
    if (col0 + 32 <= p.n && (p.ldc & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 v;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(r[kBase + j]), __uint_as_float(r[kBase + j + 1]));
        __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(r[kBase + j + 2]), __uint_as_float(r[kBase + j + 3]));
        __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(r[kBase + j + 4]), __uint_as_float(r[kBase + j + 5]));
        __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(r[kBase + j + 6]), __uint_as_float(r[kBase + j + 7]));
        v.x = *reinterpret_cast<uint32_t*>(&t0); v.y = *reinterpret_cast<uint32_t*>(&t1);
        v.z = *reinterpret_cast<uint32_t*>(&t2); v.w = *reinterpret_cast<uint32_t*>(&t3);
        *reinterpret_cast<uint4*>(dst + j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.n) dst[j] = __float2bfloat16_rn(__uint_as_float(r[kBase + j]));
    }
  } else {
    float* dst = static_cast<float*>(p.c) + zoff + static_cast<long long>(row + p.c_row_off) * p.ldc + col0;
    const bool acc = p.out_mode == kAccumF32;
    if (col0 + 32 <= p.n && (p.ldc & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 v = make_float4(__uint_as_float(r[kBase + j]), __uint_as_float(r[kBase + j + 1]),
                               __uint_as_float(r[kBase + j + 2]), __uint_as_float(r[kBase + j + 3]));
        if (acc) {
          const float4 o = *reinterpret_cast<const float4*>(dst + j);
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
        *reinterpret_cast<float4*>(dst + j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.n) dst[j] = (acc ? dst[j] : 0.0f) + __uint_as_float(r[kBase + j]);
    }
  }
}

// Gate epilogue (kGateActF16): turns this lane's 64 accumulator columns into finished gates,
//   gate_j = act((acc_j + a_j) + b_j),
// and leaves them packed as 32 half2 words in r[0..32).  A 64-column step lies inside one gate block (act_h is a
// multiple of 64).  The pre-activation is summed in fp32; the activation itself runs on packed fp16 pairs with the
// special-function unit's tanh (one operation per two gates; sigmoid(x) = 0.5 tanh(0.5 x) + 0.5): the gates are
// stored as fp16 anyway, and an epilogue warp has its scheduler to itself, so instruction and special-function
// counts decide whether the epilogue hides under the next tile's products.
__device__ __forceinline__ uint32_t TanhHalf2(uint32_t x) {
  uint32_t y;
  asm("tanh.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ void GateActivate(const Params& p, uint32_t (&r)[64], int row, int col0) {
  const int gcol = p.act_col0 + col0;
  const int g = gcol / p.act_h, j = gcol - g * p.act_h;
  const int bias_block = g == 0 ? 0 : (g == 1 ? 3 : (g == 2 ? 2 : 1));   // gates i,o,u,f <- bias i,f,u,o
  const float* bias = p.act_bias + bias_block * p.act_h + j;
  const int t = p.act_t_off + row / p.act_rpv;
  const size_t ar = p.act_a_row != nullptr ? static_cast<size_t>(__ldg(p.act_a_row + t)) : static_cast<size_t>(t);
  const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(p.act_a) + ar * 4 * p.act_h + gcol;
  const bool is_tanh = g == 2;
  const __half2 half = __floats2half2_rn(0.5f, 0.5f);
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const uint4 av = __ldg(reinterpret_cast<const uint4*>(a + 8 * q));
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias + 8 * q));
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(bias + 8 * q) + 1);
    const float2 a01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&av.x));
    const float2 a23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&av.y));
    const float2 a45 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&av.z));
    const float2 a67 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&av.w));
    const float av8[8] = {a01.x, a01.y, a23.x, a23.y, a45.x, a45.y, a67.x, a67.y};
    const float bv8[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      const float x0 = (av8[e] + __uint_as_float(r[8 * q + e])) + bv8[e];
      const float x1 = (av8[e + 1] + __uint_as_float(r[8 * q + e + 1])) + bv8[e + 1];
      __half2 x = __floats2half2_rn(x0, x1);
      if (!is_tanh) x = __hmul2(x, half);
      const uint32_t th = TanhHalf2(*reinterpret_cast<uint32_t*>(&x));
      __half2 y = *reinterpret_cast<const __half2*>(&th);
      if (!is_tanh) y = __hfma2(y, half, half);
      r[4 * q + e / 2] = *reinterpret_cast<uint32_t*>(&y);   // slot 4q + e/2 <= 8q + e: never ahead of the reads
    }
  }
}
// Writes this lane's 128-byte row of already packed 16-bit pairs (r[0..32)) at 128-byte-swizzled positions.
__device__ __forceinline__ void StageRowPacked(uint32_t slot, int lane, const uint32_t (&r)[64]) {
  const uint32_t row = slot + lane * 128;
  const uint32_t sw = lane & 7;
#pragma unroll
  for (int w = 0; w < 8; ++w)
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row + ((w ^ sw) << 4)), "r"(r[4 * w]), "r"(r[4 * w + 1]),
                 "r"(r[4 * w + 2]), "r"(r[4 * w + 3]) : "memory");
}

// Scatter epilogue.  A lane serves row i = it * 4 + lane / 8 of the warp's 32 rows (it = 0..7) and the 16-byte
// column group lane % 8, so eight lanes cover a row's 128 bytes and every global access is a full line.
// ScatterTargets: output row and addend row of the lane's eight rows, loaded once per tile.
__device__ __forceinline__ void ScatterTargets(const Params& p, int lane, int row0, int (&dst_row)[8], int (&add_row)[8]) {
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int gr = row0 + it * 4 + (lane >> 3);
    const int t = gr / p.sc_slots, c = gr - t * p.sc_slots;
    add_row[it] = t;
    dst_row[it] = gr < p.m ? __ldg(p.sc_child + static_cast<long long>(c) * p.sc_n_total + p.sc_off + t) : -1;
  }
}
// ScatterAddends: the addend values of a 32-column chunk for the lane's eight rows (issued early: the loads are
// in flight while the accumulator chunk is read and staged).
__device__ __forceinline__ void ScatterAddends(const Params& p, int lane, int col0, const int (&dst_row)[8], const int (&add_row)[8],
                                               float4 (&a)[8]) {
  const int col = col0 + (lane & 7) * 4;
#pragma unroll
  for (int it = 0; it < 8; ++it)
    a[it] = (p.sc_addend != nullptr && dst_row[it] >= 0 && col + 4 <= p.n)
                ? __ldg(reinterpret_cast<const float4*>(p.sc_addend + static_cast<long long>(add_row[it]) * p.sc_addend_ld + col))
                : make_float4(0.f, 0.f, 0.f, 0.f);
}
// ScatterRows: staged rows leave shared memory four per instruction:
//   out[dst_row][col..] = addend + staged value  (addend first: the separate scatter kernel computes ds + dq).
__device__ __forceinline__ void ScatterRows(const Params& p, uint32_t slot, int lane, int col0, const int (&dst_row)[8],
                                            const float4 (&a)[8]) {
  const int q = lane & 7;
  const int col = col0 + q * 4;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int i = it * 4 + (lane >> 3);
    if (dst_row[it] < 0 || col + 4 > p.n) continue;
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(slot + i * 128 + ((q ^ (i & 7)) << 4))
                 : "memory");
    *reinterpret_cast<float4*>(static_cast<float*>(p.c) + static_cast<long long>(dst_row[it]) * p.ldc + col) =
        make_float4(a[it].x + v.x, a[it].y + v.y, a[it].z + v.z, a[it].w + v.w);
  }
}

// Persistent kernel: each CTA walks work items w = blockIdx.x, blockIdx.x + gridDim.x, ...;
// work item -> (tile, K-split) with the N tile index fastest, so the CTAs of one wave share A
// row blocks through L2.  Two TMEM accumulators alternate between tiles: while the epilogue
// warps drain one, the MMA warp already fills the other, and the TMA ring never drains.
// kDual: the launch carries a second, independent product (its own operand / output maps and Params p1) with the
// same tile shape and operand majors; its tiles follow the first product's in the work list, so two small products
// of a level (the two gate products; the two gradient products) fill the machine as one launch and pay the launch
// and pipeline-fill latency once.  The second product is never K-split.
template <int kBN, int kAMajor, int kBMajor, int kMB, bool kDual>
__device__ __forceinline__ void GemmBody(const CUtensorMap* ma0, const CUtensorMap* mb0, const CUtensorMap* mc0, const Params& p,
                                         const CUtensorMap* ma1, const CUtensorMap* mb1, const CUtensorMap* mc1, const Params& p1) {
  using S = Smem<kBN, kMB>;
  static_assert(kMB == 1 || (kMB == 2 && kBN == 256), "two row blocks need both 256-column accumulators");
  constexpr int kTileM = kBM * kMB;
  ChainRelease(p.chain_early);
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle needs 1024-byte aligned tiles.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBarOff);
  uint64_t* full_bar = bars;                          // [kStages] TMA -> MMA
  uint64_t* empty_bar = bars + S::kStages;            // [kStages] MMA -> TMA
  uint64_t* acc_full = bars + 2 * S::kStages;         // [2] MMA -> epilogue
  uint64_t* acc_empty = bars + 2 * S::kStages + 2;    // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S::kStages + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const Params& p_first = p;
  const int n_tiles_n0 = (p.n + kBN - 1) / kBN;
  const int n_work0 = ((p.m + kTileM - 1) / kTileM) * n_tiles_n0 * p.n_splits;
  const int n_tiles_n1 = kDual ? (p1.n + kBN - 1) / kBN : 1;
  const int n_work = n_work0 + (kDual ? ((p1.m + kTileM - 1) / kTileM) * n_tiles_n1 : 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      MbarInit(SmemAddr(full_bar + s), 1);
      MbarInit(SmemAddr(empty_bar + s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      MbarInit(SmemAddr(acc_full + a), 1);
      MbarInit(SmemAddr(acc_empty + a), 4);   // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(tmem_slot)), "r"(2 * kBN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t spin = p.spin_limit != 0 ? p.spin_limit : kSpinLimit;
  bool ok = true;
  // Everything above touched only this CTA's shared memory and TMEM; operands and outputs in global
  // memory belong to the preceding kernel until here.
  ChainAcquire();

  if (warp == 0) {
    if (ElectOne() && !p.withhold_loads) {
      uint32_t it = 0;   // ring position, continuous across work items
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const bool second = kDual && w >= n_work0;
        const Params& q = second ? p1 : p;
        const CUtensorMap* map_a = second ? ma1 : ma0;
        const CUtensorMap* map_b = second ? mb1 : mb0;
        const int wl = second ? w - n_work0 : w;
        const int n_tiles_n = second ? n_tiles_n1 : n_tiles_n0;
        const int z = wl % q.n_splits, tile = wl / q.n_splits;
        const int m0 = (tile / n_tiles_n) * kTileM, n0 = (tile % n_tiles_n) * kBN;
        const int kb_begin = z * q.kb_per_split;
        const int kb_count = min(q.kb_per_split, (q.k + kBK - 1) / kBK - kb_begin);
        for (int i = 0; i < kb_count; ++i, ++it) {
          const int s = it % S::kStages;
          const uint32_t phase = (it / S::kStages) & 1;
          ok = MbarWait(SmemAddr(empty_bar + s), phase ^ 1, spin);
          if (!ok) break;
          const uint32_t bar = SmemAddr(full_bar + s);
          MbarExpectTx(bar, S::kStage);
          const uint32_t a_dst = SmemAddr(smem + s * S::kStage);
          const uint32_t b_dst = a_dst + S::kATile;
          const int k0 = (kb_begin + i) * kBK;
          if (kAMajor == kMajorK) {
#pragma unroll
            for (int mb = 0; mb < kMB; ++mb)                                          // box {64 k, 128 rows}
              TmaLoad2d(a_dst + mb * (kBM * kBK * 2), map_a, bar, k0, m0 + kBM * mb + q.a_row_off);
          } else {
#pragma unroll
            for (int j = 0; j < kTileM / 64; ++j) TmaLoad2d(a_dst + j * 8192, map_a, bar, m0 + 64 * j, k0);  // box {64 mn, 64 k}
          }
          if (kBMajor == kMajorK) {
            TmaLoad2d(b_dst, map_b, bar, k0, n0);                                    // box {64 k, kBN rows}
          } else {
#pragma unroll
            for (int j = 0; j < kBN / 64; ++j) TmaLoad2d(b_dst + j * 8192, map_b, bar, n0 + 64 * j, k0);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (ElectOne()) {
      constexpr uint32_t idesc = InstrDesc(kAMajor, kBMajor, kBN, kBM);
      constexpr uint32_t a_step = (kAMajor == kMajorK) ? (kUmmaK * 2 >> 4) : (kUmmaK * 128 >> 4);
      constexpr uint32_t b_step = (kBMajor == kMajorK) ? (kUmmaK * 2 >> 4) : (kUmmaK * 128 >> 4);
      uint32_t it = 0, t_local = 0;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++t_local) {
        const bool second = kDual && w >= n_work0;
        const Params& q = second ? p1 : p;
        const int z = (second ? w - n_work0 : w) % q.n_splits;
        const int kb_begin = z * q.kb_per_split;
        const int kb_count = min(q.kb_per_split, (q.k + kBK - 1) / kBK - kb_begin);
        // kMB = 1: two accumulators alternate between tiles; kMB = 2: one accumulator pair, reused by every tile
        const uint32_t acc = kMB == 2 ? 0 : (t_local & 1), acc_phase = kMB == 2 ? (t_local & 1) : ((t_local >> 1) & 1);
        ok = MbarWait(SmemAddr(acc_empty + acc), acc_phase ^ 1, spin);   // epilogue has drained this accumulator
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int i = 0; i < kb_count; ++i, ++it) {
          const int s = it % S::kStages;
          const uint32_t phase = (it / S::kStages) & 1;
          ok = MbarWait(SmemAddr(full_bar + s), phase, spin);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = SmemAddr(smem + s * S::kStage);
          const uint64_t a_desc = SmemDesc(a_addr, kAMajor);
          const uint64_t b_desc = SmemDesc(a_addr + S::kATile, kBMajor);
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk)
#pragma unroll
            for (int mb = 0; mb < kMB; ++mb)   // row block mb: its A half starts 16 KB further, its accumulator kBN columns further
              UmmaBf16(d_tmem + mb * kBN, a_desc + mb * ((kBM * kBK * 2) >> 4) + kk * a_step, b_desc + kk * b_step, idesc,
                       (i > 0 || kk > 0) ? 1u : 0u);
          UmmaCommit(SmemAddr(empty_bar + s));   // frees the stage once these MMAs have read it
        }
        if (ok) UmmaCommit(SmemAddr(acc_full + acc));   // accumulator complete
      }
    }
    __syncwarp();
  } else {
    // Epilogue warps 2..5 own TMEM lane quarters (warp % 4).
    const int quarter = warp & 3;
    uint32_t t_local = 0;
    uint32_t n_stores = 0;   // bulk stores issued by this warp; picks the staging slot (alternating)
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++t_local) {
      const bool second = kDual && w >= n_work0;
      const Params& p = second ? p1 : p_first;          // this work item's product (shadows the first product's)
      const CUtensorMap* map_c = second ? mc1 : mc0;
      const int wl = second ? w - n_work0 : w;
      const int n_tiles_n = second ? n_tiles_n1 : n_tiles_n0;
      const int z = wl % p.n_splits, tile = wl / p.n_splits;
      const int m0_tile = (tile / n_tiles_n) * kTileM, n0 = (tile % n_tiles_n) * kBN;
      const uint32_t acc = kMB == 2 ? 0 : (t_local & 1), acc_phase = kMB == 2 ? (t_local & 1) : ((t_local >> 1) & 1);
      int sc_dst[8], sc_add[8];
      if (p.out_mode == kScatterF32) ScatterTargets(p, lane, m0_tile + quarter * 32, sc_dst, sc_add);   // before the wait (kMB = 1 only)
      ok = MbarWait(SmemAddr(acc_full + acc), acc_phase, spin);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const long long zoff = static_cast<long long>(z) * p.split_stride;
#pragma unroll 1
      for (int mb = 0; mb < kMB; ++mb) {
      const int m0 = m0_tile + mb * kBM;
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_addr = tmem_base + (acc + mb) * kBN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (p.tma_store) {
        // Registers -> swizzled shared staging -> TMA store: every global write is a full 128-byte
        // row segment, and the tensor map clips the M / N tails.  Two slots per warp alternate on
        // every store; before a slot is rewritten, all but the most recent bulk group (which reads
        // the other slot) must have finished reading shared memory.
        const uint32_t slots = SmemAddr(smem + S::kCOff) + (warp - 2) * 2 * S::kCSlot;
        const int row0 = m0 + quarter * 32;
        const bool bf16_out = p.out_mode == kStoreBf16;
        const bool gate_out = p.out_mode == kGateActF16;
#pragma unroll 1
        for (int c0 = 0; c0 < kBN; c0 += 64) {
          if (n0 + c0 >= p.n) break;   // warp-uniform
          uint32_t r[64];
          TmemLoad64(t_addr + c0, r);
          if (row0 < p.m) {
            if (bf16_out || gate_out) {
              // 64 columns of 16-bit values = one 128-byte row: one slot, one store
              if (gate_out && row < p.m) GateActivate(p, r, row, n0 + c0);
              if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
              __syncwarp();
              const uint32_t slot = slots + (n_stores++ & 1) * S::kCSlot;
              if (gate_out) StageRowPacked(slot, lane, r); else StageRow<0, 1>(slot, lane, r);
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) {
                TmaStore2d(map_c, slot, n0 + c0, row0 + p.c_row_off);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              }
            } else {
              // two 32-column fp32 halves, one slot and one bulk group each; a slot is rewritten
              // once the group issued two stores ago has finished reading it
              if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
              __syncwarp();
              const uint32_t slot_a = slots + (n_stores++ & 1) * S::kCSlot;
              StageRow<0, 0>(slot_a, lane, r);
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) {
                TmaStore2d(map_c, slot_a, n0 + c0, row0 + p.c_row_off);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              }
              if (n0 + c0 + 32 < p.n) {
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                __syncwarp();
                const uint32_t slot_b = slots + (n_stores++ & 1) * S::kCSlot;
                StageRow<32, 0>(slot_b, lane, r);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                  TmaStore2d(map_c, slot_b, n0 + c0 + 32, row0 + p.c_row_off);
                  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
              }
            }
          }
        }
      } else if (p.out_mode == kScatterF32) {
        // Registers -> swizzled shared staging (one 128-byte row per lane) -> coalesced row scatter.  The
        // addends of a 64-column step are requested before the accumulator chunk is read.
        const uint32_t slot = SmemAddr(smem + S::kCOff) + (warp - 2) * 2 * S::kCSlot;
#pragma unroll 1
        for (int c0 = 0; c0 < kBN; c0 += 64) {
          if (n0 + c0 >= p.n) break;   // warp-uniform
          float4 add0[8], add1[8];
          ScatterAddends(p, lane, n0 + c0, sc_dst, sc_add, add0);
          ScatterAddends(p, lane, n0 + c0 + 32, sc_dst, sc_add, add1);
          uint32_t r[64];
          TmemLoad64(t_addr + c0, r);
          if (m0 + quarter * 32 < p.m) {
            __syncwarp();                      // the previous step has been read out of both slots
            StageRow<0, 0>(slot, lane, r);
            StageRow<32, 0>(slot + S::kCSlot, lane, r);
            __syncwarp();
            ScatterRows(p, slot, lane, n0 + c0, sc_dst, add0);
            ScatterRows(p, slot + S::kCSlot, lane, n0 + c0 + 32, sc_dst, add1);
          }
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < kBN; c0 += 64) {
          if (n0 + c0 >= p.n) break;   // warp-uniform
          uint32_t r[64];
          TmemLoad64(t_addr + c0, r);
          StoreChunk<0>(p, r, row, n0 + c0, zoff);
          StoreChunk<32>(p, r, row, n0 + c0 + 32, zoff);
        }
      }
      }   // row blocks
      // All of this warp's TMEM reads are complete (wait::ld above): hand the accumulator back.
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) MbarArrive(SmemAddr(acc_empty + acc));
    }
  }
  if (warp >= 2 && lane == 0 && (p.tma_store || (kDual && p1.tma_store))) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  if (!ok && p.status != nullptr) atomicExch(p.status, 1);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * kBN));
  }
}

template <int kBN, int kAMajor, int kBMajor, int kMB = 1>
__global__ void __launch_bounds__(kThreads, 1)
GemmBf16Kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const Params p) {
  GemmBody<kBN, kAMajor, kBMajor, kMB, false>(&map_a, &map_b, &map_c, p, &map_a, &map_b, &map_c, p);
}

template <int kBN, int kAMajor, int kBMajor>
__global__ void __launch_bounds__(kThreads, 1)
GemmBf16DualKernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_c, const Params p, const __grid_constant__ CUtensorMap map_a1,
                   const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_c1, const Params p1) {
  GemmBody<kBN, kAMajor, kBMajor, 1, true>(&map_a, &map_b, &map_c, p, &map_a1, &map_b1, &map_c1, p1);
}

}  // namespace tc
}  // namespace cavs_b200
#endif
