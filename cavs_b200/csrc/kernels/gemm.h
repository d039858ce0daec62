// Internal C++ interface of the two GEMM paths (shared by the C ABI and the engine).
#ifndef CAVS_B200_KERNELS_GEMM_H_
#define CAVS_B200_KERNELS_GEMM_H_

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace cavs_b200 {

// bf16 x bf16 -> fp32 on tcgen05.  Operand majors: 0 = K-major (A is [m,k] / B is [n,k],
// row-major), 1 = MN-major (A is [k,m] / B is [k,n], row-major).
struct GemmBf16Args {
  void* c = nullptr;          // [m,n] row-major, fp32 (out_mode 0 store, 1 accumulate) or bf16 (2)
  long long ldc = 0;
  int out_mode = 0;
  const void* a = nullptr;
  long long lda = 0;
  int a_major = 0;
  const void* b = nullptr;
  long long ldb = 0;
  int b_major = 0;
  int m = 0, n = 0, k = 0;
  int splits = 1;             // >1: K split across CTAs, partials in scratch, fixed-order reduce
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  int* status = nullptr;      // device word raised when a bounded wait expires
  // Wait self-test (cavs_gemm_bf16_wait_selftest): polls per bounded wait (0 = default) and a producer that
  // issues no operand load, so that every consumer wait runs out and the kernel's unwind path executes.
  unsigned wait_poll_limit = 0;
  int withhold_loads = 0;
};
int GemmBf16(const GemmBf16Args& args, cudaStream_t stream);

// A TMA tensor map of one operand, encoded once and reused across launches: building one costs
// microseconds of host time, which dominates the small GEMMs of deep, narrow levels.
struct TcOperandMap {
  alignas(64) unsigned char bytes[128];   // CUtensorMap
  int major = 0;                          // 0 K-major, 1 MN-major
  int tile_rows = 0;                      // K-major: rows per box (128 for A, the N tile for B)
};
// base: row-major matrix with pitch ld.  K-major: [rows, k] -> extents (k, rows); MN-major: [k, rows].
// tile_rows: 128 for an A operand; for a K-major B operand the N tile the GEMM will use (GemmBf16TileN).
int EncodeTcOperand(TcOperandMap* out, const void* base, long long rows, long long k, long long ld, int major, int tile_rows);
inline int GemmBf16TileN(int n) { return n > 128 ? 256 : 128; }
// N tile for an (m, n, k) problem: a short-K GEMM small enough that 64-column tiles still fit one wave is
// bound by how fast one SM can pull its operand tiles out of L2, so it runs 64-column tiles on four times
// as many SMs (measured: 7.9 -> 5.6 us for [128,1024]x[1024,3072], 17.8 -> 10.7 us for [8,3072]x[3072,1024]);
// everything else keeps GemmBf16TileN(n).
int GemmBf16TileNFor(int m, int n, int k);
struct GemmBf16MappedArgs {
  void* c = nullptr;
  long long ldc = 0;
  int out_mode = 0;
  const TcOperandMap* a = nullptr;
  int a_row_off = 0;          // first row of this GEMM's A view inside the mapped arena (K-major A only)
  const TcOperandMap* b = nullptr;
  // Optional second map of a K-major B encoded for 64-row tiles (the small-problem tiling); without it a
  // K-major B keeps the default tiling.  An MN-major B needs no second map.
  const TcOperandMap* b_small = nullptr;
  // out_mode 3 (scatter): row r = t * scatter_slots + c of the product, plus scatter_addend[t, :], is written to
  // row scatter_child[c * scatter_n_total + scatter_off + t] of c (pitch ldc); negative targets are skipped.
  const int32_t* scatter_child = nullptr;
  const float* scatter_addend = nullptr;
  long long scatter_addend_ld = 0;
  int scatter_n_total = 0, scatter_off = 0, scatter_slots = 0;
  // Optional pre-encoded map of the output (EncodeTcOutput over [>= m rows, n] at c); when null and
  // the TMA-store epilogue applies, one is encoded per call.  The map's row extent clips the M tail,
  // so it must cover exactly the rows this GEMM may write.
  const TcOperandMap* c_map = nullptr;
  int m = 0, n = 0, k = 0;
  int splits = 1;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  int* status = nullptr;
  unsigned wait_poll_limit = 0;   // see GemmBf16Args
  int withhold_loads = 0;
  // out_mode 4 (gate epilogue): instead of pre-activations the product stores finished LSTM gates as fp16,
  //   gate = act((product + act_a[row(t), act_col0 + n]) + bias),  t = act_t_off + r / act_rows_per_vertex,
  // sigmoid for the i, o, f column blocks and tanh for u (columns in the order i,o,u,f, act_hidden per block, a
  // multiple of 64); act_a: bf16 [*, 4 act_hidden] input projection with one row per vertex, or per act_a_row[t];
  // act_bias: [4 act_hidden] fp32 in the order i,f,u,o.  Needs c_map (16-bit elements); c_row_off shifts the rows
  // the map is written at, so that c_map can cover a whole arena -- the last 32-row slab of a product is stored
  // whole, so up to 31 arena rows behind the product's last row are overwritten with meaningless values: only for
  // arenas whose following rows are rewritten before they are next read (the saved gates of later levels).
  const void* act_a = nullptr;
  const int32_t* act_a_row = nullptr;
  const float* act_bias = nullptr;
  int act_col0 = 0, act_hidden = 0, act_rows_per_vertex = 1, act_t_off = 0;
  int c_row_off = 0;
};
int EncodeTcOutput(TcOperandMap* out, void* base, long long m, long long n, long long ldc, bool bf16);
int GemmBf16Mapped(const GemmBf16MappedArgs& args, cudaStream_t stream);
// Two independent products of equal operand layout in ONE launch (the two gate products of a level, or its two
// gradient products): their tiles share the persistent grid, so a small level pays the launch and pipeline-fill
// latency once.  Each product: K-major A map, no K split, output through c_map or the scatter epilogue.
int GemmBf16MappedDual(const GemmBf16MappedArgs& first, const GemmBf16MappedArgs& second, cudaStream_t stream);
size_t GemmBf16ScratchBytes(int m, int n, int splits);
int GemmBf16SplitsFor(int m, int n, int k);
int GemmBf16SplitsForTile(int m, int n, int k, int tile_m);   // the same choice for tiles of tile_m rows
// Long-K products of two MN-major operands (weight gradients) into fp32 run 256 x 256 tiles when split-K scratch
// is available: a third fewer operand bytes per flop out of L2.
bool GemmBf16UsesTallTiles(int m, int n, int k, int a_major, int b_major, int out_mode);

// fp32 GEMM on the CUDA cores with arbitrary element strides:
// C[i,j] (+)= sum_p A[i*a_rs + p*a_cs] * B[p*b_rs + j*b_cs].
struct GemmF32Args {
  float* c = nullptr;
  long long ldc = 0;
  int accumulate = 0;
  const float* a = nullptr;
  long long a_rs = 0, a_cs = 0;
  const float* b = nullptr;
  long long b_rs = 0, b_cs = 0;
  int m = 0, n = 0, k = 0;
  // Optional scratch for splitting k across CTAs when the output has too few tiles to occupy the machine (a level of
  // a few rows against wide weights is otherwise one long serial k loop on a handful of SMs): partial products go to
  // scratch [splits, m, n] and are summed in split order by a second kernel.  Without scratch k is never split.
  float* scratch = nullptr;
  size_t scratch_bytes = 0;
  int k_per_split = 0;   // set by GemmF32 (0: no split)
};
int GemmF32(const GemmF32Args& args, cudaStream_t stream);

}  // namespace cavs_b200
#endif
