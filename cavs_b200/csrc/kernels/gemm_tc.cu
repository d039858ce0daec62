// Host side of the tcgen05 GEMM: tensor-map encoding, tile-shape choice, optional
// deterministic split-K, and the C ABI entry point.
#include "kernels/gemm_tc.cuh"

#include <mutex>

#include "abi_common.h"
#include "kernels/gemm.h"
#include "kernels/launch.h"

namespace cavs_b200 {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver entry point; it is fetched through the runtime so
// the library carries no link-time dependency on libcuda.
EncodeFn GetEncodeFn(std::string* err) {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  static std::string once_err;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || sym == nullptr)
      once_err = std::string("cuTensorMapEncodeTiled unavailable: ") + cudaGetErrorString(e);
    else
      fn = reinterpret_cast<EncodeFn>(sym);
  });
  if (!fn) *err = once_err;
  return fn;
}

// 2-D bf16 tensor map over a row-major matrix [outer, inner] with row pitch ld elements,
// 128-byte swizzle, zero fill outside the extents.
int EncodeBf16(CUtensorMap* map, const void* base, long long inner, long long outer, long long ld, int box_inner,
               int box_outer) {
  std::string err;
  EncodeFn fn = GetEncodeFn(&err);
  if (!fn) return Fail(CAVS_ERR_CUDA, err);
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Fail(CAVS_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(r));
  return CAVS_OK;
}

// Tensor map of the output for the TMA-store epilogue: boxes of 32 rows x 128 bytes, 128-byte swizzle.
int EncodeC(CUtensorMap* map, void* base, long long n, long long m, long long ldc, bool bf16) {
  std::string err;
  EncodeFn fn = GetEncodeFn(&err);
  if (!fn) return Fail(CAVS_ERR_CUDA, err);
  const size_t elt = bf16 ? 2 : 4;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldc) * elt};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elt), 32};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Fail(CAVS_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult " + std::to_string(r));
  return CAVS_OK;
}

__global__ void __launch_bounds__(256) SplitKReduce(float* __restrict__ c, long long ldc, const float* __restrict__ part,
                                                    int m, int n, int splits, int accumulate) {
  const long long total = static_cast<long long>(m) * n;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    float acc = 0.0f;
    for (int z = 0; z < splits; ++z) acc += part[z * total + i];   // fixed order: deterministic
    float* dst = c + (i / n) * ldc + (i % n);
    *dst = accumulate ? *dst + acc : acc;
  }
}

template <int kBN, int kAMajor, int kBMajor, int kMB = 1>
int Launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const tc::Params& p, dim3 grid, cudaStream_t stream) {
  using S = tc::Smem<kBN, kMB>;
  auto kern = tc::GemmBf16Kernel<kBN, kAMajor, kBMajor, kMB>;
  static bool configured[kMaxDevices] = {};   // per instantiation and device: the attribute belongs to the device's copy
  const int dev = CurrentDevice();
  if (!configured[dev]) {
    CAVS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes));
    configured[dev] = true;
  }
  CAVS_CUDA(LaunchChained(kern, grid, dim3(tc::kThreads), S::kBytes, stream, ma, mb, mc, p));
  CAVS_LAUNCH_CHECK("gemm_bf16");
  return CAVS_OK;
}

template <int kBN>
int Dispatch(int a_major, int b_major, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const tc::Params& p,
             dim3 grid, cudaStream_t stream) {
  if (a_major == tc::kMajorK && b_major == tc::kMajorK) return Launch<kBN, 0, 0>(ma, mb, mc, p, grid, stream);
  if (a_major == tc::kMajorK && b_major == tc::kMajorMN) return Launch<kBN, 0, 1>(ma, mb, mc, p, grid, stream);
  if (a_major == tc::kMajorMN && b_major == tc::kMajorK) return Launch<kBN, 1, 0>(ma, mb, mc, p, grid, stream);
  return Launch<kBN, 1, 1>(ma, mb, mc, p, grid, stream);
}

bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int kBN, int kAMajor, int kBMajor>
int LaunchDual(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const tc::Params& p, const CUtensorMap& ma1,
               const CUtensorMap& mb1, const CUtensorMap& mc1, const tc::Params& p1, dim3 grid, cudaStream_t stream) {
  using S = tc::Smem<kBN, 1>;
  auto kern = tc::GemmBf16DualKernel<kBN, kAMajor, kBMajor>;
  static bool configured[kMaxDevices] = {};
  const int dev = CurrentDevice();
  if (!configured[dev]) {
    CAVS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes));
    configured[dev] = true;
  }
  CAVS_CUDA(LaunchChained(kern, grid, dim3(tc::kThreads), S::kBytes, stream, ma, mb, mc, p, ma1, mb1, mc1, p1));
  CAVS_LAUNCH_CHECK("gemm_bf16 (two products)");
  return CAVS_OK;
}

}  // namespace

size_t GemmBf16ScratchBytes(int m, int n, int splits) {
  return splits > 1 ? static_cast<size_t>(splits) * m * n * sizeof(float) : 0;
}

int GemmBf16TileNFor(int m, int n, int k) {
  const int base = GemmBf16TileN(n);
  const long long tiles64 = static_cast<long long>((m + tc::kBM - 1) / tc::kBM) * ((n + 63) / 64);
  const int nkb = (k + tc::kBK - 1) / tc::kBK;
  return (n > 64 && nkb <= 64 && tiles64 <= SmCount()) ? 64 : base;   // one wave of 64-column tiles
}

// 256 x 256 tiles: long-K products with both operands MN-major (the weight gradients X^T dY) and an fp32 output.
bool GemmBf16UsesTallTiles(int m, int n, int k, int a_major, int b_major, int out_mode) {
  return a_major == tc::kMajorMN && b_major == tc::kMajorMN && out_mode != tc::kStoreBf16 && out_mode != tc::kScatterF32 &&
         m >= 256 && n > 128 && k >= 64 * tc::kBK;
}

int GemmBf16SplitsFor(int m, int n, int k) {
  return GemmBf16SplitsForTile(m, n, k, tc::kBM);
}

int GemmBf16SplitsForTile(int m, int n, int k, int tile_m) {
  // The kernel is persistent over (tile, split) work items.  Splitting K costs partial traffic, a
  // plain-store epilogue and a reduce pass, so it is used only when the tile grid leaves more than a
  // quarter of the SMs idle; then the smallest split count that fills whole waves to >= 90 % wins,
  // keeping each split >= 32 K blocks.
  const int bn = GemmBf16TileN(n);
  const long long tiles = static_cast<long long>((m + tile_m - 1) / tile_m) * ((n + bn - 1) / bn);
  const int nkb = (k + tc::kBK - 1) / tc::kBK;
  const int sms = SmCount();
  auto fill = [&](long long items) { return static_cast<double>(items) / (((items + sms - 1) / sms) * sms); };
  if (fill(tiles) >= 0.75) return 1;
  int best = 1;
  double best_fill = fill(tiles);
  for (int s = 2; s <= 16 && nkb / s >= 32; ++s) {
    const double f = fill(tiles * s);
    if (f > best_fill + 0.04) { best = s; best_fill = f; }
    if (best_fill >= 0.9) break;
  }
  return best;
}

int EncodeTcOperand(TcOperandMap* out, const void* base, long long rows, long long k, long long ld, int major, int tile_rows) {
  CAVS_REQUIRE(out && base && rows > 0 && k > 0, CAVS_ERR_BAD_ARG, "gemm_bf16: bad operand");
  CAVS_REQUIRE(major == 0 || major == 1, CAVS_ERR_BAD_ARG, "gemm_bf16: operand major must be 0 (K) or 1 (MN)");
  // TMA: 16-byte aligned base and row pitch (8 bf16 elements).
  CAVS_REQUIRE(Aligned16(base) && ld % 8 == 0, CAVS_ERR_BAD_ARG,
               "gemm_bf16: operands need 16-byte aligned bases and row pitches that are multiples of 8 elements");
  static_assert(sizeof(CUtensorMap) <= sizeof(out->bytes), "tensor map storage");
  out->major = major;
  out->tile_rows = tile_rows;
  CUtensorMap* map = reinterpret_cast<CUtensorMap*>(out->bytes);
  if (major == tc::kMajorK) return EncodeBf16(map, base, k, rows, ld, tc::kBK, tile_rows);   // [rows, k]
  return EncodeBf16(map, base, rows, k, ld, 64, tc::kBK);                                     // [k, rows]
}

int EncodeTcOutput(TcOperandMap* out, void* base, long long m, long long n, long long ldc, bool bf16) {
  CAVS_REQUIRE(out && base && m > 0 && n > 0 && ldc >= n, CAVS_ERR_BAD_ARG, "gemm_bf16: bad output");
  CAVS_REQUIRE(Aligned16(base) && (ldc * (bf16 ? 2 : 4)) % 16 == 0, CAVS_ERR_BAD_ARG, "gemm_bf16: output map needs 16-byte aligned rows");
  out->major = -1;
  out->tile_rows = bf16 ? 2 : 4;
  return EncodeC(reinterpret_cast<CUtensorMap*>(out->bytes), base, n, m, ldc, bf16);
}

int GemmBf16Mapped(const GemmBf16MappedArgs& g, cudaStream_t stream) {
  CAVS_REQUIRE(g.m >= 0 && g.n >= 0 && g.k >= 0, CAVS_ERR_BAD_ARG, "gemm_bf16: negative dimension");
  if (g.m == 0 || g.n == 0) return CAVS_OK;
  CAVS_REQUIRE(g.k > 0, CAVS_ERR_BAD_ARG, "gemm_bf16: k must be positive");
  CAVS_REQUIRE(g.a && g.b && g.c, CAVS_ERR_BAD_ARG, "gemm_bf16: null pointer");
  CAVS_REQUIRE(g.out_mode >= 0 && g.out_mode <= 4, CAVS_ERR_BAD_ARG, "gemm_bf16: bad out_mode");
  CAVS_REQUIRE(g.out_mode != tc::kGateActF16 ||
                   (g.c_map && g.act_a && g.act_bias && g.act_hidden > 0 && g.act_hidden % 64 == 0 && g.act_col0 % 64 == 0 &&
                    g.act_col0 + g.n <= 4 * g.act_hidden && g.act_rows_per_vertex >= 1 && std::max(1, g.splits) == 1 &&
                    Aligned16(g.act_a) && Aligned16(g.act_bias)),
               CAVS_ERR_BAD_ARG,
               "gemm_bf16: the gate epilogue needs an output map, the input projection and bias (16-byte aligned), a hidden size "
               "that is a multiple of 64 and no K split");
  CAVS_REQUIRE(g.ldc >= g.n, CAVS_ERR_BAD_ARG, "gemm_bf16: ldc < n");
  CAVS_REQUIRE(g.out_mode != tc::kScatterF32 ||
                   (g.scatter_child && g.scatter_slots >= 1 && std::max(1, g.splits) == 1 && g.n % 4 == 0 && g.ldc % 4 == 0 &&
                    Aligned16(g.c) &&
                    (g.scatter_addend == nullptr ||
                     (g.scatter_addend_ld >= g.n && g.scatter_addend_ld % 4 == 0 && Aligned16(g.scatter_addend)))),
               CAVS_ERR_BAD_ARG,
               "gemm_bf16: scatter output needs the child table, 16-byte aligned output (and addend) rows (n, pitches multiples of 4) and no K split");
  CAVS_REQUIRE(g.a_row_off == 0 || g.a->major == tc::kMajorK, CAVS_ERR_BAD_ARG, "gemm_bf16: row offsets need a K-major A");
  int splits = std::max(1, g.splits);
  int bn = GemmBf16TileN(g.n);
  const TcOperandMap* bmap = g.b;
  if (splits == 1 && GemmBf16TileNFor(g.m, g.n, g.k) == 64) {
    if (g.b->major == tc::kMajorMN) bn = 64;
    else if (g.b->tile_rows == 64) bn = 64;
    else if (g.b_small != nullptr && g.b_small->major == tc::kMajorK && g.b_small->tile_rows == 64) { bn = 64; bmap = g.b_small; }
  }
  // Long-K weight gradients with split-K scratch available run 256 x 256 tiles; the split count is then chosen for
  // that tile grid.
  const bool tall_wgrad = bn == 256 && g.scratch != nullptr && splits > 1 &&
                          GemmBf16UsesTallTiles(g.m, g.n, g.k, g.a->major, bmap->major, g.out_mode);
  if (tall_wgrad) {
    splits = GemmBf16SplitsForTile(g.m, g.n, g.k, 2 * tc::kBM);
    while (splits > 1 && g.scratch_bytes < GemmBf16ScratchBytes(g.m, g.n, splits)) --splits;
  }
  // The same tiles for the deep-K gradient products of large levels (dY W^T with both operands K-major, fp32 out):
  // 32+ k-blocks per tile make the unhidden epilogue cheap, and there is at least one full wave of tiles.
  const bool tall_dgrad = bn == 256 && splits == 1 && g.a->major == tc::kMajorK &&
                          (g.out_mode == tc::kStoreF32 || g.out_mode == tc::kStoreBf16) && g.k >= 16 * tc::kBK &&
                          static_cast<long long>((g.m + 2 * tc::kBM - 1) / (2 * tc::kBM)) * ((g.n + bn - 1) / bn) >= SmCount();
  const bool tall = tall_wgrad || tall_dgrad;
  const int tile_m = tall ? 2 * tc::kBM : tc::kBM;
  CAVS_REQUIRE(g.a->major != tc::kMajorK || g.a->tile_rows == tc::kBM, CAVS_ERR_BAD_ARG, "gemm_bf16: A map was not encoded for 128-row tiles");
  CAVS_REQUIRE(bmap->major != tc::kMajorK || bmap->tile_rows == bn, CAVS_ERR_BAD_ARG, "gemm_bf16: B map was encoded for a different N tile");
  CAVS_REQUIRE(splits == 1 || g.out_mode != tc::kStoreBf16, CAVS_ERR_BAD_ARG, "gemm_bf16: split-K needs an fp32 output");
  CAVS_REQUIRE(splits == 1 || (g.scratch && g.scratch_bytes >= GemmBf16ScratchBytes(g.m, g.n, splits)), CAVS_ERR_CAPACITY,
               "gemm_bf16: split-K scratch too small");
  const CUtensorMap& ma = *reinterpret_cast<const CUtensorMap*>(g.a->bytes);
  const CUtensorMap& mb = *reinterpret_cast<const CUtensorMap*>(bmap->bytes);

  const int nkb = (g.k + tc::kBK - 1) / tc::kBK;
  const int kb_per = (nkb + splits - 1) / splits;
  const int eff_splits = (nkb + kb_per - 1) / kb_per;
  tc::Params p{};
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.kb_per_split = kb_per;
  p.n_splits = eff_splits;
  p.a_row_off = g.a_row_off;
  p.status = g.status;
  p.spin_limit = g.wait_poll_limit;
  p.withhold_loads = g.withhold_loads;
  p.chain_early = ChainEarly();
  p.sc_child = g.scatter_child; p.sc_addend = g.scatter_addend; p.sc_addend_ld = g.scatter_addend_ld;
  p.sc_n_total = g.scatter_n_total; p.sc_off = g.scatter_off; p.sc_slots = std::max(1, g.scatter_slots);
  p.act_a = g.act_a; p.act_a_row = g.act_a_row; p.act_bias = g.act_bias;
  p.act_col0 = g.act_col0; p.act_h = g.act_hidden; p.act_rpv = std::max(1, g.act_rows_per_vertex); p.act_t_off = g.act_t_off;
  p.c_row_off = g.c_row_off;
  if (eff_splits > 1) {
    p.c = g.scratch; p.ldc = g.n; p.split_stride = static_cast<long long>(g.m) * g.n; p.out_mode = tc::kStoreF32;
  } else {
    p.c = g.c; p.ldc = g.ldc; p.split_stride = 0; p.out_mode = g.out_mode;
  }
  // TMA-store epilogue: plain stores (no accumulate, no K split) into a 16-byte aligned output.
  CUtensorMap mc_local;
  const CUtensorMap* mc = &ma;   // placeholder when unused
  const size_t c_elt = (g.out_mode == tc::kStoreBf16 || g.out_mode == tc::kGateActF16) ? 2 : 4;
  p.tma_store = 0;
  if (eff_splits == 1 && g.out_mode != tc::kAccumF32 && g.out_mode != tc::kScatterF32 && Aligned16(g.c) && (g.ldc * c_elt) % 16 == 0) {
    if (g.c_map) {
      mc = reinterpret_cast<const CUtensorMap*>(g.c_map->bytes);
    } else {
      if (int erc = EncodeC(&mc_local, g.c, g.n, g.m, g.ldc, c_elt == 2)) return erc;
      mc = &mc_local;
    }
    p.tma_store = 1;
  }
  const long long n_work = static_cast<long long>((g.n + bn - 1) / bn) * ((g.m + tile_m - 1) / tile_m) * eff_splits;
  dim3 grid(static_cast<unsigned>(std::min<long long>(n_work, SmCount())));
  int rc = tall_wgrad  ? Launch<256, 1, 1, 2>(ma, mb, *mc, p, grid, stream)
           : tall_dgrad ? (bmap->major == tc::kMajorK ? Launch<256, 0, 0, 2>(ma, mb, *mc, p, grid, stream)
                                                      : Launch<256, 0, 1, 2>(ma, mb, *mc, p, grid, stream))
           : bn == 256 ? Dispatch<256>(g.a->major, bmap->major, ma, mb, *mc, p, grid, stream)
           : bn == 128 ? Dispatch<128>(g.a->major, bmap->major, ma, mb, *mc, p, grid, stream)
                       : Dispatch<64>(g.a->major, bmap->major, ma, mb, *mc, p, grid, stream);
  if (rc) return rc;
  if (eff_splits > 1) {
    const size_t total = static_cast<size_t>(g.m) * g.n;
    SplitKReduce<<<GridForElems(total, 256), 256, 0, stream>>>(static_cast<float*>(g.c), g.ldc,
                                                               static_cast<const float*>(g.scratch), g.m, g.n, eff_splits,
                                                               g.out_mode == tc::kAccumF32 ? 1 : 0);
    CAVS_LAUNCH_CHECK("gemm_bf16 split-K reduce");
  }
  return CAVS_OK;
}

// Two independent products in one launch (see GemmBf16DualKernel).  Both: K-major A through an arena map, the same B
// major, no K split, outputs through c_map (TMA store or gate epilogue) or the scatter epilogue.
int GemmBf16MappedDual(const GemmBf16MappedArgs& g0, const GemmBf16MappedArgs& g1, cudaStream_t stream) {
  const GemmBf16MappedArgs* gs[2] = {&g0, &g1};
  if (g0.m == 0 || g0.n == 0) return GemmBf16Mapped(g1, stream);
  if (g1.m == 0 || g1.n == 0) return GemmBf16Mapped(g0, stream);
  for (const auto* g : gs) {
    CAVS_REQUIRE(g->m > 0 && g->n > 0 && g->k > 0 && g->a && g->b && g->c, CAVS_ERR_BAD_ARG, "gemm_bf16 (two products): bad product");
    CAVS_REQUIRE(std::max(1, g->splits) == 1 && g->a->major == tc::kMajorK && g->a->tile_rows == tc::kBM, CAVS_ERR_BAD_ARG,
                 "gemm_bf16 (two products): needs K-major A maps for 128-row tiles and no K split");
    CAVS_REQUIRE(g->out_mode == tc::kScatterF32 || g->c_map != nullptr, CAVS_ERR_BAD_ARG,
                 "gemm_bf16 (two products): outputs go through a pre-encoded map or the scatter epilogue");
    CAVS_REQUIRE(g->out_mode != tc::kAccumF32, CAVS_ERR_BAD_ARG, "gemm_bf16 (two products): no accumulating output");
  }
  CAVS_REQUIRE(g0.b->major == g1.b->major, CAVS_ERR_BAD_ARG, "gemm_bf16 (two products): the B operands must share a major");
  // one tile width for both: 64 columns when that still fits one wave, else 256 (128 for narrow outputs)
  const long long tiles64 = static_cast<long long>((g0.m + tc::kBM - 1) / tc::kBM) * ((g0.n + 63) / 64) +
                            static_cast<long long>((g1.m + tc::kBM - 1) / tc::kBM) * ((g1.n + 63) / 64);
  int bn = std::max(GemmBf16TileN(g0.n), GemmBf16TileN(g1.n));
  const TcOperandMap* bmaps[2] = {g0.b, g1.b};
  const bool kmajor_b = g0.b->major == tc::kMajorK;
  if (tiles64 <= SmCount() && std::max(g0.k, g1.k) <= 64 * tc::kBK && std::min(g0.n, g1.n) > 64 &&
      (!kmajor_b || (g0.b_small && g1.b_small && g0.b_small->tile_rows == 64 && g1.b_small->tile_rows == 64))) {
    bn = 64;
    if (kmajor_b) { bmaps[0] = g0.b_small; bmaps[1] = g1.b_small; }
  }
  for (int i = 0; i < 2; ++i)
    CAVS_REQUIRE(bmaps[i]->major != tc::kMajorK || bmaps[i]->tile_rows == bn, CAVS_ERR_BAD_ARG,
                 "gemm_bf16 (two products): a B map was encoded for a different N tile");
  tc::Params ps[2];
  const CUtensorMap* mcs[2];
  long long n_work = 0;
  for (int i = 0; i < 2; ++i) {
    const GemmBf16MappedArgs& g = *gs[i];
    tc::Params p{};
    p.m = g.m; p.n = g.n; p.k = g.k;
    p.kb_per_split = (g.k + tc::kBK - 1) / tc::kBK;
    p.n_splits = 1;
    p.a_row_off = g.a_row_off;
    p.status = g.status;
    p.spin_limit = g.wait_poll_limit;
    p.withhold_loads = g.withhold_loads;
    p.chain_early = ChainEarly();
    p.sc_child = g.scatter_child; p.sc_addend = g.scatter_addend; p.sc_addend_ld = g.scatter_addend_ld;
    p.sc_n_total = g.scatter_n_total; p.sc_off = g.scatter_off; p.sc_slots = std::max(1, g.scatter_slots);
    p.act_a = g.act_a; p.act_a_row = g.act_a_row; p.act_bias = g.act_bias;
    p.act_col0 = g.act_col0; p.act_h = g.act_hidden; p.act_rpv = std::max(1, g.act_rows_per_vertex); p.act_t_off = g.act_t_off;
    p.c_row_off = g.c_row_off;
    p.c = g.c; p.ldc = g.ldc; p.split_stride = 0; p.out_mode = g.out_mode;
    p.tma_store = g.out_mode == tc::kScatterF32 ? 0 : 1;
    CAVS_REQUIRE(g.out_mode != tc::kGateActF16 || (g.act_a && g.act_bias && g.act_hidden % 64 == 0 && g.act_col0 % 64 == 0),
                 CAVS_ERR_BAD_ARG, "gemm_bf16 (two products): incomplete gate epilogue");
    CAVS_REQUIRE(g.out_mode != tc::kScatterF32 || (g.scatter_child && g.n % 4 == 0 && g.ldc % 4 == 0 && Aligned16(g.c) &&
                                                   (g.scatter_addend == nullptr || (g.scatter_addend_ld % 4 == 0 && Aligned16(g.scatter_addend)))),
                 CAVS_ERR_BAD_ARG, "gemm_bf16 (two products): incomplete scatter epilogue");
    ps[i] = p;
    mcs[i] = g.c_map ? reinterpret_cast<const CUtensorMap*>(g.c_map->bytes) : reinterpret_cast<const CUtensorMap*>(g.a->bytes);
    n_work += static_cast<long long>((g.n + bn - 1) / bn) * ((g.m + tc::kBM - 1) / tc::kBM);
  }
  const CUtensorMap& ma0 = *reinterpret_cast<const CUtensorMap*>(g0.a->bytes);
  const CUtensorMap& ma1 = *reinterpret_cast<const CUtensorMap*>(g1.a->bytes);
  const CUtensorMap& mb0 = *reinterpret_cast<const CUtensorMap*>(bmaps[0]->bytes);
  const CUtensorMap& mb1 = *reinterpret_cast<const CUtensorMap*>(bmaps[1]->bytes);
  dim3 grid(static_cast<unsigned>(std::min<long long>(n_work, SmCount())));
#define CAVS_DUAL(BN)                                                                                                            \
  (kmajor_b ? LaunchDual<BN, 0, 0>(ma0, mb0, *mcs[0], ps[0], ma1, mb1, *mcs[1], ps[1], grid, stream)                            \
            : LaunchDual<BN, 0, 1>(ma0, mb0, *mcs[0], ps[0], ma1, mb1, *mcs[1], ps[1], grid, stream))
  return bn == 256 ? CAVS_DUAL(256) : (bn == 128 ? CAVS_DUAL(128) : CAVS_DUAL(64));
#undef CAVS_DUAL
}

int GemmBf16(const GemmBf16Args& g, cudaStream_t stream) {
  CAVS_REQUIRE(g.m >= 0 && g.n >= 0 && g.k >= 0, CAVS_ERR_BAD_ARG, "gemm_bf16: negative dimension");
  if (g.m == 0 || g.n == 0) return CAVS_OK;
  CAVS_REQUIRE(g.k > 0, CAVS_ERR_BAD_ARG, "gemm_bf16: k must be positive");
  CAVS_REQUIRE(g.a && g.b && g.c, CAVS_ERR_BAD_ARG, "gemm_bf16: null pointer");
  TcOperandMap ma, mb;
  if (int rc = EncodeTcOperand(&ma, g.a, g.m, g.k, g.lda, g.a_major, tc::kBM)) return rc;
  const int tile_n = std::max(1, g.splits) == 1 ? GemmBf16TileNFor(g.m, g.n, g.k) : GemmBf16TileN(g.n);
  if (int rc = EncodeTcOperand(&mb, g.b, g.n, g.k, g.ldb, g.b_major, tile_n)) return rc;
  GemmBf16MappedArgs a;
  a.c = g.c; a.ldc = g.ldc; a.out_mode = g.out_mode;
  a.a = &ma; a.b = &mb;
  a.m = g.m; a.n = g.n; a.k = g.k;
  a.splits = g.splits; a.scratch = g.scratch; a.scratch_bytes = g.scratch_bytes; a.status = g.status;
  a.wait_poll_limit = g.wait_poll_limit; a.withhold_loads = g.withhold_loads;
  return GemmBf16Mapped(a, stream);
}

}  // namespace cavs_b200

extern "C" int cavs_gemm_bf16(void* c, long long ldc, int out_mode, const void* a, long long lda, int a_major,
                              const void* b, long long ldb, int b_major, int m, int n, int k, int splits, void* scratch,
                              size_t scratch_bytes, int* status, void* stream) {
  cavs_b200::GemmBf16Args g{};
  g.c = c; g.ldc = ldc; g.out_mode = out_mode;
  g.a = a; g.lda = lda; g.a_major = a_major;
  g.b = b; g.ldb = ldb; g.b_major = b_major;
  g.m = m; g.n = n; g.k = k;
  g.splits = splits; g.scratch = scratch; g.scratch_bytes = scratch_bytes; g.status = status;
  return cavs_b200::GemmBf16(g, static_cast<cudaStream_t>(stream));
}

extern "C" int cavs_gemm_bf16_wait_selftest(void* c, long long ldc, const void* a, long long lda, const void* b, long long ldb, int m,
                                            int n, int k, int* status, void* stream) {
  CAVS_REQUIRE(status != nullptr, CAVS_ERR_BAD_ARG, "gemm_bf16_wait_selftest: a status word is required");
  cavs_b200::GemmBf16Args g{};
  g.c = c; g.ldc = ldc; g.out_mode = 0;
  g.a = a; g.lda = lda; g.a_major = 0;
  g.b = b; g.ldb = ldb; g.b_major = 1;
  g.m = m; g.n = n; g.k = k;
  g.status = status;
  g.wait_poll_limit = 1u << 14;   // a few milliseconds per wait instead of a third of a second
  g.withhold_loads = 1;
  return cavs_b200::GemmBf16(g, static_cast<cudaStream_t>(stream));
}

extern "C" size_t cavs_gemm_bf16_scratch_bytes(int m, int n, int splits) {
  return cavs_b200::GemmBf16ScratchBytes(m, n, splits);
}
