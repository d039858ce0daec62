// Synthetic workloads with the shapes of the datasets the reference's apps read
// (SST trees: apps/paper/tree-lstm-cavs.cc:13,22-24; PTB chains:
// apps/paper/seq-lstm-cavs-varLength.cc:14,25), which are not distributed with it.
// One documented generator (SplitMix64) so that every consumer -- CUDA path, CPU
// oracle, tests -- sees identical inputs; no std::*_distribution (library-dependent).
#include <cmath>
#include <cstring>
#include <vector>

#include "abi_common.h"

namespace {

struct SplitMix64 {
  uint64_t s;
  explicit SplitMix64(uint64_t seed) : s(seed) {}
  uint64_t next() {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  // uniform integer in [lo, hi]
  int range(int lo, int hi) { return lo + static_cast<int>(next() % static_cast<uint64_t>(hi - lo + 1)); }
  // uniform in [0,1) with 24 random mantissa bits (exact in fp32)
  float unit24() { return static_cast<float>(next() >> 40) * (1.0f / 16777216.0f); }
  double unit53() { return static_cast<double>(next() >> 11) * (1.0 / 9007199254740992.0); }
};

struct TreeBuilder {
  SplitMix64* rng;
  int32_t* parent;
  uint8_t* leaf;
  int max_arity;
  int next_id = 0;
  // Emits the subtree over `leaves` leaves in post-order; returns the id of its root.
  int build(int leaves, bool allow_unary) {
    if (leaves == 1) {
      if (leaf) leaf[next_id] = 1;
      return next_id++;
    }
    int arity = 2;
    if (max_arity != 2) {
      const int lo = allow_unary ? 1 : 2;
      const int hi = max_arity < leaves ? max_arity : leaves;
      arity = rng->range(lo, hi < lo ? lo : hi);
    }
    int kids[cavs_b200_max_slots];
    int remaining = leaves;
    for (int c = 0; c < arity; ++c) {
      const int parts_left = arity - c - 1;
      const int take = parts_left == 0 ? remaining : rng->range(1, remaining - parts_left);
      kids[c] = build(take, arity != 1);
      remaining -= take;
    }
    const int me = next_id++;
    if (leaf) leaf[me] = 0;
    for (int c = 0; c < arity; ++c) parent[kids[c]] = me;
    return me;
  }
  static constexpr int cavs_b200_max_slots = 4;
};

}  // namespace

extern "C" int cavs_synth_trees(uint64_t seed, int batch, int leaf_lo, int leaf_hi, int max_arity, int max_len,
                                int32_t* parents, uint8_t* is_leaf) {
  CAVS_REQUIRE(parents && batch >= 0 && leaf_lo >= 1 && leaf_hi >= leaf_lo && max_arity >= 2 && max_arity <= 4,
               CAVS_ERR_BAD_ARG, "synth_trees: bad argument");
  const int worst = max_arity == 2 ? 2 * leaf_hi - 1 : 4 * leaf_hi - 2;
  CAVS_REQUIRE(max_len >= worst && max_len >= 1, CAVS_ERR_CAPACITY,
               "synth_trees: max_len must be at least " + std::to_string(worst));
  SplitMix64 rng(seed);
  for (int i = 0; i < batch; ++i) {
    int32_t* row = parents + static_cast<size_t>(i) * max_len;
    uint8_t* lrow = is_leaf ? is_leaf + static_cast<size_t>(i) * max_len : nullptr;
    for (int j = 0; j < max_len; ++j) row[j] = -1;
    if (lrow) std::memset(lrow, 0, static_cast<size_t>(max_len));
    TreeBuilder tb{&rng, row, lrow, max_arity};
    const int leaves = rng.range(leaf_lo, leaf_hi);
    const int root = tb.build(leaves, true);
    row[root] = -1;
  }
  return CAVS_OK;
}

extern "C" int cavs_synth_chains(uint64_t seed, int batch, int len_lo, int len_hi, int max_len, int32_t* parents) {
  CAVS_REQUIRE(parents && batch >= 0 && len_lo >= 1 && len_hi >= len_lo, CAVS_ERR_BAD_ARG, "synth_chains: bad argument");
  CAVS_REQUIRE(max_len >= len_hi, CAVS_ERR_CAPACITY, "synth_chains: max_len smaller than len_hi");
  SplitMix64 rng(seed);
  for (int i = 0; i < batch; ++i) {
    int32_t* row = parents + static_cast<size_t>(i) * max_len;
    const int len = rng.range(len_lo, len_hi);
    for (int j = 0; j < max_len; ++j) row[j] = (j + 1 < len) ? j + 1 : -1;
  }
  return CAVS_OK;
}

extern "C" int cavs_synth_zipf(uint64_t seed, double s, int vocab, int32_t* out, size_t count) {
  CAVS_REQUIRE(out && vocab >= 1 && s > 0.0, CAVS_ERR_BAD_ARG, "synth_zipf: bad argument");
  std::vector<double> cdf(static_cast<size_t>(vocab));
  double acc = 0.0;
  for (int r = 1; r <= vocab; ++r) { acc += std::pow(static_cast<double>(r), -s); cdf[r - 1] = acc; }
  SplitMix64 rng(seed);
  for (size_t i = 0; i < count; ++i) {
    const double u = rng.unit53() * acc;
    size_t lo = 0, hi = static_cast<size_t>(vocab) - 1;
    while (lo < hi) { const size_t mid = (lo + hi) / 2; if (cdf[mid] > u) hi = mid; else lo = mid + 1; }
    out[i] = static_cast<int32_t>(lo);
  }
  return CAVS_OK;
}

extern "C" int cavs_synth_uniform_int(uint64_t seed, int bound, int32_t* out, size_t count) {
  CAVS_REQUIRE(out && bound >= 1, CAVS_ERR_BAD_ARG, "synth_uniform_int: bad argument");
  SplitMix64 rng(seed);
  for (size_t i = 0; i < count; ++i) out[i] = rng.range(0, bound - 1);
  return CAVS_OK;
}

extern "C" int cavs_synth_uniform_float(uint64_t seed, float scale, float* out, size_t count) {
  CAVS_REQUIRE(out, CAVS_ERR_BAD_ARG, "synth_uniform_float: null output");
  SplitMix64 rng(seed);
  for (size_t i = 0; i < count; ++i) out[i] = (2.0f * rng.unit24() - 1.0f) * scale;
  return CAVS_OK;
}
