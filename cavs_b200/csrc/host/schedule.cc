#include "host/schedule.h"

#include <algorithm>
#include <cstring>

#include "abi_common.h"

namespace cavs_b200 {

int LevelSchedule::Load(const int32_t* parents, int batch, int max_len, int n_slots, std::string* err) {
  if (parents == nullptr || batch < 0 || max_len <= 0 || n_slots < 1 || n_slots > kMaxSlots) {
    *err = "schedule: bad argument (parents null, batch < 0, max_len <= 0 or slots outside 1..4)";
    return CAVS_ERR_BAD_ARG;
  }
  batch_ = batch; max_len_ = max_len; n_slots_ = n_slots;
  sample_off_.assign(static_cast<size_t>(batch) + 1, 0);
  // Pass 1: sample lengths.  The root carries -1 and must be the sample's last vertex.
  for (int i = 0; i < batch; ++i) {
    const int32_t* row = parents + static_cast<size_t>(i) * max_len;
    const int32_t* end = std::find(row, row + max_len, -1);
    if (end == row + max_len) {
      *err = "schedule: sample " + std::to_string(i) + " has no -1 terminator";
      return CAVS_ERR_BAD_GRAPH;
    }
    sample_off_[i + 1] = sample_off_[i] + static_cast<int32_t>(end - row) + 1;
  }
  const int n = n_total_ = sample_off_[batch];
  const size_t nz = static_cast<size_t>(n);
  parent_g_.assign(nz, -1);
  nchild_g_.assign(nz, 0);
  child_g_.assign(nz * n_slots, -1);
  // Pass 2: adjacency in global-id space; children land in ascending id order.
  for (int i = 0; i < batch; ++i) {
    const int32_t* row = parents + static_cast<size_t>(i) * max_len;
    const int base = sample_off_[i], len = sample_off_[i + 1] - base;
    for (int j = 0; j + 1 < len; ++j) {
      const int p = row[j];
      if (p < 0 || p >= len || p == j) {
        *err = "schedule: sample " + std::to_string(i) + " vertex " + std::to_string(j) + " has parent index " +
               std::to_string(p) + " outside the sample";
        return CAVS_ERR_BAD_GRAPH;
      }
      const int pg = base + p;
      parent_g_[base + j] = pg;
      int& k = nchild_g_[pg];
      if (k >= n_slots) {
        *err = "schedule: sample " + std::to_string(i) + " vertex " + std::to_string(p) + " has more than " +
               std::to_string(n_slots) + " children";
        return CAVS_ERR_BAD_GRAPH;
      }
      child_g_[static_cast<size_t>(k) * nz + pg] = base + j;
      ++k;
    }
  }
  // Pass 3: wavefront.  t2j doubles as the frontier queue: level l occupies
  // t2j[level_off[l] .. level_off[l+1]) and is scanned to discover level l+1.
  t2j_.assign(nz, 0);
  j2t_.assign(nz, -1);
  hits_.assign(nz, 0);
  level_off_.clear();
  level_off_.push_back(0);
  int placed = 0;
  for (int g = 0; g < n; ++g)
    if (nchild_g_[g] == 0 && parent_g_[g] >= 0) { j2t_[g] = placed; t2j_[placed++] = g; }
  max_level_rows_ = placed;
  int begin = 0;
  while (placed > begin) {
    level_off_.push_back(placed);
    max_level_rows_ = std::max(max_level_rows_, placed - begin);
    const int end = placed;
    for (int t = begin; t < end; ++t) {
      const int p = parent_g_[t2j_[t]];
      if (p >= 0 && ++hits_[p] == nchild_g_[p]) { j2t_[p] = placed; t2j_[placed++] = p; }
    }
    begin = end;
  }
  n_sched_ = placed;
  if (placed != n) {
    for (int g = 0; g < n; ++g)
      if (j2t_[g] < 0 && !(nchild_g_[g] == 0 && parent_g_[g] < 0)) {
        *err = "schedule: vertex " + std::to_string(g) + " is on a cycle (never becomes ready)";
        return CAVS_ERR_BAD_GRAPH;
      }
  }
  // Pass 4: adjacency in tensor-id space.
  child_t_.assign(nz * n_slots, -1);
  parent_t_.assign(nz, -1);
  n_roots_ = 0;
  for (int t = 0; t < n_sched_; ++t) {
    const int g = t2j_[t];
    const int p = parent_g_[g];
    if (p >= 0) parent_t_[t] = j2t_[p]; else ++n_roots_;
    for (int c = 0; c < nchild_g_[g]; ++c) child_t_[static_cast<size_t>(c) * nz + t] = j2t_[child_g_[static_cast<size_t>(c) * nz + g]];
  }
  return CAVS_OK;
}

void LevelSchedule::RefGather(int level, int slot, std::vector<int32_t>* out) const {
  out->clear();
  if (level <= 0 || slot >= n_slots_) return;
  const size_t nz = static_cast<size_t>(n_total_);
  for (int t = level_off_[level]; t < level_off_[level + 1]; ++t) {
    const int c = child_t_[static_cast<size_t>(slot) * nz + t];
    if (c >= 0) out->push_back(c);
  }
}

void LevelSchedule::RefScatter(int level, std::vector<int32_t>* out) const {
  out->clear();
  for (int t = level_off_[level]; t < level_off_[level + 1]; ++t)
    if (parent_t_[t] >= 0) out->push_back(t);
}

void LevelSchedule::RefRoots(std::vector<int32_t>* out) const {
  out->clear();
  for (int t = 0; t < n_sched_; ++t)
    if (parent_t_[t] < 0) out->push_back(t);
}

void LevelSchedule::Tables(TableMode mode, int32_t* fg, int32_t* fs, int32_t* bg, int32_t* bs) const {
  const size_t nz = static_cast<size_t>(n_total_);
  std::fill(fg, fg + nz * n_slots_, -1);
  std::fill(bs, bs + nz * n_slots_, -1);
  std::fill(fs, fs + nz, -1);
  std::fill(bg, bg + nz, -1);
  if (mode == kAligned) {
    for (int c = 0; c < n_slots_; ++c)
      for (int t = 0; t < n_sched_; ++t) fg[c * nz + t] = bs[c * nz + t] = child_t_[c * nz + t];
    for (int t = 0; t < n_sched_; ++t)
      if (parent_t_[t] >= 0) fs[t] = bg[t] = t;
    return;
  }
  std::vector<int32_t> list;
  for (int l = 0; l < n_levels(); ++l) {
    const int off = level_off_[l];
    for (int c = 0; c < n_slots_; ++c) {
      RefGather(l, c, &list);
      for (size_t b = 0; b < list.size(); ++b) fg[c * nz + off + b] = bs[c * nz + off + b] = list[b];
    }
    RefScatter(l, &list);
    for (size_t b = 0; b < list.size(); ++b) fs[off + b] = bg[off + b] = list[b];
  }
}

void LevelSchedule::RefStream(std::vector<int32_t>* out) const {
  out->clear();
  auto put = [out](const std::vector<int32_t>& v) {
    out->push_back(static_cast<int32_t>(v.size()));
    out->insert(out->end(), v.begin(), v.end());
  };
  auto put_range = [out](const int32_t* p, int n) {
    out->push_back(n);
    out->insert(out->end(), p, p + n);
  };
  const int L = n_levels();
  out->push_back(n_total_);
  out->push_back(L);
  out->insert(out->end(), level_off_.begin(), level_off_.end());
  const int n0 = L > 0 ? level_off_[1] : 0;
  std::vector<int32_t> list;
  for (int l = 0; l < L; ++l) {
    put_range(t2j_.data() + level_off_[l], level_off_[l + 1] - level_off_[l]);
    for (int c = 0; c < 2; ++c) { RefGather(l, c, &list); put(list); }
    RefScatter(l, &list); put(list);
    put_range(t2j_.data(), n0);
  }
  out->insert(out->end(), t2j_.begin(), t2j_.end());
  std::vector<int32_t> roots;
  RefRoots(&roots);
  for (int l = L - 1; l >= 0; --l) {
    out->push_back(level_off_[l]);
    put_range(t2j_.data() + level_off_[l], level_off_[l + 1] - level_off_[l]);
    RefScatter(l, &list); put(list);
    for (int c = 0; c < 2; ++c) { RefGather(l, c, &list); put(list); }
    put(roots);
  }
}

}  // namespace cavs_b200
