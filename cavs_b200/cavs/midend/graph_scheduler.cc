#include "cavs/midend/graph_scheduler.h"

#include <cuda_runtime.h>

#include "cavs_b200.h"

namespace midend {

struct GraphSchedulerBase::Impl {
  cavs_sched* sched = nullptr;
  int n_total = 0, n_sched = 0, n_levels = 0, max_rows = 0;
  std::vector<int> level_off, t2j, roots;
  // Per level: compact lists (the reference's), and where they sit in the device blob.
  struct Level { std::vector<int> g[2], s; size_t dev_g[2], dev_s; };
  std::vector<Level> levels;
  // Device blob: t2j | fg aligned [2,N] | fs aligned [N] | roots | compact lists...
  std::vector<int> blob;     // host image of the device blob
  int* dev = nullptr;
  bool dev_fresh = false;    // device copy matches `blob`
  size_t dev_cap = 0, off_fg = 0, off_fs = 0, off_roots = 0;
  // One-vertex-per-round mode (tensor id == job id).  Blob: identity [N] | forward jobs | backward jobs |
  // child 0 by job [N] | child 1 by job [N] | own id where the vertex has a parent, else -1 [N].
  bool serial = false;
  std::vector<int> sweep[2], sweep_init[2], parent_j, child_j[2];
  size_t off_sweep[2] = {0, 0}, off_child[2] = {0, 0}, off_self = 0;
  // Uploads the blob on first use after a LoadGraph, so host-only users never touch CUDA.
  const int* Device() {
    if (!dev_fresh) {
      if (blob.size() > dev_cap) {
        if (dev) cudaFree(dev);
        dev_cap = blob.size() * 2 + 64;
        cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&dev), dev_cap * sizeof(int));
        CHECK(e == cudaSuccess) << cudaGetErrorString(e);
      }
      if (!blob.empty()) {
        cudaError_t e = cudaMemcpy(dev, blob.data(), blob.size() * sizeof(int), cudaMemcpyHostToDevice);
        CHECK(e == cudaSuccess) << cudaGetErrorString(e);
      }
      dev_fresh = true;
    }
    return dev;
  }
  ~Impl() {
    if (sched) cavs_sched_destroy(sched);
    if (dev) cudaFree(dev);
  }
};

GraphSchedulerBase::GraphSchedulerBase() : impl_(new Impl()) {
  tids_for_gather_init_.resize(2);
  tids_for_gather_.resize(2);
  tids_for_scatter_.resize(2);
  CHECK(cavs_sched_create(&impl_->sched) == CAVS_OK);
}
GraphSchedulerBase::~GraphSchedulerBase() {}

int GraphSchedulerBase::LoadGraph(const Tensor& graph_struct) {
  CHECK(graph_struct.dims() == 2) << graph_struct.debug_info();
  CHECK(graph_struct.device_type() == CPU) << graph_struct.debug_info();
  Impl& m = *impl_;
  batch_size_ = graph_struct.dims(0);
  const int rc = cavs_sched_load(m.sched, graph_struct.data<int>(), graph_struct.dims(0), graph_struct.dims(1), 2);
  CHECK(rc == CAVS_OK) << cavs_last_error();
  CHECK(cavs_sched_counts(m.sched, &m.n_total, &m.n_sched, &m.n_levels, &m.max_rows) == CAVS_OK);
  total_length_ = m.n_total;
  const int n = m.n_total;
  m.level_off.assign(m.n_levels + 1, 0);
  CHECK(cavs_sched_level_offsets(m.sched, m.level_off.data(), m.n_levels + 1) == CAVS_OK);
  m.t2j.assign(n, 0);
  std::vector<int> j2t(n), fg(2 * static_cast<size_t>(n)), fs(n), bg(n), bs(2 * static_cast<size_t>(n));
  if (n > 0) {
    CHECK(cavs_sched_maps(m.sched, m.t2j.data(), j2t.data(), n) == CAVS_OK);
    CHECK(cavs_sched_tables(m.sched, 0, fg.data(), fs.data(), bg.data(), bs.data(), n) == CAVS_OK);
  }
  tids_to_jobids_ = m.t2j;
  m.roots.clear();
  for (int t = 0; t < m.n_sched; t++) if (fs[t] < 0) m.roots.push_back(t);
  // Host blob mirrors the device layout.
  std::vector<int>& blob = m.blob;
  blob.clear();
  blob.insert(blob.end(), m.t2j.begin(), m.t2j.end());
  m.off_fg = blob.size(); blob.insert(blob.end(), fg.begin(), fg.end());
  m.off_fs = blob.size(); blob.insert(blob.end(), fs.begin(), fs.end());
  m.off_roots = blob.size(); blob.insert(blob.end(), m.roots.begin(), m.roots.end());
  m.levels.assign(m.n_levels, Impl::Level());
  std::vector<int> tmp(m.max_rows > 0 ? m.max_rows : 1);
  for (int l = 0; l < m.n_levels; l++) {
    Impl::Level& lv = m.levels[l];
    int cnt = 0;
    for (int c = 0; c < 2; c++) {
      CHECK(cavs_sched_ref_gather(m.sched, l, c, tmp.data(), static_cast<int>(tmp.size()), &cnt) == CAVS_OK);
      lv.g[c].assign(tmp.begin(), tmp.begin() + cnt);
      lv.dev_g[c] = blob.size();
      blob.insert(blob.end(), lv.g[c].begin(), lv.g[c].end());
    }
    CHECK(cavs_sched_ref_scatter(m.sched, l, tmp.data(), static_cast<int>(tmp.size()), &cnt) == CAVS_OK);
    lv.s.assign(tmp.begin(), tmp.begin() + cnt);
    lv.dev_s = blob.size();
    blob.insert(blob.end(), lv.s.begin(), lv.s.end());
  }
  m.serial = OneVertexPerRound();
  if (m.serial) {
    const int cap = n > 0 ? n : 1;
    m.parent_j.assign(cap, -1);
    std::vector<int> child(2 * static_cast<size_t>(cap), -1);
    if (n > 0) CHECK(cavs_sched_adjacency(m.sched, m.parent_j.data(), child.data(), cap) == CAVS_OK);
    for (int c = 0; c < 2; c++) m.child_j[c].assign(child.begin() + c * cap, child.begin() + (c + 1) * cap);
    for (int d = 0; d < 2; d++) {
      int rounds = 0;
      m.sweep[d].assign(cap, 0);
      m.sweep_init[d].assign(cap, -1);
      CHECK(cavs_sched_serial_rounds(m.sched, d, m.sweep[d].data(), m.sweep_init[d].data(), cap, &rounds) == CAVS_OK);
      m.sweep[d].resize(rounds);
      m.sweep_init[d].resize(rounds);
    }
    if (m.sweep[0].empty()) m.sweep[1].clear();     // nothing ran forward: nothing to differentiate
    tids_to_jobids_.assign(n, 0);
    for (int g : m.sweep[0]) tids_to_jobids_[g] = g;
    blob.clear();
    for (int g = 0; g < n; g++) blob.push_back(g);
    for (int d = 0; d < 2; d++) { m.off_sweep[d] = blob.size(); blob.insert(blob.end(), m.sweep[d].begin(), m.sweep[d].end()); }
    for (int c = 0; c < 2; c++) { m.off_child[c] = blob.size(); blob.insert(blob.end(), m.child_j[c].begin(), m.child_j[c].begin() + n); }
    m.off_self = blob.size();
    for (int g = 0; g < n; g++) blob.push_back(m.parent_j[g] >= 0 ? g : -1);
  }
  m.dev_fresh = false;
  round_ = -1;
  forward_ = true;
  ready_to_execute_ids_.clear();
  return total_length_;
}

int GraphSchedulerBase::ReverseGraph() {
  CHECK(batch_size_ > 0);
  forward_ = false;
  return total_length_;
}

bool GraphSchedulerBase::HasChild(int job_id) const {
  // forward graph: a vertex has children iff it is not on level 0
  CHECK(job_id >= 0 && job_id < total_length_);
  const Impl& m = *impl_;
  if (m.serial) return forward_ ? m.child_j[0][job_id] >= 0 : m.parent_j[job_id] >= 0;   // the reversed graph swaps the roles
  for (int t = 0; t < (m.n_levels > 0 ? m.level_off[1] : 0); t++)
    if (m.t2j[t] == job_id) return false;
  return true;
}

void GraphSchedulerBase::SetRound(int level, bool forward) {
  const Impl& m = *impl_;
  round_ = level;
  for (auto& v : tids_for_gather_) v.clear();
  for (auto& v : tids_for_scatter_) v.clear();
  ready_to_execute_ids_.clear();
  if (level < 0 || level >= m.n_levels) return;
  ready_to_execute_ids_.assign(m.t2j.begin() + m.level_off[level], m.t2j.begin() + m.level_off[level + 1]);
  const Impl::Level& lv = m.levels[level];
  if (forward) {
    tids_for_gather_[0] = lv.g[0];
    tids_for_gather_[1] = lv.g[1];
    tids_for_scatter_[0] = lv.s;
  } else {
    // graph_scheduler.cc:194-198,246-257: gather := forward scatter list, scatter := forward gather lists
    tids_for_gather_[0] = lv.s;
    tids_for_scatter_[0] = lv.g[0];
    tids_for_scatter_[1] = lv.g[1];
  }
  tids_for_gather_init_[0].assign(m.t2j.begin(), m.t2j.begin() + (m.n_levels > 0 ? m.level_off[1] : 0));
  tids_for_gather_init_[1] = m.roots;
}

void GraphSchedulerBase::SetSerialRound(int round, bool forward) {
  const Impl& m = *impl_;
  const std::vector<int>& order = m.sweep[forward ? 0 : 1];
  round_ = round;
  for (auto& v : tids_for_gather_) v.clear();
  for (auto& v : tids_for_scatter_) v.clear();
  ready_to_execute_ids_.clear();
  if (round < 0 || round >= static_cast<int>(order.size())) return;
  const int g = order[round];
  ready_to_execute_ids_.push_back(g);
  // graph_scheduler.cc:143-166: the lists of children hold the children's ids, the list towards the
  // parent holds the vertex's own id once per parent ("only a count number").
  std::vector<std::vector<int>>& kids = forward ? tids_for_gather_ : tids_for_scatter_;
  std::vector<std::vector<int>>& self = forward ? tids_for_scatter_ : tids_for_gather_;
  for (int c = 0; c < 2; c++)
    if (m.child_j[c][g] >= 0) kids[c].push_back(m.child_j[c][g]);
  if (m.parent_j[g] >= 0) self[0].push_back(g);
  const int init = m.sweep_init[forward ? 0 : 1][round];
  tids_for_gather_init_[forward ? 0 : 1].clear();
  if (init >= 0) tids_for_gather_init_[forward ? 0 : 1].push_back(init);
}

const std::vector<int>& GraphSchedulerBase::CurrentRoundTensorIdsForGatherInitialization() const {
  return forward_ ? tids_for_gather_init_[0] : tids_for_gather_init_[1];
}
const std::vector<int>& GraphSchedulerBase::CurrentRoundTensorIdsForGather(int child_offset) const {
  CHECK(child_offset >= 0 && child_offset < 2);
  return tids_for_gather_[child_offset];
}
const std::vector<int>& GraphSchedulerBase::CurrentRoundTensorIdsForScatter(int child_offset) const {
  CHECK(child_offset >= 0 && child_offset < 2);
  return tids_for_scatter_[child_offset];
}

const int* GraphSchedulerBase::DeviceJobIds(int* count) const {
  Impl& m = *impl_;
  if (m.serial) {
    CHECK(!ready_to_execute_ids_.empty());
    *count = 1;
    return m.Device() + m.off_sweep[forward_ ? 0 : 1] + round_;
  }
  CHECK(round_ >= 0 && round_ < m.n_levels);
  *count = m.level_off[round_ + 1] - m.level_off[round_];
  return m.Device() + m.level_off[round_];
}
const int* GraphSchedulerBase::DeviceTensorIdsToJobIds(int* count) const {
  if (impl_->serial) { *count = impl_->n_total; return impl_->Device(); }   // identity
  *count = impl_->n_sched;
  return impl_->Device();
}
// One-vertex rounds: the list is the single table entry of the round's vertex (or empty when that
// entry is -1 and the caller wants the reference's compact lists).
static const int* SerialEntry(const int* dev, size_t table, const std::vector<int>& host, int job, bool aligned, int* count) {
  *count = (aligned || host[job] >= 0) ? 1 : 0;
  return dev + table + job;
}

const int* GraphSchedulerBase::DeviceIdsForGather(int child_offset, int* count) const {
  Impl& m = *impl_;
  if (m.serial) {
    CHECK(!ready_to_execute_ids_.empty());
    CHECK(child_offset >= 0 && child_offset < 2);
    const int g = ready_to_execute_ids_[0];
    if (forward_) return SerialEntry(m.Device(), m.off_child[child_offset], m.child_j[child_offset], g, aligned_, count);
    CHECK(child_offset == 0);
    return SerialEntry(m.Device(), m.off_self, m.parent_j, g, aligned_, count);
  }
  CHECK(round_ >= 0 && round_ < m.n_levels);
  CHECK(child_offset >= 0 && child_offset < 2);
  const int off = m.level_off[round_], rows = m.level_off[round_ + 1] - off;
  if (forward_) {
    if (aligned_) { *count = rows; return m.Device() + m.off_fg + static_cast<size_t>(child_offset) * m.n_total + off; }
    *count = static_cast<int>(m.levels[round_].g[child_offset].size());
    return m.Device() + m.levels[round_].dev_g[child_offset];
  }
  CHECK(child_offset == 0);
  if (aligned_) { *count = rows; return m.Device() + m.off_fs + off; }
  *count = static_cast<int>(m.levels[round_].s.size());
  return m.Device() + m.levels[round_].dev_s;
}
const int* GraphSchedulerBase::DeviceIdsForScatter(int child_offset, int* count) const {
  Impl& m = *impl_;
  if (m.serial) {
    CHECK(!ready_to_execute_ids_.empty());
    CHECK(child_offset >= 0 && child_offset < 2);
    const int g = ready_to_execute_ids_[0];
    if (!forward_) return SerialEntry(m.Device(), m.off_child[child_offset], m.child_j[child_offset], g, aligned_, count);
    CHECK(child_offset == 0);
    return SerialEntry(m.Device(), m.off_self, m.parent_j, g, aligned_, count);
  }
  CHECK(round_ >= 0 && round_ < m.n_levels);
  CHECK(child_offset >= 0 && child_offset < 2);
  const int off = m.level_off[round_], rows = m.level_off[round_ + 1] - off;
  if (forward_) {
    CHECK(child_offset == 0);
    if (aligned_) { *count = rows; return m.Device() + m.off_fs + off; }
    *count = static_cast<int>(m.levels[round_].s.size());
    return m.Device() + m.levels[round_].dev_s;
  }
  if (aligned_) { *count = rows; return m.Device() + m.off_fg + static_cast<size_t>(child_offset) * m.n_total + off; }
  *count = static_cast<int>(m.levels[round_].g[child_offset].size());
  return m.Device() + m.levels[round_].dev_g[child_offset];
}

void BatchGraphScheduler::Initialize() {
  CHECK(Terminate());
  SetRound(forward_ ? 0 : impl_->n_levels - 1, forward_);
}
void BatchGraphScheduler::ActivateNext() { SetRound(forward_ ? round_ + 1 : round_ - 1, forward_); }
int BatchGraphScheduler::GetCurrentRoundOffset() const {
  CHECK(round_ >= 0 && round_ < impl_->n_levels);
  return impl_->level_off[round_];
}

void SerialGraphScheduler::Initialize() {
  CHECK(Terminate());
  SetSerialRound(0, forward_);
}
void SerialGraphScheduler::ActivateNext() { SetSerialRound(round_ + 1, forward_); }

}  // namespace midend
