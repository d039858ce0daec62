#include "host/schedule.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "abi_common.h"
#include "host/threads.h"

namespace cavs_b200 {

namespace {

// Runs fn(begin, end) over [0, n) on up to `threads` host threads (the caller's included).
template <typename F>
void ParallelFor(int n, int threads, F fn) {
  threads = std::max(1, std::min(threads, n / 256 + 1));   // a thread costs tens of microseconds to start: few samples, few threads
  if (threads == 1) { fn(0, n); return; }
  std::vector<std::thread> pool;
  const int chunk = (n + threads - 1) / threads;
  for (int t = 1; t < threads; ++t) {
    const int b = t * chunk, e = std::min(n, b + chunk);
    if (b < e) pool.emplace_back([=] { fn(b, e); });
  }
  fn(0, std::min(n, chunk));
  for (auto& th : pool) th.join();
}

// v = n copies of value, the fill split over the host threads (the per-batch arrays are tens of megabytes together:
// filled by one thread they cost as much as the scheduling itself).
void ParallelAssign(std::vector<int32_t>* v, size_t n, int32_t value, int threads) {
  v->resize(n);
  int32_t* p = v->data();
  constexpr size_t kBlock = 1 << 15;
  const int blocks = static_cast<int>((n + kBlock - 1) / kBlock);
  ParallelFor(blocks, std::min(threads, std::max(1, blocks / 4)), [=](int b0, int b1) {
    std::fill(p + static_cast<size_t>(b0) * kBlock, p + std::min(n, static_cast<size_t>(b1) * kBlock), value);
  });
}

int HostThreads() {
  static const int n = HostThreadBudget(16);
  return n;
}

}  // namespace

// The reference discovers levels by one global wavefront over all samples
// (graph_scheduler.cc:169-258).  Its order has a structure that makes the work separable: level 0
// lists vertices in ascending global id, i.e. sample by sample, and scanning a sample-major level
// discovers the next level sample by sample too -- so EVERY level is the concatenation, over
// samples, of that sample's own wavefront order.  Each sample (a tree of at most max_len vertices,
// cache resident) is therefore scheduled independently and in parallel; a prefix sum over
// per-sample level counts then places it in the global order.  Output is identical to the
// sequential wavefront.
int LevelSchedule::Load(const int32_t* parents, int batch, int max_len, int n_slots, std::string* err) {
  if (parents == nullptr || batch < 0 || max_len <= 0 || n_slots < 1 || n_slots > kMaxSlots) {
    *err = "schedule: bad argument (parents null, batch < 0, max_len <= 0 or slots outside 1..4)";
    return CAVS_ERR_BAD_ARG;
  }
  batch_ = batch; max_len_ = max_len; n_slots_ = n_slots;
  const int threads = HostThreads();
  sample_off_.assign(static_cast<size_t>(batch) + 1, 0);

  // Phase A (parallel over samples): validate, run the sample's wavefront, record for every local
  // vertex its level and its position inside the sample's list of that level.
  // local_[i*max_len + j] = level << 16 | position  (max_len <= 65535 enforced below), -1 if unscheduled.
  if (max_len > 65535) { *err = "schedule: max_len above 65535"; return CAVS_ERR_UNSUPPORTED; }
  ParallelAssign(&local_, static_cast<size_t>(batch) * max_len, -1, threads);
  sample_len_.assign(batch, 0);
  sample_levels_.assign(batch, 0);
  // per-sample level counts, laid out [batch][max_len] lazily: only the first sample_levels_[i] entries are used
  ParallelAssign(&level_cnt_, static_cast<size_t>(batch) * max_len, 0, threads);
  std::vector<int> first_error(batch, 0);
  ParallelFor(batch, threads, [&](int b0, int b1) {
    std::vector<int32_t> nchild(max_len), hits(max_len), cur(max_len), nxt(max_len);
    for (int i = b0; i < b1; ++i) {
      const int32_t* row = parents + static_cast<size_t>(i) * max_len;
      const int32_t* end = std::find(row, row + max_len, -1);
      if (end == row + max_len) { first_error[i] = 1; continue; }        // no terminator
      const int len = static_cast<int>(end - row) + 1;
      sample_len_[i] = len;
      std::fill(nchild.begin(), nchild.begin() + len, 0);
      std::fill(hits.begin(), hits.begin() + len, 0);
      bool bad = false;
      for (int j = 0; j + 1 < len; ++j) {
        const int p = row[j];
        if (p < 0 || p >= len || p == j) { first_error[i] = 2 + (j << 4); bad = true; break; }
        if (++nchild[p] > n_slots) { first_error[i] = 3 + (p << 4); bad = true; break; }
      }
      if (bad) continue;
      int32_t* loc = local_.data() + static_cast<size_t>(i) * max_len;
      int32_t* cnt = level_cnt_.data() + static_cast<size_t>(i) * max_len;
      int n_cur = 0, placed = 0, level = 0;
      for (int j = 0; j + 1 < len; ++j)            // the root (j = len-1) has no parent: never on level 0
        if (nchild[j] == 0) cur[n_cur++] = j;
      while (n_cur > 0) {
        cnt[level] = n_cur;
        int n_nxt = 0;
        for (int b = 0; b < n_cur; ++b) {
          const int v = cur[b];
          loc[v] = (level << 16) | b;
          if (v + 1 < len) {                       // every vertex but the root has a parent
            const int p = row[v];
            if (++hits[p] == nchild[p]) nxt[n_nxt++] = p;
          }
        }
        placed += n_cur;
        cur.swap(nxt);
        n_cur = n_nxt;
        ++level;
      }
      sample_levels_[i] = level;
      // A single-vertex sample never executes (graph_scheduler.cc:180); anything else left over is a cycle.
      if (placed != len && !(len == 1)) first_error[i] = 4;
    }
  });
  for (int i = 0; i < batch; ++i) {
    if (first_error[i] == 0) continue;
    const int code = first_error[i] & 15, where = first_error[i] >> 4;
    if (code == 1) *err = "schedule: sample " + std::to_string(i) + " has no -1 terminator";
    else if (code == 2) *err = "schedule: sample " + std::to_string(i) + " vertex " + std::to_string(where) + " has a parent index outside the sample";
    else if (code == 3) *err = "schedule: sample " + std::to_string(i) + " vertex " + std::to_string(where) + " has more than " + std::to_string(n_slots) + " children";
    else *err = "schedule: sample " + std::to_string(i) + " contains a cycle (a vertex never becomes ready)";
    return CAVS_ERR_BAD_GRAPH;
  }

  // Phase B (serial, O(batch * depth)): global sizes and, per sample and level, the first global
  // position of that sample's block.
  int n_levels = 0;
  for (int i = 0; i < batch; ++i) {
    sample_off_[i + 1] = sample_off_[i] + sample_len_[i];
    n_levels = std::max(n_levels, sample_levels_[i]);
  }
  const int n = n_total_ = sample_off_[batch];
  const size_t nz = static_cast<size_t>(n);
  level_off_.assign(static_cast<size_t>(n_levels) + 1, 0);
  for (int i = 0; i < batch; ++i) {
    const int32_t* cnt = level_cnt_.data() + static_cast<size_t>(i) * max_len;
    for (int l = 0; l < sample_levels_[i]; ++l) level_off_[l + 1] += cnt[l];
  }
  max_level_rows_ = 0;
  for (int l = 0; l < n_levels; ++l) {
    max_level_rows_ = std::max(max_level_rows_, level_off_[l + 1]);
    level_off_[l + 1] += level_off_[l];
  }
  n_sched_ = level_off_[n_levels];
  // level_cnt_[i][l] becomes the global tensor id of sample i's first vertex on level l
  if (order_ == kBatched) {
    std::vector<int32_t> running(level_off_.begin(), level_off_.end() - 1);
    for (int i = 0; i < batch; ++i) {
      int32_t* cnt = level_cnt_.data() + static_cast<size_t>(i) * max_len;
      for (int l = 0; l < sample_levels_[i]; ++l) { const int c = cnt[l]; cnt[l] = running[l]; running[l] += c; }
    }
  } else {
    // One vertex per round: a sample's wavefront levels follow one another (the order a first-in
    // first-out work list visits them), samples follow one another.
    int32_t running = 0;
    for (int i = 0; i < batch; ++i) {
      int32_t* cnt = level_cnt_.data() + static_cast<size_t>(i) * max_len;
      for (int l = 0; l < sample_levels_[i]; ++l) { const int c = cnt[l]; cnt[l] = running; running += c; }
    }
    level_off_.resize(static_cast<size_t>(n_sched_) + 1);
    for (int t = 0; t <= n_sched_; ++t) level_off_[t] = t;
    max_level_rows_ = n_sched_ > 0 ? 1 : 0;
  }

  // Phase C (parallel over samples): global tensor ids and tensor-id-space adjacency.
  ParallelAssign(&t2j_, nz, 0, threads);
  ParallelAssign(&j2t_, nz, -1, threads);
  ParallelAssign(&child_t_, nz * n_slots, -1, threads);
  ParallelAssign(&parent_t_, nz, -1, threads);
  ParallelAssign(&child_j_, nz * n_slots, -1, threads);
  ParallelAssign(&parent_j_, nz, -1, threads);
  std::vector<int> roots_per_thread_sample(batch, 0);
  ParallelFor(batch, threads, [&](int b0, int b1) {
    std::vector<int32_t> slot_used(max_len);
    for (int i = b0; i < b1; ++i) {
      const int32_t* row = parents + static_cast<size_t>(i) * max_len;
      const int32_t* loc = local_.data() + static_cast<size_t>(i) * max_len;
      const int32_t* base_l = level_cnt_.data() + static_cast<size_t>(i) * max_len;
      const int len = sample_len_[i], base = sample_off_[i];
      if (sample_levels_[i] == 0) continue;       // single-vertex sample
      auto tid_of = [&](int v) { return base_l[loc[v] >> 16] + (loc[v] & 0xffff); };
      std::fill(slot_used.begin(), slot_used.begin() + len, 0);
      for (int v = 0; v < len; ++v) {
        const int t = tid_of(v);
        t2j_[t] = base + v;
        j2t_[base + v] = t;
        if (v + 1 < len) {
          const int p = row[v];
          const int pt = tid_of(p);
          parent_t_[t] = pt;
          // children land in ascending id order: v ascends, so the next free slot of p is v's slot
          child_j_[static_cast<size_t>(slot_used[p]) * nz + base + p] = base + v;
          parent_j_[base + v] = base + p;
          child_t_[static_cast<size_t>(slot_used[p]++) * nz + pt] = t;
        } else {
          roots_per_thread_sample[i] = 1;
        }
      }
    }
  });
  n_roots_ = 0;
  for (int i = 0; i < batch; ++i) n_roots_ += roots_per_thread_sample[i];
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

// The serial sweep as a work list over job ids.  "wake" edges are followed when a vertex finishes,
// "wait" edges must all have finished before a vertex runs; forward: wake = parent, wait = children,
// backward: the reverse (graph_scheduler.cc:73-81).  Details that shape the order:
//  * the list is first-in first-out and starts with sample 0's vertices that wait on nothing but wake
//    someone (:108-118), ascending id;
//  * the next sample joins when a vertex WITHOUT wake edges finishes (:135-137) -- its root in the
//    forward sweep, but every forward leaf in the backward sweep, so backward samples interleave;
//  * a sample of one vertex contributes nothing, and the sweep ends when the list runs empty (:141),
//    so forward execution stops at the first single-vertex sample;
//  * the gather-initialisation list holds the last vertex seen so far that waits on nothing (:101,153).
void LevelSchedule::SerialSweep(bool backward, std::vector<SerialRound>* rounds) const {
  rounds->clear();
  const size_t nz = static_cast<size_t>(n_total_);
  auto n_children = [&](int g) {
    int c = 0;
    while (c < n_slots_ && child_j_[static_cast<size_t>(c) * nz + g] >= 0) ++c;
    return c;
  };
  auto has_parent = [&](int g) { return parent_j_[g] >= 0 ? 1 : 0; };
  auto n_wake = [&](int g) { return backward ? n_children(g) : has_parent(g); };
  auto n_wait = [&](int g) { return backward ? has_parent(g) : n_children(g); };
  std::vector<int32_t> work, done(nz, 0);
  work.reserve(nz);
  auto admit = [&](int sample) {
    for (int g = sample_off_[sample]; g < sample_off_[sample + 1]; ++g)
      if (n_wait(g) == 0 && n_wake(g) > 0) work.push_back(g);
  };
  int sample = 0;
  int32_t init = -1;
  if (batch_ > 0) admit(0);
  for (size_t head = 0; head < work.size(); ++head) {
    const int g = work[head];
    SerialRound r;
    r.job = g;
    r.n_wake = n_wake(g);
    r.n_wait = n_wait(g);
    r.child[0] = r.child[1] = -1;
    // The two lists of neighbours a round reports: children in slot order in either direction.
    for (int c = 0; c < 2 && c < n_slots_; ++c) r.child[c] = child_j_[static_cast<size_t>(c) * nz + g];
    if (r.n_wait == 0) init = g;
    r.init = init;
    rounds->push_back(r);
    if (r.n_wake > 0) {
      if (backward) {
        for (int c = 0; c < r.n_wake; ++c) {
          const int p = child_j_[static_cast<size_t>(c) * nz + g];
          if (++done[p] == n_wait(p)) work.push_back(p);
        }
      } else {
        const int p = parent_j_[g];
        if (++done[p] == n_wait(p)) work.push_back(p);
      }
    } else if (++sample < batch_) {
      admit(sample);
    }
  }
}

void LevelSchedule::RefSerialStream(std::vector<int32_t>* out) const {
  out->clear();
  std::vector<SerialRound> fwd, bwd;
  SerialSweep(false, &fwd);
  if (!fwd.empty()) SerialSweep(true, &bwd);
  auto list = [out](int count, int32_t value) {
    out->push_back(count);
    for (int i = 0; i < count; ++i) out->push_back(value);
  };
  out->push_back(n_total_);
  out->push_back(static_cast<int32_t>(fwd.size()));
  std::vector<int32_t> ran(static_cast<size_t>(n_total_), 0);
  for (const SerialRound& r : fwd) {
    out->push_back(r.job);
    for (int c = 0; c < 2; ++c) list(r.child[c] >= 0 ? 1 : 0, r.child[c]);   // gather(c): the slot-c child
    list(r.n_wake, r.job);                                                // scatter(0): own id, once per parent
    list(r.init >= 0 ? 1 : 0, r.init);
    ran[r.job] = r.job;
  }
  out->insert(out->end(), ran.begin(), ran.end());
  out->push_back(static_cast<int32_t>(bwd.size()));
  for (const SerialRound& r : bwd) {
    out->push_back(r.job);
    list(r.n_wait, r.job);                                                // gather(0): own id, once per parent
    for (int c = 0; c < 2; ++c) list(r.child[c] >= 0 ? 1 : 0, r.child[c]);   // scatter(c): the slot-c child
    list(r.init >= 0 ? 1 : 0, r.init);
  }
}

}  // namespace cavs_b200
