// Level schedule of a batch of per-sample graphs, built in one pass.
//
// Replaces the reference's round-by-round BatchGraphScheduler
// (cavs/midend/graph_scheduler.{h,cc}): instead of discovering one level per
// ActivateNext() call -- each call reserving four 1M-entry vectors
// (graph_scheduler.cc:209-214) and each graph op uploading its index list from
// pageable memory -- every level of the batch is laid out at once as flat arrays
// in tensor-id (execution) order, ready for a single pinned upload.  Samples are scheduled
// independently on several host threads (CAVS_HOST_THREADS, default min(cores, 8)).
//
// The job order inside each level and therefore every tensor id is identical to
// the reference's (ascending id on level 0, graph_scheduler.cc:178-188; discovery
// order afterwards, :215-238), so the reference's per-round lists can be
// regenerated exactly (RefStream, ref_* accessors).
#ifndef CAVS_B200_HOST_SCHEDULE_H_
#define CAVS_B200_HOST_SCHEDULE_H_

#include <cstdint>
#include <string>
#include <vector>

namespace cavs_b200 {

constexpr int kMaxSlots = 4;

enum TableMode {
  kAligned = 0,    // row b of a level talks to its own children / itself
  kRefCompat = 1,  // the reference's positional pairing of compact lists with level rows
};

// How vertices are grouped into rounds.
enum RoundOrder {
  kBatched = 0,    // one round per level of the whole batch (BatchGraphScheduler)
  kUnbatched = 1,  // one vertex per round, sample after sample (the reference's serial mode as an
                   // execution order: tensor ids follow execution, single-vertex samples are skipped)
};

class LevelSchedule {
 public:
  // Takes effect at the next Load().
  void SetOrder(RoundOrder order) { order_ = order; }
  RoundOrder order() const { return order_; }

  // parents: [batch, max_len] int32, local parent index per vertex, -1 marks the root
  // and ends the sample (graph_scheduler.cc:39).  Returns 0 or a CAVS_ERR_* code and
  // leaves a message in *err.
  int Load(const int32_t* parents, int batch, int max_len, int n_slots, std::string* err);

  int n_total() const { return n_total_; }          // vertices in the batch (LoadGraph's return value)
  int n_scheduled() const { return n_sched_; }      // vertices that execute (single-vertex samples never do)
  int n_levels() const { return static_cast<int>(level_off_.size()) - 1; }
  int n_slots() const { return n_slots_; }
  int batch() const { return batch_; }
  int max_level_rows() const { return max_level_rows_; }
  int n_roots() const { return n_roots_; }

  const std::vector<int32_t>& level_off() const { return level_off_; }   // [L+1]
  const std::vector<int32_t>& t2j() const { return t2j_; }               // [N] tensor id -> job id
  const std::vector<int32_t>& j2t() const { return j2t_; }               // [N] job id -> tensor id or -1
  // Tensor-id-space adjacency: child_t[c*N + t] = tensor id of t's slot-c child or -1;
  // parent_t[t] = tensor id of t's parent or -1.
  const std::vector<int32_t>& child_t() const { return child_t_; }
  const std::vector<int32_t>& parent_t() const { return parent_t_; }
  const std::vector<int32_t>& sample_off() const { return sample_off_; } // [batch+1] first job id of each sample

  // Per-row index tables (see include/cavs_b200.h, cavs_sched_tables).
  void Tables(TableMode mode, int32_t* fg, int32_t* fs, int32_t* bg, int32_t* bs) const;

  // The reference's compact per-round lists.
  void RefGather(int level, int slot, std::vector<int32_t>* out) const;
  void RefScatter(int level, std::vector<int32_t>* out) const;
  void RefRoots(std::vector<int32_t>* out) const;
  // Full schedule stream in the oracle's documented layout (two child slots).
  void RefStream(std::vector<int32_t>* out) const;

  // Job-id-space adjacency (independent of the round order): parent_j[g] or -1, child_j[c*N + g] or -1.
  const std::vector<int32_t>& parent_j() const { return parent_j_; }
  const std::vector<int32_t>& child_j() const { return child_j_; }
  // The reference's SerialGraphScheduler (cavs/midend/graph_scheduler.cc:83-167): job ids in the order
  // its forward (backward = false) or backward sweep runs them, one per round, with the lists each
  // round reports.  Tensor id == job id in that mode.  Independent of SetOrder().
  struct SerialRound { int32_t job; int32_t n_wake; int32_t child[2]; int32_t n_wait; int32_t init; };
  void SerialSweep(bool backward, std::vector<SerialRound>* rounds) const;
  // Both sweeps serialised in the oracle's "serial schedule stream" layout.
  void RefSerialStream(std::vector<int32_t>* out) const;

 private:
  int batch_ = 0, max_len_ = 0, n_slots_ = 2;
  int n_total_ = 0, n_sched_ = 0, max_level_rows_ = 0, n_roots_ = 0;
  RoundOrder order_ = kBatched;
  std::vector<int32_t> sample_off_, level_off_, t2j_, j2t_, child_t_, parent_t_, parent_j_, child_j_;
  // scratch kept between Load() calls so steady-state loads do not allocate
  std::vector<int32_t> local_, sample_len_, sample_levels_, level_cnt_;
};

}  // namespace cavs_b200
#endif
