// The scheduler surface the graph ops read, with the reference's names
// (cavs/midend/graph_scheduler.h:12-77,142-158), backed by a level schedule that is built
// for the whole batch in LoadGraph: Initialize / ActivateNext only move a cursor, and every
// per-round index list also lives in device memory (uploaded once per batch), so no graph op
// has to copy its indices before launching (cf. cavs/backend/op_impl_graphop.cu:68,80,149,241,308).
//
// The per-round host vectors returned by CurrentRoundTensorIdsFor* are element-for-element the
// reference's (compact lists; see host/schedule.h).  In "aligned" mode (the default is the
// reference-compatible one) the device lists are padded with -1 so that entry b always belongs
// to row b of the level.
#ifndef CAVS_MIDEND_GRAPH_SCHEDULER_H_
#define CAVS_MIDEND_GRAPH_SCHEDULER_H_

#include <memory>
#include <vector>

#include "cavs/midend/tensor.h"
#include "cavs/util/logging.h"

namespace midend {

class GraphSchedulerBase {
 public:
  GraphSchedulerBase();
  virtual ~GraphSchedulerBase();
  virtual void Initialize() = 0;
  virtual bool Terminate() const = 0;
  virtual void ActivateNext() = 0;
  virtual int GetCurrentRoundOffset() const = 0;

  // graph_struct: host int tensor [batch, max_len] of parent indices (-1 = root / padding).
  int LoadGraph(const Tensor& graph_struct);
  int ReverseGraph();
  int batch_size() const { return batch_size_; }
  int total_length() const { return total_length_; }
  bool HasChild(int job_id) const;
  const std::vector<int>& GetJobId() const { CHECK(!Terminate()); return ready_to_execute_ids_; }
  const std::vector<int>& CurrentRoundTensorIdsForGatherInitialization() const;
  const std::vector<int>& CurrentRoundTensorIdsForGather(int child_offset) const;
  const std::vector<int>& CurrentRoundTensorIdsForScatter(int child_offset) const;
  const std::vector<int>& TensorIdsToJobIds() const { return tids_to_jobids_; }

  // Device-resident copies of the lists of the current round (valid until the next LoadGraph).
  // *count receives the list length.  In aligned mode the gather / scatter lists have one entry
  // per row of the level, -1 where the reference's compact list has no entry.
  const int* DeviceJobIds(int* count) const;
  const int* DeviceIdsForGather(int child_offset, int* count) const;
  const int* DeviceIdsForScatter(int child_offset, int* count) const;
  const int* DeviceTensorIdsToJobIds(int* count) const;
  // false (default): the reference's positional pairing of compact lists with level rows;
  // true: lists padded so rows always pair with their own children / parent.
  void SetAlignedTables(bool aligned) { aligned_ = aligned; }
  bool aligned_tables() const { return aligned_; }
  // Unused by the new graph ops; kept so code that asks for the staging buffer still links.
  int* gpu_idx_buf() const { return nullptr; }

  void SetMessagePasser(const Tensor& t) { message_passer_ = t; }
  const Tensor& GetMessagePasser(int id) { message_passer_.SetOffsetWithId(id); return message_passer_; }
  void SetFuncArg(const Tensor t) { func_arg_ = t; }
  const Tensor& GetFuncArg() { return func_arg_; }
  void SetFuncRet(const Tensor t) { func_ret_ = t; }
  const Tensor& GetFuncRet() { func_ret_.SetOffsetWithId(0); return func_ret_; }

 protected:
  struct Impl;
  std::unique_ptr<Impl> impl_;
  // true: one vertex per round with tensor id == job id (SerialGraphScheduler); LoadGraph then also
  // prepares the serial sweeps.
  virtual bool OneVertexPerRound() const { return false; }
  void SetRound(int level, bool forward);   // fills the per-round host vectors for `level`
  void SetSerialRound(int round, bool forward);
  std::vector<int> ready_to_execute_ids_;
  std::vector<std::vector<int>> tids_for_gather_init_, tids_for_gather_, tids_for_scatter_;
  std::vector<int> tids_to_jobids_;
  Tensor message_passer_, func_arg_, func_ret_;
  int round_ = -1;
  bool forward_ = true;
  bool aligned_ = false;
  int batch_size_ = 0, total_length_ = 0;
};

class BatchGraphScheduler : public GraphSchedulerBase {
 public:
  void Initialize() override;
  void ActivateNext() override;
  bool Terminate() const override { return ready_to_execute_ids_.empty(); }
  int GetCurrentRoundOffset() const override;
};

// One vertex per round, sample after sample, tensor id == job id: the reference's scheduler for a
// Session without OPT_BATCHING (cavs/midend/graph_scheduler.h:122-138, graph_scheduler.cc:83-167).
// Round order and every per-round list are the reference's, including its work-list details (the
// backward sweep interleaves samples; a single-vertex sample ends the forward sweep).
class SerialGraphScheduler : public GraphSchedulerBase {
 public:
  void Initialize() override;
  void ActivateNext() override;
  bool Terminate() const override { return ready_to_execute_ids_.empty(); }
  int GetCurrentRoundOffset() const override { return GetJobId()[0]; }

 protected:
  bool OneVertexPerRound() const override { return true; }
};

}  // namespace midend
#endif
