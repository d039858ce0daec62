// Per-operator execution context, same accessors as cavs/midend/op_context.h:14-62.
#ifndef CAVS_MIDEND_OP_CONTEXT_H_
#define CAVS_MIDEND_OP_CONTEXT_H_

#include <string>
#include <vector>

#include "cavs/midend/graph_scheduler.h"
#include "cavs/midend/tensor.h"
#include "cavs/proto/op_def.pb.h"

namespace midend {

class OpContext {
 public:
  OpContext() : stream_id_(-1), round_(0), gs_(nullptr) {}
  const Tensor& Input(int idx) const { CHECK(idx < InputSize()) << idx << "\t" << InputSize(); return *inputs_.at(idx); }
  Tensor* Output(int idx) { CHECK(idx < OutputSize()); return outputs_.at(idx); }
  int InputSize() const { return static_cast<int>(inputs_.size()); }
  int OutputSize() const { return static_cast<int>(outputs_.size()); }
  void AppendInput(const Tensor* t) { inputs_.push_back(t); }
  void AppendOutput(Tensor* t) { outputs_.push_back(t); }
  void SetStreamId(int id) { stream_id_ = id; }
  int GetStreamID() const { return stream_id_; }   // -1: the default stream
  void SetRound(int r) { round_ = r; }
  int round() const { return round_; }
  void SetGraphScheduler(GraphSchedulerBase* gs) { CHECK(gs_ == nullptr && gs); gs_ = gs; }
  GraphSchedulerBase* graph_scheduler() { return gs_; }
  static void SetDynDim(int dyn_dim) { dyn_dim_ = dyn_dim; }

  // Move every dynamic tensor's data pointer to the current round's first row
  // (cavs/midend/op_context.cc:13-40) / back to row 0.
  void SetTensorOffset();
  void ResetTensorOffset();
  // Set dims(0) of every dynamic output / input to the last SetDynDim value.
  void ScaleOutputTensor();
  void ScaleInputTensor();
  void SetZero();
  std::string debug_info() const;

 private:
  static int dyn_dim() { return dyn_dim_; }
  std::vector<const Tensor*> inputs_;
  std::vector<Tensor*> outputs_;
  int stream_id_;
  int round_;
  GraphSchedulerBase* gs_;
  static int dyn_dim_;
};

}  // namespace midend
#endif
