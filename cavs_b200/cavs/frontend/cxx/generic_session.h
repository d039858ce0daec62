// Session::Run for programs whose vertex function is not one of the fused LSTM forms: the recorded Node() runs
// operator by operator through midend::GenericFunction, the loss head is either
//     graph_output.Reduce_sum()                                   (apps/paper/tree-fc-cavs.cc:118-121), or
//     graph_output.FullyConnected(W, b).SoftmaxEntropyLoss(label) (apps/paper/tree-lstm-cavs.cc:196-204),
// optionally followed by Optimizer(vars, lr, clip) (SGD over every Variable; clip as cavs/backend/op_impl_clip.cu).
#ifndef CAVS_FRONTEND_CXX_GENERIC_SESSION_H_
#define CAVS_FRONTEND_CXX_GENERIC_SESSION_H_

#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "cavs/frontend/cxx/sym.h"
#include "cavs/midend/generic_function.h"
#include "cavs_b200.h"

namespace frontend {

class GenericSession {
 public:
  explicit GenericSession(int opt);
  ~GenericSession();
  void Run(std::vector<Sym>& outputs, const std::vector<std::pair<std::string, void*>>& feeds);
  void SetVariable(const std::string& var, const float* host, size_t count);
  void GetVariable(const std::string& var, float* host, size_t count);
  void GetGradient(const std::string& var, float* host, size_t count);   // of the last Run (after clipping, if any)
  const midend::GenericFunction& function() const { return *fn_; }

 private:
  int opt_ = 0;
  std::unique_ptr<midend::GenericFunction> fn_;
  cavs_sched* sched_ = nullptr;
  float *params_ = nullptr, *grads_ = nullptr, *scratch_ = nullptr, *loss_rows_ = nullptr, *loss_sum_ = nullptr;
  int32_t* d_label_ = nullptr;
  int max_vertices_ = 0, n_slots_ = 1, classes_ = 0;
  bool xent_ = false, has_optimizer_ = false;
  float lr_ = 0.f, clip_ = 0.f;
  std::string graph_ph_, vertex_ph_, label_ph_, graph_output_, loss_, optimizer_, fc_w_, fc_b_;
};

}  // namespace frontend
#endif
