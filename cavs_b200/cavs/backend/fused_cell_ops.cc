// The fused Tree-LSTM cell as an operator pair, `TreeLSTMCell` and `TreeLSTMCell_grad`, registered through the
// same OpImpl / OpDecl registries as every other operator (cavs/backend/op_impl.h:32-74, op_decl.h:29-43).
// A Node() body keeps its Gather / Embedding / MatMul ops and replaces the elementwise tail of
// apps/paper/tree-lstm-cavs.cc:150-171 by
//   TreeLSTMCell(xW, sU, hU_f[0..K), child[0..K), B) -> (h|c, gates)          attr "Slots" = K
// whose gradient is
//   TreeLSTMCell_grad(d(h|c), gates, h|c, child[0..K)) -> (d xW, d hU_f[0..K), d child_c[0..K))
// (d sU is the first 3H columns of d xW).  With K = 1 this is the chain LSTM cell of apps/paper/seq-lstm-cavs.cc:62-86
// up to its gate order.  Each Compute is one call into the C ABI.
#include <cuda_runtime.h>

#include <vector>

#include "cavs/backend/op_decl.h"
#include "cavs/backend/op_impl.h"
#include "cavs/util/op_def_builder.h"
#include "cavs/util/op_util.h"
#include "cavs/util/stream_event_handle_pool.h"
#include "cavs_b200.h"

namespace backend {

using ::midend::Tensor;

namespace {
void Must(int status, const char* what) { CHECK(status == CAVS_OK) << what << ": " << cavs_last_error(); }
cudaStream_t StreamOf(OpContext* context) { return StreamEventHandlePool::GetCudaStream(context->GetStreamID()); }
int Slots(const OpDef& def) {
  const int k = GetSingleArg<int>(def, "Slots");
  CHECK(k >= 1 && k <= 4) << def.DebugString();
  return k;
}
}  // namespace

// Inputs: 0 xW [n,4H], 1 sU [n,3H], 2..2+K hU_f[c] [n,H], 2+K..2+2K child[c] [n,2H], 2+2K B [4H].
// Outputs: 0 h|c [n,2H], 1 gates [n,(3+K)H].
template <typename T>
class TreeLSTMCellOp : public OpImpl {
 public:
  explicit TreeLSTMCellOp(const OpDef& def) : OpImpl(def), k_(Slots(def)) {
    CHECK(def.input_size() == 3 + 2 * k_) << def.DebugString();
    CHECK(def.output_size() == 2) << def.DebugString();
  }
  void Compute(OpContext* context) override {
    const Tensor& a = context->Input(0);
    Tensor* hc = context->Output(0);
    Tensor* gates = context->Output(1);
    const int rows = a.dims(0);
    const int hidden = a.count() / rows / 4;
    CHECK(hc->count() == rows * 2 * hidden) << hc->debug_info();
    CHECK(gates->count() == rows * (3 + k_) * hidden) << gates->debug_info();
    std::vector<const T*> q(k_), child(k_);
    for (int c = 0; c < k_; ++c) {
      q[c] = context->Input(2 + c).data<T>();
      child[c] = context->Input(2 + k_ + c).data<T>();
    }
    Must(cavs_treelstm_cell_dense_fwd(hc->mutable_data<T>(), gates->mutable_data<T>(), a.data<T>(), context->Input(1).data<T>(),
                                      q.data(), child.data(), context->Input(2 + 2 * k_).data<T>(), rows, hidden, k_,
                                      StreamOf(context)),
         "TreeLSTMCell");
  }
 private:
  int k_;
};

// Inputs: 0 d(h|c) [n,2H] (the pushed h's gradient already accumulated into its h half by the Mirror /
// Accumulate fan-in, op_decl_slice_join.cc:173-182), 1 gates, 2 h|c, 3..3+K child[c] [n,2H].
// Outputs: 0 d xW [n,4H], 1..1+K d hU_f[c] [n,H], 1+K..1+2K d child_c[c] [n,H].
template <typename T>
class TreeLSTMCellGradOp : public OpImpl {
 public:
  explicit TreeLSTMCellGradOp(const OpDef& def) : OpImpl(def), k_(Slots(def)) {
    CHECK(def.input_size() == 3 + k_) << def.DebugString();
    CHECK(def.output_size() == 1 + 2 * k_) << def.DebugString();
  }
  void Compute(OpContext* context) override {
    const Tensor& d_hc = context->Input(0);
    const int rows = d_hc.dims(0);
    const int hidden = d_hc.count() / rows / 2;
    std::vector<T*> zf(k_), dcc(k_);
    std::vector<const T*> child(k_);
    for (int c = 0; c < k_; ++c) {
      zf[c] = context->Output(1 + c)->mutable_data<T>();
      dcc[c] = context->Output(1 + k_ + c)->mutable_data<T>();
      child[c] = context->Input(3 + c).data<T>();
    }
    Must(cavs_treelstm_cell_dense_bwd(context->Output(0)->mutable_data<T>(), zf.data(), dcc.data(), d_hc.data<T>(), nullptr,
                                      context->Input(1).data<T>(), context->Input(2).data<T>(), child.data(), rows, hidden, k_,
                                      StreamOf(context)),
         "TreeLSTMCell_grad");
  }
 private:
  int k_;
};

REGISTER_OP_IMPL_BUILDER(Key("TreeLSTMCell").Device("GPU"), TreeLSTMCellOp<float>);
REGISTER_OP_IMPL_BUILDER(Key(GetGradientName("TreeLSTMCell")).Device("GPU"), TreeLSTMCellGradOp<float>);

namespace {

class TreeLSTMCellOpDecl : public OpDecl {
 public:
  explicit TreeLSTMCellOpDecl(const OpDef& def) : OpDecl(def), k_(Slots(def)) {
    CHECK(def.input_size() == 3 + 2 * k_) << def.DebugString();
    CHECK(def.output_size() == 2) << def.DebugString();
  }
  // Outputs: h|c has the shape of a child tensor; gates is [n, (3+K)H].
  void ShapeInference(std::vector<TensorShapeDef>* out, const std::vector<TensorShapeDef>& inputs) override {
    CHECK(out->empty());
    CHECK(static_cast<int>(inputs.size()) == 3 + 2 * k_);
    const TensorShapeDef& xw = inputs[0];
    CHECK(xw.dim_size() == 2 && xw.dim(1) % 4 == 0) << op_def_.DebugString();
    const int n = static_cast<int>(xw.dim(0)), hidden = static_cast<int>(xw.dim(1)) / 4;
    TensorShapeDef hc, gates;
    hc.add_dim(n); hc.add_dim(2 * hidden);
    gates.add_dim(n); gates.add_dim((3 + k_) * hidden);
    out->push_back(hc);
    out->push_back(gates);
  }
  void MakeGradient(std::vector<OpDef>* grad) override {
    std::vector<std::string> in = {GetGradientName(op_def_.output(0)), op_def_.output(1), op_def_.output(0)};
    for (int c = 0; c < k_; ++c) in.push_back(op_def_.input(2 + k_ + c));
    std::vector<std::string> out = {GetGradientName(op_def_.input(0))};
    for (int c = 0; c < k_; ++c) out.push_back(GetGradientName(op_def_.input(2 + c)));
    for (int c = 0; c < k_; ++c) out.push_back(GetGradientName(op_def_.input(2 + k_ + c)) + "_c");
    OpDef g;
    OpDefBuilder(GetGradientName("TreeLSTMCell")).Input(in).Output(out).Device(op_def_).Attr(op_def_).Finalize(&g);
    grad->push_back(g);
  }
 private:
  int k_;
};

class TreeLSTMCellGradOpDecl : public OpDecl {
 public:
  explicit TreeLSTMCellGradOpDecl(const OpDef& def) : OpDecl(def), k_(Slots(def)) {}
  void ShapeInference(std::vector<TensorShapeDef>* out, const std::vector<TensorShapeDef>& inputs) override {
    CHECK(out->empty());
    CHECK(static_cast<int>(inputs.size()) == 3 + k_);
    CHECK(inputs[0].dim_size() == 2 && inputs[0].dim(1) % 2 == 0) << op_def_.DebugString();
    const int n = static_cast<int>(inputs[0].dim(0)), hidden = static_cast<int>(inputs[0].dim(1)) / 2;
    TensorShapeDef d_xw, row;
    d_xw.add_dim(n); d_xw.add_dim(4 * hidden);
    row.add_dim(n); row.add_dim(hidden);
    out->push_back(d_xw);
    for (int c = 0; c < 2 * k_; ++c) out->push_back(row);
  }
 private:
  int k_;
};

}  // namespace

REGISTER_OP_DECL_BUILDER("TreeLSTMCell", TreeLSTMCellOpDecl);
REGISTER_OP_DECL_BUILDER(GetGradientName("TreeLSTMCell"), TreeLSTMCellGradOpDecl);

}  // namespace backend
