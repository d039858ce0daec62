// Symbolic front end: the subset of the reference's Sym class (cavs/frontend/cxx/sym.h:16-193) that
// vertex functions and their training programs are written in.  Constructing a Sym records an
// OpDef -- into the function being defined when FuncConf::CheckInFunc() (GraphSupport::Node()),
// else into the main program -- exactly like the reference (cavs/frontend/cxx/sym.cc:15-55); there
// is no protobuf serialisation behind it: Session binds the recorded program either to a fused engine or
// to the operator-by-operator executor (see session.h).
#ifndef CAVS_FRONTEND_CXX_SYM_H_
#define CAVS_FRONTEND_CXX_SYM_H_

#include <memory>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

#include "cavs/proto/op_def.pb.h"
#include "cavs/util/logging.h"

using std::string;

class Sym {
 public:
  explicit Sym(const OpDef& op_def);
  Sym(const Sym& sym) { *this = sym; }
  Sym() : node_(nullptr) {}
  Sym& operator=(const Sym& sym) { node_ = sym.node_; return *this; }

  const string& output(int idx) const { CHECK(idx < def().output_size()); return def().output(idx); }
  int output_size() const { return def().output_size(); }
  std::vector<string> output() const { return def().output(); }
  std::vector<int> shape(int idx) const;
  DataType type() const { return def().dtype(); }
  DeviceType device() const { return def().device(); }
  const string& op_name() const { return def().name(); }
  const OpDef& def() const { CHECK(node_.get()); return node_->op_def; }
  OpDef* mutable_def() { CHECK(node_.get()); return &(node_->op_def); }
  const void* data() const { CHECK(node_.get()); return node_->raw_data.data(); }

  typedef std::pair<string, std::vector<OpDef::AttrDef>> ATTRIBUTE;

  // sources
  static Sym Variable(DataType type, const std::vector<int>& shape, const ATTRIBUTE& filler = Ones(), string device = "GPU");
  static Sym Placeholder(DataType type, const std::vector<int>& shape, string device = "GPU");
  // unary
  static Sym Reduce_mean(const Sym& a, string device = "GPU");
  static Sym Reduce_sum(const Sym& a, string device = "GPU");
  static Sym Optimizer(const Sym& a, std::vector<Sym> variables, float lr, float clip = 0.f, int iters = 1,
                       const string& projections = "");
  static Sym Sigmoid(const Sym& a, string device = "GPU");
  static Sym Tanh(const Sym& a, string device = "GPU");
  static Sym Relu(const Sym& a, string device = "GPU");
  static Sym Slice(const Sym& a, int offset, int stride);
  static Sym Mirror(const Sym& a);
  static std::tuple<Sym, Sym> Split2(const Sym& a);
  static std::tuple<Sym, Sym, Sym> Split3(const Sym& a);
  static std::tuple<Sym, Sym, Sym, Sym> Split4(const Sym& a);
  // binary
  static Sym Add(const Sym& a, const Sym& b, string device = "GPU");
  static Sym Sub(const Sym& a, const Sym& b, string device = "GPU");
  static Sym Mul(const Sym& a, const Sym& b, string device = "GPU");
  static Sym MatMul(const Sym& a, const Sym& b, string device = "GPU");
  static Sym SoftmaxEntropyLoss(const Sym& a, const Sym& b, string device = "GPU");
  static Sym EmbeddingLookup(const Sym& a, const Sym& b, string device = "GPU");
  static Sym ControlDependency(const Sym& a, const Sym& b);
  static Sym Reshape(const Sym& a, const std::vector<int>& shape);
  static Sym Expand_dims(const Sym& a, int axis);
  // ternary / n-ary
  static Sym FullyConnected(const Sym& x, const Sym& w, const Sym& b, string device = "GPU");
  static Sym Concat(const std::vector<Sym>& syms, string device = "GPU");
  // fillers
  static ATTRIBUTE Ones();
  static ATTRIBUTE Zeros();
  static ATTRIBUTE Const(float c);
  static ATTRIBUTE Uniform(float minval, float maxval);
  // results of the last Session::Run that fetched this symbol (host memory)
  const void* eval() const { return data(); }
  void print();

  // member forms
  Sym Reduce_mean() { return Reduce_mean(*this); }
  Sym Reduce_sum() { return Reduce_sum(*this); }
  Sym Optimizer(std::vector<Sym> variables, float lr, float clip = 0.f, int iters = 1, const string& projection = "") {
    return Optimizer(*this, variables, lr, clip, iters, projection);
  }
  Sym Sigmoid() { return Sigmoid(*this); }
  Sym Tanh() { return Tanh(*this); }
  Sym Relu() { return Relu(*this); }
  Sym Slice(int offset, int stride) { return Slice(*this, offset, stride); }
  Sym Mirror() { return Mirror(*this); }
  std::tuple<Sym, Sym> Split2() { return Split2(*this); }
  std::tuple<Sym, Sym, Sym> Split3() { return Split3(*this); }
  std::tuple<Sym, Sym, Sym, Sym> Split4() { return Split4(*this); }
  Sym SoftmaxEntropyLoss(const Sym& b) { return SoftmaxEntropyLoss(*this, b); }
  Sym EmbeddingLookup(const Sym& b) { return EmbeddingLookup(*this, b); }
  Sym ControlDependency(const Sym& b) { return ControlDependency(*this, b); }
  Sym Reshape(const std::vector<int>& shape) { return Reshape(*this, shape); }
  Sym Expand_dims(int axis) { return Expand_dims(*this, axis); }
  Sym FullyConnected(const Sym& w, const Sym& b) { return FullyConnected(*this, w, b); }

  friend Sym operator+(const Sym& a, const Sym& b) { return Add(a, b); }
  friend Sym operator-(const Sym& a, const Sym& b) { return Sub(a, b); }
  friend Sym operator*(const Sym& a, const Sym& b) { return Mul(a, b); }

  // Session writes fetched values here.
  std::vector<char>* mutable_raw() { CHECK(node_.get()); return &node_->raw_data; }

 private:
  struct node_t {
    OpDef op_def;
    std::vector<char> raw_data;
  };
  std::shared_ptr<node_t> node_;
};

// Function-definition mode switch (cavs/frontend/cxx/sym.h:195-225).
class FuncConf {
 public:
  static void FuncDefineBegin(const string& name) { Get()->name_ = name; Get()->def_ = FunctionDef(); Get()->def_.set_name(name); }
  static FunctionDef FuncDefineEnd(const string& name) {
    CHECK(name == Get()->name_);
    FunctionDef ret = Get()->def_;
    Get()->name_.clear();
    Get()->def_ = FunctionDef();
    return ret;
  }
  static bool CheckInFunc() { return !Get()->name_.empty(); }
  static FunctionDef* mutable_funcdef() { CHECK(CheckInFunc()); return &Get()->def_; }
 private:
  static FuncConf* Get() { static FuncConf fc; return &fc; }
  string name_;
  FunctionDef def_;
};

// Everything recorded outside a function definition, in creation order (what the reference sends
// through C_AddOp / C_AddFunction / C_AddOptimizerOp, cavs/frontend/c_api.h:20-36).
namespace frontend {
struct Program {
  std::vector<OpDef> ops;
  std::vector<FunctionDef> functions;
  static Program* Get();
  static void Reset();   // start a new program (tests)
  // shape of a recorded tensor by output name, main program and functions alike
  const TensorShapeDef* ShapeOf(const string& tensor) const;
  const OpDef* Producer(const string& tensor) const;
};
}  // namespace frontend
#endif
