#include "cavs/frontend/cxx/sym.h"

#include <iostream>

#include "cavs/util/op_def_builder.h"
#include "cavs/util/op_util.h"

namespace frontend {
Program* Program::Get() { static Program* p = new Program(); return p; }
void Program::Reset() { *Get() = Program(); }
const OpDef* Program::Producer(const string& tensor) const {
  for (const auto& op : ops)
    for (const auto& o : op.output()) if (o == tensor) return &op;
  for (const auto& f : functions)
    for (const auto& op : f.ops())
      for (const auto& o : op.output()) if (o == tensor) return &op;
  return nullptr;
}
const TensorShapeDef* Program::ShapeOf(const string& tensor) const {
  const OpDef* op = Producer(tensor);
  if (!op) return nullptr;
  for (int i = 0; i < op->output_size(); i++)
    if (op->output(i) == tensor) return &op->shape(i < op->shape_size() ? i : 0);
  return nullptr;
}
}  // namespace frontend

Sym::Sym(const OpDef& op_def) {
  node_.reset(new node_t());
  node_->op_def = op_def;
  static int next_id = 0;
  if (def().output_size() == 0) mutable_def()->add_output(op_name() + "_" + std::to_string(next_id++));
  if (FuncConf::CheckInFunc()) {
    CHECK(op_name() != "Optimizer");
    *FuncConf::mutable_funcdef()->add_ops() = def();
  } else {
    frontend::Program::Get()->ops.push_back(def());
  }
}

std::vector<int> Sym::shape(int idx) const {
  CHECK(idx < def().shape_size()) << idx << "\n" << def().DebugString();
  std::vector<int> s;
  for (auto d : def().shape(idx).dim()) s.push_back(static_cast<int>(d));
  return s;
}

namespace {
int Count(const std::vector<int>& s) { int n = 1; for (int d : s) n *= d; return n; }
OpDefBuilder& Base(OpDefBuilder& b, const Sym& like, const string& device) {
  return b.Dtype(like.type()).Device(device);
}
Sym Unary(const char* name, const Sym& a, const string& device) {
  OpDefBuilder b(name);
  b.Input(a.output(0)).Shape(a.shape(0));
  return Sym(Base(b, a, device).Finalize());
}
Sym Binary(const char* name, const Sym& a, const Sym& b2, const string& device) {
  // elementwise; the smaller operand broadcasts (cavs/backend/op_impl_elementwise.cuh:135)
  OpDefBuilder b(name);
  b.Input(a.output(0)).Input(b2.output(0)).Shape(Count(a.shape(0)) >= Count(b2.shape(0)) ? a.shape(0) : b2.shape(0));
  return Sym(Base(b, a, device).Finalize());
}
std::vector<Sym> SplitN(const Sym& a, int parts) {
  const int total = Count(a.shape(0));
  CHECK(total % parts == 0) << a.def().DebugString();
  const int stride = total / parts;
  std::vector<Sym> out;
  for (int i = 0; i < parts; i++) out.push_back(Sym::Slice(a, i * stride, stride));
  return out;
}
}  // namespace

Sym Sym::Variable(DataType type, const std::vector<int>& shape, const ATTRIBUTE& filler, string device) {
  CHECK(shape.size() > 0);
  OpDefBuilder b("Variable");
  b.Dtype(type).Label(filler.first).Device(device).Shape(shape).Attr(filler.second);
  return Sym(b.Finalize());
}
Sym Sym::Placeholder(DataType type, const std::vector<int>& shape, string device) {
  CHECK(shape.size() > 0);
  OpDefBuilder b("Placeholder");
  b.Dtype(type).Device(device).Shape(shape);
  return Sym(b.Finalize());
}
Sym Sym::Reduce_mean(const Sym& a, string device) {
  OpDefBuilder b("Reduce_mean");
  b.Input(a.output(0)).Shape(std::vector<int>{1});
  return Sym(Base(b, a, device).Finalize());
}
Sym Sym::Reduce_sum(const Sym& a, string device) {
  OpDefBuilder b("Reduce_sum");
  b.Input(a.output(0)).Shape(std::vector<int>{1});
  return Sym(Base(b, a, device).Finalize());
}
Sym Sym::Optimizer(const Sym& a, std::vector<Sym> variables, float lr, float clip, int iters, const string& projections) {
  CHECK(variables.empty() || iters > 0);
  OpDefBuilder b("Optimizer");
  b.Input(a.output(0)).Shape(std::vector<int>{1});
  std::vector<string> names;
  for (const auto& v : variables) names.push_back(v.output(0));
  b.AttrSingle("Solver", "SGD").AttrSingle("lr", lr).AttrSingle("clip", clip).AttrSingle("Iters", iters);
  if (!projections.empty()) b.AttrSingle("Projection", projections);
  for (const auto& n : names) b.AttrSingle("Vars", n);
  return Sym(Base(b, a, "GPU").Finalize());
}
Sym Sym::Sigmoid(const Sym& a, string device) { return Unary("Sigmoid", a, device); }
Sym Sym::Tanh(const Sym& a, string device) { return Unary("Tanh", a, device); }
Sym Sym::Relu(const Sym& a, string device) { return Unary("Relu", a, device); }
Sym Sym::Mirror(const Sym& a) { return Unary("Mirror", a, a.device() == GPU ? "GPU" : "CPU"); }
Sym Sym::Slice(const Sym& a, int offset, int stride) {
  CHECK(offset >= 0 && stride > 0 && offset + stride <= Count(a.shape(0))) << a.def().DebugString();
  OpDefBuilder b("Slice");
  b.Input(a.output(0)).Shape(std::vector<int>{stride}).AttrSingle("Offset", offset).AttrSingle("Stride", stride);
  return Sym(Base(b, a, "GPU").Finalize());
}
std::tuple<Sym, Sym> Sym::Split2(const Sym& a) { auto v = SplitN(a, 2); return std::make_tuple(v[0], v[1]); }
std::tuple<Sym, Sym, Sym> Sym::Split3(const Sym& a) { auto v = SplitN(a, 3); return std::make_tuple(v[0], v[1], v[2]); }
std::tuple<Sym, Sym, Sym, Sym> Sym::Split4(const Sym& a) { auto v = SplitN(a, 4); return std::make_tuple(v[0], v[1], v[2], v[3]); }
Sym Sym::Add(const Sym& a, const Sym& b, string device) { return Binary("Add", a, b, device); }
Sym Sym::Sub(const Sym& a, const Sym& b, string device) { return Binary("Sub", a, b, device); }
Sym Sym::Mul(const Sym& a, const Sym& b, string device) { return Binary("Mul", a, b, device); }
Sym Sym::MatMul(const Sym& a, const Sym& b2, string device) {
  // [.., k] x [k, n]; a per-vertex vector counts as one row (cavs/backend/op_decl_matmul.cc)
  const std::vector<int> sa = a.shape(0), sb = b2.shape(0);
  CHECK(sb.size() == 2) << b2.def().DebugString();
  CHECK(sa.back() == sb[0]) << a.def().DebugString() << b2.def().DebugString();
  OpDefBuilder b("MatMul");
  b.Input(a.output(0)).Input(b2.output(0)).Shape(std::vector<int>{sa.size() == 2 ? sa[0] : 1, sb[1]});
  return Sym(Base(b, a, device).Finalize());
}
Sym Sym::SoftmaxEntropyLoss(const Sym& a, const Sym& b2, string device) {
  OpDefBuilder b("SoftmaxEntropyLoss");
  b.Input(a.output(0)).Input(b2.output(0)).Shape(std::vector<int>{a.shape(0)[0], 1});
  return Sym(Base(b, a, device).Finalize());
}
Sym Sym::EmbeddingLookup(const Sym& a, const Sym& table, string device) {
  const std::vector<int> st = table.shape(0);
  CHECK(st.size() == 2) << table.def().DebugString();
  OpDefBuilder b("EmbeddingLookup");
  b.Input(a.output(0)).Input(table.output(0)).Shape(std::vector<int>{Count(a.shape(0)), st[1]});
  return Sym(Base(b, table, device).Finalize());
}
Sym Sym::ControlDependency(const Sym& a, const Sym& b2) {
  OpDefBuilder b("ControlDependency");
  b.Input(a.output(0)).Input(b2.output(0)).Output(a.output(0)).Shape(a.shape(0));
  return Sym(Base(b, a, "GPU").Finalize());
}
Sym Sym::Reshape(const Sym& a, const std::vector<int>& shape) {
  OpDefBuilder b("Reshape");
  b.Input(a.output(0)).Shape(shape);
  return Sym(Base(b, a, "GPU").Finalize());
}
Sym Sym::Expand_dims(const Sym& a, int axis) {
  std::vector<int> s = a.shape(0);
  CHECK(axis >= 0 && axis <= static_cast<int>(s.size()));
  s.insert(s.begin() + axis, 1);
  OpDefBuilder b("Expand_dims");
  b.Input(a.output(0)).Shape(s).AttrSingle("Axis", axis);
  return Sym(Base(b, a, "GPU").Finalize());
}
Sym Sym::FullyConnected(const Sym& x, const Sym& w, const Sym& bias, string device) {
  const std::vector<int> sw = w.shape(0);   // [Out, K] (cavs/backend/op_impl_fullyconnected_cublas.cc:44-52)
  CHECK(sw.size() == 2) << w.def().DebugString();
  OpDefBuilder b("FullyConnected");
  b.Input(x.output(0)).Input(w.output(0)).Input(bias.output(0)).Shape(std::vector<int>{x.shape(0)[0], sw[0]});
  return Sym(Base(b, x, device).Finalize());
}
Sym Sym::Concat(const std::vector<Sym>& syms, string device) {
  CHECK(!syms.empty());
  int total = 0;
  OpDefBuilder b("Concat");
  for (const auto& s : syms) { b.Input(s.output(0)); total += Count(s.shape(0)); }
  b.Shape(std::vector<int>{total});
  return Sym(Base(b, syms[0], device).Finalize());
}

namespace {
Sym::ATTRIBUTE Filler(const char* label, std::vector<OpDef::AttrDef> attrs = {}) { return {label, attrs}; }
OpDef::AttrDef FloatAttr(const char* name, float v) {
  OpDef::AttrDef a;
  a.set_name(name);
  a.mutable_value()->set_f(v);
  return a;
}
}  // namespace
Sym::ATTRIBUTE Sym::Ones() { return Filler("ConstantFiller", {FloatAttr("const_value", 1.f)}); }
Sym::ATTRIBUTE Sym::Zeros() { return Filler("ConstantFiller", {FloatAttr("const_value", 0.f)}); }
Sym::ATTRIBUTE Sym::Const(float c) { return Filler("ConstantFiller", {FloatAttr("const_value", c)}); }
Sym::ATTRIBUTE Sym::Uniform(float minval, float maxval) {
  return Filler("Uniform", {FloatAttr("minval", minval), FloatAttr("maxval", maxval)});
}

void Sym::print() {
  const std::vector<char>* raw = mutable_raw();
  const float* v = reinterpret_cast<const float*>(raw->data());
  for (size_t i = 0; i < raw->size() / sizeof(float); i++) std::cout << v[i] << "\t";
  std::cout << std::endl;
}
