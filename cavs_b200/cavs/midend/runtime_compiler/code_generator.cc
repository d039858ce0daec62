#include "cavs/midend/runtime_compiler/code_generator.h"

#include <sstream>

#include "cavs/util/logging.h"

namespace midend {
namespace RTC {
namespace {

const char* kLoop =
    "  const long long total = (long long)rows * W;\n"
    "  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {\n"
    "    const int c = (int)(i % W);\n"
    "    const long long t = off + i / W;\n";

std::string Val(const EwiseOperand& o) {
  switch (o.kind) {
    case EwiseOperand::kNode: return "n" + std::to_string(o.index);
    case EwiseOperand::kInput: return "x" + std::to_string(o.index);
    default: return "v" + std::to_string(o.index);
  }
}
std::string Grad(const EwiseOperand& o) {
  switch (o.kind) {
    case EwiseOperand::kNode: return "g" + std::to_string(o.index);
    case EwiseOperand::kInput: return "gx" + std::to_string(o.index);
    default: return "gv" + std::to_string(o.index);
  }
}
int Arity(const std::string& name) { return (name == "Add" || name == "Sub" || name == "Mul") ? 2 : 1; }

// The forward expressions of the reference's fused kernels (cavs/midend/runtime_compiler/expression.h:40-72).
std::string ForwardExpr(const EwiseOp& op) {
  const std::string a = Val(op.in[0]), b = op.in.size() > 1 ? Val(op.in[1]) : "";
  if (op.name == "Add") return a + " + " + b;
  if (op.name == "Sub") return a + " - " + b;
  if (op.name == "Mul") return a + " * " + b;
  if (op.name == "Sigmoid") return "1.0f / (1.0f + expf(-" + a + "))";
  if (op.name == "Tanh") return "tanhf(" + a + ")";
  if (op.name == "Relu") return a + " > 0.0f ? " + a + " : 0.0f";
  LOG(FATAL) << "no expression for operator " << op.name;
  return "";
}

void LoadInputs(const EwiseGroup& g, std::ostringstream& s) {
  for (int j = 0; j < g.n_inputs; ++j) s << "    const float x" << j << " = in" << j << "[t * p" << j << " + c];\n";
  for (size_t q = 0; q < g.var_counts.size(); ++q)
    s << "    const float v" << q << " = var" << q << "[" << (g.var_counts[q] == 1 ? "0" : "c") << "];\n";
}

}  // namespace

bool IsElementwise(const std::string& n) {
  return n == "Add" || n == "Sub" || n == "Mul" || n == "Sigmoid" || n == "Tanh" || n == "Relu";
}

std::string GenForward(const EwiseGroup& g, const std::string& name) {
  std::ostringstream s;
  s << "extern \"C\" __global__ void " << name << "(int rows, long long off";
  for (int j = 0; j < g.n_inputs; ++j) s << ", const float* __restrict__ in" << j << ", long long p" << j;
  for (size_t q = 0; q < g.var_counts.size(); ++q) s << ", const float* __restrict__ var" << q;
  for (size_t k = 0; k < g.ops.size(); ++k) s << ", float* __restrict__ out" << k;
  s << ") {\n  const int W = " << g.width << ";\n" << kLoop;
  LoadInputs(g, s);
  for (size_t k = 0; k < g.ops.size(); ++k) {
    CHECK(static_cast<int>(g.ops[k].in.size()) == Arity(g.ops[k].name)) << g.ops[k].name;
    s << "    const float n" << k << " = " << ForwardExpr(g.ops[k]) << ";\n";
  }
  for (size_t k = 0; k < g.ops.size(); ++k) s << "    out" << k << "[t * W + c] = n" << k << ";\n";
  s << "  }\n}\n";
  return s.str();
}

std::string GenBackward(const EwiseGroup& g, const std::string& name) {
  std::ostringstream s;
  s << "extern \"C\" __global__ void " << name << "(int rows, long long off";
  for (int j = 0; j < g.n_inputs; ++j)
    s << ", const float* __restrict__ in" << j << ", long long p" << j << ", float* gin" << j;   // gradients may alias one another
  for (size_t q = 0; q < g.var_counts.size(); ++q) s << ", const float* __restrict__ var" << q << ", float* __restrict__ vrow" << q;
  for (size_t k = 0; k < g.ops.size(); ++k) s << ", const float* __restrict__ out" << k << ", const float* __restrict__ gout" << k;
  s << ") {\n  const int W = " << g.width << ";\n" << kLoop;
  LoadInputs(g, s);
  // saved outputs, and what the consumers outside the group left in the operators' gradient arenas
  for (size_t k = 0; k < g.ops.size(); ++k)
    s << "    const float n" << k << " = out" << k << "[t * W + c];\n    float g" << k << " = gout" << k << "[t * W + c];\n";
  for (int j = 0; j < g.n_inputs; ++j) s << "    float gx" << j << " = 0.0f;\n";
  for (size_t q = 0; q < g.var_counts.size(); ++q) s << "    float gv" << q << " = 0.0f;\n";
  // reverse sweep: gradient rules of cavs/backend/op_decl_elementwise_arithmetic.cc:25-109 and
  // op_decl_elementwise_activation.cc:7-27 (sigmoid' = y (1 - y), tanh' = 1 - y^2, relu' = [y > 0])
  for (int k = static_cast<int>(g.ops.size()) - 1; k >= 0; --k) {
    const EwiseOp& op = g.ops[k];
    const std::string gk = "g" + std::to_string(k), nk = "n" + std::to_string(k);
    if (op.name == "Add") {
      s << "    " << Grad(op.in[0]) << " += " << gk << ";\n    " << Grad(op.in[1]) << " += " << gk << ";\n";
    } else if (op.name == "Sub") {
      s << "    " << Grad(op.in[0]) << " += " << gk << ";\n    " << Grad(op.in[1]) << " -= " << gk << ";\n";
    } else if (op.name == "Mul") {
      s << "    " << Grad(op.in[0]) << " += " << gk << " * " << Val(op.in[1]) << ";\n";
      s << "    " << Grad(op.in[1]) << " += " << gk << " * " << Val(op.in[0]) << ";\n";
    } else if (op.name == "Sigmoid") {
      s << "    " << Grad(op.in[0]) << " += " << gk << " * " << nk << " * (1.0f - " << nk << ");\n";
    } else if (op.name == "Tanh") {
      s << "    " << Grad(op.in[0]) << " += " << gk << " * (1.0f - " << nk << " * " << nk << ");\n";
    } else if (op.name == "Relu") {
      s << "    " << Grad(op.in[0]) << " += " << nk << " > 0.0f ? " << gk << " : 0.0f;\n";
    } else {
      LOG(FATAL) << "no gradient rule for operator " << op.name;
    }
  }
  for (int j = 0; j < g.n_inputs; ++j) s << "    gin" << j << "[t * p" << j << " + c] += gx" << j << ";\n";
  for (size_t q = 0; q < g.var_counts.size(); ++q) s << "    vrow" << q << "[t * W + c] = gv" << q << ";\n";
  s << "  }\n}\n";
  return s.str();
}

// One operator as its own kernel, with the operand patterns of the reference's stand-alone elementwise operators
// (cavs/backend/op_impl_elementwise.cuh:60-76 unary, :118-206 binary): equal sizes; a one-element operand read as a
// scalar; a shorter operand repeated along the longer one (i % n).
std::string GenStandalone(const std::string& op_name, const std::string& name) {
  EwiseOp op;
  op.name = op_name;
  op.in.push_back({EwiseOperand::kInput, 0});
  if (Arity(op_name) == 2) op.in.push_back({EwiseOperand::kInput, 1});
  std::ostringstream s;
  s << "extern \"C\" __global__ void " << name
    << "(float* out, long long n, const float* in0, long long n0, const float* in1, long long n1) {\n";
  s << "  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {\n";
  s << "    const float x0 = in0[n0 == n ? i : (n0 == 1 ? 0 : i % n0)];\n";
  if (op.in.size() > 1) s << "    const float x1 = in1[n1 == n ? i : (n1 == 1 ? 0 : i % n1)];\n";
  s << "    out[i] = " << ForwardExpr(op) << ";\n  }\n}\n";
  return s.str();
}

}  // namespace RTC
}  // namespace midend
