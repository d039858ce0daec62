// CUDA source for fused groups of elementwise operators of a vertex function, forward and backward.
//
// Stands where the reference's runtime compiler does (cavs/midend/runtime_compiler/parser.cc groups consecutive
// elementwise statements, code_generator.cc:20-185 prints one kernel per group, statement_builder.cc:19-21 holds the
// per-operator expressions).  Differences: a group is described by a small value type instead of graph nodes; every
// kernel is a grid-stride loop over (row, column) of a level's rows in tensor-id-ordered arenas; and the backward
// kernel of a group is generated too (the reference differentiates first and fuses the gradient operators like any
// others) -- it re-reads the group's saved outputs, walks the group in reverse inside one thread and adds into the
// gradients of the group's inputs.
#ifndef CAVS_MIDEND_RUNTIME_COMPILER_CODE_GENERATOR_H_
#define CAVS_MIDEND_RUNTIME_COMPILER_CODE_GENERATOR_H_

#include <string>
#include <vector>

namespace midend {
namespace RTC {

struct EwiseOperand {
  enum Kind { kNode, kInput, kVar } kind;
  int index;   // kNode: operator of the group; kInput: per-vertex input of the group; kVar: variable operand
};
struct EwiseOp {
  std::string name;                 // Add, Sub, Mul, Sigmoid, Tanh, Relu
  std::vector<EwiseOperand> in;     // the operator's output is node number (its position in the group)
};
struct EwiseGroup {
  int width = 0;                    // columns of every per-vertex tensor in the group
  int n_inputs = 0;                 // distinct per-vertex inputs
  std::vector<int> var_counts;      // per variable operand: `width` (one value per column) or 1 (a scalar)
  std::vector<EwiseOp> ops;
};

bool IsElementwise(const std::string& op_name);
// Kernel arguments, in order: int rows, long long off,
//   per input:    const float* in (first column of the view), long long pitch
//   per variable: const float* var
//   per operator: float* out (arena [*, width])
std::string GenForward(const EwiseGroup& g, const std::string& kernel_name);
// Kernel arguments, in order: int rows, long long off,
//   per input:    const float* in, long long pitch, float* grad_in (same view of the gradient arena; added to)
//   per variable: const float* var, float* var_rows (arena [*, width]: this row's contribution to the variable's gradient)
//   per operator: const float* out, const float* grad_out
std::string GenBackward(const EwiseGroup& g, const std::string& kernel_name);
// One operator (IsElementwise) as a kernel of its own.  Kernel arguments, in order: float* out, long long n,
//   const float* in0, long long n0, const float* in1, long long n1 (in1 / n1 ignored by unary operators); an operand
//   with fewer elements than the output is read at i % its size.
std::string GenStandalone(const std::string& op_name, const std::string& kernel_name);

}  // namespace RTC
}  // namespace midend
#endif
