// Level-batched execution of an ARBITRARY vertex function, operator by operator.
//
// The fused engines behind the C ABI cover the LSTM / GRU vertex functions.  Every other Node() body written against
// Sym / GraphSupport runs here, the way the reference runs all of them: the recorded operators of the function are
// executed once per level over the level's rows (cavs/midend/statement.cc:43-123), consecutive elementwise operators
// fused into kernels generated and compiled at run time (cavs/midend/runtime_compiler/, op_impl_fused_kernel.cu:62-64),
// MatMul on the GEMM kernels, Gather / Scatter / Pull / Push / Slice / Concat on the row-copy kernels, weight and bias
// gradients deferred to one pass over all rows (cavs/midend/batch_weight_updater.h:10-85).  Gradients follow the
// reference's operator rules (cavs/backend/op_decl_*.cc); there is no CPU fallback.
//
// Supported in Node(): Gather, Pull (one, any width), EmbeddingLookup (of the pulled value), Slice, Reshape, Mirror,
// Expand_dims, Concat, MatMul (per-vertex row x Variable), Add, Sub, Mul (per-vertex tensors of equal width, or one
// Variable operand of that width or of one element), Sigmoid, Tanh, Relu, Scatter, Push.  fp32 throughout.
#ifndef CAVS_MIDEND_GENERIC_FUNCTION_H_
#define CAVS_MIDEND_GENERIC_FUNCTION_H_

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "cavs/backend/cudaRTC_wrapper.h"
#include "cavs/frontend/cxx/sym.h"
#include "cavs/midend/runtime_compiler/code_generator.h"

namespace midend {

class GenericFunction {
 public:
  struct Variable { std::string name; size_t offset = 0, count = 0; };

  // Plans `f` (the recorded Node()) and compiles its fused groups.  No CUDA call: works without a GPU.
  GenericFunction(const frontend::Program& prog, const FunctionDef& f, int max_vertices);
  ~GenericFunction();

  // Variables of the whole program (function and loss head), laid out in one flat buffer in declaration order.
  const std::vector<Variable>& variables() const { return vars_; }
  size_t param_count() const { return param_count_; }
  const Variable* FindVariable(const std::string& name) const;
  int out_width() const { return out_width_; }        // columns of what Push receives
  int state_width() const { return state_width_; }    // columns of what Scatter / Gather move
  int pull_width() const { return pull_width_; }      // columns of the vertex input one vertex pulls (0: no Pull)
  int n_groups() const { return static_cast<int>(groups_.size()); }
  int n_steps() const { return static_cast<int>(steps_.size()); }
  const std::string& group_source(int g, bool backward) const { return backward ? groups_[g]->bwd_src : groups_[g]->fwd_src; }

  // ---- device side (needs a GPU) ----
  void Bind(float* params, float* grads);   // flat fp32 device buffers of param_count() floats
  // Tables of one batch, in tensor-id space (cavs_sched_tables; either row-alignment mode): fg [n_slots, n] forward Gather
  // source rows, fs [n] forward Scatter target rows, bg [n] backward Gather source rows, bs [n_slots, n] backward
  // Scatter target rows (-1: zero row / no target); t2j [n]; level offsets; vertex_input: host rows [n, pull_width()] in
  // job order (may be null without a Pull).
  void LoadBatch(const int32_t* fg, const int32_t* fs, const int32_t* bg, const int32_t* bs, int n_slots, const int32_t* t2j, int n,
                 const std::vector<int32_t>& level_off, const float* vertex_input);
  void Forward();
  float* output() const { return out_val_; }          // [n, out_width()] in tensor-id order (device)
  float* output_grad() const { return out_grad_; }     // the loss head writes d(loss)/d(output) here before Backward
  // Level loop in reverse, then the deferred weight / bias / embedding gradients, ADDED into the bound gradient
  // buffer (the caller zeroes it, and may have put the loss head's own gradients there already).
  void Backward();
  int n() const { return n_; }

 private:
  struct Ref { int buf = -1; size_t var_off = 0; int col = 0, width = 0; };   // buf >= 0: per-vertex arena view; -1: variable view
  struct Buf { int width = 0; float* val = nullptr; float* grad = nullptr; };
  struct Group {
    RTC::EwiseGroup desc;
    std::vector<Ref> inputs, var_refs;
    std::vector<int> out_bufs;                 // one arena per operator
    std::vector<float*> var_rows;              // per variable operand: [max_vertices, width] per-row gradient terms
    std::string fwd_src, bwd_src, fwd_name, bwd_name;
    ::RTC::CudaRTCWrapper fwd, bwd;
  };
  enum class Kind { kGather, kPull, kEmbed, kConcat, kMatMul, kGroup, kScatter, kPush };
  struct Step {
    Kind kind;
    int slot = 0, out = -1, group = -1, k = 0, n = 0, vocab = 0, pull_offset = 0;
    Ref in, weight;
    std::vector<Ref> ins;
  };

  int NewBuf(int width);
  float* ValPtr(const Ref& r, long long row) const;
  float* GradPtr(const Ref& r, long long row) const;
  void RunLevel(int off, int rows);
  void RunLevelBackward(int off, int rows);
  void Allocate();

  int max_vertices_ = 0, n_ = 0, n_slots_ = 0;
  int out_width_ = 0, state_width_ = 0, pull_width_ = 0;
  std::vector<Variable> vars_;
  size_t param_count_ = 0;
  std::map<std::string, Ref> refs_;
  std::vector<Buf> bufs_;
  std::vector<Step> steps_;
  std::vector<std::unique_ptr<Group>> groups_;
  ::RTC::CudaRTCWrapper embed_fwd_;
  bool allocated_ = false;
  float *params_ = nullptr, *grads_ = nullptr;
  float *mailbox_ = nullptr, *dmail_ = nullptr, *out_val_ = nullptr, *out_grad_ = nullptr, *vin_ = nullptr, *tmp_ = nullptr, *col_scratch_ = nullptr;
  void* arena_ = nullptr;        // one allocation behind every per-vertex array
  size_t grad_region_off_ = 0, grad_region_bytes_ = 0;
  int32_t *d_fg_ = nullptr, *d_bs_ = nullptr, *d_fs_ = nullptr, *d_bg_ = nullptr, *d_t2j_ = nullptr;
  std::vector<int32_t> level_off_, h_tok_tid_;
  int max_slots_ = 0;
  // embedding gradient tables (device) rebuilt per batch
  int32_t* d_emb_idx_ = nullptr;
  size_t emb_idx_cap_ = 0;
  int emb_chunks_ = 0, emb_segs_ = 0;
  float* emb_scratch_ = nullptr;
};

}  // namespace midend
#endif
