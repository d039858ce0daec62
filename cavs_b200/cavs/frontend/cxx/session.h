// Session::Run with the reference's signature (cavs/frontend/cxx/session.h:13-30).  Where the reference
// compiles the recorded program into a statement list and interprets the vertex function op by op per
// level, this Session first tries to recognise the program --
//     GraphOutput(Node) -> FullyConnected -> SoftmaxEntropyLoss [-> Optimizer | Reduce_mean]
// with Node() the child-sum Tree-LSTM (apps/paper/tree-lstm-cavs.cc:129-172) or the chain LSTM
// (apps/paper/seq-lstm-cavs.cc:62-86) -- and binds it to the fused engine behind the C ABI
// (cavs_treelstm_*).  Any other vertex function (Tree-FC, apps/paper/tree-fc-cavs.cc:29-36, or a user's own) runs
// operator by operator per level with run-time-compiled fused elementwise groups (generic_session.h,
// cavs/midend/generic_function.h), on the GPU as well: there is no CPU fallback.
//
// Optimisation bits (cavs/proto/opt.proto:3-8): OPT_BATCHING is honoured as in the reference
// (cavs/midend/graph_session.h:20-24) -- with it every level of the batch is one round, without it the
// vertices run one per round in the serial scheduler's order, with identical results.  OPT_FUSION and
// OPT_STREAMMING are accepted and change nothing: the cell is always one fused kernel per level and
// direction, and the launches of a step are already chained on one stream.
#ifndef CAVS_FRONTEND_CXX_SESSION_H_
#define CAVS_FRONTEND_CXX_SESSION_H_

#include <initializer_list>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "cavs/frontend/cxx/sym.h"
#include "cavs/proto/opt.pb.h"

class Session {
 public:
  Session(int opt = 0, std::string name = "SimpleSession");
  ~Session();
  // feeds: {placeholder, host pointer} sized by the placeholder's shape.  The graph placeholder takes
  // int parent indices [batch, max_len]; the vertex and label placeholders take floats read in compact
  // job order, as Pull / the loss do in the reference (cavs/backend/op_impl_graphop.cu:214-254).
  void Run(std::vector<Sym> outputs, const std::initializer_list<std::pair<Sym&, void*>>& feed = {});
  void Run(Sym& output, const std::initializer_list<std::pair<Sym&, void*>>& feed = {}) {
    std::vector<Sym> out = {output};
    Run(out, feed);
  }
  // Not in the reference: direct access to a Variable's values in its declared layout, for parity runs
  // (the reference fills every Uniform variable from the same default-seeded engine, functor_filler.h:93-97).
  void SetVariable(const Sym& var, const float* host, size_t count);
  void GetVariable(const Sym& var, float* host, size_t count);
  // d(loss)/d(var) of the last Run, in the declared layout (after clipping, if the program clips).
  void GetGradient(const Sym& var, float* host, size_t count);

 private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
};

// Extra optimisation bit understood by this Session only: run the gate GEMMs on the tensor cores with
// bf16 operands (the default, like the reference, is fp32 throughout).
enum { OPT_BF16_GEMM = 8 };
// Extra bit: pair gathered / scattered rows with level rows the way the reference's graph ops do -- positionally, which
// shifts rows on batches whose levels mix vertices with and without a given child slot or parent
// (cavs/backend/op_impl_graphop.cu:57-76,140-157).  The default pairs every row with its own children.  Honoured by the
// operator-by-operator executor (the Session then uses it for every vertex function); the fused engines pair rows correctly.
enum { OPT_REF_COMPAT_ROWS = 16 };
#endif
