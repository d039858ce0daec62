// Shape inference and gradient pairing of the graph ops, same rules as
// cavs/backend/op_decl_graphop.cc:9-199: Gather(Child=c) <-> Scatter(Child=c),
// Pull <-> Push, GraphOutput -> GraphOutput_grad.
#include "cavs/backend/op_decl.h"
#include "cavs/util/op_def_builder.h"
#include "cavs/util/op_util.h"

namespace backend {
namespace {

// Source ops (no inputs): the output shape is the declared one.
class SourceOpDecl : public OpDecl {
 public:
  explicit SourceOpDecl(const OpDef& def) : OpDecl(def) {
    CHECK(def.shape_size() == 1) << def.DebugString();
    CHECK(def.input_size() == 0) << def.DebugString();
  }
  void ShapeInference(std::vector<TensorShapeDef>* out, const std::vector<TensorShapeDef>&) override {
    CHECK(out->empty());
    out->push_back(op_def_.shape(0));
  }
};
// Sink ops (one input): the output has the input's shape.
class SinkOpDecl : public OpDecl {
 public:
  explicit SinkOpDecl(const OpDef& def) : OpDecl(def) {
    CHECK(def.input_size() == 1) << def.DebugString();
    CHECK(def.output_size() == 1) << def.DebugString();
  }
  void ShapeInference(std::vector<TensorShapeDef>* out, const std::vector<TensorShapeDef>& inputs) override {
    CHECK(out->empty());
    CHECK(inputs.size() == 1);
    out->push_back(inputs[0]);
  }
};

class GatherOpDecl : public SourceOpDecl {
 public:
  using SourceOpDecl::SourceOpDecl;
  void MakeGradient(std::vector<OpDef>* grad) override {
    // d(Gather(c)) is scattered back to the slot-c children; the output name is free because
    // the mailbox receives it.
    OpDef scatter;
    OpDefBuilder("Scatter")
        .Input(GetGradientName(op_def_.output(0)))
        .Output("Scatter_Backward_" + std::to_string(GetHash(op_def_)))
        .Device(op_def_)
        .Attr(op_def_)
        .Finalize(&scatter);
    grad->push_back(scatter);
  }
};
class PullOpDecl : public SourceOpDecl {
 public:
  using SourceOpDecl::SourceOpDecl;
  void MakeGradient(std::vector<OpDef>* grad) override {
    OpDef push;
    OpDefBuilder("Push")
        .Input(GetGradientName(op_def_.output(0)))
        .Output("Push_Backward" + std::to_string(GetHash(op_def_)))
        .Device(op_def_)
        .Finalize(&push);
    grad->push_back(push);
  }
};
class ScatterOpDecl : public SinkOpDecl {
 public:
  using SinkOpDecl::SinkOpDecl;
  void MakeGradient(std::vector<OpDef>* grad) override {
    CHECK(op_def_.shape_size() == 1) << op_def_.DebugString();
    OpDef gather;
    OpDefBuilder("Gather")
        .Output(GetGradientName(op_def_.input(0)))
        .Shape(op_def_)
        .Attr(op_def_)
        .Device(op_def_)
        .Finalize(&gather);
    grad->push_back(gather);
  }
};
class PushOpDecl : public SinkOpDecl {
 public:
  using SinkOpDecl::SinkOpDecl;
  void MakeGradient(std::vector<OpDef>* grad) override {
    OpDef pull;
    OpDefBuilder("Pull").Output(GetGradientName(op_def_.input(0))).Shape(op_def_).Device(op_def_).Finalize(&pull);
    grad->push_back(pull);
  }
};
class GraphOutputOpDecl : public OpDecl {
 public:
  explicit GraphOutputOpDecl(const OpDef& def) : OpDecl(def) { CHECK(def.shape_size() == 1) << def.DebugString(); }
  void ShapeInference(std::vector<TensorShapeDef>* out, const std::vector<TensorShapeDef>&) override {
    CHECK(out->empty());
    out->push_back(op_def_.shape(0));
  }
  void MakeGradient(std::vector<OpDef>* grad) override {
    CHECK(op_def_.input_size() >= 2) << op_def_.DebugString();
    CHECK(op_def_.output_size() == 1) << op_def_.DebugString();
    std::vector<std::string> var, var_grad;
    for (int i = 1; i < op_def_.input_size(); i++) {   // input 0 is the graph structure
      var.push_back(op_def_.input(i));
      var_grad.push_back(GetGradientName(op_def_.input(i)));
    }
    OpDef g;
    OpDefBuilder(GetGradientName("GraphOutput"))
        .Input(GetGradientName(op_def_.output(0)))
        .Input(var)
        .Output(var_grad)
        .Device(op_def_)
        .Finalize(&g);
    grad->push_back(g);
  }
};
class GraphOutputGradOpDecl : public OpDecl {
 public:
  using OpDecl::OpDecl;
  void ShapeInference(std::vector<TensorShapeDef>* out, const std::vector<TensorShapeDef>& inputs) override {
    CHECK(out->empty());
    CHECK(inputs.size() > 1);
    for (size_t i = 1; i < inputs.size(); i++) out->push_back(inputs[i]);
  }
};

}  // namespace

REGISTER_OP_DECL_BUILDER("Gather", GatherOpDecl);
REGISTER_OP_DECL_BUILDER("Pull", PullOpDecl);
REGISTER_OP_DECL_BUILDER("Scatter", ScatterOpDecl);
REGISTER_OP_DECL_BUILDER("Push", PushOpDecl);
REGISTER_OP_DECL_BUILDER("GraphOutput", GraphOutputOpDecl);
REGISTER_OP_DECL_BUILDER(GetGradientName("GraphOutput"), GraphOutputGradOpDecl);

}  // namespace backend
