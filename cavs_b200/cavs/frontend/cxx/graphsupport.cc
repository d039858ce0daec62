#include "cavs/frontend/cxx/graphsupport.h"

#include "cavs/util/op_def_builder.h"

Sym GraphSupport::Output() {
  FuncConf::FuncDefineBegin("Node");
  this->Node();
  FunctionDef func = FuncConf::FuncDefineEnd("Node");
  // The function's result is what Push receives (cavs/midend/graph_util.cc:296-331).
  int unit = 0;
  for (const auto& op : func.ops())
    if (op.name() == "Push") {
      unit = 1;
      for (auto d : op.shape(0).dim()) unit *= static_cast<int>(d);
    }
  CHECK(unit > 0) << "Node() must Push exactly one tensor";
  frontend::Program::Get()->functions.push_back(func);
  int max_graph_node_count = 1;
  for (int d : raw_graph_.shape(0)) max_graph_node_count *= d;
  OpDefBuilder b("GraphOutput");
  b.Input(raw_graph_.output(0)).Input(raw_vertex_.output(0)).Dtype(raw_vertex_.type()).Device(raw_vertex_.device())
      .Shape(std::vector<int>{-1, unit}).AttrSingle("Wavefront", true).AttrSingle("MaxGraphNodeCount", max_graph_node_count);
  return Sym(b.Finalize());
}

Sym GraphSupport::Gather(int child, const std::vector<int>& shape) {
  CHECK(!shape.empty());
  OpDefBuilder b("Gather");
  b.Dtype(raw_vertex_.type()).Device(raw_vertex_.device()).Shape(shape).AttrSingle("Child", child);
  return Sym(b.Finalize());
}

Sym GraphSupport::Pull(int offset, const std::vector<int>& shape) {
  OpDefBuilder b("Pull");
  b.Dtype(raw_vertex_.type()).Device(raw_vertex_.device()).Shape(shape).AttrSingle("Offset", offset);
  return Sym(b.Finalize());
}

void GraphSupport::Push(const Sym& s) {
  OpDefBuilder b("Push");
  b.Input(s.output(0)).Dtype(s.type()).Device(s.device()).Shape(s.shape(0));
  Sym recorded(b.Finalize());
  (void)recorded;
}

void GraphSupport::Scatter(const Sym& s) {
  // one parent per vertex: the reference fixes Child = 0 here (cavs/frontend/cxx/graphsupport.cc:84-93)
  OpDefBuilder b("Scatter");
  b.Input(s.output(0)).Dtype(s.type()).Device(s.device()).Shape(s.shape(0)).AttrSingle("Child", 0);
  Sym recorded(b.Finalize());
  (void)recorded;
}
