// Vertex-function declaration API, same surface as cavs/frontend/cxx/graphsupport.h:9-27: derive from
// GraphSupport, describe one vertex in Node() with Gather / Pull / Scatter / Push, call Output().
#ifndef CAVS_FRONTEND_CXX_GRAPHSUPPORT_H_
#define CAVS_FRONTEND_CXX_GRAPHSUPPORT_H_

#include <string>
#include <vector>

#include "cavs/frontend/cxx/sym.h"

class GraphSupport {
 public:
  GraphSupport(const Sym& graph_ph, const Sym& vertex_ph) : raw_graph_(graph_ph), raw_vertex_(vertex_ph) {}
  virtual ~GraphSupport() {}
  virtual void Node() = 0;
  // Records Node() as function "Node" and returns the GraphOutput symbol ([-1, unit], job order).
  Sym Output();

 protected:
  Sym Gather(int child, const std::vector<int>& shape);   // child-state row of slot `child`
  Sym Pull(int offset, const std::vector<int>& shape);    // this vertex's slice of the vertex input
  void Push(const Sym& s);                                // this vertex's row of the graph output
  void Scatter(const Sym& s);                             // state handed to the parent

 private:
  Sym raw_graph_;
  Sym raw_vertex_;
};
#endif
