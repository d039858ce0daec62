// Vertex functions other than the fused LSTM forms, through the same Sym / GraphSupport / Session API: the recorded
// Node() is executed operator by operator per level, its elementwise groups as kernels generated and compiled at run time.
//
//   generic_fn_test cpu          plans and compiles (no GPU needed): Tree-FC as the reference's app declares it
//                                (apps/paper/tree-fc-cavs.cc:29-36) and a gated variant with inputs
//   generic_fn_test gpu <file>   runs both on the device through Session::Run (forward, loss, backward, clipped SGD step)
//                                and writes inputs, parameters, outputs, gradients and updated parameters to <file>
//                                for an independent check (tests/test_generic_function.py: float64 autograd)
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <tuple>
#include <vector>

#include "cavs/frontend/cxx/graphsupport.h"
#include "cavs/frontend/cxx/session.h"
#include "cavs/frontend/cxx/sym.h"
#include "cavs/midend/generic_function.h"
#include "cavs_b200.h"

static int g_failures = 0;
#define EXPECT(cond) do { if (!(cond)) { std::printf("FAILED %s:%d  %s\n", __FILE__, __LINE__, #cond); ++g_failures; } } while (0)

static const int kH = 24, kE = 16, kV = 40, kC = 3;

// The reference's Tree-FC vertex: relu([left | right] W); no vertex input, so every state is zero -- it is the app's
// timing benchmark.
class TreeFC : public GraphSupport {
 public:
  TreeFC(const Sym& g, const Sym& v) : GraphSupport(g, v) { W = Sym::Variable(DT_FLOAT, {2 * kH, kH}, Sym::Uniform(-0.1f, 0.1f)); }
  void Node() override {
    Sym left = Gather(0, {kH});
    Sym right = Gather(1, {kH});
    Sym fc = Sym::MatMul(Sym::Concat({left, right}).Reshape({1, 2 * kH}), W.Mirror());
    Sym res = fc.Relu();
    Scatter(res.Mirror());
    Push(res.Mirror());
  }
  Sym W;
};

// Tree-FC with a dense per-vertex input and a bias: res = relu([left | right] W + x Wx + b) - 0.5 left o right.
class TreeFCInput : public GraphSupport {
 public:
  TreeFCInput(const Sym& g, const Sym& v) : GraphSupport(g, v) {
    W = Sym::Variable(DT_FLOAT, {2 * kH, kH}, Sym::Uniform(-0.1f, 0.1f));
    Wx = Sym::Variable(DT_FLOAT, {kE, kH}, Sym::Uniform(-0.1f, 0.1f));
    b = Sym::Variable(DT_FLOAT, {kH}, Sym::Zeros());
    half = Sym::Variable(DT_FLOAT, {1}, Sym::Const(0.5f));
  }
  void Node() override {
    Sym left = Gather(0, {kH});
    Sym right = Gather(1, {kH});
    Sym x = Pull(0, {kE});
    Sym fc = Sym::MatMul(Sym::Concat({left, right}).Reshape({1, 2 * kH}), W.Mirror()).Reshape({kH});
    Sym fx = Sym::MatMul(x.Reshape({1, kE}), Wx.Mirror()).Reshape({kH});
    Sym res = (fc + fx + b.Mirror()).Relu() - (left * right) * half.Mirror();
    Scatter(res.Mirror());
    Push(res.Mirror());
  }
  Sym W, Wx, b, half;
};

// A gated cell on tokens: z, g = sigmoid, u = tanh of x Wx + (hl + hr) Wh + bias; c = z o u + g o (cl + cr); h = tanh(c) o z.
class GatedCell : public GraphSupport {
 public:
  GatedCell(const Sym& g, const Sym& v) : GraphSupport(g, v) {
    table = Sym::Variable(DT_FLOAT, {kV, kE}, Sym::Uniform(-0.1f, 0.1f));
    Wx = Sym::Variable(DT_FLOAT, {kE, 3 * kH}, Sym::Uniform(-0.1f, 0.1f));
    Wh = Sym::Variable(DT_FLOAT, {kH, 3 * kH}, Sym::Uniform(-0.1f, 0.1f));
    bias = Sym::Variable(DT_FLOAT, {3 * kH}, Sym::Zeros());
  }
  void Node() override {
    Sym hl, cl, hr, cr;
    std::tie(hl, cl) = Gather(0, {2 * kH}).Split2();
    std::tie(hr, cr) = Gather(1, {2 * kH}).Split2();
    Sym x = Pull(0, {1}).EmbeddingLookup(table.Mirror());
    Sym pre = Sym::MatMul(x, Wx.Mirror()).Reshape({3 * kH}) + Sym::MatMul((hl + hr).Reshape({1, kH}), Wh.Mirror()).Reshape({3 * kH}) + bias.Mirror();
    Sym z, g, u;
    std::tie(z, g, u) = pre.Split3();
    z = z.Sigmoid(); g = g.Sigmoid(); u = u.Tanh();
    Sym c = z * u + g * (cl + cr);
    Sym h = Sym::Tanh(c.Mirror()) * z;
    Scatter(Sym::Concat({h.Mirror(), c.Mirror()}));
    Push(h.Mirror());
  }
  Sym table, Wx, Wh, bias;
};

static FILE* g_out = nullptr;
static void Dump(const char* name, const float* v, size_t n) {
  const int len = static_cast<int>(std::strlen(name));
  const unsigned long long cnt = n;
  std::fwrite("f", 1, 1, g_out); std::fwrite(&len, 4, 1, g_out); std::fwrite(name, 1, len, g_out); std::fwrite(&cnt, 8, 1, g_out);
  std::fwrite(v, 4, n, g_out);
}
static void DumpInts(const char* name, const int* v, size_t n) {
  const int len = static_cast<int>(std::strlen(name));
  const unsigned long long cnt = n;
  std::fwrite("i", 1, 1, g_out); std::fwrite(&len, 4, 1, g_out); std::fwrite(name, 1, len, g_out); std::fwrite(&cnt, 8, 1, g_out);
  std::fwrite(v, 4, n, g_out);
}

static void TestPlanning() {
  {
    frontend::Program::Reset();
    Sym graph = Sym::Placeholder(DT_FLOAT, {2, 7}, "CPU");
    Sym vertex = Sym::Placeholder(DT_FLOAT, {2, 7});
    TreeFC model(graph, vertex);
    Sym out = model.Output();
    Sym loss = out.Reduce_sum();
    (void)loss;
    midend::GenericFunction fn(*frontend::Program::Get(), frontend::Program::Get()->functions.back(), 14);
    EXPECT(fn.out_width() == kH && fn.state_width() == kH && fn.pull_width() == 0);
    EXPECT(fn.n_groups() == 1 && fn.variables().size() == 1 && fn.param_count() == static_cast<size_t>(2 * kH * kH));
    EXPECT(fn.group_source(0, false).find("> 0.0f") != std::string::npos);       // the Relu expression
    EXPECT(fn.group_source(0, true).find("gin0") != std::string::npos);
  }
  {
    frontend::Program::Reset();
    Sym graph = Sym::Placeholder(DT_FLOAT, {2, 7}, "CPU");
    Sym vertex = Sym::Placeholder(DT_FLOAT, {2, 7});
    GatedCell model(graph, vertex);
    Sym out = model.Output();
    (void)out;
    midend::GenericFunction fn(*frontend::Program::Get(), frontend::Program::Get()->functions.back(), 14);
    EXPECT(fn.out_width() == kH && fn.state_width() == 2 * kH && fn.pull_width() == 1);
    // (hl + hr) | the pre-activation sum with its bias | the gates and the cell
    EXPECT(fn.n_groups() == 3 && fn.variables().size() == 4);
    EXPECT(fn.group_source(2, false).find("tanhf") != std::string::npos && fn.group_source(2, false).find("expf") != std::string::npos);
  }
}

static uint64_t g_seed = 7000;
static std::vector<float> Uniform(size_t n, float scale) {
  std::vector<float> v(n);
  cavs_synth_uniform_float(++g_seed, scale, v.data(), n);
  return v;
}

static void RunOnDevice() {
  const int B = 6, leaf_hi = 7, L = 2 * leaf_hi - 1;
  std::vector<int> parents(B * L, -1);
  EXPECT(cavs_synth_trees(4242, B, 2, leaf_hi, 2, L, parents.data(), nullptr) == CAVS_OK);
  int n = 0;
  for (int s = 0; s < B; ++s) { int len = 0; while (parents[s * L + len] != -1) ++len; n += len + 1; }
  DumpInts("parents", parents.data(), parents.size());
  const int dims[6] = {B, L, kH, kE, kV, kC};
  DumpInts("dims", dims, 6);

  {  // ---- Tree-FC with inputs, Reduce_sum loss, clipped SGD ----
    frontend::Program::Reset();
    Sym graph = Sym::Placeholder(DT_FLOAT, {B, L}, "CPU");
    Sym vertex = Sym::Placeholder(DT_FLOAT, {B, L * kE});
    TreeFCInput model(graph, vertex);
    Sym out = model.Output();
    Sym loss = out.Reduce_sum();
    const float lr = 0.05f, clip = 2.0f;
    Sym train = loss.Optimizer({}, lr, clip);
    Session sess(OPT_BATCHING);
    std::vector<float> W = Uniform(2 * kH * kH, 0.3f), Wx = Uniform(kE * kH, 0.3f), b = Uniform(kH, 0.1f), half = {0.5f};
    sess.SetVariable(model.W, W.data(), W.size()); sess.SetVariable(model.Wx, Wx.data(), Wx.size());
    sess.SetVariable(model.b, b.data(), b.size()); sess.SetVariable(model.half, half.data(), 1);
    std::vector<float> x = Uniform(static_cast<size_t>(n) * kE, 1.0f);   // compact job order
    sess.Run({train, loss, out}, {{graph, parents.data()}, {vertex, x.data()}});
    Dump("fc.W", W.data(), W.size()); Dump("fc.Wx", Wx.data(), Wx.size()); Dump("fc.b", b.data(), b.size()); Dump("fc.x", x.data(), x.size());
    const float hp[2] = {lr, clip};
    Dump("fc.lr_clip", hp, 2);
    Dump("fc.loss", reinterpret_cast<const float*>(loss.eval()), 1);
    Dump("fc.out", reinterpret_cast<const float*>(out.eval()), static_cast<size_t>(n) * kH);
    auto put = [&](const char* name, const Sym& v, size_t count, bool grad) {
      std::vector<float> tmp(count);
      if (grad) sess.GetGradient(v, tmp.data(), count); else sess.GetVariable(v, tmp.data(), count);
      Dump(name, tmp.data(), count);
    };
    put("fc.gW", model.W, W.size(), true); put("fc.gWx", model.Wx, Wx.size(), true); put("fc.gb", model.b, b.size(), true);
    put("fc.ghalf", model.half, 1, true);
    put("fc.W1", model.W, W.size(), false); put("fc.Wx1", model.Wx, Wx.size(), false); put("fc.b1", model.b, b.size(), false);
  }
  {  // ---- gated cell on tokens, classifier + softmax cross-entropy, SGD ----
    frontend::Program::Reset();
    Sym graph = Sym::Placeholder(DT_FLOAT, {B, L}, "CPU");
    Sym words = Sym::Placeholder(DT_FLOAT, {B, L});
    Sym label = Sym::Placeholder(DT_FLOAT, {B, L});
    Sym fc_w = Sym::Variable(DT_FLOAT, {kC, kH}, Sym::Uniform(-0.1f, 0.1f));
    Sym fc_b = Sym::Variable(DT_FLOAT, {1, kC}, Sym::Zeros());
    GatedCell model(graph, words);
    Sym out = model.Output();
    Sym loss = out.FullyConnected(fc_w, fc_b).SoftmaxEntropyLoss(label.Reshape({-1, 1}));
    const float lr = 0.1f;
    Sym train = loss.Optimizer({}, lr);
    Session sess(OPT_BATCHING);
    std::vector<float> table = Uniform(kV * kE, 0.4f), Wx = Uniform(kE * 3 * kH, 0.3f), Wh = Uniform(kH * 3 * kH, 0.3f), bias = Uniform(3 * kH, 0.1f),
                       wc = Uniform(kC * kH, 0.4f), bc = Uniform(kC, 0.1f);
    sess.SetVariable(model.table, table.data(), table.size()); sess.SetVariable(model.Wx, Wx.data(), Wx.size());
    sess.SetVariable(model.Wh, Wh.data(), Wh.size()); sess.SetVariable(model.bias, bias.data(), bias.size());
    sess.SetVariable(fc_w, wc.data(), wc.size()); sess.SetVariable(fc_b, bc.data(), bc.size());
    std::vector<float> tok(n), lab(n);
    for (int g = 0; g < n; ++g) { tok[g] = static_cast<float>((g * 7 + 3) % kV); lab[g] = static_cast<float>((g * 5 + 1) % kC); }
    sess.Run({train, loss, out}, {{graph, parents.data()}, {words, tok.data()}, {label, lab.data()}});
    Dump("gc.table", table.data(), table.size()); Dump("gc.Wx", Wx.data(), Wx.size()); Dump("gc.Wh", Wh.data(), Wh.size());
    Dump("gc.bias", bias.data(), bias.size()); Dump("gc.wc", wc.data(), wc.size()); Dump("gc.bc", bc.data(), bc.size());
    Dump("gc.tok", tok.data(), tok.size()); Dump("gc.lab", lab.data(), lab.size());
    Dump("gc.loss", reinterpret_cast<const float*>(loss.eval()), n);
    Dump("gc.out", reinterpret_cast<const float*>(out.eval()), static_cast<size_t>(n) * kH);
    auto put = [&](const char* name, const Sym& v, size_t count) {
      std::vector<float> tmp(count);
      sess.GetGradient(v, tmp.data(), count);
      Dump(name, tmp.data(), count);
    };
    put("gc.gtable", model.table, table.size()); put("gc.gWx", model.Wx, Wx.size()); put("gc.gWh", model.Wh, Wh.size());
    put("gc.gbias", model.bias, bias.size()); put("gc.gwc", fc_w, wc.size()); put("gc.gbc", fc_b, bc.size());
  }
  {  // ---- the reference's Tree-FC app as declared: forward only, all states zero ----
    frontend::Program::Reset();
    Sym graph = Sym::Placeholder(DT_FLOAT, {B, L}, "CPU");
    Sym vertex = Sym::Placeholder(DT_FLOAT, {B, L});
    TreeFC model(graph, vertex);
    Sym out = model.Output();
    Sym loss = out.Reduce_sum();
    Session sess(OPT_BATCHING);
    sess.Run({loss}, {{graph, parents.data()}});
    EXPECT(*reinterpret_cast<const float*>(loss.eval()) == 0.0f);
  }
}

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "cpu";
  TestPlanning();
  if (mode == "gpu") {
    EXPECT(argc > 2);
    g_out = std::fopen(argc > 2 ? argv[2] : "/dev/null", "wb");
    EXPECT(g_out != nullptr);
    if (g_out) { RunOnDevice(); std::fclose(g_out); }
  }
  if (g_failures == 0) std::printf("generic_fn_test %s: ok\n", mode.c_str());
  return g_failures == 0 ? 0 : 1;
}
