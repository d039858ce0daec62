// The F/G declaration front end (Sym, GraphSupport::Node(), Session::Run) exercised the way the reference's
// apps use it: a vertex function written against Sym, a training program around it, one Session::Run per batch.
//
//   frontend_test cpu   what Node() records (no CUDA call)
//   frontend_test gpu   one training step of a Tree-LSTM and of a chain LSTM through Session::Run, compared with
//                       the CPU oracle (loss per vertex, every updated Variable), 1e-5 relative; once bound to the
//                       fused engine and once run operator by operator (CAVS_GENERIC_SESSION=1)
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <tuple>
#include <vector>

#include "cavs/frontend/cxx/graphsupport.h"
#include "cavs/frontend/cxx/session.h"
#include "cavs/frontend/cxx/sym.h"
#include "cavs/util/op_util.h"
#include "cavs_b200.h"

extern "C" {
typedef struct { int n, n_levels, hidden, embed, vocab, classes, n_slots, gemm_bf16, loss_rows, preact_bf16; } oracle_cfg;
int cavs_oracle_tables(const int* parents, int batch, int max_len, int n_slots, int mode, int* n_total_out, int* level_off,
                       int level_cap, int* t2j, int* j2t, int* fg, int* fs, int* bg, int* bs);
int cavs_oracle_treelstm_fwd_bwd(const oracle_cfg* cfg, const int* level_off, const int* fg, const int* fs, const int* bg,
                                 const int* bs, const int* tok, const int* label, const float* Emb, const float* W,
                                 const float* U, const float* B, const float* Wc, const float* bc, float* state_out,
                                 float* loss_out, float* dEmb, float* dW, float* dU, float* dB, float* dWc, float* dbc,
                                 float* dstate_dbg);
}

static int g_failures = 0;
#define EXPECT(cond) do { if (!(cond)) { std::printf("FAILED %s:%d  %s\n", __FILE__, __LINE__, #cond); ++g_failures; } } while (0)

static const int kHidden = 12, kEmbed = 10, kVocab = 30, kClasses = 4;

// A binary child-sum Tree-LSTM vertex, declared like a user of the reference would.
class TreeCell : public GraphSupport {
 public:
  TreeCell(const Sym& graph, const Sym& words) : GraphSupport(graph, words) {
    const int H = kHidden, E = kEmbed;
    table = Sym::Variable(DT_FLOAT, {kVocab, E}, Sym::Uniform(-0.1f, 0.1f));
    w_in = Sym::Variable(DT_FLOAT, {4 * E * H}, Sym::Uniform(-0.1f, 0.1f));
    w_rec = Sym::Variable(DT_FLOAT, {4 * H * H}, Sym::Uniform(-0.1f, 0.1f));
    bias = Sym::Variable(DT_FLOAT, {4 * H}, Sym::Zeros());
  }
  void Node() override {
    const int H = kHidden, E = kEmbed;
    Sym hl, cl, hr, cr;
    std::tie(hl, cl) = Gather(0, {2 * H}).Split2();
    std::tie(hr, cr) = Gather(1, {2 * H}).Split2();
    Sym x = Pull(0, {1}).EmbeddingLookup(table.Mirror());
    Sym ai, ao, au, af;   // input projection, column blocks i,o,u,f
    std::tie(ai, ao, au, af) = Sym::MatMul(x, w_in.Reshape({E, 4 * H}).Mirror()).Reshape({4 * H}).Split4();
    Sym u_iou = w_rec.Slice(0, 3 * H * H).Reshape({H, 3 * H});
    Sym u_f = w_rec.Slice(3 * H * H, H * H).Reshape({H, H});
    Sym pi, po, pu;
    std::tie(pi, po, pu) = Sym::MatMul((hl + hr).Reshape({1, H}), u_iou.Mirror()).Reshape({3 * H}).Split3();
    Sym ql = Sym::MatMul(hl.Reshape({1, H}), u_f.Mirror()).Reshape({H});
    Sym qr = Sym::MatMul(hr.Reshape({1, H}), u_f.Mirror()).Reshape({H});
    Sym bi = bias.Slice(0, H), bf = bias.Slice(H, H), bu = bias.Slice(2 * H, H), bo = bias.Slice(3 * H, H);
    Sym i = (ai + pi + bi.Mirror()).Sigmoid();
    Sym o = (ao + po + bo.Mirror()).Sigmoid();
    Sym u = (au + pu + bu.Mirror()).Tanh();
    Sym fl = (af + ql + bf.Mirror()).Sigmoid();
    Sym fr = (af + qr + bf.Mirror()).Sigmoid();
    Sym c = i * u + fl * cl + fr * cr;
    Sym h = o * Sym::Tanh(c.Mirror());
    Scatter(Sym::Concat({h.Mirror(), c.Mirror()}));
    Push(h.Mirror());
  }
  Sym table, w_in, w_rec, bias;
};

// A chain LSTM vertex: one child slot, joint weight Variable (input part first), gate blocks i,f,u,o.
class ChainCell : public GraphSupport {
 public:
  ChainCell(const Sym& graph, const Sym& words) : GraphSupport(graph, words) {
    const int H = kHidden;
    table = Sym::Variable(DT_FLOAT, {kVocab, H}, Sym::Uniform(-0.1f, 0.1f));
    weight = Sym::Variable(DT_FLOAT, {2 * 4 * H * H}, Sym::Uniform(-0.1f, 0.1f));
    bias = Sym::Variable(DT_FLOAT, {4 * H}, Sym::Zeros());
  }
  void Node() override {
    const int H = kHidden;
    Sym ch, cc;
    std::tie(ch, cc) = Gather(0, {2 * H}).Split2();
    Sym x = Pull(0, {1}).EmbeddingLookup(table);
    Sym from_x = weight.Slice(0, 4 * H * H), from_h = weight.Slice(4 * H * H, 4 * H * H);
    Sym pre = Sym::MatMul(x, from_x.Mirror().Reshape({H, 4 * H})) + Sym::MatMul(ch.Expand_dims(0), from_h.Mirror().Reshape({H, 4 * H}));
    Sym i, f, u, o;
    std::tie(i, f, u, o) = pre.Split4();
    i = (i + bias.Slice(0, H).Mirror()).Sigmoid();
    f = (f + bias.Slice(H, H).Mirror()).Sigmoid();
    u = (u + bias.Slice(2 * H, H).Mirror()).Tanh();
    o = (o + bias.Slice(3 * H, H).Mirror()).Sigmoid();
    Sym c = i * u + f * cc;
    Sym h = o * Sym::Tanh(c.Mirror());
    Scatter(Sym::Concat({h.Mirror(), c.Mirror()}));
    Push(h.Mirror());
  }
  Sym table, weight, bias;
};

static void TestRecording() {
  frontend::Program::Reset();
  Sym graph = Sym::Placeholder(DT_FLOAT, {2, 5}, "CPU");
  Sym words = Sym::Placeholder(DT_FLOAT, {2, 5});
  TreeCell cell(graph, words);
  Sym out = cell.Output();
  EXPECT(out.op_name() == "GraphOutput");
  EXPECT(out.shape(0).size() == 2 && out.shape(0)[0] == -1 && out.shape(0)[1] == kHidden);
  EXPECT(GetSingleArg<int>(out.def(), "MaxGraphNodeCount") == 10);
  const FunctionDef& f = frontend::Program::Get()->functions.back();
  EXPECT(f.name() == "Node");
  std::map<std::string, int> n;
  for (const auto& op : f.ops()) n[op.name()]++;
  EXPECT(n["Gather"] == 2 && n["Pull"] == 1 && n["MatMul"] == 4 && n["Scatter"] == 1 && n["Push"] == 1 && n["EmbeddingLookup"] == 1);
  EXPECT(!FuncConf::CheckInFunc());
  // ops created outside Node() land in the main program, not in the function
  const size_t before = frontend::Program::Get()->ops.size();
  Sym loss_in = out.FullyConnected(Sym::Variable(DT_FLOAT, {kClasses, kHidden}), Sym::Variable(DT_FLOAT, {1, kClasses}));
  EXPECT(frontend::Program::Get()->ops.size() == before + 3 && loss_in.shape(0)[1] == kClasses);
}

static uint64_t g_seed = 1000;
static std::vector<float> Uniform(size_t n, float scale) {
  std::vector<float> v(n);
  cavs_synth_uniform_float(++g_seed, scale, v.data(), n);
  return v;
}
static double RelErr(const std::vector<float>& a, const std::vector<float>& b) {
  double err = 0, ref = 1e-30;
  for (size_t i = 0; i < a.size(); i++) { err = std::fmax(err, std::fabs((double)a[i] - b[i])); ref = std::fmax(ref, std::fabs((double)b[i])); }
  return err / ref;
}

// One training step through Session::Run vs the oracle.  `chain`: which vertex function; `opt`: the
// Session's optimisation bits (without OPT_BATCHING the vertices run one per round).
static std::vector<float> TestTrainingStep(bool chain, int opt, float clip = 0.f) {
  frontend::Program::Reset();
  const int H = kHidden, E = chain ? kHidden : kEmbed, V = kVocab, C = kClasses, K = chain ? 1 : 2;
  const int B = 3, L = 7;
  std::vector<int> parents(B * L, -1);
  if (chain) {
    const int lens[B] = {7, 4, 2};
    for (int s = 0; s < B; s++) for (int j = 0; j < L; j++) parents[s * L + j] = (j + 1 < lens[s]) ? j + 1 : -1;
  } else {
    const int t0[L] = {4, 4, 5, 5, 6, 6, -1};      // 4 leaves, balanced
    const int t1[L] = {3, 3, 4, 4, -1, -1, -1};    // 3 leaves
    const int t2[L] = {2, 2, -1, -1, -1, -1, -1};  // 2 leaves
    std::memcpy(&parents[0], t0, sizeof(t0)); std::memcpy(&parents[L], t1, sizeof(t1)); std::memcpy(&parents[2 * L], t2, sizeof(t2));
  }
  Sym graph = Sym::Placeholder(DT_FLOAT, {B, L}, "CPU");
  Sym words = Sym::Placeholder(DT_FLOAT, {B, L});
  Sym label = Sym::Placeholder(DT_FLOAT, {B, L});
  Sym fc_w = Sym::Variable(DT_FLOAT, {C, H}, Sym::Uniform(-0.1f, 0.1f));
  Sym fc_b = Sym::Variable(DT_FLOAT, {1, C}, Sym::Zeros());
  TreeCell* tree = chain ? nullptr : new TreeCell(graph, words);
  ChainCell* chn = chain ? new ChainCell(graph, words) : nullptr;
  Sym graph_output = chain ? chn->Output() : tree->Output();
  Sym label_col = label.Reshape({-1, 1});
  label_col.ControlDependency(graph_output);
  Sym loss = graph_output.FullyConnected(fc_w, fc_b).SoftmaxEntropyLoss(label_col);
  const float lr = 0.5f;
  Sym train = loss.Optimizer({}, lr, clip);
  Sym mean_loss = loss.Reduce_mean();
  Session sess(opt);

  // parameters in the DECLARED layouts
  std::vector<float> table = Uniform((size_t)V * E, 0.4f), bias = Uniform(4 * H, 0.2f), wc = Uniform((size_t)C * H, 0.4f), bc = Uniform(C, 0.2f);
  std::vector<float> w_in, w_rec, joint;
  if (chain) { joint = Uniform((size_t)8 * H * H, 0.4f); } else { w_in = Uniform((size_t)4 * E * H, 0.4f); w_rec = Uniform((size_t)4 * H * H, 0.4f); }
  if (chain) {
    sess.SetVariable(chn->table, table.data(), table.size()); sess.SetVariable(chn->weight, joint.data(), joint.size());
    sess.SetVariable(chn->bias, bias.data(), bias.size());
  } else {
    sess.SetVariable(tree->table, table.data(), table.size()); sess.SetVariable(tree->w_in, w_in.data(), w_in.size());
    sess.SetVariable(tree->w_rec, w_rec.data(), w_rec.size()); sess.SetVariable(tree->bias, bias.data(), bias.size());
  }
  sess.SetVariable(fc_w, wc.data(), wc.size()); sess.SetVariable(fc_b, bc.data(), bc.size());

  // inputs: floats in compact job order
  int n = 0, levels = 0;
  std::vector<int> level_off(L + 2), t2j(B * L), j2t(B * L), fg(K * B * L), fs(B * L), bg(B * L), bs(K * B * L);
  // row alignment of the oracle's tables: the reference's positional pairing when the Session is asked for it
  levels = cavs_oracle_tables(parents.data(), B, L, K, (opt & OPT_REF_COMPAT_ROWS) ? 1 : 0, &n, level_off.data(), (int)level_off.size(), t2j.data(), j2t.data(),
                              fg.data(), fs.data(), bg.data(), bs.data());
  EXPECT(levels > 0);
  std::vector<float> words_f(B * L, 0.f), label_f(B * L, -1.f);
  std::vector<int> tok_job(n), lab_job(n);
  for (int g = 0; g < n; g++) { tok_job[g] = (g * 7 + 3) % V; lab_job[g] = (g * 5 + 1) % C; words_f[g] = (float)tok_job[g]; label_f[g] = (float)lab_job[g]; }

  sess.Run({train, loss, mean_loss}, {{graph, parents.data()}, {label, label_f.data()}, {words, words_f.data()}});

  // oracle on the same inputs, parameters in the Tree-LSTM layout
  std::vector<float> W((size_t)4 * E * H), U((size_t)4 * H * H);
  if (chain) {
    const float* Ux = joint.data(); const float* Wh = joint.data() + (size_t)4 * H * H;
    const int order[4] = {0, 3, 2, 1};
    for (int r = 0; r < H; r++) {
      for (int k = 0; k < 4; k++) std::memcpy(&W[(size_t)r * 4 * H + k * H], Ux + (size_t)r * 4 * H + order[k] * H, H * 4);
      for (int k = 0; k < 3; k++) std::memcpy(&U[(size_t)r * 3 * H + k * H], Wh + (size_t)r * 4 * H + order[k] * H, H * 4);
      std::memcpy(&U[(size_t)3 * H * H + (size_t)r * H], Wh + (size_t)r * 4 * H + H, H * 4);
    }
  } else { W = w_in; U = w_rec; }
  std::vector<int> tok(n), lab(n);
  for (int t = 0; t < n; t++) { tok[t] = tok_job[t2j[t]]; lab[t] = lab_job[t2j[t]]; }
  oracle_cfg cfg = {n, levels, H, E, V, C, K, 0, 0, 0};
  std::vector<float> state((size_t)n * 2 * H), loss_t(n), dEmb((size_t)V * E), dW(W.size()), dU(U.size()), dB(4 * H), dWc((size_t)C * H), dbc(C);
  cavs_oracle_treelstm_fwd_bwd(&cfg, level_off.data(), fg.data(), fs.data(), bg.data(), bs.data(), tok.data(), lab.data(), table.data(),
                               W.data(), U.data(), bias.data(), wc.data(), bc.data(), state.data(), loss_t.data(), dEmb.data(), dW.data(),
                               dU.data(), dB.data(), dWc.data(), dbc.data(), nullptr);
  // fetched loss is in job order
  std::vector<float> want_loss(n), got_loss(n);
  for (int t = 0; t < n; t++) want_loss[t2j[t]] = loss_t[t];
  std::memcpy(got_loss.data(), loss.eval(), n * sizeof(float));
  EXPECT(RelErr(got_loss, want_loss) < 1e-5);
  double mean = 0; for (float v : want_loss) mean += v; mean /= n;
  EXPECT(std::fabs(*reinterpret_cast<const float*>(mean_loss.eval()) - mean) < 1e-5 * mean);

  // gradient clipping (op_impl_clip.cu:25-45): every gradient is scaled by clip / max(sum of the variables' L2 norms, clip);
  // the chain cell's joint weight is ONE variable, so its two parts share a norm
  float scale = 1.f;
  if (clip > 0.f) {
    auto sq = [](const std::vector<float>& g) { double s = 0; for (float v : g) s += (double)v * v; return s; };
    double sum = std::sqrt(sq(dEmb)) + std::sqrt(sq(dB)) + std::sqrt(sq(dWc)) + std::sqrt(sq(dbc));
    sum += chain ? std::sqrt(sq(dW) + sq(dU)) : std::sqrt(sq(dW)) + std::sqrt(sq(dU));
    scale = static_cast<float>(clip / std::fmax(sum, (double)clip));
    EXPECT(scale < 0.9f);   // the case must actually clip
  }
  // updated variables: w - lr * scale * g, compared in the declared layouts
  auto sgd = [&](std::vector<float> w, const std::vector<float>& g) { for (size_t i = 0; i < w.size(); i++) w[i] -= lr * scale * g[i]; return w; };
  auto fetch = [&](const Sym& v, size_t count) { std::vector<float> out(count); sess.GetVariable(v, out.data(), count); return out; };
  EXPECT(RelErr(fetch(chain ? chn->table : tree->table, table.size()), sgd(table, dEmb)) < 1e-5);
  EXPECT(RelErr(fetch(chain ? chn->bias : tree->bias, bias.size()), sgd(bias, dB)) < 1e-5);
  EXPECT(RelErr(fetch(fc_w, wc.size()), sgd(wc, dWc)) < 1e-5);
  EXPECT(RelErr(fetch(fc_b, bc.size()), sgd(bc, dbc)) < 1e-5);
  if (chain) {
    // map the oracle's Tree-layout gradients back to the joint declared layout
    std::vector<float> gj(joint.size());
    const int order[4] = {0, 3, 2, 1};
    for (int r = 0; r < H; r++) {
      for (int k = 0; k < 4; k++) std::memcpy(&gj[(size_t)r * 4 * H + order[k] * H], &dW[(size_t)r * 4 * H + k * H], H * 4);
      for (int k = 0; k < 3; k++) std::memcpy(&gj[(size_t)4 * H * H + (size_t)r * 4 * H + order[k] * H], &dU[(size_t)r * 3 * H + k * H], H * 4);
      std::memcpy(&gj[(size_t)4 * H * H + (size_t)r * 4 * H + H], &dU[(size_t)3 * H * H + (size_t)r * H], H * 4);
    }
    EXPECT(RelErr(fetch(chn->weight, joint.size()), sgd(joint, gj)) < 1e-5);
  } else {
    EXPECT(RelErr(fetch(tree->w_in, w_in.size()), sgd(w_in, dW)) < 1e-5);
    EXPECT(RelErr(fetch(tree->w_rec, w_rec.size()), sgd(w_rec, dU)) < 1e-5);
  }
  delete tree; delete chn;
  return got_loss;
}

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "cpu";
  TestRecording();
  if (mode == "gpu") {
    TestTrainingStep(false, OPT_BATCHING);
    TestTrainingStep(true, OPT_BATCHING | OPT_FUSION | OPT_STREAMMING);
    TestTrainingStep(false, OPT_NONE);
    TestTrainingStep(true, OPT_FUSION);
    TestTrainingStep(false, OPT_BATCHING, 0.05f);   // Optimizer(vars, lr, clip)
    TestTrainingStep(true, OPT_BATCHING, 0.05f);
    // The same two programs through the operator-by-operator executor (run-time-compiled elementwise groups) instead
    // of the fused engine: same oracle, same tolerance.
    setenv("CAVS_GENERIC_SESSION", "1", 1);
    TestTrainingStep(false, OPT_BATCHING);
    TestTrainingStep(true, OPT_BATCHING);
    TestTrainingStep(false, OPT_NONE);
    TestTrainingStep(true, OPT_BATCHING, 0.05f);
    unsetenv("CAVS_GENERIC_SESSION");
    // Row alignment of the reference's graph ops (positional pairing: rows shift on this batch of three different tree
    // shapes) against the oracle on the reference-compatible tables; the losses must differ from the aligned run's.
    const std::vector<float> aligned = TestTrainingStep(false, OPT_BATCHING);
    const std::vector<float> shifted = TestTrainingStep(false, OPT_BATCHING | OPT_REF_COMPAT_ROWS);
    EXPECT(RelErr(shifted, aligned) > 1e-3);
    TestTrainingStep(true, OPT_BATCHING | OPT_REF_COMPAT_ROWS);   // ragged chains: shorter chains first, rows shift too
  }
  if (g_failures == 0) std::printf("frontend_test %s: ok\n", mode.c_str());
  return g_failures == 0 ? 0 : 1;
}
