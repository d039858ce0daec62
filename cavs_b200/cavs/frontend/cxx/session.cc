#include "cavs/frontend/cxx/session.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <set>
#include <unordered_map>

#include "cavs/frontend/cxx/generic_session.h"
#include "cavs/util/op_util.h"
#include "cavs_b200.h"

namespace {

using frontend::Program;

void Must(int status, const char* what) { CHECK(status == CAVS_OK) << what << ": " << cavs_last_error(); }
void MustCuda(cudaError_t e, const char* what) { CHECK(e == cudaSuccess) << what << ": " << cudaGetErrorString(e); }

int Count(const TensorShapeDef& s) {
  int n = 1;
  for (auto d : s.dim()) n *= static_cast<int>(d);
  return n;
}

// Follows view-like ops (Mirror, Reshape, Expand_dims, ControlDependency) back to the tensor they alias
// and accumulates Slice offsets, until a Variable / Placeholder / computed tensor is reached.
struct Origin {
  const OpDef* op = nullptr;   // producing op that is not a view
  int offset = 0;              // element offset into it (sum of Slice offsets)
};
Origin Trace(const Program& prog, const std::string& tensor) {
  Origin o;
  std::string cur = tensor;
  for (int guard = 0; guard < 64; ++guard) {
    const OpDef* op = prog.Producer(cur);
    CHECK(op != nullptr) << "tensor " << cur << " has no producer";
    const std::string& n = op->name();
    if (n == "Mirror" || n == "Reshape" || n == "Expand_dims" || n == "ControlDependency") { cur = op->input(0); continue; }
    if (n == "Slice") { o.offset += GetSingleArg<int>(*op, "Offset"); cur = op->input(0); continue; }
    o.op = op;
    return o;
  }
  LOG(FATAL) << "view chain too deep at " << tensor;
  return o;
}

enum class Kind { kTreeLstm, kChainLstm };

struct Recognised {
  Kind kind;
  int H = 0, E = 0, V = 0, C = 0, K = 0, max_vertices = 0;
  float lr = 0.f, clip = 0.f;
  bool has_optimizer = false;
  std::string graph_ph, vertex_ph, label_ph;
  std::string emb, w, u, b, fc_w, fc_b;   // Variable tensor names (chain LSTM: w == u == the joint weight variable)
  std::string graph_output, fc_out, loss, optimizer;
};

std::map<std::string, int> OpCounts(const FunctionDef& f) {
  std::map<std::string, int> c;
  for (const auto& op : f.ops()) c[op.name()]++;
  return c;
}

// True when Node() has the operator census of one of the two LSTM forms the fused engine implements.
bool LooksLikeFusedLstm(const Program& prog) {
  if (prog.functions.empty()) return false;
  const auto counts = OpCounts(prog.functions.back());
  auto cnt = [&](const char* n) { auto it = counts.find(n); return it == counts.end() ? 0 : it->second; };
  const bool tree = cnt("Gather") == 2 && cnt("MatMul") == 4 && cnt("Sigmoid") == 4 && cnt("Tanh") == 2 && cnt("Mul") == 4;
  const bool chain = cnt("Gather") == 1 && cnt("MatMul") == 2 && cnt("Sigmoid") == 3 && cnt("Tanh") == 2 && cnt("Mul") == 3;
  if (!((tree || chain) && cnt("Pull") == 1 && cnt("EmbeddingLookup") == 1 && cnt("Scatter") == 1 && cnt("Push") == 1 && cnt("Concat") == 1 &&
        cnt("Relu") == 0))
    return false;
  return true;
}

Recognised Recognise(const Program& prog) {
  Recognised r;
  const OpDef* go = nullptr;
  for (const auto& op : prog.ops) if (op.name() == "GraphOutput") go = &op;
  CHECK(go != nullptr) << "the program has no GraphOutput (GraphSupport::Output() was never called)";
  CHECK(!prog.functions.empty());
  const FunctionDef& f = prog.functions.back();
  r.graph_output = go->output(0);
  r.graph_ph = go->input(0);
  r.vertex_ph = go->input(1);
  r.max_vertices = GetSingleArg<int>(*go, "MaxGraphNodeCount");

  const auto counts = OpCounts(f);
  auto cnt = [&](const char* n) { auto it = counts.find(n); return it == counts.end() ? 0 : it->second; };
  const bool tree = cnt("Gather") == 2 && cnt("MatMul") == 4 && cnt("Sigmoid") == 4 && cnt("Tanh") == 2 && cnt("Mul") == 4;
  const bool chain = cnt("Gather") == 1 && cnt("MatMul") == 2 && cnt("Sigmoid") == 3 && cnt("Tanh") == 2 && cnt("Mul") == 3;
  CHECK((tree || chain) && cnt("Pull") == 1 && cnt("EmbeddingLookup") == 1 && cnt("Scatter") == 1 && cnt("Push") == 1 && cnt("Concat") == 1)
      << "vertex function not recognised: this build binds the child-sum Tree-LSTM (two Gather slots, four MatMul) and the "
         "chain LSTM (one Gather slot, two MatMul) forms to fused kernels and has no generic interpreter";
  r.kind = tree ? Kind::kTreeLstm : Kind::kChainLstm;
  r.K = tree ? 2 : 1;

  std::set<std::string> weight_vars;
  for (const auto& op : f.ops()) {
    if (op.name() == "Gather") {
      const int w = Count(op.shape(0));
      CHECK(w % 2 == 0);
      CHECK(r.H == 0 || r.H == w / 2) << "Gather slots disagree on the state width";
      r.H = w / 2;
    } else if (op.name() == "EmbeddingLookup") {
      const Origin o = Trace(prog, op.input(1));
      CHECK(o.op->name() == "Variable" && o.op->shape(0).dim_size() == 2) << "embedding table must be a 2-D Variable";
      r.emb = o.op->output(0);
      r.V = static_cast<int>(o.op->shape(0).dim(0));
      r.E = static_cast<int>(o.op->shape(0).dim(1));
    } else if (op.name() == "MatMul") {
      const Origin o = Trace(prog, op.input(1));
      CHECK(o.op->name() == "Variable") << "MatMul weight must come from a Variable";
      weight_vars.insert(o.op->output(0));
      const Origin lhs = Trace(prog, op.input(0));
      if (lhs.op->name() == "EmbeddingLookup") r.w = o.op->output(0); else r.u = o.op->output(0);
    } else if (op.name() == "Add") {
      for (const auto& in : op.input()) {
        const Origin o = Trace(prog, in);
        if (o.op->name() == "Variable" && Count(o.op->shape(0)) == 4 * r.H) r.b = o.op->output(0);
      }
    }
  }
  CHECK(r.H > 0 && r.E > 0 && !r.w.empty() && !r.u.empty() && !r.b.empty()) << "could not bind the vertex function's parameters";
  if (tree) {
    CHECK(r.w != r.u) << "Tree-LSTM expects separate input and recurrent weight Variables";
    CHECK(Count(*prog.ShapeOf(r.w)) == 4 * r.E * r.H && Count(*prog.ShapeOf(r.u)) == 4 * r.H * r.H);
  } else {
    CHECK(r.w == r.u && r.E == r.H) << "chain LSTM expects one joint weight Variable [2*4*H*H] and embedding == hidden";
    CHECK(Count(*prog.ShapeOf(r.w)) == 8 * r.H * r.H);
  }

  // Loss head in the main program.
  for (const auto& op : prog.ops) {
    if (op.name() == "FullyConnected" && Trace(prog, op.input(0)).op->output(0) == r.graph_output) {
      r.fc_out = op.output(0);
      r.fc_w = Trace(prog, op.input(1)).op->output(0);
      r.fc_b = Trace(prog, op.input(2)).op->output(0);
      r.C = static_cast<int>(prog.ShapeOf(r.fc_w)->dim(0));
      CHECK(static_cast<int>(prog.ShapeOf(r.fc_w)->dim(1)) == r.H) << "classifier weight must be [classes, hidden]";
    }
  }
  CHECK(!r.fc_out.empty()) << "expected graph_output.FullyConnected(weight, bias)";
  for (const auto& op : prog.ops) {
    if (op.name() == "SoftmaxEntropyLoss" && op.input(0) == r.fc_out) {
      r.loss = op.output(0);
      const Origin lab = Trace(prog, op.input(1));
      CHECK(lab.op->name() == "Placeholder") << "labels must be fed through a Placeholder";
      r.label_ph = lab.op->output(0);
    }
  }
  CHECK(!r.loss.empty()) << "expected .SoftmaxEntropyLoss(label)";
  for (const auto& op : prog.ops) {
    if (op.name() == "Optimizer" && op.input(0) == r.loss) {
      r.optimizer = op.output(0);
      r.has_optimizer = true;
      r.lr = GetSingleArg<float>(op, "lr");
      r.clip = GetSingleArg<float>(op, "clip", 0.f);
      CHECK(r.clip >= 0.f);
    }
  }
  return r;
}

}  // namespace

struct Session::Impl {
  int opt = 0;
  bool compiled = false;
  std::unique_ptr<frontend::GenericSession> generic;   // set when the program is not one of the fused forms
  Recognised r;
  cavs_treelstm_config cfg{};
  cavs_treelstm* engine = nullptr;
  cavs_sched* sched = nullptr;
  void* workspace = nullptr;
  float *params = nullptr, *grads = nullptr;   // device, engine layout: Emb | W | U | B | Wc | bc
  float* clip_scratch = nullptr;
  size_t n_params = 0;
  std::vector<float> host_params;              // staging for Set/GetVariable
  std::vector<int32_t> tok_job, label_job, t2j, j2t;
  int n_total = 0;

  size_t OffW() const { return static_cast<size_t>(r.V) * r.E; }
  size_t OffU() const { return OffW() + static_cast<size_t>(r.E) * 4 * r.H; }
  size_t OffB() const { return OffU() + static_cast<size_t>(4) * r.H * r.H; }
  size_t OffWc() const { return OffB() + static_cast<size_t>(4) * r.H; }
  size_t Offbc() const { return OffWc() + static_cast<size_t>(r.C) * r.H; }

  ~Impl() {
    if (engine) cavs_treelstm_destroy(engine);
    if (sched) cavs_sched_destroy(sched);
    if (workspace) cudaFree(workspace);
    if (params) cudaFree(params);
    if (grads) cudaFree(grads);
    if (clip_scratch) cudaFree(clip_scratch);
  }

  // ---- declared (app) layout <-> engine layout, on the host ----
  // Tree-LSTM: the declared layout IS the engine's.  Chain LSTM: the joint weight holds U [H,4H]
  // (multiplies x) then W [H,4H] (multiplies the child's h), column blocks i,f,u,o; the engine wants the
  // input weight with blocks i,o,u,f and the recurrent weight as U_iou [H,3H] followed by U_f [H,H].
  void PackVariable(const std::string& var, const float* src, size_t count, std::vector<float>* flat) const {
    const int H = r.H;
    auto blk = [&](const float* m, int row, int k) { return m + static_cast<size_t>(row) * 4 * H + static_cast<size_t>(k) * H; };
    if (var == r.emb) { CHECK(count == OffW()); std::memcpy(flat->data(), src, count * 4); return; }
    if (var == r.b) { CHECK(count == static_cast<size_t>(4 * H)); std::memcpy(flat->data() + OffB(), src, count * 4); return; }
    if (var == r.fc_w) { CHECK(count == static_cast<size_t>(r.C) * H); std::memcpy(flat->data() + OffWc(), src, count * 4); return; }
    if (var == r.fc_b) { CHECK(count == static_cast<size_t>(r.C)); std::memcpy(flat->data() + Offbc(), src, count * 4); return; }
    if (r.kind == Kind::kTreeLstm) {
      if (var == r.w) { CHECK(count == static_cast<size_t>(4) * r.E * H); std::memcpy(flat->data() + OffW(), src, count * 4); return; }
      if (var == r.u) { CHECK(count == static_cast<size_t>(4) * H * H); std::memcpy(flat->data() + OffU(), src, count * 4); return; }
    } else if (var == r.w) {
      CHECK(count == static_cast<size_t>(8) * H * H);
      const float* Ux = src;                       // [H,4H] for x
      const float* Wh = src + static_cast<size_t>(4) * H * H;   // [H,4H] for h
      float* W = flat->data() + OffW();
      float* Uiou = flat->data() + OffU();
      float* Uf = Uiou + static_cast<size_t>(3) * H * H;
      const int order_w[4] = {0, 3, 2, 1};         // engine blocks i,o,u,f <- declared blocks i,f,u,o
      for (int row = 0; row < H; ++row) {
        for (int k = 0; k < 4; ++k) std::memcpy(W + static_cast<size_t>(row) * 4 * H + static_cast<size_t>(k) * H, blk(Ux, row, order_w[k]), H * 4);
        for (int k = 0; k < 3; ++k) std::memcpy(Uiou + static_cast<size_t>(row) * 3 * H + static_cast<size_t>(k) * H, blk(Wh, row, order_w[k]), H * 4);
        std::memcpy(Uf + static_cast<size_t>(row) * H, blk(Wh, row, 1), H * 4);
      }
      return;
    }
    LOG(FATAL) << "variable " << var << " is not a parameter of the recognised program";
  }
  void UnpackVariable(const std::string& var, const std::vector<float>& flat, float* dst, size_t count) const {
    const int H = r.H;
    if (var == r.emb) { std::memcpy(dst, flat.data(), count * 4); return; }
    if (var == r.b) { std::memcpy(dst, flat.data() + OffB(), count * 4); return; }
    if (var == r.fc_w) { std::memcpy(dst, flat.data() + OffWc(), count * 4); return; }
    if (var == r.fc_b) { std::memcpy(dst, flat.data() + Offbc(), count * 4); return; }
    if (r.kind == Kind::kTreeLstm) {
      if (var == r.w) { std::memcpy(dst, flat.data() + OffW(), count * 4); return; }
      if (var == r.u) { std::memcpy(dst, flat.data() + OffU(), count * 4); return; }
    } else if (var == r.w) {
      float* Ux = dst;
      float* Wh = dst + static_cast<size_t>(4) * H * H;
      const float* W = flat.data() + OffW();
      const float* Uiou = flat.data() + OffU();
      const float* Uf = Uiou + static_cast<size_t>(3) * H * H;
      const int order_w[4] = {0, 3, 2, 1};
      for (int row = 0; row < H; ++row) {
        for (int k = 0; k < 4; ++k) std::memcpy(Ux + static_cast<size_t>(row) * 4 * H + static_cast<size_t>(order_w[k]) * H, W + static_cast<size_t>(row) * 4 * H + static_cast<size_t>(k) * H, H * 4);
        for (int k = 0; k < 3; ++k) std::memcpy(Wh + static_cast<size_t>(row) * 4 * H + static_cast<size_t>(order_w[k]) * H, Uiou + static_cast<size_t>(row) * 3 * H + static_cast<size_t>(k) * H, H * 4);
        std::memcpy(Wh + static_cast<size_t>(row) * 4 * H + static_cast<size_t>(1) * H, Uf + static_cast<size_t>(row) * H, H * 4);
      }
      return;
    }
    LOG(FATAL) << "variable " << var << " is not a parameter of the recognised program";
  }

  void Compile() {
    const Program& prog = *Program::Get();
    if (!LooksLikeFusedLstm(prog) || (opt & OPT_REF_COMPAT_ROWS) || std::getenv("CAVS_GENERIC_SESSION") != nullptr) {
      generic.reset(new frontend::GenericSession(opt));
      compiled = true;
      return;
    }
    r = Recognise(prog);
    cfg.hidden = r.H; cfg.embed = r.E; cfg.vocab = r.V; cfg.classes = r.C; cfg.n_slots = r.K;
    cfg.gemm_bf16 = (opt & OPT_BF16_GEMM) ? 1 : 0;
    cfg.max_vertices = r.max_vertices;
    cfg.max_level_rows = r.max_vertices;
    n_params = cavs_treelstm_param_count(&cfg);
    const size_t ws = cavs_treelstm_workspace_bytes(&cfg);
    CHECK(n_params > 0 && ws > 0) << cavs_last_error();
    MustCuda(cudaMalloc(&workspace, ws), "workspace");
    MustCuda(cudaMalloc(reinterpret_cast<void**>(&params), n_params * sizeof(float)), "params");
    MustCuda(cudaMalloc(reinterpret_cast<void**>(&grads), n_params * sizeof(float)), "grads");
    MustCuda(cudaMemset(grads, 0, n_params * sizeof(float)), "grads");
    Must(cavs_treelstm_create(&cfg, workspace, ws, &engine), "cavs_treelstm_create");
    Must(cavs_treelstm_bind(engine, params, grads), "cavs_treelstm_bind");
    Must(cavs_sched_create(&sched), "cavs_sched_create");
    // cavs/midend/graph_session.h:20-24: OPT_BATCHING selects the level scheduler, its absence the serial one.
    Must(cavs_sched_set_order(sched, (opt & OPT_BATCHING) ? 0 : 1), "cavs_sched_set_order");
    // Variable fillers (cavs/backend/functor_filler.h): constant or uniform; one seeded stream per variable.
    host_params.assign(n_params, 0.f);
    uint64_t seed = 0x5eed0000;
    std::set<std::string> vars = {r.emb, r.w, r.u, r.b, r.fc_w, r.fc_b};
    for (const auto& v : vars) {
      const OpDef* op = prog.Producer(v);
      const size_t count = static_cast<size_t>(Count(op->shape(0)));
      std::vector<float> init(count, 0.f);
      if (op->label() == "Uniform") {
        const float lo = GetSingleArg<float>(*op, "minval"), hi = GetSingleArg<float>(*op, "maxval");
        Must(cavs_synth_uniform_float(++seed, 1.0f, init.data(), count), "cavs_synth_uniform_float");
        for (auto& x : init) x = 0.5f * (lo + hi) + 0.5f * (hi - lo) * x;
      } else {
        const float c = GetSingleArg<float>(*op, "const_value", 0.f);
        std::fill(init.begin(), init.end(), c);
      }
      PackVariable(v, init.data(), count, &host_params);
    }
    Upload();
    compiled = true;
  }
  void Upload() {
    MustCuda(cudaMemcpy(params, host_params.data(), n_params * sizeof(float), cudaMemcpyHostToDevice), "upload parameters");
    Must(cavs_treelstm_refresh_weights(engine, nullptr), "cavs_treelstm_refresh_weights");
  }
  void Download() {
    MustCuda(cudaMemcpy(host_params.data(), params, n_params * sizeof(float), cudaMemcpyDeviceToHost), "download parameters");
  }
};

Session::Session(int opt, std::string name) : impl_(new Impl()) {
  CHECK(name == "SimpleSession") << "only SimpleSession is provided (data parallelism uses one process per GPU and NCCL)";
  impl_->opt = opt;
}
Session::~Session() {}

void Session::SetVariable(const Sym& var, const float* host, size_t count) {
  if (!impl_->compiled) impl_->Compile();
  if (impl_->generic) { impl_->generic->SetVariable(var.output(0), host, count); return; }
  impl_->Download();
  impl_->PackVariable(var.output(0), host, count, &impl_->host_params);
  impl_->Upload();
}
void Session::GetVariable(const Sym& var, float* host, size_t count) {
  if (!impl_->compiled) impl_->Compile();
  if (impl_->generic) { impl_->generic->GetVariable(var.output(0), host, count); return; }
  impl_->Download();
  impl_->UnpackVariable(var.output(0), impl_->host_params, host, count);
}

void Session::GetGradient(const Sym& var, float* host, size_t count) {
  if (!impl_->compiled) impl_->Compile();
  if (impl_->generic) { impl_->generic->GetGradient(var.output(0), host, count); return; }
  std::vector<float> flat(impl_->n_params);
  MustCuda(cudaMemcpy(flat.data(), impl_->grads, impl_->n_params * sizeof(float), cudaMemcpyDeviceToHost), "download gradients");
  impl_->UnpackVariable(var.output(0), flat, host, count);
}

void Session::Run(std::vector<Sym> outputs, const std::initializer_list<std::pair<Sym&, void*>>& feed) {
  Impl& m = *impl_;
  if (!m.compiled) m.Compile();
  if (m.generic) {
    std::vector<std::pair<std::string, void*>> named;
    for (const auto& f : feed) named.emplace_back(f.first.output(0), f.second);
    m.generic->Run(outputs, named);
    return;
  }
  const Recognised& r = m.r;
  const Program& prog = *Program::Get();
  const void *graph = nullptr, *vertex = nullptr, *label = nullptr;
  for (const auto& f : feed) {
    const std::string& name = f.first.output(0);
    if (name == r.graph_ph) graph = f.second;
    else if (name == r.vertex_ph) vertex = f.second;
    else if (name == r.label_ph) label = f.second;
    else LOG(FATAL) << "feed for " << name << " is not an input of the recognised program";
  }
  CHECK(graph && vertex && label) << "Run needs feeds for the graph, vertex-input and label placeholders";
  const TensorShapeDef* gs = prog.ShapeOf(r.graph_ph);
  CHECK(gs && gs->dim_size() == 2);
  const int batch = static_cast<int>(gs->dim(0)), max_len = static_cast<int>(gs->dim(1));
  Must(cavs_sched_load(m.sched, static_cast<const int32_t*>(graph), batch, max_len, r.K), "cavs_sched_load");
  int n_sched = 0, n_levels = 0, max_rows = 0;
  Must(cavs_sched_counts(m.sched, &m.n_total, &n_sched, &n_levels, &max_rows), "cavs_sched_counts");
  const int n = m.n_total;
  m.tok_job.resize(n); m.label_job.resize(n); m.t2j.resize(n); m.j2t.resize(n);
  const float* vf = static_cast<const float*>(vertex);
  const float* lf = static_cast<const float*>(label);
  // Token ids and labels are carried as floats and cast (op_impl_embedding_lookup.cu:27,
  // op_impl_softmax_entropy_logits_loss.cu:101); Pull reads the vertex input at the compact job id.
  for (int g = 0; g < n; ++g) { m.tok_job[g] = static_cast<int32_t>(vf[g]); m.label_job[g] = static_cast<int32_t>(lf[g]); }
  Must(cavs_treelstm_load_batch(m.engine, m.sched, m.tok_job.data(), m.label_job.data(), n, nullptr), "cavs_treelstm_load_batch");
  Must(cavs_treelstm_forward(m.engine, nullptr), "cavs_treelstm_forward");
  Must(cavs_treelstm_backward(m.engine, nullptr), "cavs_treelstm_backward");
  float loss_sum = 0.f;
  int status = 0;
  Must(cavs_treelstm_read_loss(m.engine, &loss_sum, &status, nullptr), "cavs_treelstm_read_loss");

  bool update = false;
  for (auto& out : outputs) {
    const std::string& name = out.output(0);
    const OpDef* op = prog.Producer(name);
    CHECK(op != nullptr);
    if (name == r.optimizer) { update = true; continue; }
    std::vector<char>* raw = out.mutable_raw();
    if (name == r.loss) {
      // per-vertex loss, permuted from execution order back to job order (FunctionPopRet)
      const void* dev = nullptr; size_t bytes = 0;
      // leaves may share loss-head rows per token: have the per-vertex values written out first
      Must(cavs_treelstm_materialize_state(m.engine, nullptr), "cavs_treelstm_materialize_state");
      Must(cavs_treelstm_peek(m.engine, 1, &dev, &bytes), "cavs_treelstm_peek");
      std::vector<float> tid(n_sched);
      MustCuda(cudaMemcpy(tid.data(), dev, n_sched * sizeof(float), cudaMemcpyDeviceToHost), "fetch loss");
      Must(cavs_sched_maps(m.sched, m.t2j.data(), m.j2t.data(), n), "cavs_sched_maps");
      raw->assign(static_cast<size_t>(n) * sizeof(float), 0);
      float* dst = reinterpret_cast<float*>(raw->data());
      for (int t = 0; t < n_sched; ++t) dst[m.t2j[t]] = tid[t];
    } else if ((op->name() == "Reduce_mean" || op->name() == "Reduce_sum") && op->input(0) == r.loss) {
      // the reference reduces with an absolute sum (cavs/backend/op_impl_blas1_cublas.cc:71); losses are >= 0
      const float v = op->name() == "Reduce_mean" ? std::fabs(loss_sum) / static_cast<float>(std::max(n, 1)) : std::fabs(loss_sum);
      raw->assign(sizeof(float), 0);
      std::memcpy(raw->data(), &v, sizeof(float));
    } else if (name == r.graph_output) {
      const void* dev = nullptr; size_t bytes = 0;
      // leaves may share state rows per token: have the per-vertex rows written out first
      Must(cavs_treelstm_materialize_state(m.engine, nullptr), "cavs_treelstm_materialize_state");
      Must(cavs_treelstm_peek(m.engine, 0, &dev, &bytes), "cavs_treelstm_peek");
      std::vector<float> state(static_cast<size_t>(n_sched) * 2 * r.H);
      MustCuda(cudaMemcpy(state.data(), dev, state.size() * sizeof(float), cudaMemcpyDeviceToHost), "fetch graph output");
      Must(cavs_sched_maps(m.sched, m.t2j.data(), m.j2t.data(), n), "cavs_sched_maps");
      raw->assign(static_cast<size_t>(n) * r.H * sizeof(float), 0);
      float* dst = reinterpret_cast<float*>(raw->data());
      for (int t = 0; t < n_sched; ++t) std::memcpy(dst + static_cast<size_t>(m.t2j[t]) * r.H, state.data() + static_cast<size_t>(t) * 2 * r.H, r.H * sizeof(float));
    } else {
      LOG(FATAL) << "cannot fetch " << name << " (" << op->name() << "): fetchable are the loss, its Reduce_mean / Reduce_sum, "
                    "the graph output and the optimizer";
    }
  }
  if (update) {
    CHECK(r.has_optimizer);
    if (r.clip > 0.f) {
      // Clip (cavs/backend/op_impl_clip.cu:25-45): scale by clip / max(sum of the per-VARIABLE L2 norms, clip).  The
      // engine's blocks are the declared variables, except that the chain LSTM's joint weight is W and U together.
      std::vector<unsigned long long> offs = {0, m.OffW()};
      if (r.kind == Kind::kTreeLstm) offs.push_back(m.OffU());
      offs.push_back(m.OffB()); offs.push_back(m.OffWc()); offs.push_back(m.Offbc()); offs.push_back(m.n_params);
      const int n_blocks = static_cast<int>(offs.size()) - 1;
      if (!m.clip_scratch) MustCuda(cudaMalloc(reinterpret_cast<void**>(&m.clip_scratch), cavs_clip_gradients_scratch_bytes(8)), "clip scratch");
      Must(cavs_clip_gradients(m.grads, offs.data(), n_blocks, r.clip, m.clip_scratch, nullptr), "cavs_clip_gradients");
    }
    // one SGD launch over the flat parameter buffer (every Variable, as `Optimizer({}, lr)` asks: c_api.cc:123-137)
    Must(cavs_sgd(m.params, m.grads, m.n_params, r.lr, nullptr), "cavs_sgd");
    Must(cavs_treelstm_refresh_weights(m.engine, nullptr), "cavs_treelstm_refresh_weights");
  }
  MustCuda(cudaDeviceSynchronize(), "Session::Run");   // the reference synchronises once per Run (session_simple.cc:106-107)
}
