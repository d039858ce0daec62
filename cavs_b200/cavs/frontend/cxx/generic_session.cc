#include "cavs/frontend/cxx/generic_session.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstring>

#include "cavs/frontend/cxx/session.h"
#include "cavs/proto/opt.pb.h"
#include "cavs/util/op_util.h"

namespace frontend {
namespace {

void Must(int status, const char* what) { CHECK(status == CAVS_OK) << what << ": " << cavs_last_error(); }
void MustCuda(cudaError_t e, const char* what) { CHECK(e == cudaSuccess) << what << ": " << cudaGetErrorString(e); }
int Count(const TensorShapeDef& s) {
  int n = 1;
  for (auto d : s.dim()) n *= static_cast<int>(d);
  return n;
}
// the Variable a (possibly viewed) tensor of the main program comes from
std::string VariableOf(const Program& prog, std::string tensor) {
  for (int guard = 0; guard < 64; ++guard) {
    const OpDef* op = prog.Producer(tensor);
    CHECK(op != nullptr) << "tensor " << tensor << " has no producer";
    if (op->name() == "Variable") return op->output(0);
    CHECK(op->name() == "Mirror" || op->name() == "Reshape" || op->name() == "Expand_dims") << "expected a Variable behind " << tensor;
    tensor = op->input(0);
  }
  LOG(FATAL) << "view chain too deep";
  return "";
}

}  // namespace

GenericSession::GenericSession(int opt) : opt_(opt) {
  const Program& prog = *Program::Get();
  const OpDef* go = nullptr;
  for (const auto& op : prog.ops) if (op.name() == "GraphOutput") go = &op;
  CHECK(go != nullptr && !prog.functions.empty()) << "the program has no GraphOutput";
  graph_output_ = go->output(0);
  graph_ph_ = go->input(0);
  vertex_ph_ = go->input(1);
  max_vertices_ = GetSingleArg<int>(*go, "MaxGraphNodeCount");
  fn_.reset(new midend::GenericFunction(prog, prog.functions.back(), max_vertices_));
  for (const auto& op : prog.functions.back().ops())
    if (op.name() == "Gather") n_slots_ = std::max(n_slots_, GetSingleArg<int>(op, "Child") + 1);
  // loss head
  for (const auto& op : prog.ops) {
    if (op.name() == "Reduce_sum" && op.input(0) == graph_output_) loss_ = op.output(0);
    if (op.name() == "FullyConnected" && op.input(0) == graph_output_) {
      fc_w_ = VariableOf(prog, op.input(1));
      fc_b_ = VariableOf(prog, op.input(2));
      classes_ = static_cast<int>(prog.ShapeOf(fc_w_)->dim(0));
      CHECK(static_cast<int>(prog.ShapeOf(fc_w_)->dim(1)) == fn_->out_width()) << "classifier weight must be [classes, width of the pushed tensor]";
      CHECK(classes_ >= 1 && classes_ <= 8) << "the generic path's loss head takes at most 8 classes";
      for (const auto& l : prog.ops)
        if (l.name() == "SoftmaxEntropyLoss" && l.input(0) == op.output(0)) {
          loss_ = l.output(0);
          xent_ = true;
          std::string cur = l.input(1);
          const OpDef* lab = prog.Producer(cur);
          for (int guard = 0; guard < 16 && lab && lab->name() != "Placeholder"; ++guard) { cur = lab->input(0); lab = prog.Producer(cur); }
          CHECK(lab && lab->name() == "Placeholder") << "labels must be fed through a Placeholder";
          label_ph_ = lab->output(0);
        }
    }
  }
  CHECK(!loss_.empty()) << "expected graph_output.Reduce_sum() or graph_output.FullyConnected(w, b).SoftmaxEntropyLoss(label)";
  for (const auto& op : prog.ops)
    if (op.name() == "Optimizer" && op.input(0) == loss_) {
      optimizer_ = op.output(0);
      has_optimizer_ = true;
      lr_ = GetSingleArg<float>(op, "lr");
      clip_ = GetSingleArg<float>(op, "clip", 0.f);
    }
  const size_t np = std::max<size_t>(fn_->param_count(), 4);
  MustCuda(cudaMalloc(reinterpret_cast<void**>(&params_), np * sizeof(float)), "parameters");
  MustCuda(cudaMalloc(reinterpret_cast<void**>(&grads_), np * sizeof(float)), "gradients");
  MustCuda(cudaMemset(params_, 0, np * sizeof(float)), "parameters");
  MustCuda(cudaMemset(grads_, 0, np * sizeof(float)), "gradients");
  size_t scratch = 4096 + cavs_clip_gradients_scratch_bytes(static_cast<int>(fn_->variables().size()));
  if (xent_) scratch = std::max(scratch, cavs_fc_softmax_xent_scratch_bytes(fn_->out_width(), classes_));
  MustCuda(cudaMalloc(reinterpret_cast<void**>(&scratch_), scratch), "scratch");
  MustCuda(cudaMalloc(reinterpret_cast<void**>(&loss_rows_), (static_cast<size_t>(max_vertices_) + 4) * sizeof(float)), "loss rows");
  MustCuda(cudaMalloc(reinterpret_cast<void**>(&loss_sum_), 4 * sizeof(float)), "loss sum");
  MustCuda(cudaMalloc(reinterpret_cast<void**>(&d_label_), static_cast<size_t>(max_vertices_) * sizeof(int32_t)), "labels");
  Must(cavs_sched_create(&sched_), "cavs_sched_create");
  Must(cavs_sched_set_order(sched_, (opt_ & OPT_BATCHING) ? 0 : 1), "cavs_sched_set_order");
  // Variable fillers (cavs/backend/functor_filler.h): constant or uniform, one seeded stream per variable.
  uint64_t seed = 0x5eed1000;
  for (const auto& v : fn_->variables()) {
    const OpDef* op = prog.Producer(v.name);
    std::vector<float> init(v.count, 0.f);
    if (op->label() == "Uniform") {
      const float lo = GetSingleArg<float>(*op, "minval"), hi = GetSingleArg<float>(*op, "maxval");
      Must(cavs_synth_uniform_float(++seed, 1.0f, init.data(), v.count), "cavs_synth_uniform_float");
      for (auto& x : init) x = 0.5f * (lo + hi) + 0.5f * (hi - lo) * x;
    } else {
      std::fill(init.begin(), init.end(), GetSingleArg<float>(*op, "const_value", 0.f));
    }
    MustCuda(cudaMemcpy(params_ + v.offset, init.data(), v.count * sizeof(float), cudaMemcpyHostToDevice), "variable init");
  }
  fn_->Bind(params_, grads_);
}

GenericSession::~GenericSession() {
  if (sched_) cavs_sched_destroy(sched_);
  for (void* p : {static_cast<void*>(params_), static_cast<void*>(grads_), static_cast<void*>(scratch_), static_cast<void*>(loss_rows_),
                  static_cast<void*>(loss_sum_), static_cast<void*>(d_label_)})
    if (p) cudaFree(p);
}

void GenericSession::SetVariable(const std::string& var, const float* host, size_t count) {
  const auto* v = fn_->FindVariable(var);
  CHECK(v != nullptr && v->count == count) << "no Variable " << var << " of " << count << " values";
  MustCuda(cudaMemcpy(params_ + v->offset, host, count * sizeof(float), cudaMemcpyHostToDevice), "SetVariable");
}
void GenericSession::GetVariable(const std::string& var, float* host, size_t count) {
  const auto* v = fn_->FindVariable(var);
  CHECK(v != nullptr && v->count == count) << "no Variable " << var << " of " << count << " values";
  MustCuda(cudaMemcpy(host, params_ + v->offset, count * sizeof(float), cudaMemcpyDeviceToHost), "GetVariable");
}
void GenericSession::GetGradient(const std::string& var, float* host, size_t count) {
  const auto* v = fn_->FindVariable(var);
  CHECK(v != nullptr && v->count == count) << "no Variable " << var << " of " << count << " values";
  MustCuda(cudaMemcpy(host, grads_ + v->offset, count * sizeof(float), cudaMemcpyDeviceToHost), "GetGradient");
}

void GenericSession::Run(std::vector<Sym>& outputs, const std::vector<std::pair<std::string, void*>>& feeds) {
  const Program& prog = *Program::Get();
  const void *graph = nullptr, *vertex = nullptr, *label = nullptr;
  for (const auto& f : feeds) {
    if (f.first == graph_ph_) graph = f.second;
    else if (f.first == vertex_ph_) vertex = f.second;
    else if (f.first == label_ph_) label = f.second;
    else LOG(FATAL) << "feed for " << f.first << " is not an input of the program";
  }
  CHECK(graph != nullptr) << "Run needs a feed for the graph placeholder";
  CHECK(!xent_ || label != nullptr) << "Run needs a feed for the label placeholder";
  const TensorShapeDef* gs = prog.ShapeOf(graph_ph_);
  CHECK(gs && gs->dim_size() == 2);
  Must(cavs_sched_load(sched_, static_cast<const int32_t*>(graph), static_cast<int>(gs->dim(0)), static_cast<int>(gs->dim(1)), n_slots_), "cavs_sched_load");
  int n_total = 0, n = 0, n_levels = 0, max_rows = 0;
  Must(cavs_sched_counts(sched_, &n_total, &n, &n_levels, &max_rows), "cavs_sched_counts");
  std::vector<int32_t> level_off(n_levels + 1), t2j(n_total), j2t(n_total), fg(static_cast<size_t>(n_slots_) * n_total), fs(n_total), bg(n_total),
      bs(static_cast<size_t>(n_slots_) * n_total);
  Must(cavs_sched_level_offsets(sched_, level_off.data(), n_levels + 1), "cavs_sched_level_offsets");
  Must(cavs_sched_maps(sched_, t2j.data(), j2t.data(), n_total), "cavs_sched_maps");
  // Row alignment: 0 = every row pairs with its own children / parent; 1 = the reference's positional pairing of its compact
  // per-round lists with level rows (op_impl_graphop.cu:62-76,144-157), which shifts rows on skewed batches.
  Must(cavs_sched_tables(sched_, (opt_ & OPT_REF_COMPAT_ROWS) ? 1 : 0, fg.data(), fs.data(), bg.data(), bs.data(), n_total), "cavs_sched_tables");
  // compact the slot-major tables to the scheduled rows
  std::vector<int32_t> cfg(static_cast<size_t>(n_slots_) * std::max(n, 1)), cbs(cfg.size());
  for (int c = 0; c < n_slots_; ++c)
    for (int t = 0; t < n; ++t) {
      cfg[static_cast<size_t>(c) * n + t] = fg[static_cast<size_t>(c) * n_total + t];
      cbs[static_cast<size_t>(c) * n + t] = bs[static_cast<size_t>(c) * n_total + t];
    }
  fn_->LoadBatch(cfg.data(), fs.data(), bg.data(), cbs.data(), n_slots_, t2j.data(), n, level_off, static_cast<const float*>(vertex));
  fn_->Forward();
  const int wo = fn_->out_width();
  MustCuda(cudaMemsetAsync(grads_, 0, std::max<size_t>(fn_->param_count(), 4) * sizeof(float), nullptr), "zero gradients");
  if (xent_) {
    std::vector<int32_t> lab(std::max(n, 1));
    const float* lf = static_cast<const float*>(label);
    for (int t = 0; t < n; ++t) lab[t] = static_cast<int32_t>(lf[t2j[t]]);   // labels are floats in job order (op_impl_softmax_entropy_logits_loss.cu:101)
    MustCuda(cudaMemcpy(d_label_, lab.data(), sizeof(int32_t) * n, cudaMemcpyHostToDevice), "labels");
    const auto* w = fn_->FindVariable(fc_w_);
    const auto* b = fn_->FindVariable(fc_b_);
    Must(cavs_fc_softmax_xent(loss_rows_, loss_sum_, fn_->output_grad(), grads_ + w->offset, grads_ + b->offset, fn_->output(), wo, d_label_,
                              params_ + w->offset, params_ + b->offset, n, wo, classes_, 1.0f / static_cast<float>(std::max(n, 1)), scratch_, nullptr),
         "cavs_fc_softmax_xent");
  } else {
    // Reduce_sum is a sum of absolute values (cublasSasum, op_impl_blas1_cublas.cc:48-77) and its gradient a Fill with
    // the upstream value, 1 (op_decl_reduction.cc:19-28, graph_util.cc:106-112).
    Must(cavs_abs_sum(loss_sum_, fn_->output(), static_cast<size_t>(n) * wo, scratch_, nullptr), "cavs_abs_sum");
    Must(cavs_fill(fn_->output_grad(), static_cast<size_t>(n) * wo, 1.0f, nullptr), "cavs_fill");
  }
  fn_->Backward();
  float loss_sum = 0.f;
  MustCuda(cudaMemcpy(&loss_sum, loss_sum_, sizeof(float), cudaMemcpyDeviceToHost), "fetch loss");

  bool update = false;
  for (auto& out : outputs) {
    const std::string& name = out.output(0);
    const OpDef* op = prog.Producer(name);
    CHECK(op != nullptr);
    std::vector<char>* raw = out.mutable_raw();
    if (name == optimizer_ && has_optimizer_) { update = true; continue; }
    if (name == loss_ && !xent_) {
      raw->assign(sizeof(float), 0);
      std::memcpy(raw->data(), &loss_sum, sizeof(float));
    } else if (name == loss_) {
      std::vector<float> tid(std::max(n, 1));
      MustCuda(cudaMemcpy(tid.data(), loss_rows_, n * sizeof(float), cudaMemcpyDeviceToHost), "fetch loss rows");
      raw->assign(static_cast<size_t>(n_total) * sizeof(float), 0);
      float* dst = reinterpret_cast<float*>(raw->data());
      for (int t = 0; t < n; ++t) dst[t2j[t]] = tid[t];
    } else if ((op->name() == "Reduce_mean" || op->name() == "Reduce_sum") && op->input(0) == loss_) {
      const float count = xent_ ? static_cast<float>(std::max(n_total, 1)) : 1.0f;
      const float v = op->name() == "Reduce_mean" ? std::fabs(loss_sum) / count : std::fabs(loss_sum);
      raw->assign(sizeof(float), 0);
      std::memcpy(raw->data(), &v, sizeof(float));
    } else if (name == graph_output_) {
      std::vector<float> tid(static_cast<size_t>(std::max(n, 1)) * wo);
      MustCuda(cudaMemcpy(tid.data(), fn_->output(), static_cast<size_t>(n) * wo * sizeof(float), cudaMemcpyDeviceToHost), "fetch graph output");
      raw->assign(static_cast<size_t>(n_total) * wo * sizeof(float), 0);
      float* dst = reinterpret_cast<float*>(raw->data());
      for (int t = 0; t < n; ++t) std::memcpy(dst + static_cast<size_t>(t2j[t]) * wo, tid.data() + static_cast<size_t>(t) * wo, wo * sizeof(float));
    } else {
      LOG(FATAL) << "cannot fetch " << name << " (" << op->name() << ")";
    }
  }
  if (update) {
    if (clip_ > 0.f) {
      std::vector<unsigned long long> offs;
      for (const auto& v : fn_->variables()) offs.push_back(v.offset);
      offs.push_back(fn_->param_count());
      Must(cavs_clip_gradients(grads_, offs.data(), static_cast<int>(offs.size()) - 1, clip_, scratch_, nullptr), "cavs_clip_gradients");
    }
    Must(cavs_sgd(params_, grads_, fn_->param_count(), lr_, nullptr), "cavs_sgd");
  }
  MustCuda(cudaDeviceSynchronize(), "Session::Run");
}

}  // namespace frontend
