#include "cavs/midend/generic_function.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <numeric>

#include "cavs/util/logging.h"
#include "cavs/util/op_util.h"
#include "cavs_b200.h"

namespace midend {
namespace {

constexpr int kEmbedChunkRows = 256;   // rows per chunk of the segmented embedding gradient (cavs_embed_bwd_segmented)

int Count(const TensorShapeDef& s) {
  int n = 1;
  for (auto d : s.dim()) n *= static_cast<int>(d);
  return n;
}
void Must(int status, const char* what) { CHECK(status == CAVS_OK) << what << ": " << cavs_last_error(); }
void MustCuda(cudaError_t e, const char* what) { CHECK(e == cudaSuccess) << what << ": " << cudaGetErrorString(e); }
size_t Align(size_t bytes) { return (bytes + 255) & ~static_cast<size_t>(255); }

const char* kEmbedFwdSource =
    "extern \"C\" __global__ void generic_embed_fwd(int rows, long long off, const float* __restrict__ ids, long long pitch,\n"
    "                                              const float* __restrict__ table, int vocab, int E, float* __restrict__ out) {\n"
    "  const long long total = (long long)rows * E;\n"
    "  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {\n"
    "    const int c = (int)(i % E);\n"
    "    const long long t = off + i / E;\n"
    "    int id = (int)ids[t * pitch];\n"          // token ids travel as floats (op_impl_embedding_lookup.cu:27)
    "    if (id < 0 || id >= vocab) id = 0;\n"
    "    out[t * E + c] = table[(long long)id * E + c];\n"
    "  }\n"
    "}\n";

unsigned GridFor(long long elems) { return static_cast<unsigned>(std::max<long long>(1, std::min<long long>((elems + 255) / 256, 148 * 8))); }

}  // namespace

int GenericFunction::NewBuf(int width) {
  CHECK(width > 0);
  bufs_.push_back(Buf{width, nullptr, nullptr});
  return static_cast<int>(bufs_.size()) - 1;
}

const GenericFunction::Variable* GenericFunction::FindVariable(const std::string& name) const {
  for (const auto& v : vars_) if (v.name == name) return &v;
  return nullptr;
}

GenericFunction::GenericFunction(const frontend::Program& prog, const FunctionDef& f, int max_vertices) : max_vertices_(max_vertices) {
  CHECK(max_vertices > 0);
  // Every Variable of the program, in declaration order, in one flat buffer (blocks start on 16-byte boundaries).
  for (const auto& op : prog.ops) {
    if (op.name() != "Variable") continue;
    Variable v;
    v.name = op.output(0);
    v.count = static_cast<size_t>(Count(op.shape(0)));
    v.offset = param_count_;
    param_count_ += (v.count + 3) & ~static_cast<size_t>(3);
    vars_.push_back(v);
    Ref r; r.buf = -1; r.var_off = v.offset; r.col = 0; r.width = static_cast<int>(v.count);
    refs_[v.name] = r;
  }
  // Views of Variables recorded in the main program (a Slice / Reshape / Mirror outside Node()).
  for (const auto& op : prog.ops) {
    const std::string& n = op.name();
    if ((n == "Slice" || n == "Reshape" || n == "Mirror" || n == "Expand_dims") && refs_.count(op.input(0))) {
      Ref r = refs_[op.input(0)];
      if (n == "Slice") { r.var_off += GetSingleArg<int>(op, "Offset"); r.width = GetSingleArg<int>(op, "Stride"); }
      refs_[op.output(0)] = r;
    }
  }
  auto ref_of = [&](const std::string& name) -> Ref {
    auto it = refs_.find(name);
    CHECK(it != refs_.end()) << "tensor " << name << " is used before it is produced";
    return it->second;
  };
  Group* open = nullptr;   // the elementwise group that the next elementwise operator may join
  int pull_buf = -1;
  for (const auto& op : f.ops()) {
    const std::string& n = op.name();
    const int out_w = op.shape_size() ? Count(op.shape(0)) : 0;
    if (RTC::IsElementwise(n)) {
      if (open == nullptr || open->desc.width != out_w) {
        groups_.emplace_back(new Group());
        open = groups_.back().get();
        open->desc.width = out_w;
        Step st; st.kind = Kind::kGroup; st.group = static_cast<int>(groups_.size()) - 1;
        steps_.push_back(st);
      }
      RTC::EwiseOp eop;
      eop.name = n;
      for (const auto& in : op.input()) {
        const Ref r = ref_of(in);
        RTC::EwiseOperand o;
        if (r.buf >= 0) {
          CHECK(r.width == out_w) << n << ": operand " << in << " has " << r.width << " columns, the result " << out_w;
          // an operand produced inside this group is a node; anything else an input of the group
          int node = -1;
          for (size_t k = 0; k < open->out_bufs.size(); ++k)
            if (open->out_bufs[k] == r.buf && r.col == 0) node = static_cast<int>(k);
          if (node >= 0) {
            o = {RTC::EwiseOperand::kNode, node};
          } else {
            int idx = -1;
            for (size_t j = 0; j < open->inputs.size(); ++j)
              if (open->inputs[j].buf == r.buf && open->inputs[j].col == r.col) idx = static_cast<int>(j);
            if (idx < 0) { open->inputs.push_back(r); idx = static_cast<int>(open->inputs.size()) - 1; }
            o = {RTC::EwiseOperand::kInput, idx};
          }
        } else {
          CHECK(r.width == out_w || r.width == 1) << n << ": a Variable operand must have the result's width or one element";
          int idx = -1;
          for (size_t q = 0; q < open->var_refs.size(); ++q)
            if (open->var_refs[q].var_off == r.var_off && open->var_refs[q].width == r.width) idx = static_cast<int>(q);
          if (idx < 0) { open->var_refs.push_back(r); open->desc.var_counts.push_back(r.width); idx = static_cast<int>(open->var_refs.size()) - 1; }
          o = {RTC::EwiseOperand::kVar, idx};
        }
        eop.in.push_back(o);
      }
      open->desc.ops.push_back(eop);
      const int b = NewBuf(out_w);
      open->out_bufs.push_back(b);
      Ref r; r.buf = b; r.width = out_w;
      refs_[op.output(0)] = r;
      continue;
    }
    // views: no operator runs
    if (n == "Reshape" || n == "Mirror" || n == "Expand_dims" || n == "ControlDependency") { refs_[op.output(0)] = ref_of(op.input(0)); continue; }
    if (n == "Slice") {
      Ref r = ref_of(op.input(0));
      const int o = GetSingleArg<int>(op, "Offset"), w = GetSingleArg<int>(op, "Stride");
      CHECK(o >= 0 && o + w <= r.width);
      if (r.buf >= 0) r.col += o; else r.var_off += o;
      r.width = w;
      refs_[op.output(0)] = r;
      continue;
    }
    open = nullptr;   // any other operator ends the group
    Step st;
    if (n == "Gather") {
      st.kind = Kind::kGather; st.slot = GetSingleArg<int>(op, "Child"); st.out = NewBuf(out_w);
      CHECK(state_width_ == 0 || state_width_ == out_w) << "Gather slots disagree on the state width";
      state_width_ = out_w;
      max_slots_ = std::max(max_slots_, st.slot + 1);
    } else if (n == "Pull") {
      CHECK(pull_buf < 0) << "one Pull per vertex function";
      st.kind = Kind::kPull; st.out = NewBuf(out_w); st.pull_offset = GetSingleArg<int>(op, "Offset");
      pull_width_ = out_w; pull_buf = st.out;
    } else if (n == "EmbeddingLookup") {
      st.kind = Kind::kEmbed; st.in = ref_of(op.input(0)); st.weight = ref_of(op.input(1));
      CHECK(st.in.buf == pull_buf && st.in.width == 1) << "EmbeddingLookup takes the pulled token id";
      CHECK(st.weight.buf < 0 && op.shape(0).dim_size() == 2);
      st.n = static_cast<int>(op.shape(0).dim(1));
      CHECK(st.weight.width % st.n == 0);
      st.vocab = st.weight.width / st.n;
      st.out = NewBuf(st.n);
    } else if (n == "Concat") {
      st.kind = Kind::kConcat;
      int total = 0;
      for (const auto& in : op.input()) { st.ins.push_back(ref_of(in)); CHECK(st.ins.back().buf >= 0); total += st.ins.back().width; }
      CHECK(total == out_w);
      st.out = NewBuf(out_w);
    } else if (n == "MatMul") {
      st.kind = Kind::kMatMul; st.in = ref_of(op.input(0)); st.weight = ref_of(op.input(1));
      CHECK(st.in.buf >= 0 && st.weight.buf < 0) << "MatMul multiplies a per-vertex row by a Variable";
      st.k = st.in.width; st.n = out_w;
      CHECK(st.weight.width == st.k * st.n) << "MatMul: the weight holds " << st.weight.width << " values, expected " << st.k << " x " << st.n;
      st.out = NewBuf(out_w);
    } else if (n == "Scatter") {
      st.kind = Kind::kScatter; st.in = ref_of(op.input(0));
      CHECK(st.in.buf >= 0);
      CHECK(state_width_ == 0 || state_width_ == st.in.width) << "Scatter and Gather disagree on the state width";
      state_width_ = st.in.width;
    } else if (n == "Push") {
      st.kind = Kind::kPush; st.in = ref_of(op.input(0));
      CHECK(st.in.buf >= 0 && out_width_ == 0);
      out_width_ = st.in.width;
    } else {
      LOG(FATAL) << "operator " << n << " is not supported inside a vertex function (fused LSTM / GRU engines aside, Node() may use "
                    "Gather, Pull, EmbeddingLookup, Slice, Reshape, Mirror, Expand_dims, Concat, MatMul, Add, Sub, Mul, Sigmoid, Tanh, "
                    "Relu, Scatter, Push)";
    }
    if (st.out >= 0) { Ref r; r.buf = st.out; r.width = bufs_[st.out].width; refs_[op.output(0)] = r; }
    steps_.push_back(st);
  }
  CHECK(out_width_ > 0) << "Node() must Push a tensor";
  CHECK(state_width_ > 0) << "Node() must Gather or Scatter a state";
  max_slots_ = std::max(max_slots_, 1);
  // Generate and compile the fused groups (and the lookup kernel, if used).
  for (size_t g = 0; g < groups_.size(); ++g) {
    Group& grp = *groups_[g];
    grp.desc.n_inputs = static_cast<int>(grp.inputs.size());
    grp.fwd_name = "generic_group" + std::to_string(g) + "_fwd";
    grp.bwd_name = "generic_group" + std::to_string(g) + "_bwd";
    grp.fwd_src = RTC::GenForward(grp.desc, grp.fwd_name);
    grp.bwd_src = RTC::GenBackward(grp.desc, grp.bwd_name);
    grp.fwd.Compile(grp.fwd_name, grp.fwd_src);
    grp.bwd.Compile(grp.bwd_name, grp.bwd_src);
  }
  for (const auto& st : steps_)
    if (st.kind == Kind::kEmbed && !embed_fwd_.compiled()) embed_fwd_.Compile("generic_embed_fwd", kEmbedFwdSource);
}

GenericFunction::~GenericFunction() {
  if (arena_) cudaFree(arena_);
  if (d_emb_idx_) cudaFree(d_emb_idx_);
  if (emb_scratch_) cudaFree(emb_scratch_);
}

void GenericFunction::Allocate() {
  if (allocated_) return;
  const size_t N = static_cast<size_t>(max_vertices_);
  // pass 1 sizes, pass 2 carves; the gradient arrays are contiguous so that one memset clears them
  for (int pass = 0; pass < 2; ++pass) {
    size_t used = 0;
    uint8_t* base = static_cast<uint8_t*>(arena_);
    auto take = [&](size_t floats) { float* p = base ? reinterpret_cast<float*>(base + used) : nullptr; used += Align(floats * sizeof(float)); return p; };
    for (auto& b : bufs_) b.val = take(N * b.width);
    mailbox_ = take(N * state_width_);
    out_val_ = take(N * out_width_);
    vin_ = take(N * std::max(pull_width_, 1));
    int max_w = 1;
    for (auto& g : groups_) max_w = std::max(max_w, g->desc.width);
    tmp_ = take(static_cast<size_t>(max_w));
    col_scratch_ = take(cavs_column_sum_scratch_bytes(max_w) / sizeof(float) + 4);
    d_fg_ = reinterpret_cast<int32_t*>(take(N * max_slots_));
    d_bs_ = reinterpret_cast<int32_t*>(take(N * max_slots_));
    d_fs_ = reinterpret_cast<int32_t*>(take(N));
    d_bg_ = reinterpret_cast<int32_t*>(take(N));
    d_t2j_ = reinterpret_cast<int32_t*>(take(N));
    grad_region_off_ = used;
    for (auto& b : bufs_) b.grad = take(N * b.width);
    dmail_ = take(N * state_width_);
    out_grad_ = take(N * out_width_);
    for (auto& g : groups_) {
      g->var_rows.resize(g->var_refs.size());
      for (size_t q = 0; q < g->var_refs.size(); ++q) g->var_rows[q] = take(N * g->desc.width);
    }
    grad_region_bytes_ = used - grad_region_off_;
    if (pass == 0) {
      MustCuda(cudaMalloc(&arena_, used), "generic function arenas");
      MustCuda(cudaMemset(arena_, 0, used), "generic function arenas");
    }
  }
  allocated_ = true;
}

void GenericFunction::Bind(float* params, float* grads) {
  params_ = params;
  grads_ = grads;
  Allocate();
}

float* GenericFunction::ValPtr(const Ref& r, long long row) const {
  if (r.buf < 0) return params_ + r.var_off;
  return bufs_[r.buf].val + row * bufs_[r.buf].width + r.col;
}
float* GenericFunction::GradPtr(const Ref& r, long long row) const {
  if (r.buf < 0) return grads_ + r.var_off;
  return bufs_[r.buf].grad + row * bufs_[r.buf].width + r.col;
}

void GenericFunction::LoadBatch(const int32_t* fg, const int32_t* fs, const int32_t* bg, const int32_t* bs, int n_slots,
                                const int32_t* t2j, int n, const std::vector<int32_t>& level_off, const float* vertex_input) {
  CHECK(params_ != nullptr) << "Bind() first";
  CHECK(n <= max_vertices_) << "batch of " << n << " vertices exceeds the declared maximum " << max_vertices_;
  CHECK(n_slots >= max_slots_) << "the vertex function gathers slot " << max_slots_ - 1 << " but the schedule has " << n_slots << " slots";
  n_ = n; n_slots_ = n_slots; level_off_ = level_off;
  MustCuda(cudaMemcpy(d_fg_, fg, sizeof(int32_t) * n * max_slots_, cudaMemcpyHostToDevice), "gather table");
  MustCuda(cudaMemcpy(d_bs_, bs, sizeof(int32_t) * n * max_slots_, cudaMemcpyHostToDevice), "gradient scatter table");
  MustCuda(cudaMemcpy(d_fs_, fs, sizeof(int32_t) * n, cudaMemcpyHostToDevice), "scatter table");
  MustCuda(cudaMemcpy(d_bg_, bg, sizeof(int32_t) * n, cudaMemcpyHostToDevice), "gradient gather table");
  MustCuda(cudaMemcpy(d_t2j_, t2j, sizeof(int32_t) * n, cudaMemcpyHostToDevice), "t2j");
  // a mailbox row that no vertex of this batch writes reads as zeros (the reference zero-fills, op_impl_graphop.cu:77-86)
  MustCuda(cudaMemset(mailbox_, 0, sizeof(float) * static_cast<size_t>(std::max(n, 1)) * state_width_), "mailbox");
  if (pull_width_ > 0) {
    CHECK(vertex_input != nullptr) << "the vertex function pulls its input: feed the vertex placeholder";
    MustCuda(cudaMemcpy(vin_, vertex_input, sizeof(float) * static_cast<size_t>(n) * pull_width_, cudaMemcpyHostToDevice), "vertex input");
  }
  // Segments of the embedding gradient: rows grouped by token (stable, so sums run in tensor-id order), chunks of at
  // most 256 rows; replaces the atomicAdd of BatchedSparseUpdate (op_impl_embedding_lookup.cu:91-103).
  for (const auto& st : steps_) {
    if (st.kind != Kind::kEmbed) continue;
    std::vector<int32_t> tok(n), order(n);
    for (int t = 0; t < n; ++t) {
      int id = static_cast<int>(vertex_input[static_cast<size_t>(t2j[t]) * pull_width_ + st.in.col]);
      tok[t] = (id < 0 || id >= st.vocab) ? 0 : id;
    }
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return tok[a] < tok[b]; });
    std::vector<int32_t> chunk_off, seg_first, seg_tok;
    for (int i = 0; i < n;) {
      int j = i;
      while (j < n && tok[order[j]] == tok[order[i]]) ++j;
      seg_first.push_back(static_cast<int32_t>(chunk_off.size()));
      seg_tok.push_back(tok[order[i]]);
      for (int b = i; b < j; b += kEmbedChunkRows) chunk_off.push_back(b);
      i = j;
    }
    seg_first.push_back(static_cast<int32_t>(chunk_off.size()));
    chunk_off.push_back(n);
    emb_chunks_ = static_cast<int>(chunk_off.size()) - 1;
    emb_segs_ = static_cast<int>(seg_tok.size());
    std::vector<int32_t> blob;
    blob.insert(blob.end(), order.begin(), order.end());
    blob.insert(blob.end(), chunk_off.begin(), chunk_off.end());
    blob.insert(blob.end(), seg_first.begin(), seg_first.end());
    blob.insert(blob.end(), seg_tok.begin(), seg_tok.end());
    if (blob.size() > emb_idx_cap_) {
      if (d_emb_idx_) cudaFree(d_emb_idx_);
      if (emb_scratch_) cudaFree(emb_scratch_);
      emb_idx_cap_ = 4 * static_cast<size_t>(max_vertices_) + 16;
      MustCuda(cudaMalloc(reinterpret_cast<void**>(&d_emb_idx_), emb_idx_cap_ * sizeof(int32_t)), "embedding gradient tables");
      MustCuda(cudaMalloc(reinterpret_cast<void**>(&emb_scratch_), (static_cast<size_t>(max_vertices_) + 1) * st.n * sizeof(float)), "embedding gradient scratch");
    }
    MustCuda(cudaMemcpy(d_emb_idx_, blob.data(), blob.size() * sizeof(int32_t), cudaMemcpyHostToDevice), "embedding gradient tables");
  }
}

void GenericFunction::RunLevel(int off, int rows) {
  for (auto& st : steps_) {
    switch (st.kind) {
      case Kind::kGather: {
        // out[b] = mailbox[child_slot(t)], zeros without a child (op_impl_graphop.cu:32-90)
        const int w = bufs_[st.out].width;
        Must(cavs_copy_rows_2d(bufs_[st.out].val + static_cast<size_t>(off) * w, w, nullptr, mailbox_, state_width_,
                               d_fg_ + static_cast<size_t>(st.slot) * n_ + off, rows, w, 0, nullptr), "Gather");
        break;
      }
      case Kind::kPull: {
        // out[b] = vertex_input[job id of t] (op_impl_graphop.cu:214-254)
        const int w = bufs_[st.out].width;
        Must(cavs_copy_rows_2d(bufs_[st.out].val + static_cast<size_t>(off) * w, w, nullptr, vin_ + st.pull_offset, pull_width_, d_t2j_ + off,
                               rows, w, 0, nullptr), "Pull");
        break;
      }
      case Kind::kEmbed: {
        int r = rows, vocab = st.vocab, E = st.n;
        long long o = off, pitch = bufs_[st.in.buf].width;
        const float* ids = bufs_[st.in.buf].val + st.in.col;
        const float* table = params_ + st.weight.var_off;
        float* out = bufs_[st.out].val;
        std::vector<void*> args = {&r, &o, &ids, &pitch, &table, &vocab, &E, &out};
        embed_fwd_.Launch(args, GridFor(static_cast<long long>(rows) * E), 256, nullptr);
        break;
      }
      case Kind::kConcat: {
        const int W = bufs_[st.out].width;
        int pos = 0;
        for (const auto& in : st.ins) {
          Must(cavs_copy_rows_2d(bufs_[st.out].val + static_cast<size_t>(off) * W + pos, W, nullptr, ValPtr(in, off), bufs_[in.buf].width, nullptr,
                                 rows, in.width, 0, nullptr), "Concat");
          pos += in.width;
        }
        break;
      }
      case Kind::kMatMul:
        // [rows, k] x [k, n] (cavs/backend/op_impl_blas3_cublas.cc:35-70)
        Must(cavs_gemm_f32(bufs_[st.out].val + static_cast<size_t>(off) * st.n, st.n, 0, ValPtr(st.in, off), bufs_[st.in.buf].width, 1,
                           params_ + st.weight.var_off, st.n, 1, rows, st.n, st.k, nullptr), "MatMul");
        break;
      case Kind::kGroup: {
        Group& g = *groups_[st.group];
        int r = rows; long long o = off;
        std::vector<const float*> in_ptr(g.inputs.size()), var_ptr(g.var_refs.size());
        std::vector<long long> pitch(g.inputs.size());
        std::vector<float*> out_ptr(g.out_bufs.size());
        std::vector<void*> args = {&r, &o};
        for (size_t j = 0; j < g.inputs.size(); ++j) {
          in_ptr[j] = bufs_[g.inputs[j].buf].val + g.inputs[j].col; pitch[j] = bufs_[g.inputs[j].buf].width;
          args.push_back(&in_ptr[j]); args.push_back(&pitch[j]);
        }
        for (size_t q = 0; q < g.var_refs.size(); ++q) { var_ptr[q] = params_ + g.var_refs[q].var_off; args.push_back(&var_ptr[q]); }
        for (size_t k = 0; k < g.out_bufs.size(); ++k) { out_ptr[k] = bufs_[g.out_bufs[k]].val; args.push_back(&out_ptr[k]); }
        g.fwd.Launch(args, GridFor(static_cast<long long>(rows) * g.desc.width), 256, nullptr);
        break;
      }
      case Kind::kScatter:
        // the state a parent will gather: mailbox[fs[t]] = row t (op_impl_graphop.cu:108-161); roots have no target
        Must(cavs_copy_rows_2d(mailbox_, state_width_, d_fs_ + off, ValPtr(st.in, off), bufs_[st.in.buf].width, nullptr, rows,
                               state_width_, 0, nullptr), "Scatter");
        break;
      case Kind::kPush:
        Must(cavs_copy_rows_2d(out_val_ + static_cast<size_t>(off) * out_width_, out_width_, nullptr, ValPtr(st.in, off),
                               bufs_[st.in.buf].width, nullptr, rows, out_width_, 0, nullptr), "Push");
        break;
    }
  }
}

void GenericFunction::Forward() {
  CHECK(n_ >= 0 && !level_off_.empty());
  for (size_t l = 0; l + 1 < level_off_.size(); ++l) RunLevel(level_off_[l], level_off_[l + 1] - level_off_[l]);
}

void GenericFunction::RunLevelBackward(int off, int rows) {
  for (auto it = steps_.rbegin(); it != steps_.rend(); ++it) {
    const Step& st = *it;
    switch (st.kind) {
      case Kind::kPush:     // Pull_grad of the output gradient (op_decl_graphop.cc:89-111)
        Must(cavs_copy_rows_2d(GradPtr(st.in, off), bufs_[st.in.buf].width, nullptr, out_grad_ + static_cast<size_t>(off) * out_width_, out_width_,
                               nullptr, rows, out_width_, 1, nullptr), "Push gradient");
        break;
      case Kind::kScatter:  // what the parent left for this vertex; zeros for roots (op_decl_graphop.cc:49-69)
        Must(cavs_copy_rows_2d(GradPtr(st.in, off), bufs_[st.in.buf].width, nullptr, dmail_, state_width_, d_bg_ + off, rows, state_width_, 1,
                               nullptr), "Scatter gradient");
        break;
      case Kind::kGroup: {
        Group& g = *groups_[st.group];
        int r = rows; long long o = off;
        const size_t ni = g.inputs.size(), nv = g.var_refs.size(), nk = g.out_bufs.size();
        std::vector<const float*> in_ptr(ni), var_ptr(nv), out_ptr(nk), gout_ptr(nk);
        std::vector<float*> gin_ptr(ni), vrow_ptr(nv);
        std::vector<long long> pitch(ni);
        std::vector<void*> args = {&r, &o};
        for (size_t j = 0; j < ni; ++j) {
          const Buf& b = bufs_[g.inputs[j].buf];
          in_ptr[j] = b.val + g.inputs[j].col; gin_ptr[j] = b.grad + g.inputs[j].col; pitch[j] = b.width;
          args.push_back(&in_ptr[j]); args.push_back(&pitch[j]); args.push_back(&gin_ptr[j]);
        }
        for (size_t q = 0; q < nv; ++q) {
          var_ptr[q] = params_ + g.var_refs[q].var_off; vrow_ptr[q] = g.var_rows[q];
          args.push_back(&var_ptr[q]); args.push_back(&vrow_ptr[q]);
        }
        for (size_t k = 0; k < nk; ++k) {
          out_ptr[k] = bufs_[g.out_bufs[k]].val; gout_ptr[k] = bufs_[g.out_bufs[k]].grad;
          args.push_back(&out_ptr[k]); args.push_back(&gout_ptr[k]);
        }
        g.bwd.Launch(args, GridFor(static_cast<long long>(rows) * g.desc.width), 256, nullptr);
        break;
      }
      case Kind::kMatMul:   // dX += dY W^T (op_decl_matmul.cc:21-31); dW is deferred
        Must(cavs_gemm_f32(GradPtr(st.in, off), bufs_[st.in.buf].width, 1, bufs_[st.out].grad + static_cast<size_t>(off) * st.n, st.n, 1,
                           params_ + st.weight.var_off, 1, st.n, rows, st.k, st.n, nullptr), "MatMul gradient");
        break;
      case Kind::kConcat: { // every input takes its columns of the output gradient (op_decl_slice_join.cc:80-98)
        const int W = bufs_[st.out].width;
        int pos = 0;
        for (const auto& in : st.ins) {
          Must(cavs_copy_rows_2d(GradPtr(in, off), bufs_[in.buf].width, nullptr, bufs_[st.out].grad + static_cast<size_t>(off) * W + pos, W, nullptr,
                                 rows, in.width, 1, nullptr), "Concat gradient");
          pos += in.width;
        }
        break;
      }
      case Kind::kGather: { // Scatter(Child = slot) of the gathered state's gradient to the child's row (op_decl_graphop.cc:25-41)
        const int w = bufs_[st.out].width;
        Must(cavs_copy_rows_2d(dmail_, state_width_, d_bs_ + static_cast<size_t>(st.slot) * n_ + off, bufs_[st.out].grad + static_cast<size_t>(off) * w,
                               w, nullptr, rows, w, 0, nullptr), "Gather gradient");
        break;
      }
      case Kind::kEmbed:
      case Kind::kPull:
        break;
    }
  }
}

void GenericFunction::Backward() {
  // every gradient array starts at zero except d(output), which the loss head has just written
  uint8_t* base = static_cast<uint8_t*>(arena_) + grad_region_off_;
  uint8_t* keep = reinterpret_cast<uint8_t*>(out_grad_);
  MustCuda(cudaMemsetAsync(base, 0, static_cast<size_t>(keep - base), nullptr), "zero gradients");
  uint8_t* after = keep + Align(static_cast<size_t>(max_vertices_) * out_width_ * sizeof(float));
  MustCuda(cudaMemsetAsync(after, 0, grad_region_bytes_ - static_cast<size_t>(after - base), nullptr), "zero gradients");
  for (int l = static_cast<int>(level_off_.size()) - 2; l >= 0; --l) RunLevelBackward(level_off_[l], level_off_[l + 1] - level_off_[l]);
  // Deferred gradients over all rows at once (cavs/midend/batch_weight_updater.h:10-85).
  for (const auto& st : steps_) {
    if (st.kind == Kind::kMatMul) {
      // dW += X^T dY (op_decl_matmul.cc:33-43): A = X transposed through strides
      Must(cavs_gemm_f32(grads_ + st.weight.var_off, st.n, 1, ValPtr(st.in, 0), 1, bufs_[st.in.buf].width, bufs_[st.out].grad, st.n, 1, st.k, st.n,
                         n_, nullptr), "MatMul weight gradient");
    } else if (st.kind == Kind::kGroup) {
      Group& g = *groups_[st.group];
      for (size_t q = 0; q < g.var_refs.size(); ++q) {
        const int w = g.desc.width;
        Must(cavs_column_sum(tmp_, g.var_rows[q], 0, w, n_, w, col_scratch_, nullptr), "bias gradient");
        if (g.var_refs[q].width == 1) {   // a scalar variable takes the sum over columns too
          Must(cavs_column_sum(tmp_, tmp_, 0, 1, w, 1, col_scratch_, nullptr), "scalar gradient");
          Must(cavs_axpy(grads_ + g.var_refs[q].var_off, tmp_, 1, 1.0f, nullptr), "scalar gradient");
        } else {
          Must(cavs_axpy(grads_ + g.var_refs[q].var_off, tmp_, static_cast<size_t>(w), 1.0f, nullptr), "bias gradient");
        }
      }
    } else if (st.kind == Kind::kEmbed && n_ > 0) {
      const int32_t* order = d_emb_idx_;
      const int32_t* chunk_off = order + n_;
      const int32_t* seg_first = chunk_off + emb_chunks_ + 1;
      const int32_t* seg_tok = seg_first + emb_segs_ + 1;
      Must(cavs_embed_bwd_segmented(grads_ + st.weight.var_off, bufs_[st.out].grad, order, chunk_off, emb_chunks_, seg_first, seg_tok, emb_segs_,
                                    emb_scratch_, st.n, nullptr), "embedding gradient");
    }
  }
}

}  // namespace midend
