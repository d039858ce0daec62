// Graph-op tests written against the reference's operator interface (OpDef -> CreateOp ->
// OpImpl::Compute(OpContext*)), in the style of the reference's own *_test.cc executables.
//
//   graph_ops_test cpu   registry, gradient pairing and the scheduler facade (no CUDA call)
//   graph_ops_test gpu   Gather / Scatter / Pull / Push / FunctionPopRet on a device, compared
//                        bit-for-bit with the CPU oracle's row ops driven by the same lists; the fused
//                        TreeLSTMCell / TreeLSTMCell_grad operators against a host restatement
//
// Links the product host library and the test oracle (oracle/libcavs_oracle.so).
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <vector>

#include "cavs/backend/op_decl.h"
#include "cavs/backend/op_impl.h"
#include "cavs/midend/graph_scheduler.h"
#include "cavs/util/op_def_builder.h"

extern "C" {
int cavs_oracle_schedule_stream(const int* parents, int batch, int max_len, int* out, int capacity);
int cavs_oracle_serial_stream(const int* parents, int batch, int max_len, int* out, int capacity);
void cavs_oracle_gather_rows(float* out, const float* inp, const int* ids, int n_ids, int row);
void cavs_oracle_scatter_rows(float* out, const int* ids, const float* inp, int n_ids, int row);
void cavs_oracle_zero_rows(float* out, int n_ids, int row);
}

using backend::CreateOp;
using backend::OpImpl;
using midend::BatchGraphScheduler;
using midend::OpContext;
using midend::SerialGraphScheduler;
using midend::Tensor;
using midend::TensorShape;

static int g_failures = 0;
#define EXPECT(cond)                                                          \
  do {                                                                        \
    if (!(cond)) { std::printf("FAILED %s:%d  %s\n", __FILE__, __LINE__, #cond); ++g_failures; } \
  } while (0)

// Tree A (2 leaves) and tree B (3 leaves): level 1 mixes A's root with B's inner vertex, the case
// where the reference's compact lists shift rows.
static const int kSkew[2][5] = {{2, 2, -1, -1, -1}, {3, 3, 4, 4, -1}};
static const int kBatch = 2, kMaxLen = 5;

static OpDef GraphOp(const char* name, int child, const std::vector<int>& shape, bool source) {
  OpDefBuilder b(name);
  if (source) b.Output(std::string(name) + "_out").Shape(shape);
  else b.Input(std::string(name) + "_in").Output(std::string(name) + "_out").Shape(shape);
  if (child >= 0) b.AttrSingle("Child", child);
  return b.Device("GPU").Finalize();
}

static void TestRegistryAndDecls() {
  for (const char* name : {"Gather", "Scatter", "Pull", "Push", "FunctionPushArg", "FunctionPopRet"}) {
    OpDef def = GraphOp(name, 0, {4}, false);
    if (std::string(name) == "Gather") def = GraphOp(name, 0, {4}, true);
    std::unique_ptr<OpImpl> op(CreateOp(def));
    EXPECT(op != nullptr);
    if (op) EXPECT(op->name() == name);
  }
  OpDef unknown = OpDefBuilder("NoSuchOp").Device("GPU").Finalize();
  EXPECT(CreateOp(unknown) == nullptr);
  OpDef cpu_gather = OpDefBuilder("Gather").Output("g").Shape(std::vector<int>{4}).AttrSingle("Child", 0).Device("CPU").Finalize();
  EXPECT(CreateOp(cpu_gather) == nullptr);   // GPU only, like the reference

  // Gather(Child=1) <-> Scatter(Child=1)
  OpDef gather = GraphOp("Gather", 1, {8}, true);
  std::vector<OpDef> g = backend::MakeGradient(gather);
  EXPECT(g.size() == 1 && g[0].name() == "Scatter");
  EXPECT(g[0].input(0) == GetGradientName("Gather_out"));
  EXPECT(GetSingleArg<int>(g[0], "Child") == 1);
  OpDef scatter = GraphOp("Scatter", 0, {8}, false);
  g = backend::MakeGradient(scatter);
  EXPECT(g.size() == 1 && g[0].name() == "Gather" && g[0].output(0) == GetGradientName("Scatter_in"));
  EXPECT(g[0].shape(0).dim(0) == 8 && GetSingleArg<int>(g[0], "Child") == 0);
  // Pull <-> Push
  g = backend::MakeGradient(GraphOp("Pull", -1, {1}, true));
  EXPECT(g.size() == 1 && g[0].name() == "Push");
  g = backend::MakeGradient(GraphOp("Push", -1, {6}, false));
  EXPECT(g.size() == 1 && g[0].name() == "Pull" && g[0].shape(0).dim(0) == 6);
  // GraphOutput -> GraphOutput_grad over the variables it closes over
  OpDef go = OpDefBuilder("GraphOutput").Input("graph").Input("x").Input("W").Output("y").Shape({-1, 6}).Device("GPU").Finalize();
  g = backend::MakeGradient(go);
  EXPECT(g.size() == 1 && g[0].name() == "GraphOutput_grad" && g[0].input_size() == 3 && g[0].output_size() == 2);
  EXPECT(g[0].output(1) == "W_grad");
  std::vector<TensorShapeDef> shp = backend::ShapeInference(gather, {});
  EXPECT(shp.size() == 1 && shp[0].dim(0) == 8);
}

// Walks the facade like GraphStatement::Run / GraphGradStatement::Run and rebuilds the oracle's
// schedule stream from what the accessors return.
static void TestSchedulerFacade() {
  Tensor graph("graph", CPU, DT_INT32, TensorShape({kBatch, kMaxLen}), const_cast<int*>(&kSkew[0][0]));
  BatchGraphScheduler gs;
  const int total = gs.LoadGraph(graph);
  std::vector<int> offs, body;
  auto put = [&body](const std::vector<int>& v) { body.push_back((int)v.size()); body.insert(body.end(), v.begin(), v.end()); };
  int levels = 0, sched = 0;
  gs.Initialize();
  while (!gs.Terminate()) {
    offs.push_back(gs.GetCurrentRoundOffset());
    sched = gs.GetCurrentRoundOffset() + (int)gs.GetJobId().size();
    put(gs.GetJobId());
    put(gs.CurrentRoundTensorIdsForGather(0));
    put(gs.CurrentRoundTensorIdsForGather(1));
    put(gs.CurrentRoundTensorIdsForScatter(0));
    put(gs.CurrentRoundTensorIdsForGatherInitialization());
    gs.ActivateNext();
    ++levels;
  }
  offs.push_back(sched);
  body.insert(body.end(), gs.TensorIdsToJobIds().begin(), gs.TensorIdsToJobIds().end());
  gs.ReverseGraph();
  gs.Initialize();
  while (!gs.Terminate()) {
    body.push_back(gs.GetCurrentRoundOffset());
    put(gs.GetJobId());
    put(gs.CurrentRoundTensorIdsForGather(0));
    put(gs.CurrentRoundTensorIdsForScatter(0));
    put(gs.CurrentRoundTensorIdsForScatter(1));
    put(gs.CurrentRoundTensorIdsForGatherInitialization());
    gs.ActivateNext();
  }
  std::vector<int> mine = {total, levels};
  mine.insert(mine.end(), offs.begin(), offs.end());
  mine.insert(mine.end(), body.begin(), body.end());
  std::vector<int> want(4096);
  const int n = cavs_oracle_schedule_stream(&kSkew[0][0], kBatch, kMaxLen, want.data(), (int)want.size());
  EXPECT(n == (int)mine.size());
  EXPECT(n > 0 && std::memcmp(want.data(), mine.data(), sizeof(int) * mine.size()) == 0);
}

// The same walk over the one-vertex-per-round scheduler, against the oracle's serial stream.  The
// second batch holds a single-vertex sample in the middle: the forward sweep ends there, the backward
// sweep (which admits a new sample at every leaf) does not.
static const int kHole[3][5] = {{2, 2, -1, -1, -1}, {-1, -1, -1, -1, -1}, {3, 3, 4, 4, -1}};
static void SerialFacadeCase(const int* parents, int batch) {
  Tensor graph("graph", CPU, DT_INT32, TensorShape({batch, kMaxLen}), const_cast<int*>(parents));
  SerialGraphScheduler gs;
  const int total = gs.LoadGraph(graph);
  std::vector<int> mine = {total, 0};
  auto put = [&mine](const std::vector<int>& v) { mine.push_back((int)v.size()); mine.insert(mine.end(), v.begin(), v.end()); };
  int rounds = 0;
  gs.Initialize();
  while (!gs.Terminate()) {
    EXPECT(gs.GetJobId().size() == 1);
    mine.push_back(gs.GetCurrentRoundOffset());
    put(gs.CurrentRoundTensorIdsForGather(0));
    put(gs.CurrentRoundTensorIdsForGather(1));
    put(gs.CurrentRoundTensorIdsForScatter(0));
    put(gs.CurrentRoundTensorIdsForGatherInitialization());
    EXPECT(gs.HasChild(gs.GetJobId()[0]) == !gs.CurrentRoundTensorIdsForGather(0).empty());
    gs.ActivateNext();
    ++rounds;
  }
  mine[1] = rounds;
  mine.insert(mine.end(), gs.TensorIdsToJobIds().begin(), gs.TensorIdsToJobIds().end());
  const size_t at = mine.size();
  mine.push_back(0);
  rounds = 0;
  gs.ReverseGraph();
  gs.Initialize();
  while (!gs.Terminate()) {
    mine.push_back(gs.GetCurrentRoundOffset());
    put(gs.CurrentRoundTensorIdsForGather(0));
    put(gs.CurrentRoundTensorIdsForScatter(0));
    put(gs.CurrentRoundTensorIdsForScatter(1));
    put(gs.CurrentRoundTensorIdsForGatherInitialization());
    gs.ActivateNext();
    ++rounds;
  }
  mine[at] = rounds;
  std::vector<int> want(4096);
  const int n = cavs_oracle_serial_stream(parents, batch, kMaxLen, want.data(), (int)want.size());
  EXPECT(n == (int)mine.size());
  EXPECT(n > 0 && std::memcmp(want.data(), mine.data(), sizeof(int) * mine.size()) == 0);
}
static void TestSerialSchedulerFacade() {
  SerialFacadeCase(&kSkew[0][0], kBatch);
  SerialFacadeCase(&kHole[0][0], 3);
}

static std::vector<float> ToHost(const Tensor& t, size_t elems) {
  std::vector<float> h(elems);
  cudaMemcpy(h.data(), t.data<float>(), elems * sizeof(float), cudaMemcpyDeviceToHost);
  return h;
}

// One forward sweep of a toy vertex function y = g0 + 2*g1 + x (combined on the host) through the
// real operators, against the same sweep done with the oracle's row ops on the host.
static void TestGraphOpsOnDevice(bool aligned) {
  const int W = 12;   // mailbox row width (floats)
  Tensor graph("graph", CPU, DT_INT32, TensorShape({kBatch, kMaxLen}), const_cast<int*>(&kSkew[0][0]));
  BatchGraphScheduler gs;
  gs.SetAlignedTables(aligned);
  const int total = gs.LoadGraph(graph);
  const int cap = kBatch * kMaxLen;

  // Arenas [cap, W]; per-vertex tensors are dynamic, the vertex input is job-ordered.
  auto arena = [&](const char* name) { Tensor t(name, GPU, DT_FLOAT, TensorShape({cap, W})); t.SetAsDynamic(); return t; };
  Tensor mailbox = arena("mailbox"), g0 = arena("g0"), g1 = arena("g1"), xin = arena("x"), y = arena("y"), pushed = arena("pushed");
  Tensor func_arg("arg", GPU, DT_FLOAT, TensorShape({cap, W}));
  Tensor graph_out("out", GPU, DT_FLOAT, TensorShape({cap, W}));
  std::vector<float> h_arg((size_t)cap * W);
  for (size_t i = 0; i < h_arg.size(); i++) h_arg[i] = 0.25f * (float)((i * 2654435761u) % 97) - 3.0f;
  cudaMemcpy(func_arg.mutable_data<float>(), h_arg.data(), h_arg.size() * sizeof(float), cudaMemcpyHostToDevice);
  gs.SetMessagePasser(mailbox);

  std::unique_ptr<OpImpl> gather0(CreateOp(GraphOp("Gather", 0, {W}, true))), gather1(CreateOp(GraphOp("Gather", 1, {W}, true)));
  std::unique_ptr<OpImpl> pull(CreateOp(GraphOp("Pull", -1, {W}, true))), scatter(CreateOp(GraphOp("Scatter", 0, {W}, false)));
  std::unique_ptr<OpImpl> push(CreateOp(GraphOp("Push", -1, {W}, false)));
  std::unique_ptr<OpImpl> pusharg(CreateOp(GraphOp("FunctionPushArg", -1, {W}, false))), popret(CreateOp(GraphOp("FunctionPopRet", -1, {W}, false)));
  auto ctx = [&](std::vector<const Tensor*> in, std::vector<Tensor*> out) {
    std::unique_ptr<OpContext> c(new OpContext());
    for (auto* t : in) c->AppendInput(t);
    for (auto* t : out) c->AppendOutput(t);
    c->SetGraphScheduler(&gs);
    return c;
  };
  auto c_g0 = ctx({}, {&g0}), c_g1 = ctx({}, {&g1}), c_pull = ctx({}, {&xin}), c_sc = ctx({&y}, {&mailbox}), c_push = ctx({&y}, {&pushed});
  auto c_arg = ctx({&func_arg}, {}), c_ret = ctx({}, {&graph_out});

  // Host model of the same sweep with the oracle's row ops.
  std::vector<float> m_mail((size_t)cap * W, 0.f), m_g0((size_t)cap * W, 0.f), m_g1((size_t)cap * W, 0.f), m_x((size_t)cap * W, 0.f),
      m_y((size_t)cap * W, 0.f), m_out((size_t)cap * W, 0.f);

  pusharg->Compute(c_arg.get());
  gs.Initialize();
  while (!gs.Terminate()) {
    const int off = gs.GetCurrentRoundOffset(), rows = (int)gs.GetJobId().size();
    for (OpContext* c : {c_g0.get(), c_g1.get(), c_pull.get(), c_sc.get(), c_push.get()}) c->SetTensorOffset();
    gather0->Compute(c_g0.get());
    gather1->Compute(c_g1.get());
    pull->Compute(c_pull.get());
    // oracle side of the three source ops
    for (int c = 0; c < 2; c++) {
      std::vector<float>& mg = c == 0 ? m_g0 : m_g1;
      const std::vector<int>& ids = gs.CurrentRoundTensorIdsForGather(c);
      if (aligned) {
        // row b pairs with its own slot-c child: rebuild the padded list from the compact one
        // by walking the level (children exist exactly for the first |ids| jobs that own the slot).
        std::vector<float> tmp((size_t)rows * W, 0.f);
        // The facade's aligned device list is what the product used; model it from the schedule:
        // a job owns slot c iff it has > c children, which for this batch is read off the parent array.
        int k = 0;
        for (int b = 0; b < rows; b++) {
          const int job = gs.GetJobId()[b];
          int n_child = 0;
          const int sample = job < 3 ? 0 : 1, base = sample == 0 ? 0 : 3, len = sample == 0 ? 3 : 5;
          for (int j = 0; j < len; j++) if (kSkew[sample][j] == job - base) n_child++;
          if (c < n_child) { std::memcpy(&tmp[(size_t)b * W], &m_mail[(size_t)ids[k] * W], W * sizeof(float)); k++; }
        }
        std::memcpy(&mg[(size_t)off * W], tmp.data(), tmp.size() * sizeof(float));
      } else if (!ids.empty()) {
        cavs_oracle_gather_rows(&mg[(size_t)off * W], m_mail.data(), ids.data(), (int)ids.size(), W);
      } else {
        cavs_oracle_zero_rows(&mg[(size_t)off * W], (int)gs.CurrentRoundTensorIdsForGatherInitialization().size(), W);
      }
    }
    cavs_oracle_gather_rows(&m_x[(size_t)off * W], h_arg.data(), gs.GetJobId().data(), rows, W);
    // toy vertex function on the host, from the DEVICE results of the source ops
    std::vector<float> d_g0 = ToHost(g0, (size_t)rows * W), d_g1 = ToHost(g1, (size_t)rows * W), d_x = ToHost(xin, (size_t)rows * W);
    EXPECT(std::memcmp(d_g0.data(), &m_g0[(size_t)off * W], d_g0.size() * sizeof(float)) == 0);
    EXPECT(std::memcmp(d_g1.data(), &m_g1[(size_t)off * W], d_g1.size() * sizeof(float)) == 0);
    EXPECT(std::memcmp(d_x.data(), &m_x[(size_t)off * W], d_x.size() * sizeof(float)) == 0);
    std::vector<float> hy((size_t)rows * W);
    for (size_t i = 0; i < hy.size(); i++) hy[i] = d_g0[i] + 2.0f * d_g1[i] + d_x[i];
    std::memcpy(&m_y[(size_t)off * W], hy.data(), hy.size() * sizeof(float));
    y.ScaleDynamicDimension(rows);
    cudaMemcpy(y.mutable_data<float>(), hy.data(), hy.size() * sizeof(float), cudaMemcpyHostToDevice);
    scatter->Compute(c_sc.get());
    push->Compute(c_push.get());
    // oracle side of Scatter
    const std::vector<int>& sids = gs.CurrentRoundTensorIdsForScatter(0);
    if (aligned) {
      int k = 0;
      for (int b = 0; b < rows; b++) {
        const int job = gs.GetJobId()[b];
        const bool root = (job == 2 || job == 7);
        if (!root) { std::memcpy(&m_mail[(size_t)sids[k] * W], &hy[(size_t)b * W], W * sizeof(float)); k++; }
      }
    } else if (!sids.empty()) {
      cavs_oracle_scatter_rows(m_mail.data(), sids.data(), hy.data(), (int)sids.size(), W);
    }
    gs.ActivateNext();
  }
  for (OpContext* c : {c_g0.get(), c_g1.get(), c_pull.get(), c_sc.get(), c_push.get()}) c->ResetTensorOffset();
  popret->Compute(c_ret.get());
  cavs_oracle_scatter_rows(m_out.data(), gs.TensorIdsToJobIds().data(), m_y.data(), total, W);
  cudaDeviceSynchronize();
  mailbox.SetOffsetWithId(0);
  std::vector<float> d_mail = ToHost(mailbox, (size_t)cap * W), d_out = ToHost(graph_out, (size_t)cap * W);
  EXPECT(std::memcmp(d_mail.data(), m_mail.data(), d_mail.size() * sizeof(float)) == 0);
  EXPECT(std::memcmp(d_out.data(), m_out.data(), (size_t)total * W * sizeof(float)) == 0);
  EXPECT(cudaGetLastError() == cudaSuccess);
}

// The forward sweep of the same toy vertex function, one vertex per round (tensor id == job id), with the
// reference's compact one-entry lists.
static void TestSerialOpsOnDevice() {
  const int W = 12;
  Tensor graph("graph", CPU, DT_INT32, TensorShape({kBatch, kMaxLen}), const_cast<int*>(&kSkew[0][0]));
  SerialGraphScheduler gs;
  const int total = gs.LoadGraph(graph);
  const int cap = kBatch * kMaxLen;
  auto arena = [&](const char* name) { Tensor t(name, GPU, DT_FLOAT, TensorShape({cap, W})); t.SetAsDynamic(); return t; };
  Tensor mailbox = arena("mailbox"), g0 = arena("g0"), g1 = arena("g1"), xin = arena("x"), y = arena("y"), pushed = arena("pushed");
  Tensor func_arg("arg", GPU, DT_FLOAT, TensorShape({cap, W}));
  Tensor graph_out("out", GPU, DT_FLOAT, TensorShape({cap, W}));
  std::vector<float> h_arg((size_t)cap * W);
  for (size_t i = 0; i < h_arg.size(); i++) h_arg[i] = 0.125f * (float)((i * 2246822519u) % 89) - 5.0f;
  cudaMemcpy(func_arg.mutable_data<float>(), h_arg.data(), h_arg.size() * sizeof(float), cudaMemcpyHostToDevice);
  gs.SetMessagePasser(mailbox);
  std::unique_ptr<OpImpl> gather0(CreateOp(GraphOp("Gather", 0, {W}, true))), gather1(CreateOp(GraphOp("Gather", 1, {W}, true)));
  std::unique_ptr<OpImpl> pull(CreateOp(GraphOp("Pull", -1, {W}, true))), scatter(CreateOp(GraphOp("Scatter", 0, {W}, false)));
  std::unique_ptr<OpImpl> push(CreateOp(GraphOp("Push", -1, {W}, false)));
  std::unique_ptr<OpImpl> pusharg(CreateOp(GraphOp("FunctionPushArg", -1, {W}, false))), popret(CreateOp(GraphOp("FunctionPopRet", -1, {W}, false)));
  auto ctx = [&](std::vector<const Tensor*> in, std::vector<Tensor*> out) {
    std::unique_ptr<OpContext> c(new OpContext());
    for (auto* t : in) c->AppendInput(t);
    for (auto* t : out) c->AppendOutput(t);
    c->SetGraphScheduler(&gs);
    return c;
  };
  auto c_g0 = ctx({}, {&g0}), c_g1 = ctx({}, {&g1}), c_pull = ctx({}, {&xin}), c_sc = ctx({&y}, {&mailbox}), c_push = ctx({&y}, {&pushed});
  auto c_arg = ctx({&func_arg}, {}), c_ret = ctx({}, {&graph_out});
  std::vector<float> m_mail((size_t)cap * W, 0.f), m_y((size_t)cap * W, 0.f), m_out((size_t)cap * W, 0.f);

  pusharg->Compute(c_arg.get());
  int rounds = 0;
  gs.Initialize();
  while (!gs.Terminate()) {
    const int job = gs.GetCurrentRoundOffset();
    for (OpContext* c : {c_g0.get(), c_g1.get(), c_pull.get(), c_sc.get(), c_push.get()}) c->SetTensorOffset();
    gather0->Compute(c_g0.get());
    gather1->Compute(c_g1.get());
    pull->Compute(c_pull.get());
    std::vector<float> want[2] = {std::vector<float>(W, 0.f), std::vector<float>(W, 0.f)};
    for (int c = 0; c < 2; c++) {
      const std::vector<int>& ids = gs.CurrentRoundTensorIdsForGather(c);
      EXPECT(ids.size() <= 1);
      if (!ids.empty()) cavs_oracle_gather_rows(want[c].data(), m_mail.data(), ids.data(), 1, W);
    }
    std::vector<float> d_g0 = ToHost(g0, W), d_g1 = ToHost(g1, W), d_x = ToHost(xin, W);
    // a childless vertex zero-fills its gather outputs through the initialisation list; a vertex with
    // one child leaves the other slot's row as the allocator left it (zero: fresh arena)
    EXPECT(std::memcmp(d_g0.data(), want[0].data(), W * sizeof(float)) == 0);
    EXPECT(std::memcmp(d_g1.data(), want[1].data(), W * sizeof(float)) == 0);
    EXPECT(std::memcmp(d_x.data(), &h_arg[(size_t)job * W], W * sizeof(float)) == 0);
    std::vector<float> hy(W);
    for (int i = 0; i < W; i++) hy[i] = d_g0[i] + 2.0f * d_g1[i] + d_x[i];
    std::memcpy(&m_y[(size_t)job * W], hy.data(), W * sizeof(float));
    y.ScaleDynamicDimension(1);
    cudaMemcpy(y.mutable_data<float>(), hy.data(), W * sizeof(float), cudaMemcpyHostToDevice);
    scatter->Compute(c_sc.get());
    push->Compute(c_push.get());
    const std::vector<int>& sids = gs.CurrentRoundTensorIdsForScatter(0);
    if (!sids.empty()) cavs_oracle_scatter_rows(m_mail.data(), sids.data(), hy.data(), 1, W);
    gs.ActivateNext();
    ++rounds;
  }
  EXPECT(rounds == total);
  for (OpContext* c : {c_g0.get(), c_g1.get(), c_pull.get(), c_sc.get(), c_push.get()}) c->ResetTensorOffset();
  popret->Compute(c_ret.get());
  cavs_oracle_scatter_rows(m_out.data(), gs.TensorIdsToJobIds().data(), m_y.data(), total, W);
  cudaDeviceSynchronize();
  mailbox.SetOffsetWithId(0);
  std::vector<float> d_mail = ToHost(mailbox, (size_t)cap * W), d_out = ToHost(graph_out, (size_t)cap * W);
  EXPECT(std::memcmp(d_mail.data(), m_mail.data(), d_mail.size() * sizeof(float)) == 0);
  EXPECT(std::memcmp(d_out.data(), m_out.data(), (size_t)total * W * sizeof(float)) == 0);
  EXPECT(cudaGetLastError() == cudaSuccess);
}

// The fused cell operators: registration, shape inference and gradient definition (no CUDA call).
static OpDef FusedCellDef(int k) {
  OpDefBuilder b("TreeLSTMCell");
  b.Input("xW").Input("sU");
  for (int c = 0; c < k; ++c) b.Input("hUf" + std::to_string(c));
  for (int c = 0; c < k; ++c) b.Input("child" + std::to_string(c));
  b.Input("B").Output("hc").Output("gates").AttrSingle("Slots", k);
  return b.Device("GPU").Finalize();
}
static void TestFusedCellDecl() {
  const int K = 2, H = 6, n = 5;
  OpDef def = FusedCellDef(K);
  std::unique_ptr<OpImpl> op(CreateOp(def));
  EXPECT(op != nullptr);
  auto shape = [](int a, int b) { TensorShapeDef s; s.add_dim(a); s.add_dim(b); return s; };
  std::vector<TensorShapeDef> in = {shape(n, 4 * H), shape(n, 3 * H), shape(n, H), shape(n, H), shape(n, 2 * H), shape(n, 2 * H)};
  TensorShapeDef bias; bias.add_dim(4 * H); in.push_back(bias);
  std::vector<TensorShapeDef> out = backend::ShapeInference(def, in);
  EXPECT(out.size() == 2 && out[0].dim(0) == n && out[0].dim(1) == 2 * H && out[1].dim(1) == (3 + K) * H);
  std::vector<OpDef> g = backend::MakeGradient(def);
  EXPECT(g.size() == 1 && g[0].name() == GetGradientName("TreeLSTMCell"));
  EXPECT(g[0].input_size() == 3 + K && g[0].output_size() == 1 + 2 * K);
  EXPECT(g[0].input(0) == GetGradientName("hc") && g[0].input(1) == "gates" && g[0].input(3) == "child0");
  EXPECT(g[0].output(0) == GetGradientName("xW") && g[0].output(1) == GetGradientName("hUf0"));
  EXPECT(GetSingleArg<int>(g[0], "Slots") == K);
  std::unique_ptr<OpImpl> gop(CreateOp(g[0]));
  EXPECT(gop != nullptr);
}

// Forward and gradient of the fused cell on a device against a host restatement of
// apps/paper/tree-lstm-cavs.cc:150-171 and its gradient rules.
static void TestFusedCellOnDevice() {
  const int K = 2, H = 20, n = 7, G = (3 + K) * H;
  auto fill = [](std::vector<float>& v, unsigned seed, float scale) {
    for (size_t i = 0; i < v.size(); i++) { seed = seed * 1664525u + 1013904223u; v[i] = scale * ((float)(seed >> 8) / 8388608.0f - 1.0f); }
  };
  std::vector<float> hA((size_t)n * 4 * H), hP((size_t)n * 3 * H), hQ[2], hC[2], hB(4 * H), hD((size_t)n * 2 * H);
  fill(hA, 1, 1.0f); fill(hP, 2, 1.0f); fill(hB, 3, 0.3f); fill(hD, 4, 0.5f);
  for (int c = 0; c < K; c++) { hQ[c].resize((size_t)n * H); hC[c].resize((size_t)n * 2 * H); fill(hQ[c], 10 + c, 1.0f); fill(hC[c], 20 + c, 1.0f); }
  auto dev = [&](const char* name, std::vector<int> shape, const std::vector<float>* src) {
    Tensor t(name, GPU, DT_FLOAT, TensorShape(shape));
    if (src) cudaMemcpy(t.mutable_data<float>(), src->data(), src->size() * sizeof(float), cudaMemcpyHostToDevice);
    return t;
  };
  Tensor A = dev("xW", {n, 4 * H}, &hA), P = dev("sU", {n, 3 * H}, &hP), B = dev("B", {4 * H}, &hB), D = dev("d_hc", {n, 2 * H}, &hD);
  Tensor Q0 = dev("q0", {n, H}, &hQ[0]), Q1 = dev("q1", {n, H}, &hQ[1]), C0 = dev("c0", {n, 2 * H}, &hC[0]), C1 = dev("c1", {n, 2 * H}, &hC[1]);
  Tensor hc = dev("hc", {n, 2 * H}, nullptr), gates = dev("gates", {n, G}, nullptr);
  Tensor dA = dev("dA", {n, 4 * H}, nullptr), zf0 = dev("zf0", {n, H}, nullptr), zf1 = dev("zf1", {n, H}, nullptr);
  Tensor dc0 = dev("dc0", {n, H}, nullptr), dc1 = dev("dc1", {n, H}, nullptr);
  OpDef def = FusedCellDef(K);
  std::unique_ptr<OpImpl> op(CreateOp(def)), gop(CreateOp(backend::MakeGradient(def)[0]));
  OpContext fwd, bwd;
  for (const Tensor* t : {&A, &P, &Q0, &Q1, &C0, &C1, &B}) fwd.AppendInput(t);
  fwd.AppendOutput(&hc); fwd.AppendOutput(&gates);
  for (const Tensor* t : {&D, &gates, &hc, &C0, &C1}) bwd.AppendInput(t);
  for (Tensor* t : {&dA, &zf0, &zf1, &dc0, &dc1}) bwd.AppendOutput(t);
  op->Compute(&fwd);
  gop->Compute(&bwd);
  EXPECT(cudaDeviceSynchronize() == cudaSuccess);
  auto host = [&](const Tensor& t) { std::vector<float> v(t.count()); cudaMemcpy(v.data(), t.data<float>(), v.size() * sizeof(float), cudaMemcpyDeviceToHost); return v; };
  std::vector<float> g_hc = host(hc), g_dA = host(dA), g_zf[2] = {host(zf0), host(zf1)}, g_dc[2] = {host(dc0), host(dc1)};
  auto sig = [](float x) { return 1.0f / (1.0f + std::exp(-x)); };
  // max-norm relative error over everything compared (the contract of the fp32 configurations)
  double max_diff = 0, max_want = 0;
  auto cmp = [&](float got, float want) {
    max_diff = std::fmax(max_diff, std::fabs((double)got - want));
    max_want = std::fmax(max_want, std::fabs((double)want));
  };
  for (int b = 0; b < n; b++)
    for (int j = 0; j < H; j++) {
      const float* a = &hA[(size_t)b * 4 * H];
      const float* p = &hP[(size_t)b * 3 * H];
      float gi = sig((a[j] + p[j]) + hB[j]), go = sig((a[H + j] + p[H + j]) + hB[3 * H + j]);
      float gu = std::tanh((a[2 * H + j] + p[2 * H + j]) + hB[2 * H + j]);
      float gf[2], cc = gi * gu;
      for (int c = 0; c < K; c++) { gf[c] = sig((a[3 * H + j] + hQ[c][(size_t)b * H + j]) + hB[H + j]); cc = cc + gf[c] * hC[c][(size_t)b * 2 * H + H + j]; }
      float th = std::tanh(cc);
      cmp(g_hc[(size_t)b * 2 * H + j], go * th);
      cmp(g_hc[(size_t)b * 2 * H + H + j], cc);
      float dh = hD[(size_t)b * 2 * H + j], mc = hD[(size_t)b * 2 * H + H + j];
      float dc = mc + (dh * go) * (1.0f - th * th);
      float zfs = 0;
      for (int c = 0; c < K; c++) {
        float z = (dc * hC[c][(size_t)b * 2 * H + H + j]) * gf[c] * (1.0f - gf[c]);
        zfs += z;
        cmp(g_zf[c][(size_t)b * H + j], z);
        cmp(g_dc[c][(size_t)b * H + j], dc * gf[c]);
      }
      cmp(g_dA[(size_t)b * 4 * H + j], (dc * gu) * gi * (1.0f - gi));
      cmp(g_dA[(size_t)b * 4 * H + H + j], (dh * th) * go * (1.0f - go));
      cmp(g_dA[(size_t)b * 4 * H + 2 * H + j], (dc * gi) * (1.0f - gu * gu));
      cmp(g_dA[(size_t)b * 4 * H + 3 * H + j], zfs);
    }
  EXPECT(max_want > 0.1 && max_diff / max_want < 1e-5);
}

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "cpu";
  TestRegistryAndDecls();
  TestFusedCellDecl();
  TestSchedulerFacade();
  TestSerialSchedulerFacade();
  if (mode == "gpu") {
    TestGraphOpsOnDevice(false);   // the reference's positional lists
    TestGraphOpsOnDevice(true);    // aligned lists
    TestSerialOpsOnDevice();
    TestFusedCellOnDevice();
  }
  if (g_failures == 0) std::printf("graph_ops_test %s: ok\n", mode.c_str());
  return g_failures == 0 ? 0 : 1;
}
