// Stand-alone vertex-function operators (MatMul, Add / Sub / Mul, Sigmoid / Tanh / Relu, Slice, Concat, Mirror)
// through the reference's operator interface: OpDef -> CreateOp -> OpImpl::Compute(OpContext*).
//
//   vertex_ops_test cpu   the operators are registered under the reference's keys, GPU only; the generated source of
//                         every elementwise kernel compiles for sm_100a (no CUDA call)
//   vertex_ops_test gpu   each operator on a device against a host computation of the cited reference semantics:
//                         copies bit-exact, elementwise within 2 ulp of libm, MatMul within 1e-5 of an fp64 product
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <random>
#include <vector>

#include "cavs/backend/cudaRTC_wrapper.h"
#include "cavs/backend/op_impl.h"
#include "cavs/midend/op_context.h"
#include "cavs/midend/runtime_compiler/code_generator.h"
#include "cavs/util/op_def_builder.h"

using backend::CreateOp;
using backend::OpImpl;
using midend::OpContext;
using midend::Tensor;
using midend::TensorShape;

static int g_failures = 0;
#define EXPECT(cond)                                                          \
  do {                                                                        \
    if (!(cond)) { std::printf("FAILED %s:%d  %s\n", __FILE__, __LINE__, #cond); ++g_failures; } \
  } while (0)

static const char* kNames[] = {"MatMul", "Add", "Sub", "Mul", "Sigmoid", "Tanh", "Relu", "Slice", "Concat", "Mirror"};

static OpDef Def(const char* name, int n_in, const std::vector<int>& shape) {
  OpDefBuilder b(name);
  for (int i = 0; i < n_in; ++i) b.Input(std::string(name) + "_in" + std::to_string(i));
  b.Output(std::string(name) + "_out").Shape(shape);
  return b.Device("GPU").Finalize();
}

static void TestRegistry() {
  for (const char* name : kNames) {
    const bool unary = !std::strcmp(name, "Sigmoid") || !std::strcmp(name, "Tanh") || !std::strcmp(name, "Relu") ||
                       !std::strcmp(name, "Slice") || !std::strcmp(name, "Mirror");
    OpDefBuilder b(name);
    b.Input("a");
    if (!unary) b.Input("b");
    b.Output("y").Shape(std::vector<int>{4});
    if (!std::strcmp(name, "Slice")) b.AttrSingle("Offset", 0).AttrSingle("Stride", 4);
    std::unique_ptr<OpImpl> op(CreateOp(b.Device("GPU").Finalize()));
    EXPECT(op != nullptr);
    if (op) EXPECT(op->name() == name);
    OpDefBuilder c(name);
    c.Input("a").Output("y").Shape(std::vector<int>{4});
    EXPECT(CreateOp(c.Device("CPU").Finalize()) == nullptr);   // GPU only, like the reference
  }
  for (const char* name : {"Add", "Sub", "Mul", "Sigmoid", "Tanh", "Relu"}) {
    const std::string kname = std::string("k_") + name;
    const std::string src = midend::RTC::GenStandalone(name, kname);
    EXPECT(src.find("extern \"C\" __global__ void " + kname) != std::string::npos);
    RTC::CudaRTCWrapper w;
    w.Compile(kname, src);     // NVRTC only: runs without a GPU
    EXPECT(w.compiled() && w.cubin_bytes() > 0);
  }
}

namespace {
struct Dev {
  Tensor t;
  Dev(const char* name, const std::vector<int>& shape, const std::vector<float>* src, bool dynamic)
      : t(name, GPU, DT_FLOAT, TensorShape(shape)) {
    if (dynamic) t.SetAsDynamic();
    if (src) cudaMemcpy(t.mutable_data<float>(), src->data(), src->size() * sizeof(float), cudaMemcpyHostToDevice);
  }
  std::vector<float> host() const {
    std::vector<float> v(t.count());
    cudaMemcpy(v.data(), t.data<float>(), v.size() * sizeof(float), cudaMemcpyDeviceToHost);
    return v;
  }
};
std::vector<float> Random(size_t n, unsigned seed) {
  std::mt19937 rng(seed);
  std::normal_distribution<float> d(0.f, 1.f);
  std::vector<float> v(n);
  for (auto& x : v) x = d(rng);
  return v;
}
bool SameBits(const std::vector<float>& a, const std::vector<float>& b) {
  return a.size() == b.size() && std::memcmp(a.data(), b.data(), a.size() * sizeof(float)) == 0;
}
float UlpDiff(float a, float b) {
  if (a == b) return 0.f;
  const float scale = std::ldexp(1.0f, std::ilogb(std::fmax(std::fabs(a), std::fabs(b))) - 23);
  return std::fabs(a - b) / scale;
}
void Run(const OpDef& def, std::initializer_list<const Tensor*> in, Tensor* out) {
  std::unique_ptr<OpImpl> op(CreateOp(def));
  EXPECT(op != nullptr);
  if (!op) return;
  OpContext ctx;
  for (auto* t : in) ctx.AppendInput(t);
  ctx.AppendOutput(out);
  op->Compute(&ctx);
  EXPECT(cudaDeviceSynchronize() == cudaSuccess);
}
}  // namespace

static void TestElementwise() {
  const int rows = 37, W = 150;
  const std::vector<float> ha = Random(rows * W, 1), hb = Random(rows * W, 2), hrow = Random(W, 3), hs = {0.75f};
  Dev a("a", {rows, W}, &ha, true), b("b", {rows, W}, &hb, true), row("row", {W}, &hrow, false), s("s", {1}, &hs, false);
  struct Bin { const char* name; float (*f)(float, float); };
  const Bin bins[] = {{"Add", [](float x, float y) { return x + y; }}, {"Sub", [](float x, float y) { return x - y; }},
                      {"Mul", [](float x, float y) { return x * y; }}};
  for (const Bin& bn : bins) {
    Dev y("y", {rows, W}, nullptr, true);
    Run(Def(bn.name, 2, {rows, W}), {&a.t, &b.t}, &y.t);                 // equal sizes
    std::vector<float> want(rows * W), got = y.host();
    for (int i = 0; i < rows * W; ++i) want[i] = bn.f(ha[i], hb[i]);
    EXPECT(SameBits(got, want));
    Run(Def(bn.name, 2, {rows, W}), {&a.t, &s.t}, &y.t);                 // second operand a scalar
    got = y.host();
    for (int i = 0; i < rows * W; ++i) want[i] = bn.f(ha[i], hs[0]);
    EXPECT(SameBits(got, want));
    Run(Def(bn.name, 2, {rows, W}), {&row.t, &b.t}, &y.t);               // first operand repeated per row (i % n0)
    got = y.host();
    for (int i = 0; i < rows * W; ++i) want[i] = bn.f(hrow[i % W], hb[i]);
    EXPECT(SameBits(got, want));
  }
  struct Un { const char* name; float (*f)(float); float ulps; };
  const Un uns[] = {{"Sigmoid", [](float x) { return 1.0f / (1.0f + std::exp(-x)); }, 4.f},
                    {"Tanh", [](float x) { return std::tanh(x); }, 4.f},
                    {"Relu", [](float x) { return x > 0.f ? x : 0.f; }, 0.f}};
  for (const Un& un : uns) {
    Dev y("y", {rows, W}, nullptr, true);
    Run(Def(un.name, 1, {rows, W}), {&a.t}, &y.t);
    const std::vector<float> got = y.host();
    float worst = 0.f;
    for (int i = 0; i < rows * W; ++i) worst = std::fmax(worst, UlpDiff(got[i], un.f(ha[i])));
    EXPECT(worst <= un.ulps);
  }
}

static void TestMatMul() {
  const int M = 33, K = 150, N = 70;
  struct Case { bool ta, tb; };
  for (const Case& c : {Case{false, false}, Case{true, false}, Case{false, true}, Case{true, true}}) {
    const std::vector<float> ha = Random(M * K, 5), hb = Random(K * N, 6);
    Dev A("A", c.ta ? std::vector<int>{K, M} : std::vector<int>{M, K}, &ha, false);
    Dev B("B", c.tb ? std::vector<int>{N, K} : std::vector<int>{K, N}, &hb, false);
    Dev C("C", {M, N}, nullptr, false);
    OpDefBuilder b("MatMul");
    b.Input("A").Input("B").Output("C").Shape(std::vector<int>{M, N});
    std::vector<int> tr;
    if (c.ta) tr.push_back(0);
    if (c.tb) tr.push_back(1);
    if (!tr.empty()) b.AttrList("Transpose", tr);
    Run(b.Device("GPU").Finalize(), {&A.t, &B.t}, &C.t);
    const std::vector<float> got = C.host();
    double worst = 0, scale = 0;
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) {
        double acc = 0;
        for (int p = 0; p < K; ++p)
          acc += static_cast<double>(c.ta ? ha[p * M + i] : ha[i * K + p]) * (c.tb ? hb[j * K + p] : hb[p * N + j]);
        worst = std::fmax(worst, std::fabs(acc - got[i * N + j]));
        scale = std::fmax(scale, std::fabs(acc));
      }
    EXPECT(worst <= 1e-5 * scale);
  }
}

static void TestSliceConcat() {
  const int rows = 41, W = 600;     // a Tree-LSTM pre-activation row of hidden size 150: i | o | u | f
  const std::vector<float> hx = Random(rows * W, 9);
  Dev x("x", {rows, W}, &hx, true);
  // dynamic Slice, Split / Index form (op_impl_slice_join.cu:44-69): quarter `index` of every row
  std::vector<Dev*> parts;
  for (int index = 0; index < 4; ++index) {
    Dev* y = new Dev("y", {rows, W / 4}, nullptr, true);
    OpDefBuilder b("Slice");
    b.Input("x").Output("y").Shape(std::vector<int>{rows, W / 4}).AttrSingle("Split", 4).AttrSingle("Index", index);
    Run(b.Device("GPU").Finalize(), {&x.t}, &y->t);
    std::vector<float> want(rows * (W / 4));
    for (int r = 0; r < rows; ++r) std::memcpy(&want[r * (W / 4)], &hx[r * W + index * (W / 4)], (W / 4) * sizeof(float));
    EXPECT(SameBits(y->host(), want));
    parts.push_back(y);
  }
  // dynamic Slice, Offset / Stride form: columns [150, 450) of every row
  {
    Dev y("y", {rows, 300}, nullptr, true);
    OpDefBuilder b("Slice");
    b.Input("x").Output("y").Shape(std::vector<int>{rows, 300}).AttrSingle("Offset", 150).AttrSingle("Stride", 300);
    Run(b.Device("GPU").Finalize(), {&x.t}, &y.t);
    std::vector<float> want(rows * 300);
    for (int r = 0; r < rows; ++r) std::memcpy(&want[r * 300], &hx[r * W + 150], 300 * sizeof(float));
    EXPECT(SameBits(y.host(), want));
  }
  // dynamic Concat of the four quarters gives the rows back (op_impl_slice_join.cu:111-130)
  {
    Dev y("y", {rows, W}, nullptr, true);
    Run(Def("Concat", 4, {rows, W}), {&parts[0]->t, &parts[1]->t, &parts[2]->t, &parts[3]->t}, &y.t);
    EXPECT(SameBits(y.host(), hx));
  }
  for (Dev* p : parts) delete p;
  // static tensors: Slice is one contiguous range of the whole tensor, Concat lays the inputs end to end
  {
    const std::vector<float> hv = Random(1200, 11), hw = Random(300, 12);
    Dev v("v", {1200}, &hv, false), w("w", {300}, &hw, false), y("y", {300}, nullptr, false), z("z", {1500}, nullptr, false);
    OpDefBuilder b("Slice");
    b.Input("v").Output("y").Shape(std::vector<int>{300}).AttrSingle("Offset", 600).AttrSingle("Stride", 300);
    Run(b.Device("GPU").Finalize(), {&v.t}, &y.t);
    EXPECT(SameBits(y.host(), std::vector<float>(hv.begin() + 600, hv.begin() + 900)));
    Run(Def("Concat", 2, {1500}), {&v.t, &w.t}, &z.t);
    std::vector<float> want = hv;
    want.insert(want.end(), hw.begin(), hw.end());
    EXPECT(SameBits(z.host(), want));
  }
}

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "cpu";
  TestRegistry();
  if (mode == "gpu") {
    TestElementwise();
    TestMatMul();
    TestSliceConcat();
  }
  std::printf("%s: %s\n", argv[0], g_failures ? "FAILED" : "ok");
  return g_failures ? 1 : 0;
}
