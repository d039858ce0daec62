// The six graph operators behind the vertex-function API -- Gather, Scatter, Pull, Push,
// FunctionPushArg, FunctionPopRet -- registered under the reference's keys
// (cavs/backend/op_impl_graphop.cu:329-334) and with its Compute semantics (:32-327).
// Each Compute is one call into the C ABI (include/cavs_b200.h): the index list is already on
// the device (uploaded once per batch by the scheduler), so there is no per-launch host-to-device
// copy, and rows move as 128-bit words.
#include <cuda_runtime.h>

#include <unordered_map>

#include "cavs/backend/op_impl.h"
#include "cavs/midend/graph_scheduler.h"
#include "cavs/util/stream_event_handle_pool.h"
#include "cavs_b200.h"

cudaStream_t StreamEventHandlePool::GetCudaStream(int id) {
  static std::unordered_map<int, cudaStream_t> pool;
  if (id < 0) return cudaStreamDefault;
  auto it = pool.find(id);
  if (it != pool.end()) return it->second;
  cudaStream_t s;
  cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  CHECK(e == cudaSuccess) << cudaGetErrorString(e);
  pool[id] = s;
  return s;
}

namespace backend {

using ::midend::GraphSchedulerBase;
using ::midend::Tensor;

namespace {
// Errors of the C ABI become fatal, like the reference's checkCudaError (cavs/util/macros_gpu.h:10-28).
void Must(int status, const char* what) { CHECK(status == CAVS_OK) << what << ": " << cavs_last_error(); }
cudaStream_t StreamOf(OpContext* context) { return StreamEventHandlePool::GetCudaStream(context->GetStreamID()); }
int RowElems(const Tensor& t) { return t.count() / t.dims(0); }
}  // namespace

template <typename T>
class GraphGatherOp : public OpImpl {
 public:
  explicit GraphGatherOp(const OpDef& def) : OpImpl(def), count_(1) {
    CHECK(def.input_size() == 0);
    CHECK(def.output_size() == 1);
    CHECK(def.shape_size() == 1);
    for (auto d : def.shape(0).dim()) count_ *= static_cast<int>(d);
    child_offset_ = GetSingleArg<int>(def, "Child");
    CHECK(child_offset_ >= 0);
  }
  void Compute(OpContext* context) override {
    Tensor* out = context->Output(0);
    GraphSchedulerBase* gs = CHECK_NOTNULL(context->graph_scheduler());
    const Tensor& mailbox = gs->GetMessagePasser(0);
    // A source op sizes its output to the level itself (op_impl_graphop.cu:38-40).
    context->SetDynDim(static_cast<int>(gs->GetJobId().size()));
    context->ScaleOutputTensor();
    const int stride = RowElems(*out);
    CHECK(stride == count_) << out->debug_info() << op_def_.DebugString();
    int n_ids = 0;
    const int* ids = gs->DeviceIdsForGather(child_offset_, &n_ids);
    if (n_ids > 0) {
      Must(cavs_gather_rows(out->mutable_data<T>(), mailbox.data<T>(), ids, n_ids, stride * sizeof(T), StreamOf(context)), "Gather");
    } else {
      // Empty list: clear as many rows as the initialisation list is long (op_impl_graphop.cu:77-86).
      const int n_zero = static_cast<int>(gs->CurrentRoundTensorIdsForGatherInitialization().size());
      Must(cavs_zero_rows(out->mutable_data<T>(), n_zero, stride * sizeof(T), StreamOf(context)), "Gather (zero fill)");
    }
  }
 private:
  int count_;
  int child_offset_;
};

template <typename T>
class GraphScatterOp : public OpImpl {
 public:
  explicit GraphScatterOp(const OpDef& def) : OpImpl(def) {
    child_offset_ = GetSingleArg<int>(def, "Child");
    CHECK(child_offset_ >= 0);
  }
  void Compute(OpContext* context) override {
    const Tensor& inp = context->Input(0);
    Tensor* out = context->Output(0);
    CHECK(inp.IsDynamicShape());
    CHECK(out->IsDynamicShape());
    const int stride = RowElems(*out);
    CHECK(stride == RowElems(inp));
    out->SetOffsetWithId(0);   // the mailbox is addressed by absolute tensor id (op_impl_graphop.cu:123)
    GraphSchedulerBase* gs = CHECK_NOTNULL(context->graph_scheduler());
    int n_ids = 0;
    const int* ids = gs->DeviceIdsForScatter(child_offset_, &n_ids);
    if (n_ids > 0)
      Must(cavs_scatter_rows(out->mutable_data<T>(), ids, inp.data<T>(), n_ids, stride * sizeof(T), StreamOf(context)), "Scatter");
  }
 private:
  int child_offset_;
};

template <typename T>
class GraphPushOp : public OpImpl {
 public:
  explicit GraphPushOp(const OpDef& def) : OpImpl(def) {}
  void Compute(OpContext* context) override {
    GraphSchedulerBase* gs = CHECK_NOTNULL(context->graph_scheduler());
    const Tensor& inp = context->Input(0);
    Tensor* out = context->Output(0);
    CHECK(!out->IsFullShape());
    cudaError_t e = cudaMemcpyAsync(out->mutable_data<T>(), inp.data<T>(), inp.count() * sizeof(T), cudaMemcpyDeviceToDevice,
                                    StreamOf(context));
    CHECK(e == cudaSuccess) << cudaGetErrorString(e);
    gs->SetFuncRet(*out);
  }
};

template <typename T>
class GraphPullOp : public OpImpl {
 public:
  explicit GraphPullOp(const OpDef& def) : OpImpl(def) {}
  void Compute(OpContext* context) override {
    GraphSchedulerBase* gs = CHECK_NOTNULL(context->graph_scheduler());
    const Tensor& inp = gs->GetFuncArg();
    Tensor* out = context->Output(0);
    int n_jobs = 0;
    const int* job_ids = gs->DeviceJobIds(&n_jobs);
    context->SetDynDim(n_jobs);
    context->ScaleOutputTensor();
    CHECK(out->dims(0) == n_jobs);
    CHECK(inp.count() >= out->count()) << inp.debug_info() << out->debug_info();
    const int stride = RowElems(*out);
    Must(cavs_gather_rows(out->mutable_data<T>(), inp.data<T>(), job_ids, n_jobs, stride * sizeof(T), StreamOf(context)), "Pull");
  }
};

template <typename T>
class FunctionPushArgOp : public OpImpl {
 public:
  explicit FunctionPushArgOp(const OpDef& def) : OpImpl(def) {}
  void Compute(OpContext* context) override {
    CHECK_NOTNULL(context->graph_scheduler())->SetFuncArg(context->Input(0));
  }
};

template <typename T>
class FunctionPopRetOp : public OpImpl {
 public:
  explicit FunctionPopRetOp(const OpDef& def) : OpImpl(def) {}
  void Compute(OpContext* context) override {
    GraphSchedulerBase* gs = CHECK_NOTNULL(context->graph_scheduler());
    const Tensor& inp = gs->GetFuncRet();
    Tensor* out = context->Output(0);
    CHECK(inp.IsDynamicShape());
    const int stride = RowElems(inp);
    // Tensor-id order -> job order over the vertices that executed.  (The reference walks all
    // total_length entries of the map, including the never-written tail left by single-vertex
    // samples, op_impl_graphop.cu:297-318; those rows are skipped here.)
    int n = 0;
    const int* t2j = gs->DeviceTensorIdsToJobIds(&n);
    if (n > 0)
      Must(cavs_scatter_rows(out->mutable_data<T>(), t2j, inp.data<T>(), n, stride * sizeof(T), StreamOf(context)), "FunctionPopRet");
  }
};

REGISTER_OP_IMPL_BUILDER(Key("Pull").Device("GPU"), GraphPullOp<float>);
REGISTER_OP_IMPL_BUILDER(Key("Push").Device("GPU"), GraphPushOp<float>);
REGISTER_OP_IMPL_BUILDER(Key("Scatter").Device("GPU"), GraphScatterOp<float>);
REGISTER_OP_IMPL_BUILDER(Key("Gather").Device("GPU"), GraphGatherOp<float>);
REGISTER_OP_IMPL_BUILDER(Key("FunctionPushArg").Device("GPU"), FunctionPushArgOp<float>);
REGISTER_OP_IMPL_BUILDER(Key("FunctionPopRet").Device("GPU"), FunctionPopRetOp<float>);

}  // namespace backend
