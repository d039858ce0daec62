// Stand-alone operators a vertex function is written in -- MatMul, Add / Sub / Mul, Sigmoid / Tanh / Relu, Slice,
// Concat, Mirror -- registered under the reference's keys with its Compute semantics, for callers that run an
// operator list one statement at a time (cavs/midend/statement.cc:43-123).  Session::Run does not use them: it
// executes whole levels through the fused engines or the planned executor (cavs/midend/generic_function.h).
//
//   MatMul            cavs/backend/op_impl_blas3_cublas.cc:13-86   -> cavs_gemm_f32 (strides absorb the transposes)
//   Add / Sub / Mul   cavs/backend/op_impl_elementwise.cu:14-19    -> one generated kernel per operator name
//   Sigmoid / Tanh / Relu  cavs/backend/op_impl_activation_cudnn.cu (cuDNN activations; here the expressions of the
//                     reference's own fused kernels, cavs/midend/runtime_compiler/expression.h:40-72)
//   Slice / Concat    cavs/backend/op_impl_slice_join.cu:13-149    -> cavs_copy_rows_2d
//   Mirror            cavs/backend/op_impl_slice_join.cu:228-233   (no work: the output aliases the input)
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "cavs/backend/cudaRTC_wrapper.h"
#include "cavs/backend/op_impl.h"
#include "cavs/midend/runtime_compiler/code_generator.h"
#include "cavs/util/op_util.h"
#include "cavs/util/stream_event_handle_pool.h"
#include "cavs_b200.h"

namespace backend {

using ::midend::Tensor;

namespace {

void Must(int status, const char* what) { CHECK(status == CAVS_OK) << what << ": " << cavs_last_error(); }
cudaStream_t StreamOf(OpContext* context) { return StreamEventHandlePool::GetCudaStream(context->GetStreamID()); }

// One compiled kernel per operator name, shared by every instance of the operator.
::RTC::CudaRTCWrapper* KernelFor(const std::string& op_name) {
  static std::mutex mu;
  static std::map<std::string, std::unique_ptr<::RTC::CudaRTCWrapper>> kernels;
  std::lock_guard<std::mutex> lock(mu);
  auto& slot = kernels[op_name];
  if (!slot) {
    slot.reset(new ::RTC::CudaRTCWrapper());
    const std::string name = "cavs_standalone_" + op_name;
    slot->Compile(name, ::midend::RTC::GenStandalone(op_name, name));
  }
  return slot.get();
}

void LaunchElementwise(const std::string& op_name, float* out, long long n, const float* in0, long long n0, const float* in1,
                       long long n1, cudaStream_t stream) {
  if (n == 0) return;
  // operand patterns of the reference: equal sizes, a scalar, or a shorter operand repeated along the longer one
  CHECK(n0 == n || n0 == 1 || (n0 < n && n % n0 == 0)) << op_name << ": Unrecognized Pattern: " << n0 << " vs " << n;
  CHECK(in1 == nullptr || n1 == n || n1 == 1 || (n1 < n && n % n1 == 0)) << op_name << ": Unrecognized Pattern: " << n1 << " vs " << n;
  std::vector<void*> args = {&out, &n, &in0, &n0, &in1, &n1};
  const unsigned block = 256;
  const unsigned grid = static_cast<unsigned>(std::min<long long>((n + block - 1) / block, 148 * 8));
  KernelFor(op_name)->Launch(args, grid, block, stream);
}

}  // namespace

class ElementwiseUnaryOp : public OpImpl {
 public:
  explicit ElementwiseUnaryOp(const OpDef& def) : OpImpl(def) { CHECK(def.input_size() == 1 && def.output_size() == 1); }
  void Compute(OpContext* context) override {
    const Tensor& inp = context->Input(0);
    Tensor* out = context->Output(0);
    LaunchElementwise(op_def_.name(), out->mutable_data<float>(), out->count(), inp.data<float>(), inp.count(), nullptr, 0,
                      StreamOf(context));
  }
};

class ElementwiseBinaryOp : public OpImpl {
 public:
  explicit ElementwiseBinaryOp(const OpDef& def) : OpImpl(def) { CHECK(def.input_size() == 2 && def.output_size() == 1); }
  void Compute(OpContext* context) override {
    const Tensor& a = context->Input(0);
    const Tensor& b = context->Input(1);
    Tensor* out = context->Output(0);
    LaunchElementwise(op_def_.name(), out->mutable_data<float>(), out->count(), a.data<float>(), a.count(), b.data<float>(),
                      b.count(), StreamOf(context));
  }
};

class MatMulOp : public OpImpl {
 public:
  explicit MatMulOp(const OpDef& def) : OpImpl(def) {
    for (int t : GetListArg<int>(def, "Transpose")) {
      if (t == 0) trans_a_ = true;
      if (t == 1) trans_b_ = true;
    }
  }
  void Compute(OpContext* context) override {
    const Tensor& A = context->Input(0);
    const Tensor& B = context->Input(1);
    Tensor* C = context->Output(0);
    CHECK(A.dims() == 2 && B.dims() == 2 && C->dims() == 2);
    const int MA = trans_a_ ? A.dims(1) : A.dims(0), KA = trans_a_ ? A.dims(0) : A.dims(1);
    const int KB = trans_b_ ? B.dims(1) : B.dims(0), NB = trans_b_ ? B.dims(0) : B.dims(1);
    CHECK(KA == KB);
    CHECK(C->dims(0) == MA) << "C.dims(0): " << C->dims(0) << "\tMA: " << MA;
    CHECK(C->dims(1) == NB) << "C.dims(1): " << C->dims(1) << "\tNB: " << NB;
    if (MA == 0 || NB == 0) return;
    const long long lda = A.dims(1), ldb = B.dims(1);
    Must(cavs_gemm_f32(C->mutable_data<float>(), NB, 0, A.data<float>(), trans_a_ ? 1 : lda, trans_a_ ? lda : 1, B.data<float>(),
                       trans_b_ ? 1 : ldb, trans_b_ ? ldb : 1, MA, NB, KA, StreamOf(context)), "MatMul");
  }
 private:
  bool trans_a_ = false, trans_b_ = false;
};

class SliceOp : public OpImpl {
 public:
  explicit SliceOp(const OpDef& def) : OpImpl(def) {
    CHECK(GetSingleArg<int>(def, "Axis", 0) == 0);
    if (GetSingleArg<int>(def, "Split", 0) != 0) {
      split_ = GetSingleArg<int>(def, "Split");
      index_ = GetSingleArg<int>(def, "Index");
      CHECK(split_ > 0 && index_ >= 0 && index_ < split_);
    } else {
      offset_ = GetSingleArg<int>(def, "Offset");
      stride_ = GetSingleArg<int>(def, "Stride");
      CHECK(offset_ >= 0 && stride_ > 0);
    }
  }
  void Compute(OpContext* context) override {
    const Tensor& x = context->Input(0);
    Tensor* y = context->Output(0);
    if (x.IsDynamicShape()) {
      // one slice per row of the level: columns [offset, offset + stride) of every row.  The reference handles the
      // Split / Index form only (op_impl_slice_join.cu:44-47); the Offset / Stride form follows the same row rule.
      CHECK(y->IsDynamicShape() && x.dims() == 2 && y->dims() == 2 && y->dims(0) == x.dims(0));
      const int rows = x.dims(0), x_stride = rows ? x.count() / rows : 0;
      int y_stride, x_offset;
      if (split_ > 0) {
        CHECK(x_stride % split_ == 0);
        y_stride = x_stride / split_; x_offset = y_stride * index_;
      } else {
        y_stride = stride_; x_offset = offset_;
        CHECK(x_offset + y_stride <= x_stride);
      }
      CHECK(static_cast<long long>(rows) * y_stride == y->count());
      if (rows == 0) return;
      Must(cavs_copy_rows_2d(y->mutable_data<float>(), y_stride, nullptr, x.data<float>() + x_offset, x_stride, nullptr, rows,
                             y_stride, 0, StreamOf(context)), "Slice");
    } else {
      CHECK(!y->IsDynamicShape());
      int stride = stride_, offset = offset_;
      if (split_ > 0) {
        CHECK(x.count() % split_ == 0);
        stride = x.count() / split_; offset = stride * index_;
      }
      CHECK(stride == y->count() && offset + stride <= x.count());
      Must(cavs_copy_rows_2d(y->mutable_data<float>(), stride, nullptr, x.data<float>() + offset, stride, nullptr, 1, stride, 0,
                             StreamOf(context)), "Slice");
    }
  }
 private:
  int split_ = -1, index_ = -1, offset_ = -1, stride_ = -1;
};

class ConcatOp : public OpImpl {
 public:
  explicit ConcatOp(const OpDef& def) : OpImpl(def) { CHECK(GetSingleArg<int>(def, "Axis", 0) == 0); }
  void Compute(OpContext* context) override {
    Tensor* out = context->Output(0);
    CHECK(out->count() > 0);
    long long copied = 0;
    for (int i = 0; i < context->InputSize(); ++i) {
      const Tensor& inp = context->Input(i);
      CHECK(inp.count() > 0 && copied + inp.count() <= out->count());
      if (out->IsDynamicShape()) {
        // per row: the inputs' rows side by side (op_impl_slice_join.cu:111-130)
        CHECK(inp.IsDynamicShape() && out->dims() == 2 && inp.dims() == 2 && inp.dims(0) == out->dims(0));
        const int rows = out->dims(0), out_stride = out->count() / rows, inp_stride = inp.count() / rows;
        Must(cavs_copy_rows_2d(out->mutable_data<float>() + copied / rows, out_stride, nullptr, inp.data<float>(), inp_stride, nullptr,
                               rows, inp_stride, 0, StreamOf(context)), "Concat");
      } else {
        CHECK(!inp.IsDynamicShape());
        Must(cavs_copy_rows_2d(out->mutable_data<float>() + copied, inp.count(), nullptr, inp.data<float>(), inp.count(), nullptr, 1,
                               inp.count(), 0, StreamOf(context)), "Concat");
      }
      copied += inp.count();
    }
    CHECK(out->count() == copied);
  }
};

class MirrorOp : public OpImpl {
 public:
  explicit MirrorOp(const OpDef& def) : OpImpl(def) {}
  void Compute(OpContext*) override {}
};

REGISTER_OP_IMPL_BUILDER(Key("Add").Device("GPU"), ElementwiseBinaryOp);
REGISTER_OP_IMPL_BUILDER(Key("Sub").Device("GPU"), ElementwiseBinaryOp);
REGISTER_OP_IMPL_BUILDER(Key("Mul").Device("GPU"), ElementwiseBinaryOp);
REGISTER_OP_IMPL_BUILDER(Key("Sigmoid").Device("GPU"), ElementwiseUnaryOp);
REGISTER_OP_IMPL_BUILDER(Key("Tanh").Device("GPU"), ElementwiseUnaryOp);
REGISTER_OP_IMPL_BUILDER(Key("Relu").Device("GPU"), ElementwiseUnaryOp);
REGISTER_OP_IMPL_BUILDER(Key("MatMul").Device("GPU"), MatMulOp);
REGISTER_OP_IMPL_BUILDER(Key("Slice").Device("GPU"), SliceOp);
REGISTER_OP_IMPL_BUILDER(Key("Concat").Device("GPU"), ConcatOp);
REGISTER_OP_IMPL_BUILDER(Key("Mirror").Device("GPU"), MirrorOp);

}  // namespace backend
