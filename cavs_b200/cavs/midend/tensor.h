// Device tensor handle with the interface the reference's operators use
// (cavs/midend/tensor.h:63-140): a ref-counted buffer, a shared parameter block
// (type, byte offset, dynamic flag, zero-init flag) and a shape.  Per-vertex tensors are
// arenas of [capacity, unit] rows whose data pointer is moved to a row with
// SetOffsetWithId (cavs/midend/tensor.cc:311-321) and whose leading dimension is scaled
// to the level size with ScaleDynamicDimension (:259-271).  Unlike the reference, scaling
// never reallocates: arenas are sized once from the graph's capacity and a request above
// it is a fatal error.
#ifndef CAVS_MIDEND_TENSOR_H_
#define CAVS_MIDEND_TENSOR_H_

#include <memory>
#include <string>
#include <vector>

#include "cavs/proto/op_def.pb.h"
#include "cavs/util/logging.h"

namespace midend {

class TensorShape {
 public:
  TensorShape() : n_elements_(0) {}
  explicit TensorShape(const std::vector<int>& shape);
  explicit TensorShape(const TensorShapeDef& shape);
  int n_elements() const { return n_elements_; }
  int dim() const { return static_cast<int>(shape_.size()); }
  int dim(int idx) const { return shape_.at(idx); }
  void SetDim(int d, int size);
  void AddDim(int size);
  std::string debug_info() const;
 private:
  std::vector<int> shape_;
  int n_elements_;
};

// Owns (or borrows) one device or host allocation.
class TensorBufferBase {
 public:
  TensorBufferBase(DeviceType dev, size_t bytes);                 // allocates and zero-fills
  TensorBufferBase(DeviceType dev, void* borrowed, size_t bytes); // wraps caller memory
  ~TensorBufferBase();
  void* data() const { return data_; }
  size_t size() const { return bytes_; }
  DeviceType device_type() const { return dev_; }
  void InitWithZero();
 private:
  DeviceType dev_;
  void* data_;
  size_t bytes_;
  bool owned_;
};

class Tensor {
 public:
  Tensor();
  // Allocates shape.n_elements() elements of `type` on `dev`, zero-filled
  // (the reference's allocator clears new buffers, cavs/midend/allocator.cu:17-22).
  Tensor(const std::string& name, DeviceType dev, DataType type, const TensorShape& shape);
  // Wraps caller-owned memory.
  Tensor(const std::string& name, DeviceType dev, DataType type, const TensorShape& shape, void* borrowed);
  // Shares t's buffer and parameter block under a new name.
  Tensor(const std::string& name, const Tensor& t);

  DeviceType device_type() const { return buf_->device_type(); }
  std::string name() const { return name_; }
  bool empty() const { return buf_ == nullptr; }
  bool IsDynamicShape() const { return params_->dynamic; }
  DataType data_type() const { return params_->type; }
  void SetAsDynamic() { params_->dynamic = true; }
  int count() const { return shape_.n_elements(); }
  int dims() const { return shape_.dim(); }
  int dims(int idx) const { return shape_.dim(idx); }
  size_t debug_size() const { return buf_->size(); }

  void Reshape(const std::vector<int>& dims);
  // Sets dims(0) = new_dim for a dynamic tensor; fatal if the rows no longer fit the buffer.
  bool ScaleDynamicDimension(int new_dim);
  template <typename T> T* mutable_data() const {
    return reinterpret_cast<T*>(static_cast<char*>(buf_->data()) + params_->offset);
  }
  template <typename T> const T* data() const {
    return reinterpret_cast<const T*>(static_cast<const char*>(buf_->data()) + params_->offset);
  }
  void SetZeroInitEnforced() { params_->zero_init_enforced = true; }
  bool ZeroInitEnforced() const { return params_->zero_init_enforced; }
  bool InitWithZero(int iteration);
  // data pointer := buffer + id * (bytes of one leading-dimension row)
  void SetOffsetWithId(int id);
  // true for a tensor whose leading dimension was declared -1 (deduced at run time)
  bool IsFullShape() const { return full_shape_; }
  void SetFullShape(bool v) { full_shape_ = v; }
  std::string debug_info() const;
  template <typename T> void DebugNumerical() const {}

  struct Params {
    DataType type = DT_FLOAT;
    size_t offset = 0;
    bool dynamic = false;
    bool zero_init_enforced = false;
    int iteration = 0;
  };

 private:
  size_t ElemBytes() const { return params_->type == DT_DOUBLE ? 8 : 4; }
  std::shared_ptr<TensorBufferBase> buf_;
  std::shared_ptr<Params> params_;
  TensorShape shape_;
  std::string name_;
  bool full_shape_ = false;
};

}  // namespace midend
#endif
