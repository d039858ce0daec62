#include "cavs/midend/tensor.h"

#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

namespace midend {

TensorShape::TensorShape(const std::vector<int>& shape) : shape_(shape), n_elements_(1) {
  for (int d : shape) { CHECK(d != 0); n_elements_ *= d; }
}
TensorShape::TensorShape(const TensorShapeDef& shape) : n_elements_(1) {
  CHECK(shape.dim_size() > 0);
  for (int i = 0; i < shape.dim_size(); i++) {
    CHECK(shape.dim(i) != 0);
    shape_.push_back(static_cast<int>(shape.dim(i)));
    n_elements_ *= static_cast<int>(shape.dim(i));
  }
}
void TensorShape::SetDim(int d, int size) {
  CHECK(dim() > d);
  CHECK(size != 0);
  n_elements_ = n_elements_ / shape_[d] * size;
  shape_[d] = size;
}
void TensorShape::AddDim(int size) {
  CHECK(size != 0);
  shape_.push_back(size);
  n_elements_ = (n_elements_ == 0 ? 1 : n_elements_) * size;
}
std::string TensorShape::debug_info() const {
  std::string s;
  for (int d : shape_) s += std::to_string(d) + ",";
  return s;
}

TensorBufferBase::TensorBufferBase(DeviceType dev, size_t bytes) : dev_(dev), data_(nullptr), bytes_(bytes), owned_(true) {
  if (bytes == 0) return;
  if (dev == GPU) {
    cudaError_t e = cudaMalloc(&data_, bytes);
    CHECK(e == cudaSuccess) << "cudaMalloc(" << bytes << "): " << cudaGetErrorString(e);
    e = cudaMemset(data_, 0, bytes);
    CHECK(e == cudaSuccess) << cudaGetErrorString(e);
  } else {
    data_ = std::calloc(1, bytes);
    CHECK(data_ != nullptr);
  }
}
TensorBufferBase::TensorBufferBase(DeviceType dev, void* borrowed, size_t bytes)
    : dev_(dev), data_(borrowed), bytes_(bytes), owned_(false) {}
TensorBufferBase::~TensorBufferBase() {
  if (!owned_ || !data_) return;
  if (dev_ == GPU) cudaFree(data_); else std::free(data_);
}
void TensorBufferBase::InitWithZero() {
  if (!data_) return;
  if (dev_ == GPU) {
    cudaError_t e = cudaMemsetAsync(data_, 0, bytes_, 0);
    CHECK(e == cudaSuccess) << cudaGetErrorString(e);
  } else {
    std::memset(data_, 0, bytes_);
  }
}

Tensor::Tensor() : params_(std::make_shared<Params>()) {}
Tensor::Tensor(const std::string& name, DeviceType dev, DataType type, const TensorShape& shape)
    : params_(std::make_shared<Params>()), shape_(shape), name_(name) {
  params_->type = type;
  buf_ = std::make_shared<TensorBufferBase>(dev, static_cast<size_t>(shape.n_elements()) * ElemBytes());
}
Tensor::Tensor(const std::string& name, DeviceType dev, DataType type, const TensorShape& shape, void* borrowed)
    : params_(std::make_shared<Params>()), shape_(shape), name_(name) {
  params_->type = type;
  buf_ = std::make_shared<TensorBufferBase>(dev, borrowed, static_cast<size_t>(shape.n_elements()) * ElemBytes());
}
Tensor::Tensor(const std::string& name, const Tensor& t)
    : buf_(t.buf_), params_(t.params_), shape_(t.shape_), name_(name), full_shape_(t.full_shape_) {}

void Tensor::Reshape(const std::vector<int>& dims) {
  TensorShape s(dims);
  CHECK(static_cast<size_t>(s.n_elements()) * ElemBytes() <= buf_->size()) << debug_info();
  shape_ = s;
}
bool Tensor::ScaleDynamicDimension(int new_dim) {
  CHECK(IsDynamicShape()) << debug_info();
  CHECK(dims() > 0 && new_dim > 0);
  if (dims(0) == new_dim) return false;
  const size_t unit = static_cast<size_t>(count() / dims(0)) * ElemBytes();
  CHECK(params_->offset + unit * new_dim <= buf_->size())
      << name_ << ": " << new_dim << " rows at byte offset " << params_->offset << " exceed the arena (" << buf_->size() << " bytes)";
  shape_.SetDim(0, new_dim);
  return true;
}
bool Tensor::InitWithZero(int iteration) {
  if (!params_->zero_init_enforced || params_->iteration == iteration) return false;
  buf_->InitWithZero();
  params_->iteration = iteration;
  return true;
}
void Tensor::SetOffsetWithId(int id) {
  CHECK(dims() > 0 && dims(0) > 0);
  const size_t unit = static_cast<size_t>(count() / dims(0)) * ElemBytes();
  CHECK(unit * id <= buf_->size()) << debug_info();
  params_->offset = unit * id;
}
std::string Tensor::debug_info() const {
  return "\nname: " + name_ + "\nshape: " + shape_.debug_info() + "\ntype: " + std::to_string(params_->type);
}

}  // namespace midend
