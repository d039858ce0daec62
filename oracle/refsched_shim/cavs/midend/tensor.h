// Stand-in for midend::Tensor exposing only what graph_scheduler.{h,cc} touch:
// a host int matrix [batch, max_len] plus no-op offset hooks.  TEST INFRASTRUCTURE.
#ifndef ORACLE_SHIM_CAVS_MIDEND_TENSOR_H_
#define ORACLE_SHIM_CAVS_MIDEND_TENSOR_H_
#include <string>
#include "cavs/proto/devices.pb.h"
#include "cavs/util/logging.h"
namespace midend {
class Tensor {
 public:
  Tensor() : base_(nullptr), rows_(0), cols_(0) {}
  Tensor(const int* base, int rows, int cols) : base_(base), rows_(rows), cols_(cols) {}
  int dims() const { return 2; }
  int dims(int axis) const { return axis == 0 ? rows_ : cols_; }
  DeviceType device_type() const { return CPU; }
  template <typename T> const T* data() const { return reinterpret_cast<const T*>(base_); }
  bool IsFullShape() const { return false; }
  void SetOffsetWithId(int) {}
  std::string debug_info() const { return "shim tensor"; }
 private:
  const int* base_;
  int rows_, cols_;
};
}  // namespace midend
#endif
