// Operator implementation interface and its string-keyed registry, same contract as
// cavs/backend/op_impl.h:14-74: an implementation derives from OpImpl, overrides Compute,
// and is registered at static-initialisation time under "name:device:label".
#ifndef CAVS_BACKEND_OP_IMPL_H_
#define CAVS_BACKEND_OP_IMPL_H_

#include <string>
#include <vector>

#include "cavs/midend/op_context.h"
#include "cavs/proto/op_def.pb.h"
#include "cavs/util/op_util.h"

namespace backend {

using ::midend::OpContext;

class OpImpl {
 public:
  explicit OpImpl(const OpDef& def) : op_def_(def) {}
  virtual ~OpImpl() {}
  virtual void Compute(OpContext* context) = 0;
  std::string DebugInfo(int level = V_DEBUG) const { return level == V_DEBUG ? op_def_.DebugString() : op_def_.name(); }
  std::string name() const { return op_def_.name(); }
 protected:
  OpDef op_def_;
};

// Returns NULL when no implementation is registered for the definition's key.
OpImpl* CreateOp(const OpDef& def);

#define REGISTER_OP_IMPL_BUILDER(key, ...) REGISTER_OP_IMPL_BUILDER_UNIQ(__COUNTER__, key, __VA_ARGS__)
#define REGISTER_OP_IMPL_BUILDER_UNIQ(ctr, key, ...) REGISTER_OP_IMPL_BUILDER_CONCAT(ctr, key, __VA_ARGS__)
#define REGISTER_OP_IMPL_BUILDER_CONCAT(ctr, key, ...)                                            \
  static ::backend::op_factory::OpImplRegister register_body_##ctr##_op_impl(                     \
      ::backend::op_factory::key.ToString(),                                                      \
      [](const OpDef& def) -> ::backend::OpImpl* { return new __VA_ARGS__(def); });

namespace op_factory {

class Key {
 public:
  Key(const std::string& name) : op_name_(name) {}
  Key(const char* name) : op_name_(name) {}
  Key(const OpDef& def) : op_name_(def.name()), dev_(DeviceTypeToString(def.device())), label_(def.label()) {}
  Key& Device(std::string dev) { dev_ = dev; return *this; }
  Key& Label(std::string label) { label_ = label; return *this; }
  std::string ToString() const { return op_name_ + ":" + dev_ + ":" + label_; }
 private:
  std::string op_name_, dev_, label_;
};

class OpImplRegister {
 public:
  typedef OpImpl* (*Factory)(const OpDef& def);
  OpImplRegister(const std::string& name, Factory factory);
};

}  // namespace op_factory
}  // namespace backend
#endif
