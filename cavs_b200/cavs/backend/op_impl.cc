#include "cavs/backend/op_impl.h"

#include <unordered_map>

namespace backend {
namespace op_factory {
namespace {
std::unordered_map<std::string, OpImplRegister::Factory>& Registry() {
  static auto* r = new std::unordered_map<std::string, OpImplRegister::Factory>();
  return *r;
}
}  // namespace
OpImplRegister::OpImplRegister(const std::string& name, Factory factory) { Registry().emplace(name, factory); }
}  // namespace op_factory

OpImpl* CreateOp(const OpDef& def) {
  auto& r = op_factory::Registry();
  auto it = r.find(op_factory::Key(def).ToString());
  return it == r.end() ? nullptr : it->second(def);
}
}  // namespace backend
