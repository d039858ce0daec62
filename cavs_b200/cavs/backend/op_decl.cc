#include "cavs/backend/op_decl.h"

#include <memory>
#include <unordered_map>

namespace backend {
namespace op_factory {
namespace {
std::unordered_map<std::string, OpDeclRegister::Factory>& Registry() {
  static auto* r = new std::unordered_map<std::string, OpDeclRegister::Factory>();
  return *r;
}
}  // namespace
OpDeclRegister::OpDeclRegister(const std::string& name, Factory factory) { Registry().emplace(name, factory); }
}  // namespace op_factory

std::vector<OpDef> MakeGradient(const OpDef& def) {
  auto& r = op_factory::Registry();
  CHECK(r.count(def.name()) > 0) << def.name();
  std::unique_ptr<OpDecl> decl(r.at(def.name())(def));
  std::vector<OpDef> out;
  decl->MakeGradient(&out);
  return out;
}

std::vector<TensorShapeDef> ShapeInference(const OpDef& def, const std::vector<TensorShapeDef>& inputs) {
  auto& r = op_factory::Registry();
  CHECK(r.count(def.name()) > 0) << def.name();
  std::unique_ptr<OpDecl> decl(r.at(def.name())(def));
  std::vector<TensorShapeDef> out;
  decl->ShapeInference(&out, inputs);
  return out;
}
}  // namespace backend
