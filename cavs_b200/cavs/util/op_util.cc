#include "cavs/util/op_util.h"

#include <functional>

#include "cavs/util/logging.h"

namespace {
const OpDef::AttrDef* FindAttr(const OpDef& def, const std::string& key) {
  for (const auto& a : def.attr())
    if (a.name() == key) return &a;
  return nullptr;
}
template <typename T> T Scalar(const OpDef::AttrType& v);
template <> int Scalar<int>(const OpDef::AttrType& v) { return static_cast<int>(v.i()); }
template <> int64_t Scalar<int64_t>(const OpDef::AttrType& v) { return v.i(); }
template <> float Scalar<float>(const OpDef::AttrType& v) { return v.f(); }
template <> bool Scalar<bool>(const OpDef::AttrType& v) { return v.b(); }
template <> std::string Scalar<std::string>(const OpDef::AttrType& v) { return v.s(); }
}  // namespace

template <typename T> T GetSingleArg(const OpDef& op_def, const std::string& key) {
  const OpDef::AttrDef* a = FindAttr(op_def, key);
  CHECK(a != nullptr) << "attribute " << key << " missing in\n" << op_def.DebugString();
  return Scalar<T>(a->value());
}
template <typename T> T GetSingleArg(const OpDef& op_def, const std::string& key, T value) {
  const OpDef::AttrDef* a = FindAttr(op_def, key);
  return a ? Scalar<T>(a->value()) : value;
}
template <> std::vector<int> GetListArg<int>(const OpDef& op_def, const std::string& key) {
  const OpDef::AttrDef* a = FindAttr(op_def, key);
  std::vector<int> out;
  if (a) for (auto v : a->value().list().i()) out.push_back(static_cast<int>(v));
  return out;
}
template <> std::vector<float> GetListArg<float>(const OpDef& op_def, const std::string& key) {
  const OpDef::AttrDef* a = FindAttr(op_def, key);
  return a ? a->value().list().f() : std::vector<float>();
}

#define INSTANTIATE(T)                                                        \
  template T GetSingleArg<T>(const OpDef&, const std::string&);              \
  template T GetSingleArg<T>(const OpDef&, const std::string&, T);
INSTANTIATE(int)
INSTANTIATE(int64_t)
INSTANTIATE(float)
INSTANTIATE(bool)
INSTANTIATE(std::string)
#undef INSTANTIATE

static const char kGradSuffix[] = "_grad";

std::string GetGradientName(const std::string& op) { return op + kGradSuffix; }
std::string GetOriginName(const std::string& op) {
  CHECK(IsGradientName(op)) << op;
  return op.substr(0, op.size() - (sizeof(kGradSuffix) - 1));
}
bool IsGradientName(const std::string& edge) {
  const size_t n = sizeof(kGradSuffix) - 1;
  return edge.size() >= n && edge.compare(edge.size() - n, n, kGradSuffix) == 0;
}
const char* DeviceTypeToString(DeviceType type) { return type == GPU ? "GPU" : "CPU"; }
size_t GetHash(const OpDef& op_def) { return std::hash<std::string>()(op_def.DebugString()); }
