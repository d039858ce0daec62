// Fluent OpDef construction, same surface as cavs/util/op_def_builder.h:12-55.
#ifndef CAVS_UTIL_OP_DEF_BUILDER_H_
#define CAVS_UTIL_OP_DEF_BUILDER_H_

#include <string>
#include <vector>

#include "cavs/proto/op_def.pb.h"

class OpDefBuilder {
 public:
  explicit OpDefBuilder(const std::string& op_name) { op_def_.set_name(op_name); }
  OpDefBuilder(const OpDefBuilder&) = delete;
  OpDefBuilder& operator=(const OpDefBuilder&) = delete;
  OpDefBuilder& Input(const std::string& input) { op_def_.add_input(input); return *this; }
  OpDefBuilder& Input(const std::vector<std::string>& inputs) { for (auto& s : inputs) op_def_.add_input(s); return *this; }
  OpDefBuilder& Input(const OpDef& def) { return Input(def.input()); }
  OpDefBuilder& Output(const std::string& output) { op_def_.add_output(output); return *this; }
  OpDefBuilder& Output(const std::vector<std::string>& outputs) { for (auto& s : outputs) op_def_.add_output(s); return *this; }
  OpDefBuilder& Output(const OpDef& def) { return Output(def.output()); }
  OpDefBuilder& Device(const std::string& dev) { op_def_.set_device(dev == "CPU" ? CPU : GPU); return *this; }
  OpDefBuilder& Device(const DeviceType type) { op_def_.set_device(type); return *this; }
  OpDefBuilder& Device(const OpDef& def) { op_def_.set_device(def.device()); return *this; }
  OpDefBuilder& Shape(const std::vector<int>& shape) {
    TensorShapeDef* s = op_def_.add_shape();
    for (int d : shape) s->add_dim(d);
    return *this;
  }
  OpDefBuilder& Shape(const TensorShapeDef& shape) { *op_def_.add_shape() = shape; return *this; }
  OpDefBuilder& Shape(const std::vector<TensorShapeDef>& shapes) { for (auto& s : shapes) Shape(s); return *this; }
  OpDefBuilder& Shape(const OpDef& def) { return Shape(def.shape()); }
  OpDefBuilder& Dtype(const DataType type) { op_def_.set_dtype(type); return *this; }
  OpDefBuilder& Label(const std::string& label) { op_def_.set_label(label); return *this; }
  OpDefBuilder& Attr(const OpDef& def) { for (auto& a : def.attr()) *op_def_.add_attr() = a; return *this; }
  OpDefBuilder& Attr(const OpDef::AttrDef& def) { *op_def_.add_attr() = def; return *this; }
  OpDefBuilder& Attr(const std::vector<OpDef::AttrDef>& defs) { for (auto& a : defs) Attr(a); return *this; }
  OpDefBuilder& AttrSingle(const std::string& key, int value) { Named(key)->mutable_value()->set_i(value); return *this; }
  OpDefBuilder& AttrSingle(const std::string& key, int64_t value) { Named(key)->mutable_value()->set_i(value); return *this; }
  OpDefBuilder& AttrSingle(const std::string& key, float value) { Named(key)->mutable_value()->set_f(value); return *this; }
  OpDefBuilder& AttrSingle(const std::string& key, bool value) { Named(key)->mutable_value()->set_b(value); return *this; }
  OpDefBuilder& AttrSingle(const std::string& key, const std::string& value) { Named(key)->mutable_value()->set_s(value); return *this; }
  OpDefBuilder& AttrSingle(const std::string& key, const char* value) { Named(key)->mutable_value()->set_s(value); return *this; }
  OpDefBuilder& AttrList(const std::string& key, const std::vector<int>& value) {
    auto* l = Named(key)->mutable_value()->mutable_list();
    for (int v : value) l->add_i(v);
    return *this;
  }
  OpDefBuilder& AttrList(const std::string& key, const std::vector<float>& value) {
    auto* l = Named(key)->mutable_value()->mutable_list();
    for (float v : value) l->add_f(v);
    return *this;
  }
  const OpDef& Finalize() const { return op_def_; }
  void Finalize(OpDef* op_def) { *op_def = op_def_; }

 private:
  OpDef::AttrDef* Named(const std::string& key) {
    OpDef::AttrDef* a = op_def_.add_attr();
    a->set_name(key);
    return a;
  }
  OpDef op_def_;
};
#endif
