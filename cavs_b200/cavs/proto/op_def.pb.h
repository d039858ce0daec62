// Protobuf-free OpDef / TensorShapeDef / FunctionDef with the accessor names protoc
// generates for the reference's messages (cavs/proto/op_def.proto:7-35,
// cavs/proto/tensor_shape.proto:3-5, cavs/proto/func_def.proto:5-8,
// cavs/proto/types.proto:3-7, cavs/proto/devices.proto), so operator code written against
// the generated classes compiles unchanged.  No wire format: definitions stay in process.
#ifndef CAVS_PROTO_OP_DEF_PB_H_
#define CAVS_PROTO_OP_DEF_PB_H_

#include <cstdint>
#include <sstream>
#include <string>
#include <vector>

enum DeviceType { CPU = 0, GPU = 1 };
enum DataType { DT_FLOAT = 0, DT_DOUBLE = 1, DT_INT32 = 2 };

class TensorShapeDef {
 public:
  int dim_size() const { return static_cast<int>(dim_.size()); }
  int64_t dim(int i) const { return dim_.at(i); }
  const std::vector<int64_t>& dim() const { return dim_; }
  void add_dim(int64_t d) { dim_.push_back(d); }
  void set_dim(int i, int64_t d) { dim_.at(i) = d; }
  void clear_dim() { dim_.clear(); }
 private:
  std::vector<int64_t> dim_;
};

class OpDef {
 public:
  class AttrType {
   public:
    class ListValue {
     public:
      const std::vector<std::string>& s() const { return s_; }
      const std::vector<int64_t>& i() const { return i_; }
      const std::vector<float>& f() const { return f_; }
      const std::vector<bool>& b() const { return b_; }
      void add_s(const std::string& v) { s_.push_back(v); }
      void add_i(int64_t v) { i_.push_back(v); }
      void add_f(float v) { f_.push_back(v); }
      void add_b(bool v) { b_.push_back(v); }
     private:
      std::vector<std::string> s_;
      std::vector<int64_t> i_;
      std::vector<float> f_;
      std::vector<bool> b_;
    };
    enum TypeCase { TYPE_NOT_SET = 0, kS = 1, kI = 2, kF = 3, kB = 4, kList = 5 };
    TypeCase type_case() const { return case_; }
    const std::string& s() const { return s_; }
    int64_t i() const { return i_; }
    float f() const { return f_; }
    bool b() const { return b_; }
    const ListValue& list() const { return list_; }
    void set_s(const std::string& v) { s_ = v; case_ = kS; }
    void set_i(int64_t v) { i_ = v; case_ = kI; }
    void set_f(float v) { f_ = v; case_ = kF; }
    void set_b(bool v) { b_ = v; case_ = kB; }
    ListValue* mutable_list() { case_ = kList; return &list_; }
   private:
    TypeCase case_ = TYPE_NOT_SET;
    std::string s_;
    int64_t i_ = 0;
    float f_ = 0.f;
    bool b_ = false;
    ListValue list_;
  };
  class AttrDef {
   public:
    const std::string& name() const { return name_; }
    void set_name(const std::string& n) { name_ = n; }
    const AttrType& value() const { return value_; }
    AttrType* mutable_value() { return &value_; }
   private:
    std::string name_;
    AttrType value_;
  };

  const std::string& name() const { return name_; }
  void set_name(const std::string& n) { name_ = n; }
  int input_size() const { return static_cast<int>(input_.size()); }
  const std::string& input(int i) const { return input_.at(i); }
  const std::vector<std::string>& input() const { return input_; }
  void add_input(const std::string& s) { input_.push_back(s); }
  void set_input(int i, const std::string& s) { input_.at(i) = s; }
  void clear_input() { input_.clear(); }
  int output_size() const { return static_cast<int>(output_.size()); }
  const std::string& output(int i) const { return output_.at(i); }
  const std::vector<std::string>& output() const { return output_; }
  void add_output(const std::string& s) { output_.push_back(s); }
  void set_output(int i, const std::string& s) { output_.at(i) = s; }
  void clear_output() { output_.clear(); }
  int shape_size() const { return static_cast<int>(shape_.size()); }
  const TensorShapeDef& shape(int i) const { return shape_.at(i); }
  const std::vector<TensorShapeDef>& shape() const { return shape_; }
  TensorShapeDef* add_shape() { shape_.emplace_back(); return &shape_.back(); }
  TensorShapeDef* mutable_shape(int i) { return &shape_.at(i); }
  void clear_shape() { shape_.clear(); }
  DeviceType device() const { return device_; }
  void set_device(DeviceType d) { device_ = d; }
  DataType dtype() const { return dtype_; }
  void set_dtype(DataType t) { dtype_ = t; }
  const std::string& label() const { return label_; }
  void set_label(const std::string& l) { label_ = l; }
  int attr_size() const { return static_cast<int>(attr_.size()); }
  const AttrDef& attr(int i) const { return attr_.at(i); }
  const std::vector<AttrDef>& attr() const { return attr_; }
  AttrDef* add_attr() { attr_.emplace_back(); return &attr_.back(); }
  void clear_attr() { attr_.clear(); }

  std::string DebugString() const {
    std::ostringstream o;
    o << "name: \"" << name_ << "\"\n";
    for (const auto& s : input_) o << "input: \"" << s << "\"\n";
    for (const auto& s : output_) o << "output: \"" << s << "\"\n";
    for (const auto& sh : shape_) {
      o << "shape {";
      for (auto d : sh.dim()) o << " dim: " << d;
      o << " }\n";
    }
    o << "device: " << (device_ == GPU ? "GPU" : "CPU") << "\n";
    if (!label_.empty()) o << "label: \"" << label_ << "\"\n";
    for (const auto& a : attr_) {
      o << "attr { name: \"" << a.name() << "\" value: ";
      switch (a.value().type_case()) {
        case AttrType::kS: o << "\"" << a.value().s() << "\""; break;
        case AttrType::kI: o << a.value().i(); break;
        case AttrType::kF: o << a.value().f(); break;
        case AttrType::kB: o << (a.value().b() ? "true" : "false"); break;
        case AttrType::kList: o << "[list]"; break;
        default: o << "<unset>";
      }
      o << " }\n";
    }
    return o.str();
  }

 private:
  std::string name_;
  std::vector<std::string> input_, output_;
  std::vector<TensorShapeDef> shape_;
  DeviceType device_ = GPU;
  DataType dtype_ = DT_FLOAT;
  std::string label_;
  std::vector<AttrDef> attr_;
};

class FunctionDef {
 public:
  const std::string& name() const { return name_; }
  void set_name(const std::string& n) { name_ = n; }
  int ops_size() const { return static_cast<int>(ops_.size()); }
  const OpDef& ops(int i) const { return ops_.at(i); }
  const std::vector<OpDef>& ops() const { return ops_; }
  OpDef* add_ops() { ops_.emplace_back(); return &ops_.back(); }
 private:
  std::string name_;
  std::vector<OpDef> ops_;
};
#endif
