// NOT onnx-light. A minimal, header-only stand-in for exactly the part of onnx-light's C++
// runtime API that a kernel plug-in touches (KernelBase, RuntimeContext, Tensor, NodeProto,
// the kernel dispatch table and the node helper functions), so that the MatMulNBits
// operator class can be compiled, registered and run where onnx-light itself is not
// installed. Names, argument meaning and error behaviour follow the way the reference
// plug-in uses them (onnx_light_cpu/kernels/math/integer_matmul_kernel.cc:298-378,
// onnx_light_cpu/kernels/math/gemm_kernel.cc:462-476,
// onnx_light_cpu/kernels/kernel_registration.cc:56-85). Build against the real headers by
// putting onnx-light's include directory before this one on the include path.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#ifndef ONNX_LIGHT_NAMESPACE
#define ONNX_LIGHT_NAMESPACE onnx_light
#endif

namespace ONNX_LIGHT_NAMESPACE {

// ---- protobuf-shaped node description --------------------------------------------------
class AttributeProto {
public:
  const std::string &name() const { return name_; }
  void set_name(std::string v) { name_ = std::move(v); }
  std::int64_t i() const { return i_; }
  void set_i(std::int64_t v) {
    i_ = v;
    has_i_ = true;
  }
  float f() const { return f_; }
  void set_f(float v) {
    f_ = v;
    has_f_ = true;
  }
  bool has_i() const { return has_i_; }
  bool has_f() const { return has_f_; }

private:
  std::string name_;
  std::int64_t i_ = 0;
  float f_ = 0.0f;
  bool has_i_ = false;
  bool has_f_ = false;
};

class NodeProto {
public:
  const std::string &op_type() const { return op_type_; }
  void set_op_type(std::string v) { op_type_ = std::move(v); }
  const std::string &domain() const { return domain_; }
  void set_domain(std::string v) { domain_ = std::move(v); }
  const std::string &name() const { return name_; }
  void set_name(std::string v) { name_ = std::move(v); }
  int input_size() const { return static_cast<int>(inputs_.size()); }
  int output_size() const { return static_cast<int>(outputs_.size()); }
  const std::string &input(int i) const { return inputs_.at(static_cast<std::size_t>(i)); }
  const std::string &output(int i) const { return outputs_.at(static_cast<std::size_t>(i)); }
  void add_input(std::string v) { inputs_.push_back(std::move(v)); }
  void add_output(std::string v) { outputs_.push_back(std::move(v)); }
  int attribute_size() const { return static_cast<int>(attributes_.size()); }
  const AttributeProto &attribute(int i) const { return attributes_.at(static_cast<std::size_t>(i)); }
  AttributeProto *add_attribute() {
    attributes_.emplace_back();
    return &attributes_.back();
  }

private:
  std::string op_type_, domain_, name_;
  std::vector<std::string> inputs_, outputs_;
  std::vector<AttributeProto> attributes_;
};

inline std::string NormaliseDomain(const std::string &domain) {
  return domain.empty() ? std::string("ai.onnx") : domain;
}

namespace core {

namespace symbolic {
enum class Device : std::int32_t { kUndefined = 0, kCPU = 1, kCUDA = 2 };
inline const char *DeviceName(Device device) {
  switch (device) {
  case Device::kCPU:
    return "CPU";
  case Device::kCUDA:
    return "CUDA";
  default:
    return "UNDEFINED";
  }
}
} // namespace symbolic

namespace runtime {

// TensorProto::DataType values.
enum class DataType : std::int32_t {
  UNDEFINED = 0,
  FLOAT = 1,
  UINT8 = 2,
  INT8 = 3,
  UINT16 = 4,
  INT16 = 5,
  INT32 = 6,
  INT64 = 7,
  STRING = 8,
  BOOL = 9,
  FLOAT16 = 10,
  DOUBLE = 11,
  UINT32 = 12,
  UINT64 = 13,
  BFLOAT16 = 16,
};

using Shape = std::vector<std::int64_t>;

inline std::size_t ElementSizeOf(std::int32_t data_type) {
  switch (static_cast<DataType>(data_type)) {
  case DataType::FLOAT:
  case DataType::INT32:
  case DataType::UINT32:
    return 4;
  case DataType::DOUBLE:
  case DataType::INT64:
  case DataType::UINT64:
    return 8;
  case DataType::FLOAT16:
  case DataType::BFLOAT16:
  case DataType::INT16:
  case DataType::UINT16:
    return 2;
  case DataType::UINT8:
  case DataType::INT8:
  case DataType::BOOL:
    return 1;
  default:
    throw std::invalid_argument("onnx-light shim: unsupported tensor data type.");
  }
}

class Tensor {
public:
  std::string name;
  std::int32_t data_type = 0;
  Shape shape;

  Tensor() = default;
  Tensor(std::string tensor_name, std::int32_t dtype, Shape tensor_shape, std::vector<std::uint8_t> data)
      : name(std::move(tensor_name)), data_type(dtype), shape(std::move(tensor_shape)),
        storage_(std::move(data)) {}

  std::int64_t element_count() const {
    std::int64_t n = 1;
    for (std::int64_t d : shape) {
      n *= d;
    }
    return n;
  }
  std::size_t element_size() const { return ElementSizeOf(data_type); }
  std::size_t size_bytes() const { return storage_.size(); }
  const void *bytes() const { return storage_.data(); }
  void *mutable_bytes() { return storage_.data(); }

  const float *AsFloat() const { return reinterpret_cast<const float *>(storage_.data()); }
  float *AsFloat() { return reinterpret_cast<float *>(storage_.data()); }
  const std::uint8_t *AsUint8() const { return storage_.data(); }
  std::uint8_t *AsUint8() { return storage_.data(); }
  const std::int32_t *AsInt32() const { return reinterpret_cast<const std::int32_t *>(storage_.data()); }
  std::int32_t *AsInt32() { return reinterpret_cast<std::int32_t *>(storage_.data()); }

  template <typename T>
  static Tensor From(std::string tensor_name, std::int32_t dtype, Shape tensor_shape,
                     const std::vector<T> &values) {
    std::vector<std::uint8_t> data(values.size() * sizeof(T));
    if (!values.empty()) {
      std::memcpy(data.data(), values.data(), data.size());
    }
    return Tensor(std::move(tensor_name), dtype, std::move(tensor_shape), std::move(data));
  }
  static Tensor FromFloat(std::string tensor_name, Shape tensor_shape, const std::vector<float> &values) {
    return From<float>(std::move(tensor_name), static_cast<std::int32_t>(DataType::FLOAT),
                       std::move(tensor_shape), values);
  }

private:
  std::vector<std::uint8_t> storage_;
};

inline Tensor MakeOutputTensor(std::int32_t data_type, const Shape &shape, std::size_t bytes,
                               void * /*allocator*/) {
  return Tensor("", data_type, shape, std::vector<std::uint8_t>(bytes));
}

struct OpsetId {
  std::string domain;
  std::int64_t version = 0;
  OpsetId() = default;
  OpsetId(std::string d, std::int64_t v) : domain(std::move(d)), version(v) {}
};

inline OpsetId DefaultOpset(int version) { return OpsetId("", version); }

class KernelContext {
public:
  KernelContext() = default;
  explicit KernelContext(OpsetId opset) : opset_(std::move(opset)) {}
  const OpsetId &opset() const { return opset_; }

private:
  OpsetId opset_;
};

using TensorMap = std::map<std::string, Tensor>;

class RuntimeContext {
public:
  RuntimeContext() = default;
  explicit RuntimeContext(KernelContext ctx) : kernel_ctx_(std::move(ctx)) {}
  TensorMap &tensors() { return tensors_; }
  const TensorMap &tensors() const { return tensors_; }
  const KernelContext &kernel_ctx() const { return kernel_ctx_; }
  Tensor MakeOutputTensor(int /*slot*/, std::int32_t data_type, const Shape &shape, std::size_t bytes) {
    return ::ONNX_LIGHT_NAMESPACE::core::runtime::MakeOutputTensor(data_type, shape, bytes, nullptr);
  }
  void *execution_allocator() { return nullptr; }
  void Set(const std::string &name, Tensor tensor) {
    tensor.name = name;
    tensors_[name] = std::move(tensor);
  }
  const Tensor &Get(const std::string &name) const {
    auto it = tensors_.find(name);
    if (it == tensors_.end()) {
      throw std::invalid_argument("onnx-light shim: missing tensor '" + name + "'.");
    }
    return it->second;
  }

private:
  KernelContext kernel_ctx_;
  TensorMap tensors_;
};

class KernelBase {
public:
  explicit KernelBase(const KernelContext &ctx) : ctx_(ctx) {}
  virtual ~KernelBase() = default;
  virtual void Run(RuntimeContext &rt) = 0;
  void set_node(const NodeProto &node) { node_ = &node; }

protected:
  const NodeProto *node_ = nullptr;
  KernelContext ctx_;
};

using NodeKernelFn = std::function<std::unique_ptr<KernelBase>(const NodeProto &, RuntimeContext &)>;

struct DispatchEntry {
  symbolic::Device device = symbolic::Device::kUndefined;
  NodeKernelFn fn;
};

// Process-wide table keyed "<domain>:<op_type>".
inline std::map<std::string, DispatchEntry> &KernelDispatchTable() {
  static std::map<std::string, DispatchEntry> table;
  return table;
}

inline void RegisterKernelFn(const std::string &domain, const std::string &op_type,
                             symbolic::Device device, NodeKernelFn fn) {
  KernelDispatchTable()[NormaliseDomain(domain) + ":" + op_type] = DispatchEntry{device, std::move(fn)};
}

// ---- node helpers ------------------------------------------------------------------------
inline void RequireInputCount(const NodeProto &node, int count) {
  if (node.input_size() != count) {
    throw std::invalid_argument(node.op_type() + " expects exactly " + std::to_string(count) + " inputs.");
  }
}
inline void RequireMinInputCount(const NodeProto &node, int count) {
  if (node.input_size() < count) {
    throw std::invalid_argument(node.op_type() + " expects at least " + std::to_string(count) + " inputs.");
  }
}
inline void RequireOutputCount(const NodeProto &node, int count) {
  if (node.output_size() != count) {
    throw std::invalid_argument(node.op_type() + " expects exactly " + std::to_string(count) + " outputs.");
  }
}
inline const Tensor &GetInput(const NodeProto &node, int index, const TensorMap &tensors) {
  if (index >= node.input_size() || node.input(index).empty()) {
    throw std::invalid_argument(node.op_type() + ": required input " + std::to_string(index) + " is missing.");
  }
  auto it = tensors.find(node.input(index));
  if (it == tensors.end()) {
    throw std::invalid_argument(node.op_type() + ": input '" + node.input(index) + "' has no value.");
  }
  return it->second;
}
inline const Tensor *GetOptionalInput(const NodeProto &node, int index, const TensorMap &tensors) {
  if (index >= node.input_size() || node.input(index).empty()) {
    return nullptr;
  }
  auto it = tensors.find(node.input(index));
  return it == tensors.end() ? nullptr : &it->second;
}
inline void SetOutput(const NodeProto &node, int index, Tensor value, RuntimeContext &rt) {
  rt.Set(node.output(index), std::move(value));
}
inline std::int64_t GetAttributeIntOrDefault(const NodeProto &node, const std::string &name,
                                             std::int64_t fallback) {
  for (int i = 0; i < node.attribute_size(); ++i) {
    if (node.attribute(i).name() == name && node.attribute(i).has_i()) {
      return node.attribute(i).i();
    }
  }
  return fallback;
}
inline float GetAttributeFloatOrDefault(const NodeProto &node, const std::string &name, float fallback) {
  for (int i = 0; i < node.attribute_size(); ++i) {
    if (node.attribute(i).name() == name && node.attribute(i).has_f()) {
      return node.attribute(i).f();
    }
  }
  return fallback;
}

} // namespace runtime
} // namespace core
} // namespace ONNX_LIGHT_NAMESPACE
