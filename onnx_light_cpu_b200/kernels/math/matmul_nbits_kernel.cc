#include "onnx_light_cpu_b200/kernels/math/matmul_nbits_kernel.h"

#include "include/matmulnbits_b200.h"
#include "onnx_light_cpu_b200/kernels/kernel_registration.h"
#include "onnx_light_cpu_b200/kernels/kernel_usage.h"

#include "onnx_core/runtime/kernels/kernel_dispatch_table.h"
#include "onnx_core/runtime/kernels/node_helpers.h"
#include "onnx_core/symbolic/sym_tensor.h"

#include <atomic>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>

namespace onnx_light_cuda {

namespace rt_ns = ONNX_LIGHT_NAMESPACE::core::runtime;
namespace sym_ns = ONNX_LIGHT_NAMESPACE::core::symbolic;

using NodeProto = ONNX_LIGHT_NAMESPACE::NodeProto;
using rt_ns::DataType;
using rt_ns::NodeKernelFn;
using rt_ns::RuntimeContext;
using rt_ns::Shape;
using rt_ns::Tensor;

namespace {

std::atomic<int> g_device{0};

[[noreturn]] void Reject(const std::string &what) {
  throw std::invalid_argument(std::string(MatMulNBitsKernel::kName) + ": " + what);
}

bool IsType(const Tensor &t, DataType type) { return t.data_type == static_cast<std::int32_t>(type); }

// Converts a C ABI status into the exception the reference's kernels use.
void Check(int status) {
  if (status == MNB_OK) {
    return;
  }
  const std::string message = mnb_last_error();
  if (status == MNB_ERR_INVALID_ARGUMENT || status == MNB_ERR_UNSUPPORTED) {
    throw std::invalid_argument(message);
  }
  throw std::runtime_error(message);
}

} // namespace

namespace {

// Fingerprint of a constant operand: its size and 64-bit words sampled at up to 512 evenly spaced
// places (always the first and the last), FNV-1a. A microsecond per Run; it tells a buffer that
// was rewritten in place, or freed and reallocated at the same address with other contents, from
// the one that was uploaded. (A rewrite that leaves every sampled word as it was goes unnoticed:
// the constant operands of this operator are initializers, which a runtime does not modify.)
std::uint64_t Fingerprint(const std::uint8_t *data, std::size_t bytes) {
  std::uint64_t h = 1469598103934665603ull ^ bytes;
  if (data == nullptr || bytes == 0) {
    return h;
  }
  auto mix = [&h](std::uint64_t v) {
    h ^= v;
    h *= 1099511628211ull;
  };
  const std::size_t words = bytes / 8;
  if (words == 0) {
    for (std::size_t i = 0; i < bytes; ++i) {
      mix(data[i]);
    }
    return h;
  }
  const std::size_t samples = words < 512 ? words : 512;
  for (std::size_t i = 0; i < samples; ++i) {
    const std::size_t at = samples > 1 ? i * (words - 1) / (samples - 1) : 0;
    std::uint64_t v;
    std::memcpy(&v, data + at * 8, 8);
    mix(v);
  }
  for (std::size_t i = words * 8; i < bytes; ++i) {
    mix(data[i]);
  }
  return h;
}

std::uint64_t FingerprintOf(const Tensor *t) {
  return t != nullptr ? Fingerprint(reinterpret_cast<const std::uint8_t *>(t->bytes()), t->size_bytes()) : 0;
}

} // namespace

// The uploaded constants of the node, rebuilt when the initializer tensors change: another
// address, other attributes, or another fingerprint of their contents.
struct MatMulNBitsKernel::DeviceWeights {
  std::mutex mutex;
  mnb_weights *handle = nullptr;
  const void *key_b = nullptr;
  const void *key_scales = nullptr;
  const void *key_zp = nullptr;
  const void *key_bias = nullptr;
  MatMulNBitsAttributes key_attrs;
  std::uint64_t stamp[4] = {0, 0, 0, 0};
  const char *last_kernel = "";

  ~DeviceWeights() { mnb_weights_destroy(handle); }

  bool Matches(const Tensor &b, const Tensor &scales, const Tensor *zp, const Tensor *bias,
               const MatMulNBitsAttributes &a) const {
    return handle != nullptr && key_b == b.bytes() && key_scales == scales.bytes() &&
           key_zp == (zp != nullptr ? zp->bytes() : nullptr) &&
           key_bias == (bias != nullptr ? bias->bytes() : nullptr) && key_attrs.k == a.k &&
           key_attrs.n == a.n && key_attrs.bits == a.bits && key_attrs.block_size == a.block_size &&
           stamp[0] == FingerprintOf(&b) && stamp[1] == FingerprintOf(&scales) && stamp[2] == FingerprintOf(zp) &&
           stamp[3] == FingerprintOf(bias);
  }
};

MatMulNBitsKernel::MatMulNBitsKernel(const rt_ns::KernelContext &ctx)
    : KernelBase(ctx), weights_(std::make_unique<DeviceWeights>()) {}

MatMulNBitsKernel::~MatMulNBitsKernel() = default;

const char *MatMulNBitsKernel::last_device_kernel() const { return weights_->last_kernel; }

void SetMatMulNBitsDevice(int device) { g_device.store(device); }
int GetMatMulNBitsDevice() { return g_device.load(); }

Tensor MatMulNBitsKernel::operator()(const Tensor &a, const Tensor &b, const Tensor &scales,
                                     const Tensor *zero_points, const Tensor *bias,
                                     const MatMulNBitsAttributes &attrs, RuntimeContext *rt) const {
  if (attrs.k <= 0 || attrs.n <= 0) {
    Reject("attributes K and N must be positive.");
  }
  if (attrs.bits != 4 && attrs.bits != 8) {
    Reject("attribute bits must be 4 or 8.");
  }
  if (attrs.block_size < 16 || (attrs.block_size & (attrs.block_size - 1)) != 0) {
    Reject("attribute block_size must be a power of two >= 16.");
  }
  if (attrs.accuracy_level != 0 && attrs.accuracy_level != 4) {
    Reject("attribute accuracy_level must be 0 or 4.");
  }
  if (!IsType(a, DataType::FLOAT)) {
    Reject("input A must have FLOAT dtype.");
  }
  if (!IsType(b, DataType::UINT8)) {
    Reject("input B must have UINT8 dtype.");
  }
  if (!IsType(scales, DataType::FLOAT)) {
    Reject("input scales must have FLOAT dtype.");
  }
  if (zero_points != nullptr && !IsType(*zero_points, DataType::UINT8)) {
    Reject("input zero_points must have UINT8 dtype (packed codes).");
  }
  if (bias != nullptr && !IsType(*bias, DataType::FLOAT)) {
    Reject("input bias must have FLOAT dtype.");
  }
  if (a.shape.empty() || a.shape.back() != attrs.k) {
    Reject("the last dimension of A must equal attribute K.");
  }
  const std::int64_t n_blocks = (attrs.k + attrs.block_size - 1) / attrs.block_size;
  const std::int64_t blob = attrs.block_size * attrs.bits / 8;
  if (b.element_count() != attrs.n * n_blocks * blob) {
    Reject("B must hold N * ceil(K/block_size) * block_size*bits/8 bytes.");
  }
  if (scales.element_count() != attrs.n * n_blocks) {
    Reject("scales must hold N * ceil(K/block_size) values.");
  }
  const std::int64_t zp_row = (n_blocks * attrs.bits + 7) / 8;
  if (zero_points != nullptr && zero_points->element_count() != attrs.n * zp_row) {
    Reject("zero_points must hold N * ceil(ceil(K/block_size)*bits/8) bytes.");
  }
  if (bias != nullptr && bias->element_count() != attrs.n) {
    Reject("bias must hold N values.");
  }

  Shape out_shape(a.shape.begin(), a.shape.end() - 1);
  out_shape.push_back(attrs.n);
  const std::int64_t m = a.element_count() / attrs.k;
  const std::size_t out_bytes = static_cast<std::size_t>(m) * static_cast<std::size_t>(attrs.n) * sizeof(float);
  Tensor y = rt != nullptr
                 ? rt->MakeOutputTensor(0, static_cast<std::int32_t>(DataType::FLOAT), out_shape, out_bytes)
                 : rt_ns::MakeOutputTensor(static_cast<std::int32_t>(DataType::FLOAT), out_shape, out_bytes,
                                           nullptr);
  if (m == 0) {
    return y;
  }

  DeviceWeights &cache = *weights_;
  std::lock_guard<std::mutex> guard(cache.mutex);
  if (!cache.Matches(b, scales, zero_points, bias, attrs)) {
    mnb_weights_destroy(cache.handle);
    cache.handle = nullptr;
    Check(mnb_weights_create(GetMatMulNBitsDevice(), b.AsUint8(), scales.AsFloat(),
                             zero_points != nullptr ? zero_points->AsUint8() : nullptr,
                             bias != nullptr ? bias->AsFloat() : nullptr, attrs.n, attrs.k,
                             static_cast<int>(attrs.bits), static_cast<int>(attrs.block_size),
                             &cache.handle));
    cache.key_b = b.bytes();
    cache.key_scales = scales.bytes();
    cache.key_zp = zero_points != nullptr ? zero_points->bytes() : nullptr;
    cache.key_bias = bias != nullptr ? bias->bytes() : nullptr;
    cache.key_attrs = attrs;
    cache.stamp[0] = FingerprintOf(&b);
    cache.stamp[1] = FingerprintOf(&scales);
    cache.stamp[2] = FingerprintOf(zero_points);
    cache.stamp[3] = FingerprintOf(bias);
  }
  Check(mnb_matmul_host(cache.handle, a.AsFloat(), m, static_cast<int>(attrs.accuracy_level),
                        MNB_PATH_AUTO, y.AsFloat()));
  cache.last_kernel = mnb_last_kernel();
  return y;
}

void MatMulNBitsKernel::Run(RuntimeContext &rt) {
  RecordKernelUsage(kName);
  const NodeProto &node = *node_;
  rt_ns::RequireMinInputCount(node, 3);
  if (node.input_size() > 6) {
    Reject("expects at most six inputs.");
  }
  rt_ns::RequireOutputCount(node, 1);
  MatMulNBitsAttributes attrs;
  attrs.k = rt_ns::GetAttributeIntOrDefault(node, "K", 0);
  attrs.n = rt_ns::GetAttributeIntOrDefault(node, "N", 0);
  attrs.bits = rt_ns::GetAttributeIntOrDefault(node, "bits", 4);
  attrs.block_size = rt_ns::GetAttributeIntOrDefault(node, "block_size", 0);
  attrs.accuracy_level = rt_ns::GetAttributeIntOrDefault(node, "accuracy_level", 0);
  const Tensor &a = rt_ns::GetInput(node, 0, rt.tensors());
  const Tensor &b = rt_ns::GetInput(node, 1, rt.tensors());
  const Tensor &scales = rt_ns::GetInput(node, 2, rt.tensors());
  const Tensor *zero_points = rt_ns::GetOptionalInput(node, 3, rt.tensors());
  if (rt_ns::GetOptionalInput(node, 4, rt.tensors()) != nullptr) {
    Reject("input g_idx is not supported.");
  }
  const Tensor *bias = rt_ns::GetOptionalInput(node, 5, rt.tensors());
  rt_ns::SetOutput(node, 0, (*this)(a, b, scales, zero_points, bias, attrs, &rt), rt);
}

void RegisterMatMulNBitsKernel() {
  NodeKernelFn factory = [](const NodeProto &node, RuntimeContext &rt) -> std::unique_ptr<rt_ns::KernelBase> {
    auto kernel = std::make_unique<MatMulNBitsKernel>(rt.kernel_ctx());
    kernel->set_node(node);
    return kernel;
  };
  KernelRegistration info;
  info.domain = "com.microsoft";
  info.op_type = "MatMulNBits";
  info.device = sym_ns::Device::kCPU;
  info.kernel_name = MatMulNBitsKernel::kName;
  info.types = {DataType::FLOAT};
  RegisterKernel(std::move(info), std::move(factory));
}

} // namespace onnx_light_cuda
