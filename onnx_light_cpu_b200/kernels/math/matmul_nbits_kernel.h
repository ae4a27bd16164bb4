// com.microsoft.MatMulNBits for onnx-light, executed on a B200 GPU.
// Operator adapter in the shape of the reference's KernelBase subclasses
// (onnx_light_cpu/kernels/math/integer_matmul_kernel.h:17-32): validation, output
// allocation and tensor plumbing on the host, arithmetic behind the C ABI of
// include/matmulnbits_b200.h. Host tensors in, host tensor out, so a model evaluated through
// onnx-light needs no other change once RegisterAllKernels() has run.
#pragma once

#include "onnx_core/runtime/kernels/kernel_context.h"
#include "onnx_core/runtime/memory/simple_tensor.h"
#include "onnx_core/runtime/runtime_context.h"

#include <cstdint>
#include <memory>

#ifndef ONNX_LIGHT_NAMESPACE
#define ONNX_LIGHT_NAMESPACE onnx_light
#endif

namespace onnx_light_cuda {

/// Attributes of one MatMulNBits node.
struct MatMulNBitsAttributes {
  std::int64_t k = 0;
  std::int64_t n = 0;
  std::int64_t bits = 4;
  std::int64_t block_size = 0;
  std::int64_t accuracy_level = 0;
};

class MatMulNBitsKernel : public ONNX_LIGHT_NAMESPACE::core::runtime::KernelBase {
public:
  explicit MatMulNBitsKernel(const ONNX_LIGHT_NAMESPACE::core::runtime::KernelContext &ctx);
  ~MatMulNBitsKernel() override;

  static constexpr const char *kName = "onnx_light_cuda::MatMulNBits";

  /// Reads K, N, bits, block_size, accuracy_level from the node, inputs
  /// A, B, scales[, zero_points[, g_idx[, bias]]], and sets the single output.
  /// Throws std::invalid_argument on any contract violation (g_idx is rejected).
  void Run(ONNX_LIGHT_NAMESPACE::core::runtime::RuntimeContext &rt) override;

  /// Direct call on tensors, without a session.
  ONNX_LIGHT_NAMESPACE::core::runtime::Tensor
  operator()(const ONNX_LIGHT_NAMESPACE::core::runtime::Tensor &a,
             const ONNX_LIGHT_NAMESPACE::core::runtime::Tensor &b,
             const ONNX_LIGHT_NAMESPACE::core::runtime::Tensor &scales,
             const ONNX_LIGHT_NAMESPACE::core::runtime::Tensor *zero_points,
             const ONNX_LIGHT_NAMESPACE::core::runtime::Tensor *bias,
             const MatMulNBitsAttributes &attributes,
             ONNX_LIGHT_NAMESPACE::core::runtime::RuntimeContext *rt = nullptr) const;

  /// Name of the CUDA kernel the last call dispatched to (diagnostics).
  const char *last_device_kernel() const;

private:
  struct DeviceWeights;
  // Per-node cache of the uploaded constants (constant-weight policy: B, scales, zero_points and
  // bias are initializers). Keyed on their addresses, the attributes and a fingerprint of sampled
  // contents, so a buffer rewritten in place or recycled at the same address is uploaded again.
  std::unique_ptr<DeviceWeights> weights_;
};

/// CUDA device used by kernels constructed after the call (default 0).
void SetMatMulNBitsDevice(int device);
int GetMatMulNBitsDevice();

void RegisterMatMulNBitsKernel();

} // namespace onnx_light_cuda
