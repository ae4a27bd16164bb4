// Registration of this library's kernels into onnx-light's process-wide dispatch table.
// Same public surface as the reference plug-in (onnx_light_cpu/kernels/kernel_registration.h:
// KernelRegistration :30-56, KernelRegistrationScope :73-95, RegisterKernel :113,
// CollectRegisteredKernels :123), re-implemented for the CUDA library.
#pragma once

#include "onnx_core/runtime/kernels/kernel_dispatch_table.h"
#include "onnx_core/runtime/memory/simple_tensor.h"
#include "onnx_core/symbolic/sym_tensor.h"

#include <cstdint>
#include <optional>
#include <string>
#include <vector>

#ifndef ONNX_LIGHT_NAMESPACE
#define ONNX_LIGHT_NAMESPACE onnx_light
#endif

namespace onnx_light_cuda {

/// What one Register*Kernel() call installs: operator identity, the device the runtime
/// dispatches on, the C++ kernel class name and the accepted element types.
struct KernelRegistration {
  std::string domain;  ///< "" is normalised to "ai.onnx"
  std::string op_type;
  /// Host tensors go in and come out, so the runtime sees a CPU-device kernel; the GPU is an
  /// implementation detail behind the operator.
  ONNX_LIGHT_NAMESPACE::core::symbolic::Device device =
      ONNX_LIGHT_NAMESPACE::core::symbolic::Device::kCPU;
  std::string kernel_name;
  std::vector<ONNX_LIGHT_NAMESPACE::core::runtime::DataType> types;
  std::optional<std::int64_t> since_version;
  std::optional<std::int64_t> until_version;
};

/// Bounds one registration pass on the calling thread. The outermost scope decides whether
/// the pass installs kernels (inventory == nullptr) or only records their metadata; nested
/// scopes join the outer one. Duplicate (domain, op_type, device) triples inside one pass
/// throw std::invalid_argument.
class KernelRegistrationScope {
public:
  explicit KernelRegistrationScope(std::vector<KernelRegistration> *inventory = nullptr);
  ~KernelRegistrationScope();
  KernelRegistrationScope(const KernelRegistrationScope &) = delete;
  KernelRegistrationScope &operator=(const KernelRegistrationScope &) = delete;

private:
  bool outermost_ = false;
};

/// Installs `fn` for (info.domain, info.op_type, info.device), or - while
/// CollectRegisteredKernels() runs on this thread - records `info` only.
void RegisterKernel(KernelRegistration info, ONNX_LIGHT_NAMESPACE::core::runtime::NodeKernelFn fn);

/// Metadata of every kernel RegisterAllKernels() would install, sorted by
/// (domain, op_type, device, kernel_name). Never touches the dispatch table.
std::vector<KernelRegistration> CollectRegisteredKernels();

} // namespace onnx_light_cuda
