#include "onnx_light_cpu_b200/kernels/kernel_registration.h"

#include "onnx_light_cpu_b200/kernels/register_kernels.h"

#include "onnx_proto/onnx_helper.h"

#include <algorithm>
#include <set>
#include <stdexcept>
#include <tuple>
#include <utility>

namespace onnx_light_cuda {

namespace rt_ns = ONNX_LIGHT_NAMESPACE::core::runtime;
namespace sym_ns = ONNX_LIGHT_NAMESPACE::core::symbolic;

namespace {

// State of the registration pass running on this thread.
struct PassState {
  int depth = 0;
  std::vector<KernelRegistration> *inventory = nullptr;
  std::set<std::tuple<std::string, std::string, std::int32_t>> seen;
};

PassState &Pass() {
  static thread_local PassState state;
  return state;
}

} // namespace

KernelRegistrationScope::KernelRegistrationScope(std::vector<KernelRegistration> *inventory) {
  PassState &pass = Pass();
  if (pass.depth == 0) {
    outermost_ = true;
    pass.inventory = inventory;
    pass.seen.clear();
  }
  ++pass.depth;
}

KernelRegistrationScope::~KernelRegistrationScope() {
  PassState &pass = Pass();
  --pass.depth;
  if (outermost_) {
    pass.inventory = nullptr;
    pass.seen.clear();
  }
}

void RegisterKernel(KernelRegistration info, rt_ns::NodeKernelFn fn) {
  info.domain = ONNX_LIGHT_NAMESPACE::NormaliseDomain(info.domain);
  // A direct call outside any pass is a pass of its own.
  KernelRegistrationScope single_call_scope;
  PassState &pass = Pass();
  const auto key = std::make_tuple(info.domain, info.op_type, static_cast<std::int32_t>(info.device));
  if (!pass.seen.insert(key).second) {
    throw std::invalid_argument("onnx_light_cuda::RegisterKernel: duplicate registration for domain '" +
                                info.domain + "', operator '" + info.op_type + "', device " +
                                sym_ns::DeviceName(info.device) + ".");
  }
  if (pass.inventory != nullptr) {
    pass.inventory->push_back(std::move(info));
    return;
  }
  rt_ns::RegisterKernelFn(info.domain, info.op_type, info.device, std::move(fn));
}

std::vector<KernelRegistration> CollectRegisteredKernels() {
  std::vector<KernelRegistration> inventory;
  {
    KernelRegistrationScope scope(&inventory);
    RegisterAllKernels();
  }
  std::sort(inventory.begin(), inventory.end(), [](const KernelRegistration &l, const KernelRegistration &r) {
    return std::tie(l.domain, l.op_type, l.device, l.kernel_name) <
           std::tie(r.domain, r.op_type, r.device, r.kernel_name);
  });
  return inventory;
}

} // namespace onnx_light_cuda
