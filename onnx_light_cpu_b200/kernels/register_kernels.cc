#include "onnx_light_cpu_b200/kernels/register_kernels.h"

#include "onnx_light_cpu_b200/kernels/kernel_registration.h"
#include "onnx_light_cpu_b200/kernels/math/matmul_nbits_kernel.h"

namespace onnx_light_cuda {

void RegisterAllKernels() {
  KernelRegistrationScope scope; // joins CollectRegisteredKernels()'s scope when one is open
  RegisterMatMulNBitsKernel();
}

} // namespace onnx_light_cuda
