// Counterpart of onnx_light_cpu/kernels/register_kernels.h:22.
#pragma once

namespace onnx_light_cuda {

/// Registers every kernel of this library (currently com.microsoft.MatMulNBits) into
/// onnx-light's shared dispatch table. Idempotent.
void RegisterAllKernels();

} // namespace onnx_light_cuda
