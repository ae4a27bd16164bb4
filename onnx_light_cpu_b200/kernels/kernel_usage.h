// Kernel usage log: which of this library's kernels a model actually ran. Same surface as
// onnx_light_cpu/kernels/kernel_usage.h:14-48.
#pragma once

#include <string>
#include <string_view>
#include <utility>
#include <vector>

namespace onnx_light_cuda {

/// Appends `name` to the process-wide log (thread safe). Called by every kernel's Run().
void RecordKernelUsage(std::string_view name);
/// Names recorded since the last clear, in call order.
std::vector<std::string> UsedKernelNames();
void ClearUsedKernelNames();
/// Turns recording off for timing runs (dispatch is unchanged).
void SetKernelUsageRecording(bool enabled) noexcept;
/// {op_type, kernel class name} of every registered kernel, from CollectRegisteredKernels().
const std::vector<std::pair<std::string, std::string>> &RegisteredKernelNames();

} // namespace onnx_light_cuda
