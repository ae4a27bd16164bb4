#include "onnx_light_cpu_b200/kernels/kernel_usage.h"

#include "onnx_light_cpu_b200/kernels/kernel_registration.h"

#include <atomic>
#include <mutex>

namespace onnx_light_cuda {

namespace {

struct UsageLog {
  std::mutex mutex;
  std::vector<std::string> names;
  std::atomic<bool> enabled{true};
};

UsageLog &Log() {
  static UsageLog log;
  return log;
}

} // namespace

void RecordKernelUsage(std::string_view name) {
  UsageLog &log = Log();
  if (!log.enabled.load(std::memory_order_relaxed)) {
    return;
  }
  std::lock_guard<std::mutex> guard(log.mutex);
  log.names.emplace_back(name);
}

std::vector<std::string> UsedKernelNames() {
  UsageLog &log = Log();
  std::lock_guard<std::mutex> guard(log.mutex);
  return log.names;
}

void ClearUsedKernelNames() {
  UsageLog &log = Log();
  std::lock_guard<std::mutex> guard(log.mutex);
  log.names.clear();
}

void SetKernelUsageRecording(bool enabled) noexcept {
  Log().enabled.store(enabled, std::memory_order_relaxed);
}

const std::vector<std::pair<std::string, std::string>> &RegisteredKernelNames() {
  static const std::vector<std::pair<std::string, std::string>> names = [] {
    std::vector<std::pair<std::string, std::string>> out;
    for (const KernelRegistration &item : CollectRegisteredKernels()) {
      out.emplace_back(item.op_type, item.kernel_name);
    }
    return out;
  }();
  return names;
}

} // namespace onnx_light_cuda
