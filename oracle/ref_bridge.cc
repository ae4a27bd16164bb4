// TEST INFRASTRUCTURE ONLY. C-ABI bridge over the reference's own compiled sources so that
// Python tests can call the real reference functions that pin this project's integer
// conventions. Compiled by oracle/Makefile together with the reference translation units,
// read in place from the reference checkout (never copied), into oracle/_ref/.
//
// Reference entry points bridged:
//   IntegerMatMul4Bit2D  onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:276-299
//   IntegerMatMul2D      onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:236-274
//   FloatToBFloat16Bits  onnx_light_cpu/impl/math/half_conversion.h:80-87
//   ExecuteRanges        onnx_light_cpu/impl/execution.h:146-176, with an executor injected through
//                        ExecutionExecutorScope (:31-40) the way unittests/cc/test_execution.cc:24-75
//                        injects its InlineExecutor; here the executor is a persistent std::thread pool

#include "onnx_light_cpu/impl/execution.h"
#include "onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.h"
#include "onnx_light_cpu/impl/math/half_conversion.h"

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace {

// The executor handed to the reference: `threads` - 1 parked std::threads plus the caller. It plays
// the part of onnx-light's per-session CpuExecutor (which the reference borrows and never owns).
class ThreadExecutor {
public:
  explicit ThreadExecutor(int threads) : threads_(threads) {
    for (int i = 1; i < threads; ++i) {
      workers_.emplace_back([this] { Loop(); });
    }
    view_.context = this;
    view_.effective_threads = threads;
    view_.run_blocks = [](void *context, int64_t num_blocks, void *task_context,
                          onnx_light_cpu::ExecutionBlockFn task) {
      static_cast<ThreadExecutor *>(context)->Run(num_blocks, task_context, task);
    };
  }
  ~ThreadExecutor() {
    {
      std::lock_guard<std::mutex> lock(mutex_);
      stop_ = true;
      ++generation_;
    }
    wake_.notify_all();
    for (auto &t : workers_) {
      t.join();
    }
  }
  int threads() const { return threads_; }
  const onnx_light_cpu::ExecutionExecutorView *view() const { return &view_; }

private:
  void Run(int64_t blocks, void *task_context, onnx_light_cpu::ExecutionBlockFn task) {
    {
      std::lock_guard<std::mutex> lock(mutex_);
      task_context_ = task_context;
      task_ = task;
      blocks_ = blocks;
      next_.store(0);
      pending_ = static_cast<int>(workers_.size());
      ++generation_;
    }
    wake_.notify_all();
    Drain();
    std::unique_lock<std::mutex> lock(mutex_);
    done_.wait(lock, [this] { return pending_ == 0; });
  }
  void Drain() {
    for (;;) {
      const int64_t block = next_.fetch_add(1);
      if (block >= blocks_) {
        return;
      }
      task_(task_context_, block);
    }
  }
  void Loop() {
    std::uint64_t seen = 0;
    for (;;) {
      {
        std::unique_lock<std::mutex> lock(mutex_);
        wake_.wait(lock, [&] { return generation_ != seen; });
        seen = generation_;
        if (stop_) {
          return;
        }
      }
      Drain();
      {
        std::lock_guard<std::mutex> lock(mutex_);
        --pending_;
      }
      done_.notify_one();
    }
  }
  const int threads_;
  std::vector<std::thread> workers_;
  std::mutex mutex_;
  std::condition_variable wake_, done_;
  std::uint64_t generation_ = 0;
  bool stop_ = false;
  int pending_ = 0;
  void *task_context_ = nullptr;
  onnx_light_cpu::ExecutionBlockFn task_ = nullptr;
  int64_t blocks_ = 0;
  std::atomic<int64_t> next_{0};
  onnx_light_cpu::ExecutionExecutorView view_;
};

std::mutex g_executor_mutex;
std::unique_ptr<ThreadExecutor> g_executor;
std::atomic<long long> g_dispatches{0};

} // namespace

extern "C" {

void ref_integer_matmul_4bit_2d(const std::uint8_t *a, int a_signed, const std::uint8_t *b,
                                int b_signed, std::int32_t *c, std::int64_t rows,
                                std::int64_t cols, std::int64_t depth,
                                const std::int32_t *a_zero_point, std::int64_t a_zero_point_count,
                                const std::int32_t *b_zero_point,
                                std::int64_t b_zero_point_count) {
  onnx_light_cpu::IntegerMatMul4Bit2D(a, a_signed != 0, b, b_signed != 0, c, rows, cols, depth,
                                      a_zero_point, a_zero_point_count, b_zero_point,
                                      b_zero_point_count);
}

void ref_integer_matmul_2d(const std::uint8_t *a, int a_signed, const std::uint8_t *b,
                           int b_signed, std::int32_t *c, std::int64_t rows, std::int64_t cols,
                           std::int64_t depth, const std::int32_t *a_zero_point,
                           std::int64_t a_zero_point_count, const std::int32_t *b_zero_point,
                           std::int64_t b_zero_point_count) {
  onnx_light_cpu::IntegerMatMul2D(a, a_signed != 0, b, b_signed != 0, c, rows, cols, depth,
                                  a_zero_point, a_zero_point_count, b_zero_point,
                                  b_zero_point_count);
}

std::uint16_t ref_float_to_bf16_bits(float value) {
  return onnx_light_cpu::detail::FloatToBFloat16Bits(value);
}

int ref_uses_vnni() { return onnx_light_cpu::IntegerMatMul2DUsesVnni() ? 1 : 0; }

// Runs fn(context, begin, end) over [0, total) through the reference's ExecuteRanges, with a
// persistent std::thread executor of `threads` participants injected for the duration of the call.
// The cost per unit is chosen so that the reference's grain (32768 work units) never collapses a
// column panel into a single block for the sizes this checker is used on.
void ref_execute_ranges(std::int64_t total, int threads, void *context,
                        void (*fn)(void *, std::int64_t, std::int64_t)) {
  std::lock_guard<std::mutex> lock(g_executor_mutex);
  if (g_executor == nullptr || g_executor->threads() != threads) {
    g_executor.reset(new ThreadExecutor(threads));
  }
  onnx_light_cpu::ExecutionExecutorScope scope(g_executor->view());
  g_dispatches.fetch_add(1);
  onnx_light_cpu::ExecuteRanges(total, 1.0e6, [&](std::int64_t begin, std::int64_t end) { fn(context, begin, end); });
}

long long ref_execute_ranges_calls() { return g_dispatches.load(); }
}
