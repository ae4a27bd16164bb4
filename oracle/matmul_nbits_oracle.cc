// TEST INFRASTRUCTURE ONLY - see matmul_nbits_oracle.h for the contract, what is pinned
// against the reference and what is not ("parity unpinned" for the operator as a whole: the
// reference has no MatMulNBits).
//
// Conventions followed, by reference file:line
//   nibble order / tail nibble     onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:60-93
//   exact integer (value - zp)     onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:208-223
//   bf16 RNE + NaN quieting        onnx_light_cpu/impl/math/half_conversion.h:80-87
//   N column panels across threads onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258
//   argument validation style      onnx_light_cpu/kernels/math/integer_matmul_kernel.cc:298-314

#include "matmul_nbits_oracle.h"

#include <algorithm>
#include <cmath>
#include <limits>
#include <cstring>
#include <atomic>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace {

struct QuantView {
  const std::uint8_t *b;
  const std::uint8_t *zp; // may be null
  std::int64_t n, k;
  int bits, block_size;
  std::int64_t n_blocks, blob_bytes, row_bytes, zp_row_bytes;
  int default_zp;
};

bool MakeView(const std::uint8_t *b, const std::uint8_t *zp, std::int64_t n, std::int64_t k,
              int bits, int block_size, QuantView *view) {
  if (b == nullptr || n < 0 || k < 0) {
    return false;
  }
  if (bits != 4 && bits != 8) {
    return false;
  }
  if (block_size < 16 || (block_size & (block_size - 1)) != 0) {
    return false;
  }
  view->b = b;
  view->zp = zp;
  view->n = n;
  view->k = k;
  view->bits = bits;
  view->block_size = block_size;
  view->n_blocks = (k + block_size - 1) / block_size;
  view->blob_bytes = static_cast<std::int64_t>(block_size) * bits / 8;
  view->row_bytes = view->n_blocks * view->blob_bytes;
  view->zp_row_bytes = (view->n_blocks * bits + 7) / 8;
  view->default_zp = 1 << (bits - 1);
  return true;
}

// Quantized code of logical element (row, kk): low nibble holds the even index.
inline int ReadCode(const QuantView &v, std::int64_t row, std::int64_t kk) {
  const std::int64_t block = kk / v.block_size;
  const std::int64_t within = kk - block * v.block_size;
  const std::uint8_t *blob = v.b + row * v.row_bytes + block * v.blob_bytes;
  if (v.bits == 8) {
    return blob[within];
  }
  const std::uint8_t byte = blob[within >> 1];
  return (within & 1) ? (byte >> 4) : (byte & 0x0f);
}

inline int ReadZeroPoint(const QuantView &v, std::int64_t row, std::int64_t block) {
  if (v.zp == nullptr) {
    return v.default_zp;
  }
  const std::uint8_t *zrow = v.zp + row * v.zp_row_bytes;
  if (v.bits == 8) {
    return zrow[block];
  }
  const std::uint8_t byte = zrow[block >> 1];
  return (block & 1) ? (byte >> 4) : (byte & 0x0f);
}

// Worker threads that live as long as the process: started on first use (and again when another
// thread count is asked for), parked on a condition variable between calls. A call hands out
// block indices through an atomic counter and returns when every block is done; the calling
// thread takes blocks too. Thread start-up is therefore outside any timed call after the first.
class WorkerPool {
public:
  using BlockFn = void (*)(void *, std::int64_t);

  static WorkerPool &Get(int threads) {
    static std::mutex guard;
    static std::unique_ptr<WorkerPool> pool;
    std::lock_guard<std::mutex> lock(guard);
    if (pool == nullptr || pool->threads_ != threads) {
      pool.reset(new WorkerPool(threads));
    }
    return *pool;
  }

  ~WorkerPool() {
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

  void Run(std::int64_t blocks, void *context, BlockFn fn) {
    if (blocks <= 0) {
      return;
    }
    std::lock_guard<std::mutex> serial(run_mutex_);  // one parallel region at a time
    {
      std::lock_guard<std::mutex> lock(mutex_);
      context_ = context;
      fn_ = fn;
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

private:
  explicit WorkerPool(int threads) : threads_(threads) {
    for (int i = 1; i < threads; ++i) {
      workers_.emplace_back([this] { Loop(); });
    }
  }

  void Drain() {
    for (;;) {
      const std::int64_t block = next_.fetch_add(1);
      if (block >= blocks_) {
        return;
      }
      fn_(context_, block);
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
  std::mutex mutex_, run_mutex_;
  std::condition_variable wake_, done_;
  std::uint64_t generation_ = 0;
  bool stop_ = false;
  int pending_ = 0;
  void *context_ = nullptr;
  BlockFn fn_ = nullptr;
  std::int64_t blocks_ = 0;
  std::atomic<std::int64_t> next_{0};
};

// Optional outside dispatcher for the column panels: runner(total, threads, context, fn) must call
// fn(context, begin, end) over disjoint ranges that cover [0, total). Set from the test harness to
// the bridge that goes through the reference's ExecuteRanges (onnx_light_cpu/impl/execution.h:146-176).
using RangeFn = void (*)(void *, std::int64_t, std::int64_t);
using RangeRunner = void (*)(std::int64_t, int, void *, RangeFn);
std::atomic<RangeRunner> g_range_runner{nullptr};

// Splits the n output columns into one contiguous panel per worker ("stream B once, partition N",
// onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258).
template <typename Fn> void ForColumnPanels(std::int64_t n, int threads, Fn fn) {
  const int hw = std::max(1, threads);
  const std::int64_t workers = std::min<std::int64_t>(hw, std::max<std::int64_t>(n, 1));
  if (workers <= 1) {
    fn(std::int64_t{0}, n);
    return;
  }
  if (const RangeRunner runner = g_range_runner.load()) {
    runner(n, hw, &fn, [](void *context, std::int64_t begin, std::int64_t end) {
      (*static_cast<Fn *>(context))(begin, end);
    });
    return;
  }
  const std::int64_t panel = (n + workers - 1) / workers;
  struct Task {
    Fn *fn;
    std::int64_t panel, n;
  } task{&fn, panel, n};
  WorkerPool::Get(hw).Run((n + panel - 1) / panel, &task, [](void *context, std::int64_t block) {
    auto *t = static_cast<Task *>(context);
    const std::int64_t begin = block * t->panel;
    (*t->fn)(begin, std::min(t->n, begin + t->panel));
  });
}

inline std::uint16_t ToBf16(float value) {
  std::uint32_t u;
  std::memcpy(&u, &value, sizeof(u));
  if ((u & 0x7fffffffu) > 0x7f800000u) { // NaN: keep payload top bits, force quiet bit
    return static_cast<std::uint16_t>((u >> 16) | 0x0040u);
  }
  const std::uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return static_cast<std::uint16_t>(u >> 16);
}

inline float FromBf16(std::uint16_t bits) {
  const std::uint32_t u = static_cast<std::uint32_t>(bits) << 16;
  float value;
  std::memcpy(&value, &u, sizeof(value));
  return value;
}

} // namespace

extern "C" {

// Installs (or, with nullptr, removes) the outside dispatcher of the column panels.
void nbits_oracle_set_range_runner(void (*runner)(std::int64_t, int, void *, void (*)(void *, std::int64_t, std::int64_t))) {
  g_range_runner.store(runner);
}

std::uint16_t nbits_oracle_float_to_bf16_bits(float value) { return ToBf16(value); }
float nbits_oracle_bf16_bits_to_float(std::uint16_t bits) { return FromBf16(bits); }

int nbits_oracle_hardware_threads() {
  const unsigned hw = std::thread::hardware_concurrency();
  return hw == 0 ? 1 : static_cast<int>(hw);
}

int nbits_oracle_dequant_int(const std::uint8_t *b, const std::uint8_t *zero_points,
                             std::int64_t n, std::int64_t k, int bits, int block_size,
                             std::int32_t *out) {
  QuantView v;
  if (!MakeView(b, zero_points, n, k, bits, block_size, &v) || out == nullptr) {
    return 1;
  }
  for (std::int64_t row = 0; row < n; ++row) {
    for (std::int64_t kk = 0; kk < k; ++kk) {
      out[row * k + kk] = ReadCode(v, row, kk) - ReadZeroPoint(v, row, kk / block_size);
    }
  }
  return 0;
}

int nbits_oracle_matmul_f32(const float *a, const std::uint8_t *b, const float *scales,
                            const std::uint8_t *zero_points, const float *bias, std::int64_t m,
                            std::int64_t n, std::int64_t k, int bits, int block_size, float *y,
                            int threads) {
  QuantView v;
  if (!MakeView(b, zero_points, n, k, bits, block_size, &v) || a == nullptr ||
      scales == nullptr || y == nullptr) {
    return 1;
  }
  ForColumnPanels(n, threads, [&](std::int64_t begin, std::int64_t end) {
    for (std::int64_t col = begin; col < end; ++col) {
      for (std::int64_t row = 0; row < m; ++row) {
        float acc = 0.0f;
        for (std::int64_t kk = 0; kk < k; ++kk) {
          const std::int64_t block = kk / block_size;
          const float w = static_cast<float>(ReadCode(v, col, kk) - ReadZeroPoint(v, col, block)) *
                          scales[col * v.n_blocks + block];
          acc = std::fmaf(a[row * k + kk], w, acc);
        }
        y[row * n + col] = bias != nullptr ? acc + bias[col] : acc;
      }
    }
  });
  return 0;
}

int nbits_oracle_matmul_f64(const float *a, const std::uint8_t *b, const float *scales,
                            const std::uint8_t *zero_points, const float *bias, std::int64_t m,
                            std::int64_t n, std::int64_t k, int bits, int block_size, double *y,
                            int threads) {
  QuantView v;
  if (!MakeView(b, zero_points, n, k, bits, block_size, &v) || a == nullptr ||
      scales == nullptr || y == nullptr) {
    return 1;
  }
  ForColumnPanels(n, threads, [&](std::int64_t begin, std::int64_t end) {
    for (std::int64_t col = begin; col < end; ++col) {
      for (std::int64_t row = 0; row < m; ++row) {
        double acc = 0.0;
        for (std::int64_t kk = 0; kk < k; ++kk) {
          const std::int64_t block = kk / block_size;
          const double w =
              static_cast<double>(ReadCode(v, col, kk) - ReadZeroPoint(v, col, block)) *
              static_cast<double>(scales[col * v.n_blocks + block]);
          acc += static_cast<double>(a[row * k + kk]) * w;
        }
        y[row * n + col] = bias != nullptr ? acc + static_cast<double>(bias[col]) : acc;
      }
    }
  });
  return 0;
}

int nbits_oracle_matmul_bf16(const float *a, const std::uint8_t *b, const float *scales,
                             const std::uint8_t *zero_points, const float *bias, std::int64_t m,
                             std::int64_t n, std::int64_t k, int bits, int block_size, double *y,
                             int threads) {
  QuantView v;
  if (!MakeView(b, zero_points, n, k, bits, block_size, &v) || a == nullptr ||
      scales == nullptr || y == nullptr) {
    return 1;
  }
  std::vector<float> a_rounded(static_cast<std::size_t>(m * k));
  for (std::int64_t i = 0; i < m * k; ++i) {
    a_rounded[static_cast<std::size_t>(i)] = FromBf16(ToBf16(a[i]));
  }
  ForColumnPanels(n, threads, [&](std::int64_t begin, std::int64_t end) {
    std::vector<float> w_row(static_cast<std::size_t>(k));
    for (std::int64_t col = begin; col < end; ++col) {
      for (std::int64_t kk = 0; kk < k; ++kk) {
        const std::int64_t block = kk / block_size;
        const float w = static_cast<float>(ReadCode(v, col, kk) - ReadZeroPoint(v, col, block)) *
                        scales[col * v.n_blocks + block];
        w_row[static_cast<std::size_t>(kk)] = FromBf16(ToBf16(w));
      }
      for (std::int64_t row = 0; row < m; ++row) {
        double acc = 0.0;
        const float *a_row = a_rounded.data() + row * k;
        for (std::int64_t kk = 0; kk < k; ++kk) {
          acc += static_cast<double>(a_row[kk]) *
                 static_cast<double>(w_row[static_cast<std::size_t>(kk)]);
        }
        y[row * n + col] = bias != nullptr ? acc + static_cast<double>(bias[col]) : acc;
      }
    }
  });
  return 0;
}

int nbits_oracle_quantize_a(const float *a, std::int64_t m, std::int64_t k, int block_size,
                            std::int8_t *aq, float *a_scales) {
  if (a == nullptr || aq == nullptr || a_scales == nullptr || block_size <= 0) {
    return 1;
  }
  const std::int64_t n_blocks = (k + block_size - 1) / block_size;
  for (std::int64_t row = 0; row < m; ++row) {
    for (std::int64_t block = 0; block < n_blocks; ++block) {
      const std::int64_t k0 = block * block_size;
      const std::int64_t k1 = std::min<std::int64_t>(k, k0 + block_size);
      float amax = 0.0f;
      bool bad = false; // a NaN or an infinity in the block
      for (std::int64_t kk = k0; kk < k1; ++kk) {
        const float v = std::fabs(a[row * k + kk]);
        amax = std::fmax(amax, v);
        bad = bad || !(v <= std::numeric_limits<float>::max());
      }
      // A block with a non-finite activation has no int8 form: scale NaN, codes 0, so that every
      // output of the token is NaN (as at accuracy_level 0).
      const float sa = bad ? std::numeric_limits<float>::quiet_NaN() : amax / 127.0f;
      a_scales[row * n_blocks + block] = sa;
      for (std::int64_t kk = k0; kk < k1; ++kk) {
        int q = 0;
        if (sa > 0.0f) {
          const float r = std::nearbyintf(a[row * k + kk] / sa); // default mode: half-to-even
          q = static_cast<int>(std::fmin(127.0f, std::fmax(-127.0f, r)));
        }
        aq[row * k + kk] = static_cast<std::int8_t>(q);
      }
    }
  }
  return 0;
}

int nbits_oracle_int8_block_dots(const std::int8_t *aq, const std::uint8_t *b,
                                 const std::uint8_t *zero_points, std::int64_t m, std::int64_t n,
                                 std::int64_t k, int bits, int block_size, std::int32_t *dots,
                                 int threads) {
  QuantView v;
  if (!MakeView(b, zero_points, n, k, bits, block_size, &v) || aq == nullptr ||
      dots == nullptr) {
    return 1;
  }
  ForColumnPanels(n, threads, [&](std::int64_t begin, std::int64_t end) {
    for (std::int64_t col = begin; col < end; ++col) {
      for (std::int64_t block = 0; block < v.n_blocks; ++block) {
        const int zp = ReadZeroPoint(v, col, block);
        const std::int64_t k0 = block * block_size;
        const std::int64_t k1 = std::min<std::int64_t>(k, k0 + block_size);
        for (std::int64_t row = 0; row < m; ++row) {
          std::int32_t acc = 0;
          for (std::int64_t kk = k0; kk < k1; ++kk) {
            acc += static_cast<std::int32_t>(aq[row * k + kk]) * (ReadCode(v, col, kk) - zp);
          }
          dots[(row * n + col) * v.n_blocks + block] = acc;
        }
      }
    }
  });
  return 0;
}

int nbits_oracle_matmul_int8(const float *a, const std::uint8_t *b, const float *scales,
                             const std::uint8_t *zero_points, const float *bias, std::int64_t m,
                             std::int64_t n, std::int64_t k, int bits, int block_size, float *y,
                             int threads) {
  QuantView v;
  if (!MakeView(b, zero_points, n, k, bits, block_size, &v) || a == nullptr ||
      scales == nullptr || y == nullptr) {
    return 1;
  }
  std::vector<std::int8_t> aq(static_cast<std::size_t>(m * k));
  std::vector<float> sa(static_cast<std::size_t>(m * v.n_blocks));
  std::vector<std::int32_t> dots(static_cast<std::size_t>(m * n * v.n_blocks));
  nbits_oracle_quantize_a(a, m, k, block_size, aq.data(), sa.data());
  nbits_oracle_int8_block_dots(aq.data(), b, zero_points, m, n, k, bits, block_size, dots.data(),
                               threads);
  for (std::int64_t row = 0; row < m; ++row) {
    for (std::int64_t col = 0; col < n; ++col) {
      float acc = 0.0f;
      for (std::int64_t block = 0; block < v.n_blocks; ++block) {
        const float s = sa[static_cast<std::size_t>(row * v.n_blocks + block)] *
                        scales[col * v.n_blocks + block];
        acc = std::fmaf(
            s, static_cast<float>(dots[static_cast<std::size_t>((row * n + col) * v.n_blocks + block)]),
            acc);
      }
      y[row * n + col] = bias != nullptr ? acc + bias[col] : acc;
    }
  }
  return 0;
}

// --- throughput-oriented variant -------------------------------------------------------------

namespace {

// Unpacks one block of codes to float(q - zp). `count` <= block_size.
__attribute__((target_clones("avx512f", "avx2", "default"))) void
UnpackBlock(const std::uint8_t *blob, int bits, int count, float zp, float *dst) {
  if (bits == 8) {
    for (int i = 0; i < count; ++i) {
      dst[i] = static_cast<float>(blob[i]) - zp;
    }
    return;
  }
  const int pairs = count / 2;
  for (int i = 0; i < pairs; ++i) {
    const std::uint8_t byte = blob[i];
    dst[2 * i] = static_cast<float>(byte & 0x0f) - zp;
    dst[2 * i + 1] = static_cast<float>(byte >> 4) - zp;
  }
  if (count & 1) {
    dst[count - 1] = static_cast<float>(blob[pairs] & 0x0f) - zp;
  }
}

__attribute__((target_clones("avx512f", "avx2", "default"))) float
DotBlock(const float *x, const float *w, int count) {
  float lanes[16] = {0};
  int i = 0;
  for (; i + 16 <= count; i += 16) {
    for (int l = 0; l < 16; ++l) {
      lanes[l] += x[i + l] * w[i + l];
    }
  }
  float acc = 0.0f;
  for (int l = 0; l < 16; ++l) {
    acc += lanes[l];
  }
  for (; i < count; ++i) {
    acc += x[i] * w[i];
  }
  return acc;
}

} // namespace

int nbits_oracle_matmul_f32_fast(const float *a, const std::uint8_t *b, const float *scales,
                                 const std::uint8_t *zero_points, const float *bias,
                                 std::int64_t m, std::int64_t n, std::int64_t k, int bits,
                                 int block_size, float *y, int threads) {
  QuantView v;
  if (!MakeView(b, zero_points, n, k, bits, block_size, &v) || a == nullptr ||
      scales == nullptr || y == nullptr) {
    return 1;
  }
  ForColumnPanels(n, threads, [&](std::int64_t begin, std::int64_t end) {
    std::vector<float> w(static_cast<std::size_t>(block_size));
    std::vector<float> acc(static_cast<std::size_t>(m));
    for (std::int64_t col = begin; col < end; ++col) {
      std::fill(acc.begin(), acc.end(), 0.0f);
      for (std::int64_t block = 0; block < v.n_blocks; ++block) {
        const std::int64_t k0 = block * block_size;
        const int count = static_cast<int>(std::min<std::int64_t>(block_size, k - k0));
        UnpackBlock(v.b + col * v.row_bytes + block * v.blob_bytes, bits, count,
                    static_cast<float>(ReadZeroPoint(v, col, block)), w.data());
        const float s = scales[col * v.n_blocks + block];
        for (std::int64_t row = 0; row < m; ++row) {
          acc[static_cast<std::size_t>(row)] += s * DotBlock(a + row * k + k0, w.data(), count);
        }
      }
      for (std::int64_t row = 0; row < m; ++row) {
        y[row * n + col] = bias != nullptr ? acc[static_cast<std::size_t>(row)] + bias[col]
                                           : acc[static_cast<std::size_t>(row)];
      }
    }
  });
  return 0;
}

} // extern "C"
