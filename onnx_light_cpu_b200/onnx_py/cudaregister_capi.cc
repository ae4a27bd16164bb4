// C entry points over the C++ registration layer, loaded from Python with ctypes. Plays the
// role of the reference's nanobind module `_cpuregister`
// (onnx_light_cpu/onnx_py/_cpuregister.cc:62-114: register_all_kernels, registered_kernels,
// used_kernel_names, clear_used_kernel_names, set_kernel_usage_recording) and adds a minimal
// single-node session so that the registered factory can be constructed once and Run many
// times the way onnx-light's evaluator does it.

#include "onnx_light_cpu_b200/kernels/kernel_registration.h"
#include "onnx_light_cpu_b200/kernels/kernel_usage.h"
#include "onnx_light_cpu_b200/kernels/math/matmul_nbits_kernel.h"
#include "onnx_light_cpu_b200/kernels/parallel/peer_gather.h"
#include "onnx_light_cpu_b200/kernels/register_kernels.h"

#include "onnx_core/runtime/kernels/kernel_dispatch_table.h"
#include "onnx_core/runtime/kernels/node_helpers.h"

#include <cstdint>
#include <cstring>
#include <exception>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace rt_ns = ONNX_LIGHT_NAMESPACE::core::runtime;
namespace sym_ns = ONNX_LIGHT_NAMESPACE::core::symbolic;
using ONNX_LIGHT_NAMESPACE::NodeProto;

namespace {

thread_local std::string t_error;
thread_local std::string t_text;

// 0 ok, 1 std::invalid_argument, 2 anything else
template <typename Fn> int Guard(Fn fn) {
  try {
    fn();
    t_error.clear();
    return 0;
  } catch (const std::invalid_argument &e) {
    t_error = e.what();
    return 1;
  } catch (const std::exception &e) {
    t_error = e.what();
    return 2;
  }
}

std::string Quote(const std::string &s) {
  std::string out = "\"";
  for (char c : s) {
    if (c == '"' || c == '\\') {
      out.push_back('\\');
    }
    out.push_back(c);
  }
  out.push_back('"');
  return out;
}

struct Session {
  NodeProto node;
  rt_ns::RuntimeContext rt{rt_ns::KernelContext(rt_ns::OpsetId("com.microsoft", 1))};
  std::unique_ptr<rt_ns::KernelBase> kernel;
};

void AddInt(NodeProto *node, const char *name, std::int64_t value) {
  auto *attr = node->add_attribute();
  attr->set_name(name);
  attr->set_i(value);
}

} // namespace

extern "C" {

const char *olc_last_error(void) { return t_error.c_str(); }

int olc_register_all_kernels(void) {
  return Guard([] { onnx_light_cuda::RegisterAllKernels(); });
}

// JSON array of the registration inventory, in its deterministic order.
const char *olc_registered_kernels_json(void) {
  const int rc = Guard([] {
    std::ostringstream out;
    out << "[";
    bool first = true;
    for (const auto &item : onnx_light_cuda::CollectRegisteredKernels()) {
      if (!first) {
        out << ",";
      }
      first = false;
      out << "{\"domain\":" << Quote(item.domain) << ",\"op_type\":" << Quote(item.op_type)
          << ",\"device\":" << Quote(sym_ns::DeviceName(item.device))
          << ",\"kernel_name\":" << Quote(item.kernel_name) << ",\"types\":[";
      for (std::size_t i = 0; i < item.types.size(); ++i) {
        out << (i ? "," : "") << static_cast<int>(item.types[i]);
      }
      out << "],\"since_version\":";
      if (item.since_version) {
        out << *item.since_version;
      } else {
        out << "null";
      }
      out << ",\"until_version\":";
      if (item.until_version) {
        out << *item.until_version;
      } else {
        out << "null";
      }
      out << "}";
    }
    out << "]";
    t_text = out.str();
  });
  return rc == 0 ? t_text.c_str() : nullptr;
}

const char *olc_used_kernel_names_json(void) {
  std::ostringstream out;
  out << "[";
  bool first = true;
  for (const std::string &name : onnx_light_cuda::UsedKernelNames()) {
    out << (first ? "" : ",") << Quote(name);
    first = false;
  }
  out << "]";
  t_text = out.str();
  return t_text.c_str();
}

void olc_clear_used_kernel_names(void) { onnx_light_cuda::ClearUsedKernelNames(); }

void olc_set_kernel_usage_recording(int enabled) {
  onnx_light_cuda::SetKernelUsageRecording(enabled != 0);
}

int olc_dispatch_table_size(void) { return static_cast<int>(rt_ns::KernelDispatchTable().size()); }

int olc_dispatch_table_has(const char *key) {
  return rt_ns::KernelDispatchTable().find(key) != rt_ns::KernelDispatchTable().end() ? 1 : 0;
}

// Registers MatMulNBits twice inside one pass; returns 1 when the second call is rejected
// with std::invalid_argument (the documented behaviour), 0 otherwise.
int olc_duplicate_registration_is_rejected(void) {
  std::vector<onnx_light_cuda::KernelRegistration> inventory;
  onnx_light_cuda::KernelRegistrationScope scope(&inventory);
  onnx_light_cuda::RegisterMatMulNBitsKernel();
  try {
    onnx_light_cuda::RegisterMatMulNBitsKernel();
  } catch (const std::invalid_argument &) {
    return inventory.size() == 1 ? 1 : 0;
  }
  return 0;
}

void olc_set_device(int device) { onnx_light_cuda::SetMatMulNBitsDevice(device); }

// Builds a one-node model: initializers B, scales[, zero_points][, bias] with session
// lifetime, attributes from the arguments. `g_idx_mode` = 1 wires a g_idx input (which the
// kernel must reject at Run). The kernel is constructed through the dispatch table, so
// olc_register_all_kernels() must have run.
void *olc_session_create(const std::uint8_t *b, std::int64_t b_bytes, const float *scales,
                         std::int64_t scale_count, const std::uint8_t *zero_points,
                         std::int64_t zp_bytes, const float *bias, std::int64_t bias_count,
                         std::int64_t k, std::int64_t n, std::int64_t bits, std::int64_t block_size,
                         std::int64_t accuracy_level, int g_idx_mode) {
  Session *session = nullptr;
  const int rc = Guard([&] {
    auto owned = std::make_unique<Session>();
    NodeProto &node = owned->node;
    node.set_op_type("MatMulNBits");
    node.set_domain("com.microsoft");
    node.set_name("matmul_nbits_0");
    node.add_input("A");
    node.add_input("B");
    node.add_input("scales");
    node.add_input(zero_points != nullptr ? "zero_points" : "");
    node.add_input(g_idx_mode ? "g_idx" : "");
    node.add_input(bias != nullptr ? "bias" : "");
    node.add_output("Y");
    AddInt(&node, "K", k);
    AddInt(&node, "N", n);
    AddInt(&node, "bits", bits);
    AddInt(&node, "block_size", block_size);
    AddInt(&node, "accuracy_level", accuracy_level);
    auto u8 = static_cast<std::int32_t>(rt_ns::DataType::UINT8);
    auto f32 = static_cast<std::int32_t>(rt_ns::DataType::FLOAT);
    owned->rt.Set("B", rt_ns::Tensor("B", u8, {b_bytes}, std::vector<std::uint8_t>(b, b + b_bytes)));
    std::vector<std::uint8_t> scale_bytes(static_cast<std::size_t>(scale_count) * 4);
    std::memcpy(scale_bytes.data(), scales, scale_bytes.size());
    owned->rt.Set("scales", rt_ns::Tensor("scales", f32, {scale_count}, std::move(scale_bytes)));
    if (zero_points != nullptr) {
      owned->rt.Set("zero_points", rt_ns::Tensor("zero_points", u8, {zp_bytes},
                                                 std::vector<std::uint8_t>(zero_points, zero_points + zp_bytes)));
    }
    if (bias != nullptr) {
      std::vector<std::uint8_t> bias_bytes(static_cast<std::size_t>(bias_count) * 4);
      std::memcpy(bias_bytes.data(), bias, bias_bytes.size());
      owned->rt.Set("bias", rt_ns::Tensor("bias", f32, {bias_count}, std::move(bias_bytes)));
    }
    if (g_idx_mode) {
      owned->rt.Set("g_idx", rt_ns::Tensor("g_idx", static_cast<std::int32_t>(rt_ns::DataType::INT32), {k},
                                           std::vector<std::uint8_t>(static_cast<std::size_t>(k) * 4)));
    }
    auto &table = rt_ns::KernelDispatchTable();
    auto it = table.find("com.microsoft:MatMulNBits");
    if (it == table.end()) {
      throw std::runtime_error("com.microsoft:MatMulNBits is not registered; call register_kernels() first.");
    }
    owned->kernel = it->second.fn(owned->node, owned->rt);
    session = owned.release();
  });
  return rc == 0 ? session : nullptr;
}

// One execution: sets input A (host, fp32, `rank` dims), runs the node, copies Y out.
int olc_session_run(void *handle, const float *a, const std::int64_t *shape, int rank, float *y,
                    std::int64_t y_capacity) {
  return Guard([&] {
    auto *session = static_cast<Session *>(handle);
    if (session == nullptr) {
      throw std::invalid_argument("null session");
    }
    rt_ns::Shape a_shape(shape, shape + rank);
    std::int64_t count = 1;
    for (std::int64_t d : a_shape) {
      count *= d;
    }
    std::vector<std::uint8_t> bytes(static_cast<std::size_t>(count) * 4);
    if (count > 0) {
      std::memcpy(bytes.data(), a, bytes.size());
    }
    session->rt.Set("A", rt_ns::Tensor("A", static_cast<std::int32_t>(rt_ns::DataType::FLOAT), a_shape,
                                       std::move(bytes)));
    session->kernel->Run(session->rt);
    const rt_ns::Tensor &out = session->rt.Get("Y");
    if (out.element_count() > y_capacity) {
      throw std::invalid_argument("output buffer too small");
    }
    if (out.element_count() > 0) {
      std::memcpy(y, out.bytes(), static_cast<std::size_t>(out.element_count()) * 4);
    }
  });
}

// Test hook: overwrites the bytes of the session's initializer B in place (same buffer, same
// address), as a runtime that recycles an initializer's storage would.
int olc_session_overwrite_b(void *handle, const std::uint8_t *b, std::int64_t b_bytes) {
  return Guard([&] {
    auto *session = static_cast<Session *>(handle);
    if (session == nullptr) {
      throw std::invalid_argument("null session");
    }
    auto it = session->rt.tensors().find("B");
    if (it == session->rt.tensors().end()) {
      throw std::invalid_argument("olc_session_overwrite_b: the session has no B");
    }
    rt_ns::Tensor &tensor = it->second;
    if (static_cast<std::int64_t>(tensor.size_bytes()) != b_bytes) {
      throw std::invalid_argument("olc_session_overwrite_b: size mismatch");
    }
    std::memcpy(tensor.mutable_bytes(), b, static_cast<std::size_t>(b_bytes));
  });
}

const char *olc_session_last_device_kernel(void *handle) {
  auto *session = static_cast<Session *>(handle);
  auto *kernel = session != nullptr ? dynamic_cast<onnx_light_cuda::MatMulNBitsKernel *>(session->kernel.get())
                                    : nullptr;
  return kernel != nullptr ? kernel->last_device_kernel() : "";
}

void olc_session_destroy(void *handle) { delete static_cast<Session *>(handle); }

// ---- column-sharded nodes: buffer layout (no GPU needed) and the buffers themselves ----------

// out[0..3] = floats per slot, byte offset of the first flag array, bytes of the whole buffer,
// bytes of one writer's window.
int olc_peer_gather_layout(int world, int rank, std::int64_t m_max, std::int64_t n_shard, int slots,
                           std::int64_t *out) {
  return Guard([&] {
    const auto layout = onnx_light_cuda::PeerGatherLayout::Make(world, rank, m_max, n_shard, slots);
    out[0] = layout.SlotFloats();
    out[1] = layout.FlagsOffsetBytes();
    out[2] = layout.Bytes();
    out[3] = m_max * n_shard * 4;
  });
}

// Pointer tables of one call of `rank`: y_ranks[r] / flags_ranks[r] from the buffers' base addresses.
int olc_peer_gather_tables(int world, int rank, std::int64_t m_max, std::int64_t n_shard, int slots, int slot,
                           const std::uint64_t *bases, std::uint64_t *y_ranks, std::uint64_t *flags_ranks) {
  return Guard([&] {
    const auto layout = onnx_light_cuda::PeerGatherLayout::Make(world, rank, m_max, n_shard, slots);
    std::vector<std::uintptr_t> in(static_cast<size_t>(world)), y(static_cast<size_t>(world)),
        flags(static_cast<size_t>(world));
    for (int r = 0; r < world; ++r) {
      in[static_cast<size_t>(r)] = static_cast<std::uintptr_t>(bases[r]);
    }
    layout.Tables(in.data(), slot, y.data(), flags.data());
    for (int r = 0; r < world; ++r) {
      y_ranks[r] = y[static_cast<size_t>(r)];
      flags_ranks[r] = flags[static_cast<size_t>(r)];
    }
  });
}

int olc_shard_bounds(std::int64_t n, int world, int rank, std::int64_t *lo, std::int64_t *hi) {
  return Guard([&] { onnx_light_cuda::ShardBounds(n, world, rank, lo, hi); });
}

// Allocates this rank's buffer; handle_out receives the 64 bytes the peers need to map it.
void *olc_peer_gather_create(int world, int rank, std::int64_t m_max, std::int64_t n_shard, int slots, int device,
                             unsigned char *handle_out) {
  onnx_light_cuda::PeerGatherBuffers *buffers = nullptr;
  const int code = Guard([&] {
    const auto layout = onnx_light_cuda::PeerGatherLayout::Make(world, rank, m_max, n_shard, slots);
    buffers = new onnx_light_cuda::PeerGatherBuffers(layout, device);
    std::memcpy(handle_out, buffers->Handle(), onnx_light_cuda::kIpcHandleBytes);
  });
  return code == 0 ? buffers : nullptr;
}

int olc_peer_gather_open(void *buffers, const unsigned char *handles) {
  return Guard([&] { static_cast<onnx_light_cuda::PeerGatherBuffers *>(buffers)->Open(handles); });
}

void *olc_peer_gather_result(void *buffers, int slot) {
  void *result = nullptr;
  Guard([&] { result = static_cast<onnx_light_cuda::PeerGatherBuffers *>(buffers)->Result(slot); });
  return result;
}

int olc_peer_gather_run(void *buffers, void *weights, const float *a_dev, std::int64_t m, int accuracy_level,
                        int slot, int wait, void *stream) {
  return Guard([&] {
    static_cast<onnx_light_cuda::PeerGatherBuffers *>(buffers)->Run(static_cast<mnb_weights *>(weights), a_dev, m,
                                                                     accuracy_level, slot, wait != 0, stream);
  });
}

int olc_peer_gather_wait(void *buffers, void *weights, const int *slots, int count, void *stream) {
  return Guard([&] {
    static_cast<onnx_light_cuda::PeerGatherBuffers *>(buffers)->Wait(static_cast<mnb_weights *>(weights), slots, count,
                                                                      stream);
  });
}

int olc_peer_gather_close_peers(void *buffers) {
  return Guard([&] { static_cast<onnx_light_cuda::PeerGatherBuffers *>(buffers)->ClosePeers(); });
}

void olc_peer_gather_destroy(void *buffers) { delete static_cast<onnx_light_cuda::PeerGatherBuffers *>(buffers); }

} // extern "C"
