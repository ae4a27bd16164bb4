#include "onnx_light_cpu_b200/kernels/parallel/peer_gather.h"

#include "include/matmulnbits_b200.h"

#include <stdexcept>

namespace onnx_light_cuda {

namespace {

constexpr std::int64_t kFlagArrayBytes = 256;  // MNB_MAX_GATHER_RANKS + 1 ints, padded to a sector pair

void Check(int code, const char *what) {
  if (code != MNB_OK) {
    throw std::runtime_error(std::string(what) + ": " + mnb_last_error());
  }
}

}  // namespace

PeerGatherLayout PeerGatherLayout::Make(int world, int rank, std::int64_t m_max, std::int64_t n_shard, int slots) {
  if (world < 1 || world > MNB_MAX_GATHER_RANKS) {
    throw std::invalid_argument("peer gather: 1 to " + std::to_string(MNB_MAX_GATHER_RANKS) + " ranks");
  }
  if (rank < 0 || rank >= world) {
    throw std::invalid_argument("peer gather: rank out of range");
  }
  if (m_max < 1 || n_shard < 1 || slots < 1 || slots > MNB_MAX_GATHER_WAITS) {
    throw std::invalid_argument("peer gather: m_max, n_shard >= 1 and 1 to " +
                                std::to_string(MNB_MAX_GATHER_WAITS) + " slots");
  }
  if (m_max > (std::int64_t{1} << 40) / n_shard / world / slots) {
    throw std::invalid_argument("peer gather: buffer too large");
  }
  PeerGatherLayout layout;
  layout.world = world;
  layout.rank = rank;
  layout.m_max = m_max;
  layout.n_shard = n_shard;
  layout.slots = slots;
  return layout;
}

std::int64_t PeerGatherLayout::FlagsOffsetBytes() const {
  return (static_cast<std::int64_t>(slots) * SlotFloats() * 4 + 255) / 256 * 256;
}

std::int64_t PeerGatherLayout::Bytes() const { return FlagsOffsetBytes() + static_cast<std::int64_t>(slots) * kFlagArrayBytes; }

std::int64_t PeerGatherLayout::WindowOffsetBytes(int slot, int writer) const {
  if (slot < 0 || slot >= slots || writer < 0 || writer >= world) {
    throw std::invalid_argument("peer gather: slot or writer out of range");
  }
  return (static_cast<std::int64_t>(slot) * world + writer) * m_max * n_shard * 4;
}

std::int64_t PeerGatherLayout::FlagArrayOffsetBytes(int slot) const {
  if (slot < 0 || slot >= slots) {
    throw std::invalid_argument("peer gather: slot out of range");
  }
  return FlagsOffsetBytes() + static_cast<std::int64_t>(slot) * kFlagArrayBytes;
}

void PeerGatherLayout::Tables(const std::uintptr_t *bases, int slot, std::uintptr_t *y_ranks,
                              std::uintptr_t *flags_ranks) const {
  const std::int64_t window = WindowOffsetBytes(slot, rank);
  const std::int64_t flags = FlagArrayOffsetBytes(slot);
  for (int r = 0; r < world; ++r) {
    y_ranks[r] = bases[r] + static_cast<std::uintptr_t>(window);
    flags_ranks[r] = bases[r] + static_cast<std::uintptr_t>(flags);
  }
}

void ShardBounds(std::int64_t n, int world, int rank, std::int64_t *lo, std::int64_t *hi) {
  if (n < 1 || world < 1 || rank < 0 || rank >= world || lo == nullptr || hi == nullptr) {
    throw std::invalid_argument("shard bounds: N >= 1, 0 <= rank < world");
  }
  const std::int64_t per = n / world;
  const std::int64_t extra = n % world;
  *lo = per * rank + (rank < extra ? rank : extra);
  *hi = *lo + per + (rank < extra ? 1 : 0);
}

PeerGatherBuffers::PeerGatherBuffers(const PeerGatherLayout &layout, int device) : layout_(layout), device_(device) {
  Check(mnb_peer_buffer_create(device, static_cast<size_t>(layout.Bytes()), &own_, handle_), "peer buffer");
  bases_.assign(static_cast<size_t>(layout.world), 0);
  bases_[static_cast<size_t>(layout.rank)] = reinterpret_cast<std::uintptr_t>(own_);
}

PeerGatherBuffers::~PeerGatherBuffers() {
  if (opened_) {
    ClosePeers();
  }
  if (own_ != nullptr) {
    mnb_peer_buffer_destroy(device_, own_);
  }
}

void PeerGatherBuffers::Open(const unsigned char *handles) {
  if (opened_) {
    throw std::runtime_error("peer gather: buffers are already open");
  }
  for (int r = 0; r < layout_.world; ++r) {
    if (r == layout_.rank) {
      continue;
    }
    void *ptr = nullptr;
    Check(mnb_peer_buffer_open(device_, handles + static_cast<size_t>(r) * kIpcHandleBytes, &ptr), "peer buffer open");
    bases_[static_cast<size_t>(r)] = reinterpret_cast<std::uintptr_t>(ptr);
  }
  opened_ = true;
}

void PeerGatherBuffers::ClosePeers() {
  for (int r = 0; r < layout_.world; ++r) {
    if (r != layout_.rank && bases_[static_cast<size_t>(r)] != 0) {
      mnb_peer_buffer_close(device_, reinterpret_cast<void *>(bases_[static_cast<size_t>(r)]));
      bases_[static_cast<size_t>(r)] = 0;
    }
  }
  opened_ = false;
}

float *PeerGatherBuffers::Result(int slot) const {
  return reinterpret_cast<float *>(reinterpret_cast<std::uintptr_t>(own_) +
                                   static_cast<std::uintptr_t>(layout_.WindowOffsetBytes(slot, 0)));
}

void PeerGatherBuffers::Run(mnb_weights *weights, const float *a_dev, std::int64_t m, int accuracy_level, int slot,
                            bool wait, void *stream) {
  if (!opened_ && layout_.world > 1) {
    throw std::runtime_error("peer gather: Open() the peers' buffers first");
  }
  // a shard narrower than the window (the tail of an N that does not divide) fills its first columns
  if (m < 1 || m > layout_.m_max || mnb_weights_n(weights) > layout_.n_shard || mnb_weights_n(weights) < 1) {
    throw std::invalid_argument("peer gather: shape does not match the gather buffers");
  }
  std::uintptr_t y[MNB_MAX_GATHER_RANKS], flags[MNB_MAX_GATHER_RANKS];
  layout_.Tables(bases_.data(), slot, y, flags);
  float *y_ranks[MNB_MAX_GATHER_RANKS];
  int *flags_ranks[MNB_MAX_GATHER_RANKS];
  for (int r = 0; r < layout_.world; ++r) {
    y_ranks[r] = reinterpret_cast<float *>(y[r]);
    flags_ranks[r] = reinterpret_cast<int *>(flags[r]);
  }
  Check(mnb_matmul_device_gather_ex(weights, a_dev, m, accuracy_level, y_ranks, flags_ranks, layout_.world,
                                    layout_.rank, layout_.n_shard, 0, 0, wait ? 1 : 0, stream),
        "gathered product");
}

void PeerGatherBuffers::Wait(mnb_weights *weights, const int *slots, int count, void *stream) {
  if (count < 1 || count > MNB_MAX_GATHER_WAITS) {
    throw std::invalid_argument("peer gather: 1 to 8 slots per wait");
  }
  int *flags[MNB_MAX_GATHER_WAITS];
  for (int i = 0; i < count; ++i) {
    flags[i] = reinterpret_cast<int *>(reinterpret_cast<std::uintptr_t>(own_) +
                                       static_cast<std::uintptr_t>(layout_.FlagArrayOffsetBytes(slots[i])));
  }
  Check(mnb_gather_wait(weights, flags, nullptr, count, layout_.world, stream), "gather wait");
}

}  // namespace onnx_light_cuda
