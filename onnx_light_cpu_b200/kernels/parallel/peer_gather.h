// Column-sharded MatMulNBits over the GPUs of one box without a collective: every rank owns a
// buffer that the other ranks map, and each rank's kernels store their columns into all of them.
//
// PeerGatherLayout is the arithmetic of that buffer - where a writer's columns go, where the flag
// arrays sit - and has no dependency on a GPU. PeerGatherBuffers owns the local buffer and the
// mappings of the peers' buffers and runs a node through the C ABI of matmulnbits_b200.
//
// The reference has no multi-device path; the closest notion is the N split of
// onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258, whose threads write disjoint column ranges
// of one shared Y.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

struct mnb_weights;

namespace onnx_light_cuda {

// One buffer per rank: `slots` gathered results [world, m_max, n_shard] fp32 (writer-major, so a
// writer's window is contiguous), then one 256-byte flag array per slot.
struct PeerGatherLayout {
  int world = 0;
  int rank = 0;
  std::int64_t m_max = 0;
  std::int64_t n_shard = 0;
  int slots = 0;

  // Throws std::invalid_argument on a layout no box can hold (ranks, sizes, slots out of range).
  static PeerGatherLayout Make(int world, int rank, std::int64_t m_max, std::int64_t n_shard, int slots);

  std::int64_t SlotFloats() const { return static_cast<std::int64_t>(world) * m_max * n_shard; }
  std::int64_t FlagsOffsetBytes() const;            // first flag array
  std::int64_t Bytes() const;                       // whole buffer
  // Byte offset, inside ANY rank's buffer, of the window that `writer` fills in `slot`.
  std::int64_t WindowOffsetBytes(int slot, int writer) const;
  std::int64_t FlagArrayOffsetBytes(int slot) const;
  // Pointer tables of one call by this rank: its window and the slot's flag array in every
  // rank's buffer (bases[r] = rank r's buffer as mapped here).
  void Tables(const std::uintptr_t *bases, int slot, std::uintptr_t *y_ranks, std::uintptr_t *flags_ranks) const;
};

// Columns [lo, hi) of an N-column node that rank `rank` of `world` owns. N need not divide: the
// first N % world ranks take one column more. Throws std::invalid_argument on bad arguments.
void ShardBounds(std::int64_t n, int world, int rank, std::int64_t *lo, std::int64_t *hi);

constexpr int kIpcHandleBytes = 64;

class PeerGatherBuffers {
 public:
  // Allocates this rank's buffer on `device`; Handle() is what the peers need to map it.
  PeerGatherBuffers(const PeerGatherLayout &layout, int device);
  ~PeerGatherBuffers();
  PeerGatherBuffers(const PeerGatherBuffers &) = delete;
  PeerGatherBuffers &operator=(const PeerGatherBuffers &) = delete;

  const unsigned char *Handle() const { return handle_; }
  // handles: world x kIpcHandleBytes, in rank order, as collected over any host channel.
  void Open(const unsigned char *handles);
  // Unmaps the peers' buffers. Every rank calls it, then synchronizes with the others, before
  // any rank destroys its own buffer.
  void ClosePeers();

  const PeerGatherLayout &layout() const { return layout_; }
  // Local gathered result of a slot: [world, m_max, n_shard] fp32.
  float *Result(int slot) const;

  // This rank's shard of a node into `slot` of every rank's buffer; `wait`: also wait for the
  // other ranks' columns of this step (else call Wait before the result is read).
  void Run(mnb_weights *weights, const float *a_dev, std::int64_t m, int accuracy_level, int slot, bool wait,
           void *stream);
  // One small kernel that waits until the named slots hold every rank's columns of the last step.
  void Wait(mnb_weights *weights, const int *slots, int count, void *stream);

 private:
  PeerGatherLayout layout_;
  int device_;
  void *own_ = nullptr;
  unsigned char handle_[kIpcHandleBytes];
  std::vector<std::uintptr_t> bases_;
  bool opened_ = false;
};

}  // namespace onnx_light_cuda
