// Shared device/host definitions of the sm_100a MatMulNBits kernels.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace mnb {

// Device view of one node's constant operands (all pointers are device pointers).
//   b       [n, n_blocks, blob_bytes]   packed codes, low nibble = even element
//   scales  [n, n_blocks]               fp32
//   zp      [n, zp_row_bytes] or null   packed codes, one per block
//   bias    [n] or null
struct WeightView {
  const std::uint8_t *b;
  const float *scales;
  const std::uint8_t *zp;
  const float *bias;
  const unsigned char *meta; // prepared task-major scales / zero points (see MetaGeometryOf), or null
  const unsigned char *zp16; // prepared [n, n_blocks] bytes, 16 * zero point (direct decode kernel), or null
  std::int64_t n;
  std::int64_t k;
  int bits;
  int block_size;
  int n_blocks;
  int blob_bytes;
  int row_bytes;    // n_blocks * blob_bytes
  int zp_row_bytes; // ceil(n_blocks * bits / 8)
};

// Nodes that one grouped launch can serve (sibling projections sharing their activations).
constexpr int kMaxGroupedNodes = 3;
// Other GPUs whose result buffers a gathered step writes to.
constexpr int kMaxPeers = 7;

// Where a kernel writes its [m, n] result inside a possibly wider row-major matrix.
struct OutputView {
  float *y;
  std::int64_t ld;         // leading dimension in elements
  std::int64_t col_offset; // first column written
};

__device__ __forceinline__ void StoreOutput(const OutputView &out, std::int64_t index, float value) {
  out.y[index] = value;
}

// Error word written by kernels whose bounded waits gave up (0 = fine).
enum DeviceStatus : int {
  kDeviceOk = 0,
  kDeviceTimeoutFullBarrier = 1,
  kDeviceTimeoutEmptyBarrier = 2,
  kDeviceTimeoutMmaBarrier = 3,
  kDeviceTimeoutEpilogueBarrier = 4,
  kDeviceTimeoutPeerFlag = 5,
};

// The status word lives in page-locked host memory mapped into the device address space, so
// that the host can read it after a synchronize without a copy. A plain store is enough: any
// non-zero code means "a bounded wait gave up", and which of several reporters wins is
// irrelevant.
__device__ __forceinline__ void ReportStatus(int *word, int code) {
  *reinterpret_cast<volatile int *>(word) = code;
  __threadfence_system();
}

// Flag exchange of a gathered step (column shards stored into every rank's result through peer
// memory). Publishing: one warp tells every rank that this rank's columns of step `epoch` are
// stored. Waiting: a warp waits, bounded (about a second), until the local flag of every rank
// carries the epoch. flags[r] is rank r's flag array as mapped here: kMaxGatherRanks flags, then
// the step counter used when epoch == 0 (self-counting mode, what a replayed CUDA graph needs: the
// step number grows by one per call, in lockstep on all ranks).
constexpr int kMaxGatherRanks = 8;
struct GatherTail {
  int *flags[kMaxGatherRanks];
  int ranks;         // 0 = no gather
  int rank;
  int epoch;
  int wait;          // 1: the publishing warp also waits for everybody's flag
  unsigned *arrivals; // device counter of finished CTAs, zero between launches
  float *peers[kMaxPeers]; // the other ranks' result buffers (same window as the local one)
  int n_peers;
};

// Release / acquire fence at system scope. The sequentially consistent form (__threadfence_system)
// is not needed anywhere in the flag protocol and costs more; three of those in a row on the last
// CTA's path measured 7.8 us per node.
__device__ __forceinline__ void FenceSystem() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

__device__ __forceinline__ void StoreFlagSystem(int *address, int value) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}

__device__ __forceinline__ int LoadFlagSystem(const int *address) {
  int value;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
  return value;
}

// The caller has fenced (FenceSystem) after the stores the flags stand for and nothing needs
// ordering in between: the flags are plain system-scope stores. Returns the epoch.
__device__ __forceinline__ int PublishStep(const GatherTail &tail, int lane) {
  int epoch = tail.epoch;
  if (epoch == 0) {
    int *counter = tail.flags[tail.rank] + kMaxGatherRanks;
    epoch = *reinterpret_cast<volatile int *>(counter) + 1;
    __syncwarp();
    if (lane == 0) {
      *reinterpret_cast<volatile int *>(counter) = epoch;
    }
  }
  if (lane < tail.ranks) {
    StoreFlagSystem(tail.flags[lane] + tail.rank, epoch);
  }
  return epoch;
}

// Lane r waits for rank r's flag in the local array. Every wait is bounded; giving up sets the
// status word and returns, so the context stays usable.
__device__ __forceinline__ void WaitStep(int *local_flags, int ranks, int epoch, int lane, int *status) {
  if (lane < ranks) {
    bool arrived = false;
    for (std::uint32_t spin = 0; spin < (1u << 22); ++spin) {
      if (LoadFlagSystem(local_flags + lane) - epoch >= 0) {
        arrived = true;
        break;
      }
      __nanosleep(200);
    }
    if (!arrived) {
      ReportStatus(status, kDeviceTimeoutPeerFlag);
    }
    FenceSystem(); // acquire: what the flags stand for is visible to whatever follows
  }
}

__device__ __forceinline__ void PublishAndWait(const GatherTail &tail, int lane, int *status) {
  const int epoch = PublishStep(tail, lane);
  WaitStep(tail.flags[tail.rank], tail.ranks, epoch, lane, status);
}

// Copies the rows [row0, row1) of `tokens` token rows of the local result to the same place of
// every peer's buffer, warp-coalesced (consecutive lanes, consecutive columns: one 128-byte
// transaction over NVLink per warp instead of one packet per output). Scattered 4-byte stores from
// the arithmetic loop cost 8 us on a 36 us shard of the large-N projection; this costs under one.
// The caller has made the CTA's local stores visible to the CTA (a barrier).
__device__ __forceinline__ void PushRowsToPeers(const OutputView &out, const GatherTail &tail, std::int64_t token0,
                                                int tokens, std::int64_t row0, std::int64_t row1, int tid,
                                                int threads) {
  const std::int64_t rows = row1 - row0;
  if (tail.n_peers == 0) {
    return;
  }
  for (int token = 0; token < tokens; ++token) {
    const std::int64_t base = (token0 + token) * out.ld + out.col_offset + row0;
    for (std::int64_t i = tid; i < rows; i += threads) {
      const float v = __ldcg(out.y + base + i);
      for (int r = 0; r < tail.n_peers; ++r) {
        tail.peers[r][base + i] = v;
      }
    }
  }
}

// End of a kernel whose CTAs stored a gathered step: called by the `threads` threads (whole warps,
// numbered tid = 0 ...) of every CTA that stored outputs, after their last store. The CTA meets at
// the named barrier, ONE thread fences at system scope (cumulative over the stores the barrier
// ordered before it) and counts the CTA in; the warp of the last CTA to arrive publishes the flags
// (and waits, when tail.wait is set). No thread other than that one pays a system fence.
__device__ __forceinline__ void PublishWhenGridDone(const GatherTail &tail, int tid, int threads, int barrier_id,
                                                    unsigned ctas, int *status) {
  asm volatile("bar.sync %0, %1;" ::"r"(barrier_id), "r"(threads) : "memory");
  if (tid < 32) {
    unsigned last = 0;
    if (tid == 0) {
      // release at GPU scope: the CTA's stores (ordered before this thread by the barrier) before
      // its arrival. The one system-scope fence of the step is the last CTA's, below; it is
      // cumulative over what the arrivals it has observed stand for.
      __threadfence();
      last = atomicAdd(tail.arrivals, 1u) == ctas - 1 ? 1u : 0u;
      if (last != 0) {
        *tail.arrivals = 0; // everybody has arrived: ready for the next launch
      }
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last != 0) {
      FenceSystem(); // acquire the other CTAs' arrivals, release towards the flags
      const int epoch = PublishStep(tail, tid);
      if (tail.wait != 0) {
        WaitStep(tail.flags[tail.rank], tail.ranks, epoch, tid, status);
      }
    }
  }
}

__host__ __device__ inline int ZeroPointOf(const WeightView &w, std::int64_t row, int block) {
  if (w.zp == nullptr) {
    return 1 << (w.bits - 1);
  }
  const std::uint8_t *zrow = w.zp + row * w.zp_row_bytes;
  if (w.bits == 8) {
    return zrow[block];
  }
  const std::uint8_t byte = zrow[block >> 1];
  return (block & 1) ? (byte >> 4) : (byte & 0x0f);
}

__host__ __device__ inline int CodeOf(const WeightView &w, std::int64_t row, std::int64_t kk) {
  const int block = static_cast<int>(kk / w.block_size);
  const int within = static_cast<int>(kk - static_cast<std::int64_t>(block) * w.block_size);
  const std::uint8_t *blob = w.b + row * w.row_bytes + static_cast<std::int64_t>(block) * w.blob_bytes;
  if (w.bits == 8) {
    return blob[within];
  }
  const std::uint8_t byte = blob[within >> 1];
  return (within & 1) ? (byte >> 4) : (byte & 0x0f);
}

// ---- launchers (defined in the .cu files, called by the C ABI layer) ------------------------

// Returns a static kernel name for diagnostics, or nullptr when the shape is outside what the
// kernel supports (the caller then picks another one).
const char *LaunchGemvStream(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                             int *status_word, cudaStream_t stream, int sm_count);
// Any geometry and any token count (passes of sixteen tokens): the word-wise kernel below when the
// packed rows allow it, else one code at a time.
const char *LaunchGemvGeneric(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                              cudaStream_t stream, int sm_count);
// 8-bit weights, up to sixteen tokens: activations as three base-128 digit columns of an integer MMA whose
// other operand is the codes as they lie in B (blocks of 32 ... 256, B 16-byte aligned, K <= 32768). Two
// launches (digits, multiply); `scratch` holds the digits, their block sums and the row factors.
bool GemvU8MmaSupports(const WeightView &w, std::int64_t m);
std::size_t GemvU8MmaScratchBytes(const WeightView &w, std::int64_t m);
const char *LaunchGemvU8Mma(const WeightView &w, const float *a, std::int64_t m, unsigned char *scratch, OutputView out,
                            cudaStream_t stream, int sm_count);
// The same shapes at accuracy_level 4: `aq` / `a_scales` in the padded layout of LaunchQuantizeAPadded
// (16-byte aligned), `sums` room for m * n_blocks ints. The quantized activations are the MMA columns.
const char *LaunchGemvU8Int8Mma(const WeightView &w, const std::int8_t *aq, const float *a_scales, std::int64_t m,
                                int *sums, OutputView out, cudaStream_t stream, int sm_count);
// Groups of eight codes read straight from global memory: a warp per output column with lanes along K for
// one and two tokens, a lane per column from three tokens on; needs rows and the base of B aligned to a
// group (4 bytes for 4-bit, 8 for 8-bit weights).
const char *LaunchGemvWords(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                            cudaStream_t stream, int sm_count);
// Prepared side array used by the MMA decode kernel: per (8-row half tile, task slice) one
// record {float scale[8][scale_row_floats]; uint8 zp[8][bpt] (only with zero points)}. bytes == 0 means
// the geometry is outside what that kernel takes.
struct MetaGeometry {
  int bpt;             // quantization blocks per task
  int scale_row_floats; // floats per row of a record's scale part: bpt, plus 4 of padding when bpt * 4
                        // bytes is a multiple of 128 (rows would otherwise all start on the same bank)
  int slices;          // tasks per row tile
  int rec_bytes;
  int rec_scale_bytes;
  int half_tiles;
  std::size_t bytes;
};
MetaGeometry MetaGeometryOf(const WeightView &w);
bool LaunchPrepareMeta(const WeightView &w, unsigned char *meta, cudaStream_t stream);
// `tail` (optional): the last CTA to finish publishes the flags of a gathered step itself (and
// waits for the other ranks' flags when tail->wait is set), so no second kernel is needed.
const char *LaunchGemvMma(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                          int *status_word, cudaStream_t stream, int sm_count,
                          const GatherTail *tail = nullptr);
// Same arithmetic with two or four column tiles of tokens per pass over the weights; nullptr
// when one column tile is enough for `m` or the shape is outside what the kernel takes.
const char *LaunchGemvMmaMulti(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                               int *status_word, cudaStream_t stream, int sm_count,
                               const GatherTail *tail = nullptr);

// Decode for one or two tokens per pass on integer MMA: the activations enter as three base-128
// digits (22 bits of the row maximum), block dots are exact int32. block_size 128 ... 1024.
bool GemvImmaSupports(const WeightView &w, std::int64_t m);
const char *LaunchGemvImma(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                           int *status_word, cudaStream_t stream, int sm_count);

// Decode for one or two tokens on integer MMA with the packed weights streamed from global memory
// into each warp (cp.async into lane-private places or plain loads into registers): no staging
// ring, no producer. 4-bit, block_size 128. `dependent`: launch with programmatic stream
// serialization (the weight stream starts while the previous kernel of the stream drains; A is
// read and Y written only after that kernel has completed).
bool DecodeDirectSupports(const WeightView &w, std::int64_t m);
// Fills `out` (n * n_blocks bytes) with 16 * zero point per block; the geometry is one the kernel takes.
bool DecodeDirectWantsZeroPointBytes(const WeightView &w);
bool LaunchExpandZeroPoints(const WeightView &w, unsigned char *out, cudaStream_t stream);
const char *LaunchDecodeDirect(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                               cudaStream_t stream, int sm_count, bool dependent);

// Decode of one token with the CTA's whole share of the packed weights asked for at kernel start
// (TMA copies issued by a producer warp into shared-memory slots that are normally written once).
// block_size 128 or 32. `tail` (single node): the CTAs push their rows to the peers of a gathered
// step and the last one publishes the flags.
bool DecodeResidentSupports(const WeightView &w, std::int64_t m);
// Rows of up to 4096 k: a whole row of a tile fits a slot with ten or more warps at work. Longer
// rows leave the tile-per-warp structure with few warps (K = 14336: 18.7 us against 11.9 on the
// direct kernel, K = 8192: 10.0-11.3 against 9.5-10.0 on the fp16 kernel), and so do nodes of fewer
// than four tiles per CTA (K = 4096, block 128: N = 1024 7.6 against 3.5 us, N = 4096 6.2 against 5.6
// on the direct kernel; block 32, N = 1024: 8.0 against 6.1 on the fp16 kernel), so AUTO sends those
// elsewhere. A group of sibling nodes in one launch is judged by its rows only.
bool DecodeResidentPreferred(const WeightView &w);
bool DecodeResidentGroupPreferred(const WeightView *nodes, int count);
const char *LaunchDecodeResident(const WeightView &w, const float *a, std::int64_t m, OutputView out, int *status_word,
                                 cudaStream_t stream, int sm_count, const GatherTail *tail = nullptr);
// Up to kMaxGroupedNodes nodes that take the same activations (same K, zero points in all or in
// none) in one launch; nullptr when the group has no such kernel.
bool DecodeResidentGroupSupports(const WeightView *nodes, int count, std::int64_t m);
const char *LaunchDecodeResidentGroup(const WeightView *nodes, const OutputView *outs, int count, const float *a,
                                      std::int64_t m, int *status_word, cudaStream_t stream, int sm_count,
                                      const GatherTail *tail = nullptr);
// Drops the launch plans (tensor maps, slot shapes) cached for a node whose weights are going away.
void ForgetDecodeResidentPlans(const WeightView &w);

// Prefill. `scratch` holds GemmTcgen05ScratchBytes(...) bytes. `tiles`: which kernel takes the product.
constexpr int kGemmTileAuto = 0;      // CTA pairs for more than 128 tokens where the cost model prefers them
constexpr int kGemmTileRows128 = 1;   // the kernel with 128 weight rows per CTA
constexpr int kGemmTilePairs = 2;     // CTA pairs (4-bit weights; other widths fall back to the 128-row kernel)
const char *LaunchGemmTcgen05(const WeightView &w, const float *a, std::int64_t m,
                              std::uint16_t *scratch, OutputView out, int *status_word,
                              cudaStream_t stream, int sm_count, int tiles = kGemmTileAuto);
// Scratch of one call: bf16 activations, plus the partial products when K is shared between CTA pairs.
std::size_t GemmTcgen05ScratchBytes(const WeightView &w, std::int64_t m, int sm_count);
bool GemmTcgen05Supports(const WeightView &w, std::int64_t m);

// accuracy_level 4.
const char *LaunchQuantizeA(const float *a, std::int64_t m, std::int64_t k, int block_size,
                            std::int8_t *aq, float *a_scales, cudaStream_t stream);
const char *LaunchQuantizeAPadded(const float *a, std::int64_t m, std::int64_t k, int block_size,
                                  std::int8_t *aq_padded, float *a_scales, cudaStream_t stream);
const char *LaunchInt8BlockDots(const WeightView &w, const std::int8_t *aq, std::int64_t m,
                                std::int32_t *dots, cudaStream_t stream);
const char *LaunchInt8Matmul(const WeightView &w, const std::int8_t *aq, const float *a_scales,
                             std::int64_t m, OutputView out, cudaStream_t stream, int sm_count);

// accuracy_level 4 on integer MMA: quantizes `a` into `scratch` (Int8MmaScratchBytes, 0 when the
// shape is outside what the kernel takes) and multiplies.
std::size_t Int8MmaScratchBytes(const WeightView &w, std::int64_t m);
const char *LaunchInt8Mma(const WeightView &w, const float *a, std::int64_t m, unsigned char *scratch,
                          OutputView out, int *status_word, cudaStream_t stream, int sm_count);

// Parity instrument (m <= 8): the same quantization and the instrumented form of the same kernel,
// which also adds its exact int32 block dots to dots[m, n, n_blocks] (zeroed by the call).
const char *LaunchInt8MmaBlockDots(const WeightView &w, const float *a, std::int64_t m, unsigned char *scratch,
                                   OutputView out, std::int32_t *dots, int *status_word, cudaStream_t stream,
                                   int sm_count);

// accuracy_level 0 through the sixteen-row integer-MMA kernel: every token enters as three rows of
// base-128 digits (22 bits of its row maximum), the three partial results are added behind it.
// `scratch`: DigitsInt8MmaScratchBytes (0 when the shape is outside what the kernel takes).
std::size_t DigitsInt8MmaScratchBytes(const WeightView &w, std::int64_t m);
const char *LaunchDigitsInt8Mma(const WeightView &w, const float *a, std::int64_t m, unsigned char *scratch,
                                OutputView out, int *status_word, cudaStream_t stream, int sm_count);
// Sibling nodes that take the same activations: quantization / digit rows made once for the group.
const char *LaunchInt8MmaGroup(const WeightView *nodes, const OutputView *outs, int count, const float *a,
                               std::int64_t m, unsigned char *scratch, int *status_word, cudaStream_t stream,
                               int sm_count);
const char *LaunchDigitsInt8MmaGroup(const WeightView *nodes, const OutputView *outs, int count, const float *a,
                                     std::int64_t m, unsigned char *scratch, int *status_word, cudaStream_t stream,
                                     int sm_count);
// accuracy_level 0 for up to sixteen tokens in ONE pass over the weights: each CTA takes one 2048-k
// slice of K with all digit rows of that slice in shared memory. 0 bytes / nullptr when the shape
// is outside what the kernel takes.
std::size_t DigitSlicesScratchBytes(const WeightView &w, std::int64_t m);
std::size_t DigitSlicesGroupScratchBytes(const WeightView *nodes, int count, std::int64_t m);
const char *LaunchDigitSlicesGroup(const WeightView *nodes, const OutputView *outs, int count, const float *a,
                                   std::int64_t m, unsigned char *scratch, int *status_word, cudaStream_t stream,
                                   int sm_count);

const char *LaunchDequantInt(const WeightView &w, std::int32_t *out, cudaStream_t stream);

// Producer lanes per CTA that issue the tile loads of the ring-fed kernels: env
// MNB_GEMV_PRODUCERS (1, 2 or 4) or the kernel's own default. Measured: the pair kernel is
// fastest with one paced issuer (cfg2 M=1: 12.9 / 13.3 / 14.6 us with 1 / 2 / 4), the kernels whose
// warps share every task with four (level 4, cfg2 M=16: 16.5 vs 18.0 us).
int WantedProducers(int kernel_default);

void CountLaunch(int launches = 1);

// Set by the host-buffer entry point around its dispatch: the kernel launched just before
// (the small copy of A out of page-locked host memory) has triggered its dependents, so the
// decode kernels may be launched with programmatic stream serialization and begin streaming
// weights while that copy is still in flight. They wait for it before they read A.
void SetDependentLaunchHint(bool allowed);
bool DependentLaunchHint();

} // namespace mnb
