// accuracy_level = 4 path of MatMulNBits on integer tensor-core MMA (mma.sync m16n8k32, u8 x s8).
//
// Definition of the level (owned by this project, see nbits_int8.cu): activations are quantized
// per (token, quantization block) to int8, the block dot products sum aq * (q - zp) are exact
// int32 and are combined in fp32 as  Y += (sa * scale) * float(dot).
//
// Mapping. The 4-bit codes are the MMA "A" operand as unsigned bytes: a lane loads one 32-bit
// word (eight codes of one weight row), `w & 0x0f0f0f0f` and `(w >> 4) & 0x0f0f0f0f` are two
// A registers. That places codes 0,2,4,6 of the word in k slots 4t..4t+3 and codes 1,3,5,7 in
// slots 16+4t..16+4t+3 of the 32-wide step; the activations are stored in that order by the
// quantization kernel, so no shuffle is needed. The zero point is taken out afterwards with
// the per-block activation sums: sum aq*(q - zp) = D - zp * sum aq. A node without zero points
// (zp = 8 everywhere) skips that: its codes enter as the signed bytes 16 * (q - 8), which cost
// the same three operations per word, and the factor 16 is folded into the activation scale. One MMA step covers 32
// consecutive k, so a quantization block (32, 64, 128, ...) is a whole number of steps and the
// int32 accumulator restarts at each block.
//
// Data movement. Persistent CTA per SM, a producer lane fills a ring of 16 KB tasks (16 weight
// rows x 2048 k) with one 3-D tiled TMA load each - box {128 bytes, 16 rows, 8 segments} with
// the 128-byte swizzle, so that the eight lanes that read the same 16-byte column of eight
// different rows hit eight different banks - plus one bulk copy of the task's scales and zero
// points from the prepared side array shared with the fp32 decode kernel. The quantized
// activations of a pass (8 or 16 tokens), their scales and sums arrive with one bulk copy.
// Sixteen consumer warps share every task (one 128-k group each) and their sums are added
// through shared memory once per row tile. Every wait on data is bounded.
//
// Conventions: packed-INT4 nibble order of
// onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:60-93; u8 x s8 -> s32 dot and
// zero-point correction through sums as in the same file, :48-56 and :208-223.

#include "nbits_common.cuh"
#include "nbits_ptx.cuh"
#include "nbits_tma.cuh"

#include <cstdint>

namespace mnb {
namespace {

constexpr int kWarps = 16;                   // consumer warps = 128-k groups of a task
constexpr int kConsumerThreads = kWarps * 32;
// one issuing thread cannot keep enough tile loads in flight for the full memory bandwidth
// (measured 4.4 TB/s against 6.7 TB/s with four): four producer warps issue tasks round-robin
constexpr int kProducers = 4;
constexpr int kThreads = (kWarps + kProducers) * 32;
constexpr int kMaxSlots = 16;
constexpr int kTaskK = 2048;                 // k per task
constexpr int kTaskBytes = 16 * kTaskK / 2;  // packed weights of a task: 16 rows
constexpr int kSegments = kTaskK / 256;      // 128-byte segments per row inside a task

// Up to three sibling nodes (same K, block size, zero points in all or none) in one launch: their
// half tiles (8 rows) form one sequence that is split over the CTAs, so the activation prologue, the
// ramp-up and the tail are paid once for the group. A row tile never straddles two nodes.
constexpr int kMaxGroupTiles = 256;   // row tiles of one CTA that the tile table of a grouped launch holds

struct NodeSet {
  WeightView w[kMaxGroupedNodes];
  int halves_end[kMaxGroupedNodes];   // half tiles of the launch up to and including the node
  int nodes;
};

struct NodeMaps {
  CUtensorMap b[kMaxGroupedNodes];
};

struct TilePlace {
  int node;
  int h0;       // first half tile inside the node
  int halves;   // 1 or 2
};

// The CTA's row tiles when several nodes share the launch, packed node << 28 | halves << 24 | h0;
// built by one thread. Returns the number of tiles.
__device__ inline int BuildTileTable(const NodeSet &set, int h_begin, int h_end, int *table) {
  int h = h_begin;
  int count = 0;
  while (h < h_end && count < kMaxGroupTiles) {
    int node = 0;
    int start = 0;
    for (int i = 0; i + 1 < set.nodes; ++i) {
      if (h >= set.halves_end[i]) {
        node = i + 1;
        start = set.halves_end[i];
      }
    }
    int halves = h_end - h < 2 ? h_end - h : 2;
    halves = set.halves_end[node] - h < halves ? set.halves_end[node] - h : halves;
    table[count++] = (node << 28) | (halves << 24) | (h - start);
    h += halves;
  }
  return count;
}

__device__ __forceinline__ TilePlace PlaceOfTile(const NodeSet &set, const int *table, int h_begin, int h_end,
                                                 int tile) {
  TilePlace at;
  if (set.nodes == 1) {
    at.node = 0;
    at.h0 = h_begin + 2 * tile;
    at.halves = h_end - at.h0 < 2 ? h_end - at.h0 : 2;
  } else {
    const int packed = table[tile];
    at.node = static_cast<int>(static_cast<unsigned>(packed) >> 28);
    at.halves = (packed >> 24) & 15;
    at.h0 = packed & 0xffffff;
  }
  return at;
}

__device__ __forceinline__ int HalfTilesOf(const NodeSet &set, int node) {
  return set.halves_end[node] - (node > 0 ? set.halves_end[node - 1] : 0);
}

struct ImmaParams {
  NodeSet set;
  const unsigned char *act; // [passes][pass_bytes]: quantized activations, then scales and sums
  int m_total;
  OutputView out[kMaxGroupedNodes];
  int *status;
  int bpt;             // quantization blocks per task
  int slices;          // tasks per row tile
  int rec_bytes;
  int rec_scale_bytes;
  int slot_bytes;
  int num_slots;
  int producers;       // producer warps in use: min(kProducers, num_slots), see the producer loop
  int tp;              // tokens per pass (8 or 16)
  int act_row_bytes;   // bytes between token rows of the quantized activations
  int table_offset;    // byte offset of the scale / sum table inside a pass
  int pass_bytes;
  int groups_per_block; // 128-k groups per quantization block (block_size >= 256), else 1
  std::int32_t *dots;   // DOTS instantiations only: [m, n, n_blocks] exact block dots, zero before the launch
};
static_assert(kTaskK == kWarps * 128, "one 128-k group of a task per consumer warp");

__device__ __forceinline__ void MmaU8S8(int (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                        std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void MmaU8S8Zero(int (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                            std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Signed A operand: used when the node has no zero points, with codes stored as 16 * (q - 8).
__device__ __forceinline__ void MmaS8S8(int (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                        std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void MmaS8S8Zero(int (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                            std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// (x & 0xf0f0f0f0) ^ 0x80808080: a code in the high nibble of each byte, minus 8, times 16, as a
// signed byte (the nibble pattern q ^ 8 is q - 8 in 4-bit two's complement).
__device__ __forceinline__ std::uint32_t SignedHighNibbles(std::uint32_t x) {
  std::uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(x), "r"(0xf0f0f0f0u), "r"(0x80808080u));
  return d;
}

__device__ __forceinline__ void TmaLoad3D(void *smem_dst, const void *tensor_map, int x, int y, int z,
                                          std::uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(ptx::SmemAddr(smem_dst)),
               "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(ptx::SmemAddr(bar))
               : "memory");
}

// Byte position of activation k inside a token row: 128-k group major, then the quad lane
// t = (k / 8) % 4 that consumes it, the step s = (k / 32) % 4, then even k before odd k.
__host__ __device__ inline int ActBytePosition(int k) {
  const int j = k & 7;
  const int t = (k >> 3) & 3;
  const int s = (k >> 5) & 3;
  return ((k >> 7) << 7) + (t << 5) + (s << 3) + ((j & 1) ? 4 + (j >> 1) : (j >> 1));
}

// Launch with programmatic stream serialization: the kernel's blocks may become resident while the
// kernel before it in the stream drains; it waits (griddepcontrol.wait) before it touches anything
// that kernel wrote or still reads.
template <typename Kernel, typename... Args>
bool LaunchSerialized(Kernel kernel, dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cudaLaunchKernelEx(&config, kernel, args...) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return true;
}

// Quantizes one pass layout: one warp per (token slot, table entry) over passes * tp slots and
// the task-padded entry count. An entry covers min(block_size, 128) consecutive k: a whole
// quantization block, or a 128-k part of a larger one (same scale, its own sum). Slots beyond
// M, entries beyond the last block and k beyond K become zeros.
__global__ void __launch_bounds__(256)
    nbits_quantize_a_imma_kernel(const float *a, int m_total, std::int64_t k, int block_size, int entry_k,
                                 int entries_pad, int tp, int act_row_bytes, int table_offset, int pass_bytes,
                                 int passes, float table_scale, unsigned char *act) {
  // the multiply kernel behind this one may start (barrier set-up, first weight tiles) right away
  ptx::GridDependencyLaunch();
  // launched with programmatic serialization itself: A and the scratch are touched once the kernel
  // before this one in the stream (which may still read the scratch) has completed
  ptx::GridDependencyWait();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const std::int64_t item = static_cast<std::int64_t>(blockIdx.x) * 8 + warp;
  if (item >= static_cast<std::int64_t>(passes) * tp * entries_pad) {
    return;
  }
  const int slot = static_cast<int>(item / entries_pad);
  const int entry = static_cast<int>(item - static_cast<std::int64_t>(slot) * entries_pad);
  const int pass = slot / tp;
  const int token = slot - pass * tp;
  const int row = slot; // passes are consecutive groups of tp tokens
  const std::int64_t e0 = static_cast<std::int64_t>(entry) * entry_k;
  const std::int64_t k0 = e0 / block_size * block_size; // start of the enclosing quantization block
  const bool live = row < m_total;
  const float *src = a + static_cast<std::int64_t>(row) * k;
  float amax = 0.0f;
  bool bad = false;  // a NaN or an infinity in the block
  if (live) {
    for (int e = lane; e < block_size; e += 32) {
      if (k0 + e < k) {
        const float v = fabsf(src[k0 + e]);
        amax = fmaxf(amax, v);
        bad = bad || !(v <= 3.4028235e38f);
      }
    }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  }
  bad = __any_sync(0xffffffffu, bad);
  // a block with a non-finite activation: scale NaN, codes 0, every output of the token NaN
  const float sa = bad ? __int_as_float(0x7fc00000) : __fdiv_rn(amax, 127.0f);
  unsigned char *base = act + static_cast<std::int64_t>(pass) * pass_bytes;
  std::int8_t *dst = reinterpret_cast<std::int8_t *>(base) + static_cast<std::int64_t>(token) * act_row_bytes;
  int sum = 0;
  for (int e = lane; e < entry_k; e += 32) {
    const std::int64_t kk = e0 + e;
    int q = 0;
    if (live && kk < k && sa > 0.0f) {
      const float r = rintf(__fdiv_rn(src[kk], sa));
      q = static_cast<int>(fminf(127.0f, fmaxf(-127.0f, r)));
    }
    sum += q;
    dst[ActBytePosition(static_cast<int>(kk))] = static_cast<std::int8_t>(q);
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    sum += __shfl_xor_sync(0xffffffffu, sum, offset);
  }
  if (lane == 0) {
    unsigned char *cell = base + table_offset + static_cast<std::int64_t>(entry) * tp * 8;
    // table_scale is 1, or 1/16 for nodes without zero points, whose codes enter the MMA as
    // 16 * (q - 8): an exact power-of-two factor either way
    reinterpret_cast<float *>(cell)[token] = sa * table_scale;
    reinterpret_cast<int *>(cell + tp * 4)[token] = sum;
  }
}

// NT: 8-token column tiles per pass (tp = 8 * NT). SPB: 32-k steps per table entry: 1 / 2 for
// block_size 32 / 64, 4 for block_size >= 128.
//
// All sixteen consumer warps work on the same task: warp w takes the 128-k group w of its 2048
// k. The ring therefore only has to cover the memory latency, every warp is busy whatever the
// number of row tiles of the CTA, and the pipeline starts with the first task that lands. The
// price is a sum over the sixteen warps per row tile, done through shared memory by NT warps
// (rotating with the tile index) while the others go on with the next tile.
// DOTS: parity instrument, small shapes only. The int32 sum of every table entry (after the zero
// point has been taken out, before any scale is applied) is also added to p.dots, so that the
// block dots of THIS kernel - fragment layout, swizzled box, signed-code form and zero-point
// correction included - can be compared bit for bit with the CPU restatement.
template <int NT, int SPB, bool HAS_ZP, bool DOTS = false>
__global__ void __launch_bounds__(kThreads, 1)
    nbits_int8_mma_kernel(const __grid_constant__ NodeMaps maps, const ImmaParams p) {
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char *smem_raw = smem_dyn + ((1024u - (ptx::SmemAddr(smem_dyn) & 1023u)) & 1023u);
  // layout: [slots][activations of the pass + table][partial sums: 2 x 16 warps][barriers]
  unsigned char *slots = smem_raw;
  unsigned char *act = smem_raw + static_cast<size_t>(p.num_slots) * p.slot_bytes;
  float4 *partial = reinterpret_cast<float4 *>(act + p.pass_bytes); // [2][kWarps][NT][32]
  std::uint64_t *full_bar = reinterpret_cast<std::uint64_t *>(partial + 2 * kWarps * NT * 32);
  std::uint64_t *empty_bar = full_bar + kMaxSlots;
  std::uint64_t *act_bar = empty_bar + kMaxSlots;
  int *tile_table = reinterpret_cast<int *>(act_bar + 1);   // [kMaxGroupTiles] + the tile count (grouped launches)

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int m_base = blockIdx.y * p.tp;
  // what follows in the stream (the next call's quantization) may be scheduled as SMs free up
  ptx::GridDependencyLaunch();

  const int total_halves = p.set.halves_end[p.set.nodes - 1];
  const int h_begin = static_cast<int>(static_cast<std::int64_t>(blockIdx.x) * total_halves / gridDim.x);
  const int h_end = static_cast<int>(static_cast<std::int64_t>(blockIdx.x + 1) * total_halves / gridDim.x);

  if (warp >= kWarps) {
    // ------------------------------ producers ------------------------------
    // Producer j issues tasks j, j + kProducers, ...; producer 0 also fetches the activations.
    const int producer = warp - kWarps;
    if (producer == 0 && lane == 0) {
      for (int s = 0; s < p.num_slots; ++s) {
        ptx::MbarInit(&full_bar[s], 1);
        ptx::MbarInit(&empty_bar[s], kWarps);
      }
      ptx::MbarInit(act_bar, 1);
      ptx::FenceMbarInit();
      if (p.set.nodes > 1) {
        tile_table[kMaxGroupTiles] = BuildTileTable(p.set, h_begin, h_end, tile_table);
      }
    }
    asm volatile("bar.sync 11, %0;" ::"n"(kProducers * 32) : "memory"); // barriers initialised
    asm volatile("bar.arrive 10, %0;" ::"n"(kThreads) : "memory");
    if (lane == 0) {
      const int n_tiles = p.set.nodes == 1 ? (h_end - h_begin + 1) >> 1 : tile_table[kMaxGroupTiles];
      for (int i = 0; i < p.set.nodes; ++i) {
        ptx::PrefetchTensorMap(&maps.b[i]);
      }
      const int total = n_tiles * p.slices;
      bool ok = true;
      // The quantized activations come from the kernel launched just before this one (programmatic
      // dependent launch). Producer 0 asks for them FIRST: they are what the consumers need first, and
      // a response from L2 queues behind whatever the SM asked for earlier (asked for after the first
      // ring of weight tiles they landed 3.9 us after the CTA's start, 2.2 us of that behind 128 KB
      // of weights). The other producers start on the weight tiles at once; the weights do not
      // depend on the kernel before.
      if (producer == 0) {
        ptx::GridDependencyWait();
        ptx::MbarArriveExpectTx(act_bar, static_cast<std::uint32_t>(p.pass_bytes));
        ptx::BulkLoad(act, p.act + static_cast<std::int64_t>(blockIdx.y) * p.pass_bytes,
                      static_cast<std::uint32_t>(p.pass_bytes), act_bar);
      }
      int tile = 0;
      int s = producer;
      // A producer that has passed the wait for task T - producers knows that task
      // T - producers - num_slots is consumed. The parity wait for task T is only unambiguous
      // when task T - 2 * num_slots is consumed too, which follows when producers <= num_slots;
      // the host sets p.producers accordingly and the remaining producer warps stay idle.
      for (int task = producer; producer < p.producers && task < total && ok;
           task += p.producers, s += p.producers) {
        while (s >= p.slices) {
          s -= p.slices;
          ++tile;
        }
        const int slot = task % p.num_slots;
        const std::uint32_t round = static_cast<std::uint32_t>(task / p.num_slots);
        if (round != 0) {
          if (!ptx::MbarWait(&empty_bar[slot], (round & 1u) ^ 1u)) {
            ReportStatus(p.status, kDeviceTimeoutEmptyBarrier);
            ok = false;
            break;
          }
        }
        const TilePlace at = PlaceOfTile(p.set, tile_table, h_begin, h_end, tile);
        const int h0 = at.h0;
        const int node_halves = HalfTilesOf(p.set, at.node);
        const unsigned char *meta_src = p.set.w[at.node].meta + static_cast<std::int64_t>(h0) * p.rec_bytes +
                                        static_cast<std::int64_t>(s) * node_halves * p.rec_bytes;
        const std::uint32_t meta_bytes = (h0 + 1 < node_halves ? 2u : 1u) * static_cast<std::uint32_t>(p.rec_bytes);
        unsigned char *dst = slots + static_cast<size_t>(slot) * p.slot_bytes;
        ptx::MbarArriveExpectTx(&full_bar[slot], kTaskBytes + meta_bytes);
        TmaLoad3D(dst, &maps.b[at.node], 0, h0 * 8, s * kSegments, &full_bar[slot]);
        ptx::BulkLoad(dst + kTaskBytes, meta_src, meta_bytes, &full_bar[slot]);
      }
      // stay until every copy this lane issued has been consumed (bounded), so none lands after exit
      const int first = total - p.num_slots < 0 ? 0 : total - p.num_slots;
      for (int i = first; i < total && ok; ++i) {
        if (producer < p.producers && (i % p.producers) == producer &&
            !ptx::MbarWait(&empty_bar[i % p.num_slots], static_cast<std::uint32_t>(i / p.num_slots) & 1u)) {
          break;
        }
      }
      if (producer == 0) {
        ptx::MbarWait(act_bar, 0);
      }
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  asm volatile("bar.sync 10, %0;" ::"n"(kThreads) : "memory"); // barriers initialised
  const int n_tiles = p.set.nodes == 1 ? (h_end - h_begin + 1) >> 1 : tile_table[kMaxGroupTiles];
  bool dead = false; // a bounded wait gave up: skip the math, keep the barrier protocol
  if (!ptx::MbarWait(act_bar, 0)) {
    ReportStatus(p.status, kDeviceTimeoutFullBarrier);
    dead = true;
  }

  const int g = lane >> 2;
  const int t = lane & 3;
  const std::uint32_t nib = 0x0f0f0f0fu;
  // this warp's 128-k group inside every task: segment warp / 2, chunks 4 * (warp % 2) + step.
  // Byte offset of the lane's word for each step (rows g; rows g + 8 are 1024 bytes further):
  int word_off[4];
#pragma unroll
  for (int st = 0; st < 4; ++st) {
    const int c = (warp & 1) * 4 + st;
    word_off[st] = (warp >> 1) * 2048 + g * 128 + ((c ^ g) << 4) + 4 * t;
  }
  constexpr int kEntriesPerGroup = 4 / SPB;
  const int scale_row_bytes = p.rec_scale_bytes / 8;
  // scale / zero-point index of this warp's first block inside a task record row
  const int meta_index = p.groups_per_block > 1 ? warp / p.groups_per_block : warp * kEntriesPerGroup;
  const int entry_bytes = p.tp * 8;
  const int entries_per_task = 16 * kEntriesPerGroup;
  const unsigned char *table = act + p.table_offset + 8 * t + warp * kEntriesPerGroup * entry_bytes;
  const unsigned char *act_lane = act + g * p.act_row_bytes + t * 32 + warp * 128;

  int task = 0;
  int slot = 0;
  std::uint32_t round = 0;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const TilePlace at = PlaceOfTile(p.set, tile_table, h_begin, h_end, tile);
    const WeightView &node_w = p.set.w[at.node];
    const std::int64_t row0 = static_cast<std::int64_t>(at.h0) * 8;
    const std::int64_t row_limit = row0 + at.halves * 8 < node_w.n ? row0 + at.halves * 8 : node_w.n;
    float acc[NT][4];
    int d[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[nt][i] = 0.0f;
        d[nt][i] = 0;
      }
    }

    for (int s = 0; s < p.slices; ++s, ++task) {
      if (!dead && !ptx::MbarWait(&full_bar[slot], round & 1u)) {
        ReportStatus(p.status, kDeviceTimeoutFullBarrier);
        dead = true;
      }
      if (!dead) {
        const unsigned char *sb = slots + static_cast<size_t>(slot) * p.slot_bytes;
        std::uint32_t w_lo[4], w_hi[4];
#pragma unroll
        for (int st = 0; st < 4; ++st) {
          w_lo[st] = *reinterpret_cast<const std::uint32_t *>(sb + word_off[st]);
          w_hi[st] = *reinterpret_cast<const std::uint32_t *>(sb + word_off[st] + 1024);
        }
        const unsigned char *meta0 = sb + kTaskBytes;
        const unsigned char *meta1 = meta0 + p.rec_bytes;
        const float *sc0 = reinterpret_cast<const float *>(meta0 + g * scale_row_bytes) + meta_index;
        const float *sc1 = reinterpret_cast<const float *>(meta1 + g * scale_row_bytes) + meta_index;
        float ws_lo[kEntriesPerGroup], ws_hi[kEntriesPerGroup];
        int zp_lo[kEntriesPerGroup], zp_hi[kEntriesPerGroup];
        if constexpr (SPB == 1) {
          const float4 a4 = *reinterpret_cast<const float4 *>(sc0);
          const float4 b4 = *reinterpret_cast<const float4 *>(sc1);
          ws_lo[0] = a4.x, ws_lo[1] = a4.y, ws_lo[2] = a4.z, ws_lo[3] = a4.w;
          ws_hi[0] = b4.x, ws_hi[1] = b4.y, ws_hi[2] = b4.z, ws_hi[3] = b4.w;
        } else if constexpr (SPB == 2) {
          const float2 a2 = *reinterpret_cast<const float2 *>(sc0);
          const float2 b2 = *reinterpret_cast<const float2 *>(sc1);
          ws_lo[0] = a2.x, ws_lo[1] = a2.y, ws_hi[0] = b2.x, ws_hi[1] = b2.y;
        } else {
          ws_lo[0] = sc0[0], ws_hi[0] = sc1[0];
        }
        if constexpr (HAS_ZP) {
          const unsigned char *zr0 = meta0 + p.rec_scale_bytes + g * p.bpt + meta_index;
          const unsigned char *zr1 = meta1 + p.rec_scale_bytes + g * p.bpt + meta_index;
          if constexpr (SPB == 1) {
            const std::uint32_t za = *reinterpret_cast<const std::uint32_t *>(zr0);
            const std::uint32_t zb = *reinterpret_cast<const std::uint32_t *>(zr1);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              zp_lo[i] = static_cast<int>((za >> (8 * i)) & 0xffu);
              zp_hi[i] = static_cast<int>((zb >> (8 * i)) & 0xffu);
            }
          } else {
#pragma unroll
            for (int i = 0; i < kEntriesPerGroup; ++i) {
              zp_lo[i] = zr0[i];
              zp_hi[i] = zr1[i];
            }
          }
        }
        // activations of the four steps: 32 bytes per lane and column tile
        uint4 bq[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const unsigned char *src = act_lane + static_cast<size_t>(s) * kTaskK + nt * 8 * p.act_row_bytes;
          bq[nt][0] = *reinterpret_cast<const uint4 *>(src);
          bq[nt][1] = *reinterpret_cast<const uint4 *>(src + 16);
        }
        // the weights are in registers: hand the slot back before the arithmetic
        __syncwarp();
        if (lane == 0) {
          ptx::MbarArrive(&empty_bar[slot]);
        }
        const unsigned char *cell = table + static_cast<size_t>(s) * entries_per_task * entry_bytes;
#pragma unroll
        for (int st = 0; st < 4; ++st) {
          // with zero points: unsigned codes, zero point taken out afterwards through the sums;
          // without: 16 * (q - 8) as signed bytes, nothing to take out (same three operations)
          const std::uint32_t a0 = HAS_ZP ? (w_lo[st] & nib) : SignedHighNibbles(w_lo[st] << 4);
          const std::uint32_t a1 = HAS_ZP ? (w_hi[st] & nib) : SignedHighNibbles(w_hi[st] << 4);
          const std::uint32_t a2 = HAS_ZP ? ((w_lo[st] >> 4) & nib) : SignedHighNibbles(w_lo[st]);
          const std::uint32_t a3 = HAS_ZP ? ((w_hi[st] >> 4) & nib) : SignedHighNibbles(w_hi[st]);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4 &q = bq[nt][st >> 1];
            const std::uint32_t b0 = (st & 1) ? q.z : q.x;
            const std::uint32_t b1 = (st & 1) ? q.w : q.y;
            if constexpr (HAS_ZP) {
              if ((st % SPB) == 0) {
                MmaU8S8Zero(d[nt], a0, a1, a2, a3, b0, b1);
              } else {
                MmaU8S8(d[nt], a0, a1, a2, a3, b0, b1);
              }
            } else {
              if ((st % SPB) == 0) {
                MmaS8S8Zero(d[nt], a0, a1, a2, a3, b0, b1);
              } else {
                MmaS8S8(d[nt], a0, a1, a2, a3, b0, b1);
              }
            }
          }
          if (((st + 1) % SPB) == 0) {
            // a table entry is complete: D - zp * sum(aq), scaled, into the fp32 sums
            const int idx = st / SPB;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const float2 sa = *reinterpret_cast<const float2 *>(cell + idx * entry_bytes + nt * 32);
              int e0 = d[nt][0], e1 = d[nt][1], e2 = d[nt][2], e3 = d[nt][3];
              if constexpr (HAS_ZP) {
                const int2 sum = *reinterpret_cast<const int2 *>(cell + idx * entry_bytes + p.tp * 4 + nt * 32);
                e0 -= zp_lo[idx] * sum.x;
                e1 -= zp_lo[idx] * sum.y;
                e2 -= zp_hi[idx] * sum.x;
                e3 -= zp_hi[idx] * sum.y;
              }
              if constexpr (DOTS) {
                // entry -> quantization block; signed codes carry a factor 16
                const std::int64_t k0 = static_cast<std::int64_t>(s) * kTaskK + warp * 128 + idx * 32 * SPB;
                const std::int64_t block = k0 / node_w.block_size;
                const int shift = HAS_ZP ? 0 : 4;
                const int values[4] = {e0 >> shift, e1 >> shift, e2 >> shift, e3 >> shift};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const std::int64_t row = row0 + g + 8 * (i >> 1);
                  const std::int64_t token = static_cast<std::int64_t>(blockIdx.y) * p.tp + nt * 8 + 2 * t + (i & 1);
                  if (row < row_limit && token < p.m_total && block < node_w.n_blocks) {
                    atomicAdd(p.dots + (token * node_w.n + row) * node_w.n_blocks + block, values[i]);
                  }
                }
              }
              acc[nt][0] = fmaf(sa.x * ws_lo[idx], static_cast<float>(e0), acc[nt][0]);
              acc[nt][1] = fmaf(sa.y * ws_lo[idx], static_cast<float>(e1), acc[nt][1]);
              acc[nt][2] = fmaf(sa.x * ws_hi[idx], static_cast<float>(e2), acc[nt][2]);
              acc[nt][3] = fmaf(sa.y * ws_hi[idx], static_cast<float>(e3), acc[nt][3]);
            }
          }
        }
      }
      if (++slot == p.num_slots) {
        slot = 0;
        ++round;
      }
    }

    // ---- sum over the sixteen warps -----------------------------------------------------------
    // Buffer b = tile % 2. Named barriers 2 + b ("partials of this tile written") and 4 + b
    // ("buffer read, may be overwritten"), 512 participants each: the NT reducing warps of a
    // tile wait on the first and arrive on the second, everybody else the other way round.
    const int b = tile & 1;
    const int reducer0 = (tile * NT) & (kWarps - 1);
    const bool reduces = ((warp - reducer0) & (kWarps - 1)) < NT;
    if (tile >= 2) {
      const int previous0 = ((tile - 2) * NT) & (kWarps - 1);
      const bool reduced_previous = ((warp - previous0) & (kWarps - 1)) < NT;
      if (!reduced_previous) {
        asm volatile("bar.sync %0, %1;" ::"r"(4 + b), "n"(kConsumerThreads) : "memory");
      }
    }
    float4 *mine = partial + ((b * kWarps + warp) * NT) * 32 + lane;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      mine[nt * 32] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
    }
    if (!reduces) {
      asm volatile("bar.arrive %0, %1;" ::"r"(2 + b), "n"(kConsumerThreads) : "memory");
    } else {
      asm volatile("bar.sync %0, %1;" ::"r"(2 + b), "n"(kConsumerThreads) : "memory");
      const int nt = (warp - reducer0) & (kWarps - 1);
      const float4 *column = partial + (b * kWarps * NT + nt) * 32 + lane;
      float4 total = column[0];
#pragma unroll
      for (int w = 1; w < kWarps; ++w) {
        const float4 v = column[w * NT * 32];
        total.x += v.x, total.y += v.y, total.z += v.z, total.w += v.w;
      }
      if (tile + 2 < n_tiles) {
        asm volatile("bar.arrive %0, %1;" ::"r"(4 + b), "n"(kConsumerThreads) : "memory");
      }
      const std::int64_t r_lo = row0 + g;
      const std::int64_t r_hi = row0 + g + 8;
      const float bias_lo = (node_w.bias != nullptr && r_lo < row_limit) ? __ldg(node_w.bias + r_lo) : 0.0f;
      const float bias_hi = (node_w.bias != nullptr && r_hi < row_limit) ? __ldg(node_w.bias + r_hi) : 0.0f;
      const std::int64_t m0 = m_base + nt * 8 + 2 * t;
      const OutputView &node_out = p.out[at.node];
      float *y0 = node_out.y + m0 * node_out.ld + node_out.col_offset;
      float *y1 = y0 + node_out.ld;
      if (m0 < p.m_total) {
        if (r_lo < row_limit) {
          y0[r_lo] = total.x + bias_lo;
        }
        if (r_hi < row_limit) {
          y0[r_hi] = total.z + bias_hi;
        }
      }
      if (m0 + 1 < p.m_total) {
        if (r_lo < row_limit) {
          y1[r_lo] = total.y + bias_lo;
        }
        if (r_hi < row_limit) {
          y1[r_hi] = total.w + bias_hi;
        }
      }
    }
  }
}

bool EncodeWeightsMap3D(CUtensorMap *map, const WeightView &w) {
  EncodeTiledFn encode = GetEncodeTiled();
  if (encode == nullptr) {
    return false;
  }
  // a packed row seen as [segments][32 words]; dimension order: word, row, segment
  const cuuint64_t dims[3] = {32, static_cast<cuuint64_t>(w.n), static_cast<cuuint64_t>(w.row_bytes / 128)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(w.row_bytes), 128};
  const cuuint32_t box[3] = {32, 16, kSegments};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<std::uint8_t *>(w.b), dims, strides, box,
                elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct ImmaGeometry {
  bool ok;
  int tp;
  int passes;
  int act_row_bytes;
  int table_offset;
  int pass_bytes;
  int entry_k;      // k covered by one scale / sum table entry: min(block_size, 128)
  int entries_pad;  // table entries of a token, padded to whole tasks
  int slot_bytes;
  int num_slots;
  std::size_t smem;
};

ImmaGeometry ImmaGeometryOf(const WeightView &w, std::int64_t m) {
  ImmaGeometry geo{};
  const MetaGeometry meta = MetaGeometryOf(w);
  if (meta.bytes == 0 || meta.bpt * w.block_size != kTaskK || (w.row_bytes % 128) != 0 || m < 1 ||
      (reinterpret_cast<std::uintptr_t>(w.b) & 15u) != 0) {
    return geo;
  }
  const int k_pad = meta.slices * kTaskK;
  geo.entry_k = w.block_size < 128 ? w.block_size : 128;
  geo.entries_pad = k_pad / geo.entry_k;
  geo.slot_bytes = (kTaskBytes + 2 * meta.rec_bytes + 1023) & ~1023;
  const std::size_t limit = 225 * 1024;
  for (int tp = m > 8 ? 16 : 8; tp >= 8; tp -= 8) {
    geo.tp = tp;
    geo.act_row_bytes = k_pad + 16; // 16: rows of a column tile land on different banks
    geo.table_offset = tp * geo.act_row_bytes;
    geo.pass_bytes = geo.table_offset + geo.entries_pad * tp * 8;
    const std::size_t fixed = static_cast<std::size_t>(geo.pass_bytes) +
                              2 * kWarps * (tp / 8) * 32 * sizeof(float4) +
                              (2 * kMaxSlots + 1) * sizeof(std::uint64_t) + 64 +
                              (kMaxGroupTiles + 1) * sizeof(int);
    if (geo.pass_bytes < (1 << 20) && fixed + 2 * static_cast<std::size_t>(geo.slot_bytes) + 1024 <= limit) {
      int slots = static_cast<int>((limit - fixed - 1024) / geo.slot_bytes);
      geo.num_slots = slots > kMaxSlots ? kMaxSlots : slots;
      geo.smem = static_cast<std::size_t>(geo.num_slots) * geo.slot_bytes + fixed + 1024;
      geo.passes = static_cast<int>((m + tp - 1) / tp);
      geo.ok = true;
      return geo;
    }
  }
  return geo;
}

} // namespace

std::size_t Int8MmaScratchBytes(const WeightView &w, std::int64_t m) {
  const ImmaGeometry geo = ImmaGeometryOf(w, m);
  return geo.ok ? static_cast<std::size_t>(geo.passes) * geo.pass_bytes : 0;
}

namespace {
const char *LaunchMultiplyNodes(const WeightView *nodes, const OutputView *outs, int count, const ImmaGeometry &geo,
                                std::int64_t m, unsigned char *scratch, int *status_word, cudaStream_t stream,
                                int sm_count, std::int32_t *dots = nullptr);
const char *LaunchMultiply(const WeightView &w, const ImmaGeometry &geo, std::int64_t m, unsigned char *scratch,
                           OutputView out, int *status_word, cudaStream_t stream, int sm_count,
                           std::int32_t *dots = nullptr) {
  return LaunchMultiplyNodes(&w, &out, 1, geo, m, scratch, status_word, stream, sm_count, dots);
}
} // namespace

// Quantizes `a` into `scratch` (Int8MmaScratchBytes) and runs the integer-MMA kernel.
const char *LaunchInt8Mma(const WeightView &w, const float *a, std::int64_t m, unsigned char *scratch,
                          OutputView out, int *status_word, cudaStream_t stream, int sm_count) {
  const ImmaGeometry geo = ImmaGeometryOf(w, m);
  if (!geo.ok || w.meta == nullptr || scratch == nullptr) {
    return nullptr;
  }
  const std::int64_t items = static_cast<std::int64_t>(geo.passes) * geo.tp * geo.entries_pad;
  if (!LaunchSerialized(nbits_quantize_a_imma_kernel, dim3(static_cast<unsigned>((items + 7) / 8)), dim3(256), stream, a,
                        static_cast<int>(m), w.k, w.block_size, geo.entry_k, geo.entries_pad, geo.tp, geo.act_row_bytes,
                        geo.table_offset, geo.pass_bytes, geo.passes, w.zp != nullptr ? 1.0f : 0.0625f, scratch)) {
    return nullptr;
  }
  CountLaunch();
  return LaunchMultiply(w, geo, m, scratch, out, status_word, stream, sm_count);
}

namespace {
// Nodes of a group share one activation layout when the layout's sizes and the table scale agree.
bool SameActivationLayout(const WeightView &a, const ImmaGeometry &ga, const WeightView &b, const ImmaGeometry &gb) {
  return a.k == b.k && a.block_size == b.block_size && (a.zp != nullptr) == (b.zp != nullptr) && ga.tp == gb.tp &&
         ga.passes == gb.passes && ga.act_row_bytes == gb.act_row_bytes && ga.table_offset == gb.table_offset &&
         ga.pass_bytes == gb.pass_bytes && ga.entry_k == gb.entry_k && ga.entries_pad == gb.entries_pad;
}
} // namespace

// Sibling nodes (same K, block size, zero points in all or none): the activations are quantized
// once into `scratch` and every node's integer-MMA kernel reads them from there.
const char *LaunchInt8MmaGroup(const WeightView *nodes, const OutputView *outs, int count, const float *a,
                               std::int64_t m, unsigned char *scratch, int *status_word, cudaStream_t stream,
                               int sm_count) {
  if (count < 1 || count > kMaxGroupedNodes || scratch == nullptr) {
    return nullptr;
  }
  const WeightView &w = nodes[0];
  const ImmaGeometry geo = ImmaGeometryOf(w, m);
  if (!geo.ok) {
    return nullptr;
  }
  for (int i = 0; i < count; ++i) {
    if (nodes[i].meta == nullptr || !SameActivationLayout(w, geo, nodes[i], ImmaGeometryOf(nodes[i], m))) {
      return nullptr;
    }
  }
  const std::int64_t items = static_cast<std::int64_t>(geo.passes) * geo.tp * geo.entries_pad;
  if (!LaunchSerialized(nbits_quantize_a_imma_kernel, dim3(static_cast<unsigned>((items + 7) / 8)), dim3(256), stream, a,
                        static_cast<int>(m), w.k, w.block_size, geo.entry_k, geo.entries_pad, geo.tp, geo.act_row_bytes,
                        geo.table_offset, geo.pass_bytes, geo.passes, w.zp != nullptr ? 1.0f : 0.0625f, scratch)) {
    return nullptr;
  }
  CountLaunch();
  // one launch for the group: the nodes' row tiles form one sequence over the CTAs
  if (LaunchMultiplyNodes(nodes, outs, count, geo, m, scratch, status_word, stream, sm_count) != nullptr) {
    return "nbits_int8_mma_kernel";
  }
  cudaGetLastError();
  for (int i = 0; i < count; ++i) {
    if (LaunchMultiply(nodes[i], ImmaGeometryOf(nodes[i], m), m, scratch, outs[i], status_word, stream, sm_count) ==
        nullptr) {
      return nullptr;
    }
  }
  return "nbits_int8_mma_kernel";
}

// Parity instrument: quantizes `a` like LaunchInt8Mma and runs the instrumented form of the kernel,
// which also adds its exact int32 block dots to `dots` ([m, n, n_blocks], zeroed here). m <= 8.
const char *LaunchInt8MmaBlockDots(const WeightView &w, const float *a, std::int64_t m, unsigned char *scratch,
                                   OutputView out, std::int32_t *dots, int *status_word, cudaStream_t stream,
                                   int sm_count) {
  const ImmaGeometry geo = ImmaGeometryOf(w, m);
  if (!geo.ok || w.meta == nullptr || scratch == nullptr || dots == nullptr || geo.tp != 8) {
    return nullptr;
  }
  if (cudaMemsetAsync(dots, 0, static_cast<size_t>(m) * w.n * w.n_blocks * sizeof(std::int32_t), stream) !=
      cudaSuccess) {
    return nullptr;
  }
  const std::int64_t items = static_cast<std::int64_t>(geo.passes) * geo.tp * geo.entries_pad;
  if (!LaunchSerialized(nbits_quantize_a_imma_kernel, dim3(static_cast<unsigned>((items + 7) / 8)), dim3(256), stream, a,
                        static_cast<int>(m), w.k, w.block_size, geo.entry_k, geo.entries_pad, geo.tp, geo.act_row_bytes,
                        geo.table_offset, geo.pass_bytes, geo.passes, w.zp != nullptr ? 1.0f : 0.0625f, scratch)) {
    return nullptr;
  }
  CountLaunch();
  return LaunchMultiply(w, geo, m, scratch, out, status_word, stream, sm_count, dots);
}

namespace {
// Fills the node table of a launch: the nodes' half tiles one after the other. False when a node
// has no prepared records or the group is larger than the kernels take.
bool FillNodeSet(const WeightView *nodes, int count, NodeSet *set, NodeMaps *maps, std::int64_t *tiles) {
  if (count < 1 || count > kMaxGroupedNodes) {
    return false;
  }
  int halves = 0;
  *tiles = 0;
  for (int i = 0; i < kMaxGroupedNodes; ++i) {
    const WeightView &w = nodes[i < count ? i : 0];
    set->w[i] = w;
    if (i < count) {
      if (w.meta == nullptr || !EncodeWeightsMap3D(&maps->b[i], w)) {
        return false;
      }
      const MetaGeometry meta = MetaGeometryOf(w);
      halves += meta.half_tiles;
      *tiles += (meta.half_tiles + 1) / 2;
    } else {
      maps->b[i] = maps->b[0];
    }
    set->halves_end[i] = halves;
  }
  set->nodes = count;
  return true;
}

// The integer-MMA kernel over activations that the kernel launched just before has laid out in
// `scratch` (it is launched with programmatic stream serialization behind that kernel); one launch
// for all `count` nodes.
const char *LaunchMultiplyNodes(const WeightView *nodes, const OutputView *outs, int count, const ImmaGeometry &geo,
                                std::int64_t m, unsigned char *scratch, int *status_word, cudaStream_t stream,
                                int sm_count, std::int32_t *dots) {
  const WeightView &w = nodes[0];
  const MetaGeometry meta = MetaGeometryOf(w);
  ImmaParams p{};
  NodeMaps maps;
  std::int64_t tiles = 0;
  if (!FillNodeSet(nodes, count, &p.set, &maps, &tiles)) {
    return nullptr;
  }
  for (int i = 0; i < kMaxGroupedNodes; ++i) {
    p.out[i] = outs[i < count ? i : 0];
  }
  p.act = scratch;
  p.m_total = static_cast<int>(m);
  p.status = status_word;
  p.bpt = meta.bpt;
  p.slices = meta.slices;
  p.rec_bytes = meta.rec_bytes;
  p.rec_scale_bytes = meta.rec_scale_bytes;
  p.slot_bytes = geo.slot_bytes;
  p.num_slots = geo.num_slots;
  p.producers = geo.num_slots < WantedProducers(kProducers) ? geo.num_slots : WantedProducers(kProducers);
  p.tp = geo.tp;
  p.act_row_bytes = geo.act_row_bytes;
  p.table_offset = geo.table_offset;
  p.pass_bytes = geo.pass_bytes;
  p.groups_per_block = w.block_size >= 256 ? w.block_size / 128 : 1;
  p.dots = dots;
  if (dots != nullptr && geo.tp != 8) {
    return nullptr;  // the instrumented form exists for one column tile per pass only
  }
  const int spb = geo.entry_k / 32;

  int ctas = sm_count > 0 ? sm_count : 148;
  if (ctas > tiles) {
    ctas = static_cast<int>(tiles);
  }
  // a grouped launch keeps its row tiles in a table of kMaxGroupTiles entries per CTA
  if (count > 1 && (p.set.halves_end[count - 1] / ctas + 2) / 2 + count > kMaxGroupTiles) {
    return nullptr;
  }
  dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>(geo.passes), 1);
  cudaError_t err = cudaErrorInvalidValue;
#define MNB_IMMA_CASE(NT_, SPB_, ZP_)                                                            \
  if (geo.tp == 8 * NT_ && spb == SPB_ && (w.zp != nullptr) == ZP_) {                            \
    auto kernel = nbits_int8_mma_kernel<NT_, SPB_, ZP_>;                                         \
    if (dots != nullptr) {                                                                       \
      kernel = nbits_int8_mma_kernel<1, SPB_, ZP_, true>;                                        \
    }                                                                                            \
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,              \
                               static_cast<int>(geo.smem));                                      \
    if (err == cudaSuccess) {                                                                    \
      cudaLaunchConfig_t config = {};                                                            \
      config.gridDim = grid;                                                                     \
      config.blockDim = dim3(kThreads, 1, 1);                                                    \
      config.dynamicSmemBytes = geo.smem;                                                        \
      config.stream = stream;                                                                    \
      cudaLaunchAttribute attribute[1];                                                          \
      attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                      \
      attribute[0].val.programmaticStreamSerializationAllowed = 1;                               \
      config.attrs = attribute;                                                                  \
      config.numAttrs = 1;                                                                       \
      err = cudaLaunchKernelEx(&config, kernel, maps, p);                                        \
    }                                                                                            \
  }
#define MNB_IMMA_CASES(SPB_)                                                                     \
  MNB_IMMA_CASE(1, SPB_, true)                                                                   \
  MNB_IMMA_CASE(1, SPB_, false)                                                                  \
  MNB_IMMA_CASE(2, SPB_, true)                                                                   \
  MNB_IMMA_CASE(2, SPB_, false)
  MNB_IMMA_CASES(1)
  MNB_IMMA_CASES(2)
  MNB_IMMA_CASES(4)
#undef MNB_IMMA_CASES
#undef MNB_IMMA_CASE
  if (err != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return "nbits_int8_mma_kernel";
}
} // namespace


// ---- accuracy_level 0 through the same kernel: activations as three base-128 digits ----------
//
// A float row enters the integer MMA exactly enough for the 1e-5 bar of the fp32 decode paths when
// it is scaled so that its largest magnitude becomes kDigitRange, rounded to a 22-bit integer
// n = 16384 d0 + 128 d1 + d2 (d1, d2 in [-64, 63], |d0| <= 123) and handed to the kernel as THREE
// rows of signed bytes with the "activation scales" undo * {16384, 128, 1}: the kernel's per-block
// int32 dots are exact, its fp32 combination is the usual one, and the three partial rows are added
// (plus the bias) by a small kernel behind it. M tokens cost 3 M rows: 16 tokens take three passes
// of sixteen rows. Worth it where the fp16 kernels need one pass per token (block_size 32) or two.
namespace {

constexpr float kDigitRange = 2.0e6f;

// up[row] = factor applied to A (after `lift`, an exact power of two for rows of tiny magnitude),
// undo[row] = factor that takes the integer result back (NaN for a row with a non-finite entry).
// One CTA per row. factors = {up[m], lift[m], undo[m]} as three arrays of m_total floats.
__global__ void __launch_bounds__(256)
    nbits_digit_row_factors_kernel(const float *a, int m_total, std::int64_t k, float *factors) {
  // the digit kernel behind this one may be scheduled right away; it waits before it reads `factors`
  ptx::GridDependencyLaunch();
  __shared__ float warp_max[8];
  const int row = blockIdx.x;
  const float *src = a + static_cast<std::int64_t>(row) * k;
  float amax = 0.0f;
  bool bad = false;
  for (std::int64_t i = threadIdx.x; i < k; i += 256) {
    const float v = src[i];
    amax = fmaxf(amax, fabsf(v));
    bad = bad || (v != v);
  }
  if (bad) {
    amax = __int_as_float(0x7f800000);
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  }
  if ((threadIdx.x & 31) == 0) {
    warp_max[threadIdx.x >> 5] = amax;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) {
      amax = fmaxf(amax, warp_max[i]);
    }
    const bool finite = amax < 3.0e38f;
    const float lift = amax < 1.0e-18f ? 1.8446744e19f /* 2^64 */ : 1.0f;
    const float lifted = amax * lift;
    factors[row] = (finite && lifted > 0.0f) ? kDigitRange / lifted : 0.0f;
    factors[m_total + row] = lift;
    factors[2 * m_total + row] = finite ? (lifted / kDigitRange) / lift : __int_as_float(0x7fc00000);
  }
}

// Same work split and output layout as nbits_quantize_a_imma_kernel, for the digit rows: row
// 3 * token + digit of the pass layout holds digit `digit` of token `token`; its table entries carry
// undo * {16384, 128, 1} * table_scale and the digit sums.
__global__ void __launch_bounds__(256)
    nbits_digits_imma_kernel(const float *a, const float *factors, int m_total, std::int64_t k, int entry_k,
                             int entries_pad, int tp, int act_row_bytes, int table_offset, int pass_bytes,
                             int passes, float table_scale, unsigned char *act) {
  ptx::GridDependencyLaunch();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const std::int64_t item = static_cast<std::int64_t>(blockIdx.x) * 8 + warp;
  if (item >= static_cast<std::int64_t>(passes) * tp * entries_pad) {
    return;
  }
  const int slot = static_cast<int>(item / entries_pad);
  const int entry = static_cast<int>(item - static_cast<std::int64_t>(slot) * entries_pad);
  const int pass = slot / tp;
  const int row_in_pass = slot - pass * tp;
  const int token = slot / 3;
  const int digit = slot - 3 * token;
  const bool live = token < m_total;
  const float *src = a + static_cast<std::int64_t>(token) * k;
  const float up = live ? factors[token] : 0.0f;
  const float lift = live ? factors[m_total + token] : 1.0f;
  const float undo = live ? factors[2 * m_total + token] : 0.0f;
  unsigned char *base = act + static_cast<std::int64_t>(pass) * pass_bytes;
  std::int8_t *dst = reinterpret_cast<std::int8_t *>(base) + static_cast<std::int64_t>(row_in_pass) * act_row_bytes;
  const std::int64_t e0 = static_cast<std::int64_t>(entry) * entry_k;
  int sum = 0;
  for (int e = lane; e < entry_k; e += 32) {
    const std::int64_t kk = e0 + e;
    int q = 0;
    if (live && kk < k) {
      int n = __float2int_rn((src[kk] * lift) * up);
      const int range = static_cast<int>(kDigitRange);
      n = n > range ? range : (n < -range ? -range : n);
      const int low = ((n + 64) & 127) - 64;
      const int n1 = (n - low) >> 7;
      const int mid = ((n1 + 64) & 127) - 64;
      q = digit == 2 ? low : (digit == 1 ? mid : (n1 - mid) >> 7);
    }
    sum += q;
    dst[ActBytePosition(static_cast<int>(kk))] = static_cast<std::int8_t>(q);
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    sum += __shfl_xor_sync(0xffffffffu, sum, offset);
  }
  if (lane == 0) {
    unsigned char *cell = base + table_offset + static_cast<std::int64_t>(entry) * tp * 8;
    const float weight = digit == 0 ? 16384.0f : (digit == 1 ? 128.0f : 1.0f);
    reinterpret_cast<float *>(cell)[row_in_pass] = undo * weight * table_scale;
    reinterpret_cast<int *>(cell + tp * 4)[row_in_pass] = sum;
  }
}

// Y[token][n] = P[3 token][n] + P[3 token + 1][n] + P[3 token + 2][n] + bias[n].
__global__ void __launch_bounds__(256)
    nbits_digits_combine_kernel(const float *partial, const float *bias, int m_total, std::int64_t n, OutputView out) {
  const std::int64_t total = static_cast<std::int64_t>(m_total) * n;
  for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<std::int64_t>(gridDim.x) * 256) {
    const std::int64_t token = i / n;
    const std::int64_t col = i - token * n;
    const float *p0 = partial + (3 * token) * n + col;
    const float sum = (p0[0] + p0[n]) + p0[2 * n];
    StoreOutput(out, token * out.ld + out.col_offset + col, sum + (bias != nullptr ? bias[col] : 0.0f));
  }
}

// Same, four columns per thread and one token per blockIdx.y: N a multiple of 4 and 16-byte aligned
// rows of Y, the partial result and the bias.
__global__ void __launch_bounds__(256)
    nbits_digits_combine_vec_kernel(const float4 *partial, const float4 *bias, std::int64_t n4, OutputView out) {
  const std::int64_t token = blockIdx.y;
  const float4 *p0 = partial + 3 * token * n4;
  float4 *dst = reinterpret_cast<float4 *>(out.y + token * out.ld + out.col_offset);
  for (std::int64_t c = static_cast<std::int64_t>(blockIdx.x) * 256 + threadIdx.x; c < n4;
       c += static_cast<std::int64_t>(gridDim.x) * 256) {
    const float4 a = p0[c], b = p0[n4 + c], d = p0[2 * n4 + c];
    const float4 add = bias != nullptr ? bias[c] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    dst[c] = make_float4((a.x + b.x) + d.x + add.x, (a.y + b.y) + d.y + add.y, (a.z + b.z) + d.z + add.z,
                         (a.w + b.w) + d.w + add.w);
  }
}

std::size_t AlignUp(std::size_t v) { return (v + 255) & ~std::size_t{255}; }

// ---- accuracy_level 0, 5 ... 16 tokens, in ONE pass over the weights --------------------------------
//
// The three-pass form above keeps sixteen digit rows of the whole K in shared memory. Here a CTA
// takes ONE 2048-k slice of K (blockIdx.y) for all of its row tiles, so that all 3 x 8 NTOK digit rows
// of that slice fit (99 KB for sixteen tokens), and the digit rows are laid out digit-major: MMA
// column tile d * NTOK + j holds digit d of tokens 8 j ... 8 j + 7, which puts the three digits of a
// token in the same lane and register position. Every weight byte is read once (by the CTA of its
// slice) and feeds 3 NTOK MMAs. Per quantization block the three exact int32 dots are combined
//   block_size <= 64:  E = 16384 e0 + 128 e1 + e2 - zp * S   in int32 (|E| < 2^31; S = 16384 s0 + 128 s1 + s2
//                      comes ready from the digit kernel), one conversion and one FFMA with the scale;
//   block_size >= 128: e_d - zp * s_d per digit in int32, 16384 f0 + 128 f1 + f2 in fp32
//                      (the int32 combination could overflow), one FFMA with the scale.
// The per-token factor `undo` and the bias are applied by the kernel that adds the slices' partial
// products in slice order. Nodes without zero points use zp = 8 (unsigned codes as they are).
struct DigitsParams {
  NodeSet set;
  const unsigned char *act;   // [slices][slice_bytes]: digit rows of a slice, then its table of sums
  float *partial[kMaxGroupedNodes];   // per node [slices][tokens_pad][n]
  int m_total;
  int *status;
  int bpt;
  int slices;
  int rec_bytes;
  int rec_scale_bytes;
  int slot_bytes;
  int num_slots;
  int producers;
  int act_row_bytes;
  int table_offset;
  int slice_bytes;
  int groups_per_block;
};

template <int NTOK, int SPB, bool HAS_ZP>
__global__ void __launch_bounds__(kThreads, 1)
    nbits_digits_mma_kernel(const __grid_constant__ NodeMaps maps, const DigitsParams p) {
  constexpr int NT = 3 * NTOK;           // MMA column tiles: digit-major
  constexpr int kRows = 8 * NT;          // digit rows
  constexpr int kTableInts = SPB == 4 ? kRows : 8 * NTOK;   // per entry: sums per digit row, or combined per token
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char *smem_raw = smem_dyn + ((1024u - (ptx::SmemAddr(smem_dyn) & 1023u)) & 1023u);
  unsigned char *slots = smem_raw;
  unsigned char *act = smem_raw + static_cast<size_t>(p.num_slots) * p.slot_bytes;
  float4 *partial = reinterpret_cast<float4 *>(act + p.slice_bytes); // [2][kWarps][NTOK][32]
  std::uint64_t *full_bar = reinterpret_cast<std::uint64_t *>(partial + 2 * kWarps * NTOK * 32);
  std::uint64_t *empty_bar = full_bar + kMaxSlots;
  std::uint64_t *act_bar = empty_bar + kMaxSlots;
  int *tile_table = reinterpret_cast<int *>(act_bar + 1);   // [kMaxGroupTiles] + the tile count (grouped launches)

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int slice = blockIdx.y;
  // the kernel that adds the slices up may be scheduled as SMs free up; it waits for this grid
  ptx::GridDependencyLaunch();

  const int total_halves = p.set.halves_end[p.set.nodes - 1];
  const int h_begin = static_cast<int>(static_cast<std::int64_t>(blockIdx.x) * total_halves / gridDim.x);
  const int h_end = static_cast<int>(static_cast<std::int64_t>(blockIdx.x + 1) * total_halves / gridDim.x);

  if (warp >= kWarps) {
    // ------------------------------ producers ------------------------------
    const int producer = warp - kWarps;
    if (producer == 0 && lane == 0) {
      for (int s = 0; s < p.num_slots; ++s) {
        ptx::MbarInit(&full_bar[s], 1);
        ptx::MbarInit(&empty_bar[s], kWarps);
      }
      ptx::MbarInit(act_bar, 1);
      ptx::FenceMbarInit();
      if (p.set.nodes > 1) {
        tile_table[kMaxGroupTiles] = BuildTileTable(p.set, h_begin, h_end, tile_table);
      }
    }
    asm volatile("bar.sync 11, %0;" ::"n"(kProducers * 32) : "memory"); // barriers initialised
    asm volatile("bar.arrive 10, %0;" ::"n"(kThreads) : "memory");
    if (lane == 0) {
      const int n_tiles = p.set.nodes == 1 ? (h_end - h_begin + 1) >> 1 : tile_table[kMaxGroupTiles];
      for (int i = 0; i < p.set.nodes; ++i) {
        ptx::PrefetchTensorMap(&maps.b[i]);
      }
      bool ok = true;
      // the digit rows come from the kernel launched just before (programmatic dependent launch):
      // producer 0 asks for them first, the other producers start on the weight tiles at once
      if (producer == 0) {
        ptx::GridDependencyWait();
        ptx::MbarArriveExpectTx(act_bar, static_cast<std::uint32_t>(p.slice_bytes));
        ptx::BulkLoad(act, p.act + static_cast<std::int64_t>(slice) * p.slice_bytes,
                      static_cast<std::uint32_t>(p.slice_bytes), act_bar);
      }
      for (int task = producer; producer < p.producers && task < n_tiles && ok; task += p.producers) {
        const int slot = task % p.num_slots;
        const std::uint32_t round = static_cast<std::uint32_t>(task / p.num_slots);
        if (round != 0) {
          if (!ptx::MbarWait(&empty_bar[slot], (round & 1u) ^ 1u)) {
            ReportStatus(p.status, kDeviceTimeoutEmptyBarrier);
            ok = false;
            break;
          }
        }
        const TilePlace at = PlaceOfTile(p.set, tile_table, h_begin, h_end, task);
        const int h0 = at.h0;
        const int node_halves = HalfTilesOf(p.set, at.node);
        const unsigned char *meta_src = p.set.w[at.node].meta + static_cast<std::int64_t>(h0) * p.rec_bytes +
                                        static_cast<std::int64_t>(slice) * node_halves * p.rec_bytes;
        const std::uint32_t meta_bytes = (h0 + 1 < node_halves ? 2u : 1u) * static_cast<std::uint32_t>(p.rec_bytes);
        unsigned char *dst = slots + static_cast<size_t>(slot) * p.slot_bytes;
        ptx::MbarArriveExpectTx(&full_bar[slot], kTaskBytes + meta_bytes);
        TmaLoad3D(dst, &maps.b[at.node], 0, h0 * 8, slice * kSegments, &full_bar[slot]);
        ptx::BulkLoad(dst + kTaskBytes, meta_src, meta_bytes, &full_bar[slot]);
      }
      // stay until every copy this lane issued has been consumed (bounded), so none lands after exit
      const int first = n_tiles - p.num_slots < 0 ? 0 : n_tiles - p.num_slots;
      for (int i = first; i < n_tiles && ok; ++i) {
        if (producer < p.producers && (i % p.producers) == producer &&
            !ptx::MbarWait(&empty_bar[i % p.num_slots], static_cast<std::uint32_t>(i / p.num_slots) & 1u)) {
          break;
        }
      }
      if (producer == 0) {
        ptx::MbarWait(act_bar, 0);
      }
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  asm volatile("bar.sync 10, %0;" ::"n"(kThreads) : "memory"); // barriers initialised
  const int n_tiles = p.set.nodes == 1 ? (h_end - h_begin + 1) >> 1 : tile_table[kMaxGroupTiles];
  bool dead = false;
  if (!ptx::MbarWait(act_bar, 0)) {
    ReportStatus(p.status, kDeviceTimeoutFullBarrier);
    dead = true;
  }

  const int g = lane >> 2;
  const int t = lane & 3;
  const std::uint32_t nib = 0x0f0f0f0fu;
  int word_off[4];
#pragma unroll
  for (int st = 0; st < 4; ++st) {
    const int c = (warp & 1) * 4 + st;
    word_off[st] = (warp >> 1) * 2048 + g * 128 + ((c ^ g) << 4) + 4 * t;
  }
  constexpr int kEntriesPerGroup = 4 / SPB;
  const int scale_row_bytes = p.rec_scale_bytes / 8;
  const int meta_index = p.groups_per_block > 1 ? warp / p.groups_per_block : warp * kEntriesPerGroup;
  // sums of this warp's entries: tokens 2 t, 2 t + 1 of every column tile
  const int *table = reinterpret_cast<const int *>(act + p.table_offset) + warp * kEntriesPerGroup * kTableInts + 2 * t;
  // digit bytes: row g of every column tile, this warp's 128-k group, this lane's eight k per step
  const unsigned char *act_lane = act + g * p.act_row_bytes + warp * 128 + t * 32;

  int slot = 0;
  std::uint32_t round = 0;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const TilePlace at = PlaceOfTile(p.set, tile_table, h_begin, h_end, tile);
    const std::int64_t node_n = p.set.w[at.node].n;
    const std::int64_t row0 = static_cast<std::int64_t>(at.h0) * 8;
    const std::int64_t row_limit = row0 + at.halves * 8 < node_n ? row0 + at.halves * 8 : node_n;
    float acc[NTOK][4];
#pragma unroll
    for (int j = 0; j < NTOK; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[j][i] = 0.0f;
      }
    }
    if (!dead && !ptx::MbarWait(&full_bar[slot], round & 1u)) {
      ReportStatus(p.status, kDeviceTimeoutFullBarrier);
      dead = true;
    }
    if (!dead) {
      const unsigned char *sb = slots + static_cast<size_t>(slot) * p.slot_bytes;
      std::uint32_t w_lo[4], w_hi[4];
#pragma unroll
      for (int st = 0; st < 4; ++st) {
        w_lo[st] = *reinterpret_cast<const std::uint32_t *>(sb + word_off[st]);
        w_hi[st] = *reinterpret_cast<const std::uint32_t *>(sb + word_off[st] + 1024);
      }
      const unsigned char *meta0 = sb + kTaskBytes;
      const unsigned char *meta1 = meta0 + p.rec_bytes;
      const float *sc0 = reinterpret_cast<const float *>(meta0 + g * scale_row_bytes) + meta_index;
      const float *sc1 = reinterpret_cast<const float *>(meta1 + g * scale_row_bytes) + meta_index;
      float ws_lo[kEntriesPerGroup], ws_hi[kEntriesPerGroup];
      int zp_lo[kEntriesPerGroup], zp_hi[kEntriesPerGroup];
      if constexpr (SPB == 1) {
        const float4 a4 = *reinterpret_cast<const float4 *>(sc0);
        const float4 b4 = *reinterpret_cast<const float4 *>(sc1);
        ws_lo[0] = a4.x, ws_lo[1] = a4.y, ws_lo[2] = a4.z, ws_lo[3] = a4.w;
        ws_hi[0] = b4.x, ws_hi[1] = b4.y, ws_hi[2] = b4.z, ws_hi[3] = b4.w;
      } else if constexpr (SPB == 2) {
        const float2 a2 = *reinterpret_cast<const float2 *>(sc0);
        const float2 b2 = *reinterpret_cast<const float2 *>(sc1);
        ws_lo[0] = a2.x, ws_lo[1] = a2.y, ws_hi[0] = b2.x, ws_hi[1] = b2.y;
      } else {
        ws_lo[0] = sc0[0], ws_hi[0] = sc1[0];
      }
#pragma unroll
      for (int i = 0; i < kEntriesPerGroup; ++i) {
        zp_lo[i] = 8;
        zp_hi[i] = 8;
      }
      if constexpr (HAS_ZP) {
        const unsigned char *zr0 = meta0 + p.rec_scale_bytes + g * p.bpt + meta_index;
        const unsigned char *zr1 = meta1 + p.rec_scale_bytes + g * p.bpt + meta_index;
#pragma unroll
        for (int i = 0; i < kEntriesPerGroup; ++i) {
          zp_lo[i] = zr0[i];
          zp_hi[i] = zr1[i];
        }
      }
      // the weights are in registers: hand the slot back before the arithmetic
      __syncwarp();
      if (lane == 0) {
        ptx::MbarArrive(&empty_bar[slot]);
      }
      int d[NT][4];
#pragma unroll
      for (int st = 0; st < 4; ++st) {
        const std::uint32_t a0 = w_lo[st] & nib;
        const std::uint32_t a1 = w_hi[st] & nib;
        const std::uint32_t a2 = (w_lo[st] >> 4) & nib;
        const std::uint32_t a3 = (w_hi[st] >> 4) & nib;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint2 b = *reinterpret_cast<const uint2 *>(act_lane + nt * 8 * p.act_row_bytes + st * 8);
          if ((st % SPB) == 0) {
            MmaU8S8Zero(d[nt], a0, a1, a2, a3, b.x, b.y);
          } else {
            MmaU8S8(d[nt], a0, a1, a2, a3, b.x, b.y);
          }
        }
        if (((st + 1) % SPB) == 0) {
          const int idx = st / SPB;
          const int *sums = table + idx * kTableInts;
#pragma unroll
          for (int j = 0; j < NTOK; ++j) {
            float f[4];
            if constexpr (SPB == 4) {
              // per digit: take the zero point out in int32, combine the digits in fp32
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                f[i] = 0.0f;
              }
#pragma unroll
              for (int digit = 0; digit < 3; ++digit) {
                const int2 sd = *reinterpret_cast<const int2 *>(sums + (digit * NTOK + j) * 8);
                const int *e = d[digit * NTOK + j];
                const float weight = digit == 0 ? 16384.0f : (digit == 1 ? 128.0f : 1.0f);
                f[0] = fmaf(weight, static_cast<float>(e[0] - zp_lo[idx] * sd.x), f[0]);
                f[1] = fmaf(weight, static_cast<float>(e[1] - zp_lo[idx] * sd.y), f[1]);
                f[2] = fmaf(weight, static_cast<float>(e[2] - zp_hi[idx] * sd.x), f[2]);
                f[3] = fmaf(weight, static_cast<float>(e[3] - zp_hi[idx] * sd.y), f[3]);
              }
            } else {
              // block_size <= 64: everything in int32, S = 16384 s0 + 128 s1 + s2 from the table
              const int2 sd = *reinterpret_cast<const int2 *>(sums + j * 8);
              const int *e0 = d[j], *e1 = d[NTOK + j], *e2 = d[2 * NTOK + j];
              // (unsigned arithmetic: the parts may wrap, the result fits)
              auto combine = [](int x0, int x1, int x2, int zp, int s) {
                const unsigned v = static_cast<unsigned>(x0) * 16384u + static_cast<unsigned>(x1) * 128u +
                                   static_cast<unsigned>(x2) - static_cast<unsigned>(zp) * static_cast<unsigned>(s);
                return static_cast<float>(static_cast<int>(v));
              };
              f[0] = combine(e0[0], e1[0], e2[0], zp_lo[idx], sd.x);
              f[1] = combine(e0[1], e1[1], e2[1], zp_lo[idx], sd.y);
              f[2] = combine(e0[2], e1[2], e2[2], zp_hi[idx], sd.x);
              f[3] = combine(e0[3], e1[3], e2[3], zp_hi[idx], sd.y);
            }
            acc[j][0] = fmaf(ws_lo[idx], f[0], acc[j][0]);
            acc[j][1] = fmaf(ws_lo[idx], f[1], acc[j][1]);
            acc[j][2] = fmaf(ws_hi[idx], f[2], acc[j][2]);
            acc[j][3] = fmaf(ws_hi[idx], f[3], acc[j][3]);
          }
        }
      }
    }
    if (++slot == p.num_slots) {
      slot = 0;
      ++round;
    }

    // ---- sum over the sixteen warps (same scheme as the accuracy_level-4 kernel) ----------------
    const int b = tile & 1;
    const int reducer0 = (tile * NTOK) & (kWarps - 1);
    const bool reduces = ((warp - reducer0) & (kWarps - 1)) < NTOK;
    if (tile >= 2) {
      const int previous0 = ((tile - 2) * NTOK) & (kWarps - 1);
      const bool reduced_previous = ((warp - previous0) & (kWarps - 1)) < NTOK;
      if (!reduced_previous) {
        asm volatile("bar.sync %0, %1;" ::"r"(4 + b), "n"(kConsumerThreads) : "memory");
      }
    }
    float4 *mine = partial + ((b * kWarps + warp) * NTOK) * 32 + lane;
#pragma unroll
    for (int j = 0; j < NTOK; ++j) {
      mine[j * 32] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
    }
    if (!reduces) {
      asm volatile("bar.arrive %0, %1;" ::"r"(2 + b), "n"(kConsumerThreads) : "memory");
    } else {
      asm volatile("bar.sync %0, %1;" ::"r"(2 + b), "n"(kConsumerThreads) : "memory");
      const int j = (warp - reducer0) & (kWarps - 1);
      const float4 *column = partial + (b * kWarps * NTOK + j) * 32 + lane;
      float4 total = column[0];
#pragma unroll
      for (int w = 1; w < kWarps; ++w) {
        const float4 v = column[w * NTOK * 32];
        total.x += v.x, total.y += v.y, total.z += v.z, total.w += v.w;
      }
      if (tile + 2 < n_tiles) {
        asm volatile("bar.arrive %0, %1;" ::"r"(4 + b), "n"(kConsumerThreads) : "memory");
      }
      const std::int64_t r_lo = row0 + g;
      const std::int64_t r_hi = row0 + g + 8;
      const std::int64_t m0 = j * 8 + 2 * t;
      float *y0 = p.partial[at.node] + (static_cast<std::int64_t>(slice) * (8 * NTOK) + m0) * node_n;
      float *y1 = y0 + node_n;
      if (m0 < p.m_total) {
        if (r_lo < row_limit) {
          y0[r_lo] = total.x;
        }
        if (r_hi < row_limit) {
          y0[r_hi] = total.z;
        }
      }
      if (m0 + 1 < p.m_total) {
        if (r_lo < row_limit) {
          y1[r_lo] = total.y;
        }
        if (r_hi < row_limit) {
          y1[r_hi] = total.w;
        }
      }
    }
  }
}

// Digit rows of every K slice in the layout nbits_digits_mma_kernel reads: CTAs (token, slice,
// part of the slice's entries). A CTA first finds the row's largest magnitude (all of K: 16 KB per row, an L2 hit for
// all but the first CTA of a token), then converts its slice, one warp per table entry at a time.
// Slice layout: [24 NTOK rows][act_row_bytes] signed bytes, row (d NTOK + j) 8 + i = digit d of
// token 8 j + i, k in the MMA's order inside each 128-k group; then the table
// [entries of the slice][table_ints]: per digit row its sum (entries of 128 k), or per token the
// combined 16384 s0 + 128 s1 + s2 (entries of 32 / 64 k). factors[2 m + token] = the factor that
// takes the integer result back (NaN for a row with a non-finite entry), read by the kernel that adds
// the slices up.
__global__ void __launch_bounds__(256)
    nbits_digit_slices_kernel(const float *a, float *factors, int m_total, std::int64_t k, int entry_k,
                              int entries_per_slice, int ntok, int act_row_bytes, int table_offset,
                              int slice_bytes, int table_ints, unsigned char *act) {
  // the product kernel behind this one may start (barrier set-up, first weight tiles) right away
  ptx::GridDependencyLaunch();
  // launched with programmatic serialization itself: A and the scratch are touched once the kernel
  // before this one in the stream has completed
  ptx::GridDependencyWait();
  __shared__ float warp_max[8];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x;
  const int slice = blockIdx.y;
  const bool live = token < m_total;
  const float *src = a + static_cast<std::int64_t>(token) * k;
  float amax = 0.0f;
  bool bad = false;
  if (live) {
    for (std::int64_t i = threadIdx.x; i < k; i += 256) {
      const float v = src[i];
      amax = fmaxf(amax, fabsf(v));
      bad = bad || (v != v);
    }
  }
  if (bad) {
    amax = __int_as_float(0x7f800000);
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  }
  if (lane == 0) {
    warp_max[warp] = amax;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    amax = fmaxf(amax, warp_max[i]);
  }
  const bool finite = amax < 3.0e38f;
  const float lift = amax < 1.0e-18f ? 1.8446744e19f /* 2^64 */ : 1.0f;
  const float lifted = amax * lift;
  const float up = (live && finite && lifted > 0.0f) ? kDigitRange / lifted : 0.0f;
  if (live && slice == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
    factors[2 * m_total + token] = finite ? (lifted / kDigitRange) / lift : __int_as_float(0x7fc00000);
  }
  unsigned char *base = act + static_cast<std::int64_t>(slice) * slice_bytes;
  const int tile = token >> 3;
  const int within = token & 7;
  std::int8_t *rows[3];
#pragma unroll
  for (int digit = 0; digit < 3; ++digit) {
    rows[digit] = reinterpret_cast<std::int8_t *>(base) +
                  static_cast<std::int64_t>((digit * ntok + tile) * 8 + within) * act_row_bytes;
  }
  // gridDim.z CTAs share a slice's entries, so that even two slices of sixteen tokens fill the GPU
  const int entry_begin = static_cast<int>(blockIdx.z) * entries_per_slice / static_cast<int>(gridDim.z);
  const int entry_end = (static_cast<int>(blockIdx.z) + 1) * entries_per_slice / static_cast<int>(gridDim.z);
  for (int entry = entry_begin + warp; entry < entry_end; entry += 8) {
    int sum[3] = {0, 0, 0};
    for (int e = lane; e < entry_k; e += 32) {
      const int k_in_slice = entry * entry_k + e;
      const std::int64_t kk = static_cast<std::int64_t>(slice) * kTaskK + k_in_slice;
      int q[3] = {0, 0, 0};
      if (live && kk < k) {
        int n = __float2int_rn((src[kk] * lift) * up);
        const int range = static_cast<int>(kDigitRange);
        n = n > range ? range : (n < -range ? -range : n);
        q[2] = ((n + 64) & 127) - 64;
        const int n1 = (n - q[2]) >> 7;
        q[1] = ((n1 + 64) & 127) - 64;
        q[0] = (n1 - q[1]) >> 7;
      }
      const int at = ActBytePosition(k_in_slice);
#pragma unroll
      for (int digit = 0; digit < 3; ++digit) {
        sum[digit] += q[digit];
        rows[digit][at] = static_cast<std::int8_t>(q[digit]);
      }
    }
#pragma unroll
    for (int digit = 0; digit < 3; ++digit) {
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) {
        sum[digit] += __shfl_xor_sync(0xffffffffu, sum[digit], offset);
      }
    }
    if (lane == 0) {
      int *cell = reinterpret_cast<int *>(base + table_offset) + static_cast<std::int64_t>(entry) * table_ints;
      if (table_ints == 8 * ntok) {
        cell[token] = static_cast<int>(static_cast<unsigned>(sum[0]) * 16384u + static_cast<unsigned>(sum[1]) * 128u +
                                       static_cast<unsigned>(sum[2]));
      } else {
#pragma unroll
        for (int digit = 0; digit < 3; ++digit) {
          cell[(digit * ntok + tile) * 8 + within] = sum[digit];
        }
      }
    }
  }
}

// Y[token][n] = undo[token] * (P_0 + P_1 + ... in slice order)[token][n] + bias[n].
__global__ void __launch_bounds__(256)
    nbits_digit_slices_sum_kernel(const float *partial, int slices, int tokens_pad, const float *factors, int m_total,
                                  std::int64_t n, const float *bias, OutputView out) {
  const std::int64_t total = static_cast<std::int64_t>(m_total) * n;
  const std::int64_t slice_stride = static_cast<std::int64_t>(tokens_pad) * n;
  ptx::GridDependencyLaunch(); // what follows in the stream may be scheduled as SMs free up
  ptx::GridDependencyWait();   // the partial products come from the kernel before this one
  for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<std::int64_t>(gridDim.x) * 256) {
    const std::int64_t token = i / n;
    const std::int64_t col = i - token * n;
    float sum = partial[token * n + col];
    for (int s = 1; s < slices; ++s) {
      sum += partial[s * slice_stride + token * n + col];
    }
    const float undo = factors[2 * m_total + token];
    out.y[token * out.ld + out.col_offset + col] = fmaf(sum, undo, bias != nullptr ? bias[col] : 0.0f);
  }
}

struct DigitsGeometry {
  bool ok;
  int ntok;
  int spb;
  int entry_k;
  int entries_per_slice;
  int table_ints;
  int act_row_bytes;
  int table_offset;
  int slice_bytes;
  int slot_bytes;
  int num_slots;
  std::size_t smem;
  std::size_t act_bytes;      // all slices
  std::size_t partial_bytes;  // [slices][tokens_pad][n]
};

DigitsGeometry DigitsGeometryOf(const WeightView &w, std::int64_t m) {
  DigitsGeometry geo{};
  const MetaGeometry meta = MetaGeometryOf(w);
  if (meta.bytes == 0 || meta.bpt * w.block_size != kTaskK || (w.row_bytes % 128) != 0 || m < 1 || m > 16 ||
      (reinterpret_cast<std::uintptr_t>(w.b) & 15u) != 0) {
    return geo;
  }
  geo.ntok = m > 8 ? 2 : 1;
  geo.entry_k = w.block_size < 128 ? w.block_size : 128;
  geo.spb = geo.entry_k / 32;
  geo.entries_per_slice = kTaskK / geo.entry_k;
  geo.table_ints = geo.spb == 4 ? 24 * geo.ntok : 8 * geo.ntok;
  // 8 bytes of padding: the sixteen lanes of a half warp (four rows, four 32-byte positions) read
  // eight bytes each per step, and with rows 2056 bytes apart they fall on 32 different banks
  // (2064 made it a two-way conflict: 1.45 M conflicts in 4.12 M wavefronts)
  geo.act_row_bytes = kTaskK + 8;
  geo.table_offset = 24 * geo.ntok * geo.act_row_bytes;
  geo.slice_bytes = geo.table_offset + geo.entries_per_slice * geo.table_ints * 4;
  geo.slot_bytes = (kTaskBytes + 2 * meta.rec_bytes + 1023) & ~1023;
  const std::size_t limit = 225 * 1024;
  const std::size_t fixed = static_cast<std::size_t>(geo.slice_bytes) + 2 * kWarps * geo.ntok * 32 * sizeof(float4) +
                            (2 * kMaxSlots + 1) * sizeof(std::uint64_t) + 64 + 1024 +
                            (kMaxGroupTiles + 1) * sizeof(int);
  if ((geo.slice_bytes % 16) != 0 || fixed + 3 * static_cast<std::size_t>(geo.slot_bytes) > limit) {
    return geo;
  }
  int slots = static_cast<int>((limit - fixed) / geo.slot_bytes);
  geo.num_slots = slots > kMaxSlots ? kMaxSlots : slots;
  geo.smem = static_cast<std::size_t>(geo.num_slots) * geo.slot_bytes + fixed;
  geo.act_bytes = static_cast<std::size_t>(meta.slices) * geo.slice_bytes;
  geo.partial_bytes = static_cast<std::size_t>(meta.slices) * 8 * geo.ntok * static_cast<std::size_t>(w.n) * sizeof(float);
  geo.ok = true;
  return geo;
}

} // namespace

// Scratch of a group: the digit rows of all K slices, the row factors, every node's partial products.
std::size_t DigitSlicesGroupScratchBytes(const WeightView *nodes, int count, std::int64_t m) {
  if (count < 1 || count > kMaxGroupedNodes) {
    return 0;
  }
  const DigitsGeometry geo = DigitsGeometryOf(nodes[0], m);
  if (!geo.ok) {
    return 0;
  }
  std::size_t bytes = AlignUp(geo.act_bytes) + AlignUp(3 * m * sizeof(float));
  for (int i = 0; i < count; ++i) {
    const DigitsGeometry other = DigitsGeometryOf(nodes[i], m);
    if (!other.ok) {
      return 0;
    }
    bytes += other.partial_bytes;
  }
  return bytes;
}

std::size_t DigitSlicesScratchBytes(const WeightView &w, std::int64_t m) {
  return DigitSlicesGroupScratchBytes(&w, 1, m);
}

namespace {

// One product launch for all `count` nodes (their row tiles form one sequence over the CTAs of each
// slice), then per node the sum of its slices. partial: the nodes' [slices][tokens_pad][n] buffers one
// after the other.
const char *LaunchDigitSlicesNodes(const WeightView *nodes, const OutputView *outs, int count,
                                   const DigitsGeometry &geo, std::int64_t m, unsigned char *act, const float *factors,
                                   float *partial, int *status_word, cudaStream_t stream, int sm_count) {
  const WeightView &w = nodes[0];
  const MetaGeometry meta = MetaGeometryOf(w);
  DigitsParams p{};
  NodeMaps maps;
  std::int64_t tiles = 0;
  if (!FillNodeSet(nodes, count, &p.set, &maps, &tiles)) {
    return nullptr;
  }
  float *node_partial[kMaxGroupedNodes];
  float *next = partial;
  for (int i = 0; i < kMaxGroupedNodes; ++i) {
    node_partial[i] = i < count ? next : partial;
    p.partial[i] = node_partial[i];
    if (i < count) {
      next += static_cast<std::int64_t>(meta.slices) * 8 * geo.ntok * nodes[i].n;
    }
  }
  p.act = act;
  p.m_total = static_cast<int>(m);
  p.status = status_word;
  p.bpt = meta.bpt;
  p.slices = meta.slices;
  p.rec_bytes = meta.rec_bytes;
  p.rec_scale_bytes = meta.rec_scale_bytes;
  p.slot_bytes = geo.slot_bytes;
  p.num_slots = geo.num_slots;
  p.producers = geo.num_slots < kProducers ? geo.num_slots : kProducers;
  p.act_row_bytes = geo.act_row_bytes;
  p.table_offset = geo.table_offset;
  p.slice_bytes = geo.slice_bytes;
  p.groups_per_block = w.block_size >= 256 ? w.block_size / 128 : 1;
  int ctas = sm_count > 0 ? sm_count : 148;
  // slices run side by side: share the SMs between them so that one wave covers the launch
  ctas = ctas / meta.slices > 0 ? ctas / meta.slices : 1;
  if (ctas > tiles) {
    ctas = static_cast<int>(tiles);
  }
  if (count > 1 && (p.set.halves_end[count - 1] / ctas + 2) / 2 + count > kMaxGroupTiles) {
    return nullptr;
  }
  dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>(meta.slices), 1);
  cudaError_t err = cudaErrorInvalidValue;
#define MNB_DIGITS_CASE(NTOK_, SPB_, ZP_)                                                        \
  if (geo.ntok == NTOK_ && geo.spb == SPB_ && (w.zp != nullptr) == ZP_) {                        \
    auto kernel = nbits_digits_mma_kernel<NTOK_, SPB_, ZP_>;                                     \
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,              \
                               static_cast<int>(geo.smem));                                      \
    if (err == cudaSuccess) {                                                                    \
      cudaLaunchConfig_t config = {};                                                            \
      config.gridDim = grid;                                                                     \
      config.blockDim = dim3(kThreads, 1, 1);                                                    \
      config.dynamicSmemBytes = geo.smem;                                                        \
      config.stream = stream;                                                                    \
      cudaLaunchAttribute attribute[1];                                                          \
      attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                      \
      attribute[0].val.programmaticStreamSerializationAllowed = 1;                               \
      config.attrs = attribute;                                                                  \
      config.numAttrs = 1;                                                                       \
      err = cudaLaunchKernelEx(&config, kernel, maps, p);                                        \
    }                                                                                            \
  }
#define MNB_DIGITS_CASES(SPB_)                                                                   \
  MNB_DIGITS_CASE(1, SPB_, true)                                                                 \
  MNB_DIGITS_CASE(1, SPB_, false)                                                                \
  MNB_DIGITS_CASE(2, SPB_, true)                                                                 \
  MNB_DIGITS_CASE(2, SPB_, false)
  MNB_DIGITS_CASES(1)
  MNB_DIGITS_CASES(2)
  MNB_DIGITS_CASES(4)
#undef MNB_DIGITS_CASES
#undef MNB_DIGITS_CASE
  if (err != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  for (int i = 0; i < count; ++i) {
    const std::int64_t total = m * nodes[i].n;
    std::int64_t blocks = (total + 255) / 256;
    blocks = blocks > 148 * 4 ? 148 * 4 : blocks;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
    config.blockDim = dim3(256, 1, 1);
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    if (cudaLaunchKernelEx(&config, nbits_digit_slices_sum_kernel, static_cast<const float *>(node_partial[i]),
                           meta.slices, 8 * geo.ntok, factors, static_cast<int>(m), nodes[i].n, nodes[i].bias,
                           outs[i]) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    CountLaunch();
  }
  return "nbits_digits_mma_kernel";
}

} // namespace

// accuracy_level 0 for up to sixteen tokens in one pass over the weights: the digit rows of all K
// slices once (one kernel, shared by sibling nodes), then per node the sliced integer-MMA product and
// the sum of its slices. `scratch`: DigitSlicesGroupScratchBytes of the group.
const char *LaunchDigitSlicesGroup(const WeightView *nodes, const OutputView *outs, int count, const float *a,
                                   std::int64_t m, unsigned char *scratch, int *status_word, cudaStream_t stream,
                                   int sm_count) {
  if (count < 1 || count > kMaxGroupedNodes || scratch == nullptr) {
    return nullptr;
  }
  const WeightView &w = nodes[0];
  const DigitsGeometry geo = DigitsGeometryOf(w, m);
  if (!geo.ok) {
    return nullptr;
  }
  for (int i = 0; i < count; ++i) {
    const DigitsGeometry other = DigitsGeometryOf(nodes[i], m);
    if (!other.ok || nodes[i].meta == nullptr || nodes[i].k != w.k || nodes[i].block_size != w.block_size ||
        (nodes[i].zp != nullptr) != (w.zp != nullptr) || other.slice_bytes != geo.slice_bytes ||
        other.table_ints != geo.table_ints) {
      return nullptr;
    }
  }
  const MetaGeometry meta = MetaGeometryOf(w);
  unsigned char *act = scratch;
  float *factors = reinterpret_cast<float *>(scratch + AlignUp(geo.act_bytes));
  float *partial = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(factors) + AlignUp(3 * m * sizeof(float)));
  const unsigned parts = geo.entries_per_slice >= 32 ? 8u : 4u;
  if (!LaunchSerialized(nbits_digit_slices_kernel,
                        dim3(static_cast<unsigned>(8 * geo.ntok), static_cast<unsigned>(meta.slices), parts), dim3(256),
                        stream, a, factors, static_cast<int>(m), w.k, geo.entry_k, geo.entries_per_slice, geo.ntok,
                        geo.act_row_bytes, geo.table_offset, geo.slice_bytes, geo.table_ints, act)) {
    return nullptr;
  }
  CountLaunch();
  return LaunchDigitSlicesNodes(nodes, outs, count, geo, m, act, factors, partial, status_word, stream, sm_count);
}

namespace {

} // namespace

namespace {

struct DigitsScratch {
  unsigned char *act;
  float *factors;
  float *partial;
};

DigitsScratch DigitsScratchOf(const ImmaGeometry &geo, std::int64_t m, unsigned char *scratch) {
  DigitsScratch at{};
  at.act = scratch;
  at.factors = reinterpret_cast<float *>(scratch + AlignUp(static_cast<std::size_t>(geo.passes) * geo.pass_bytes));
  at.partial = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(at.factors) + AlignUp(3 * m * sizeof(float)));
  return at;
}

// Row factors and digit rows of `a` into the scratch area: the part that sibling nodes share.
bool LaunchDigitRows(const WeightView &w, const ImmaGeometry &geo, const float *a, std::int64_t m,
                     const DigitsScratch &at, cudaStream_t stream) {
  nbits_digit_row_factors_kernel<<<static_cast<unsigned>(m), 256, 0, stream>>>(a, static_cast<int>(m), w.k, at.factors);
  const std::int64_t items = static_cast<std::int64_t>(geo.passes) * geo.tp * geo.entries_pad;
  nbits_digits_imma_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, stream>>>(
      a, at.factors, static_cast<int>(m), w.k, geo.entry_k, geo.entries_pad, geo.tp, geo.act_row_bytes,
      geo.table_offset, geo.pass_bytes, geo.passes, w.zp != nullptr ? 1.0f : 0.0625f, at.act);
  if (cudaGetLastError() != cudaSuccess) {
    return false;
  }
  CountLaunch(2);
  return true;
}

// One node over digit rows that are already in the scratch area: three partial rows per token,
// then their sum plus the bias.
bool LaunchDigitsNode(const WeightView &w, const ImmaGeometry &geo, std::int64_t m, const DigitsScratch &at,
                      OutputView out, int *status_word, cudaStream_t stream, int sm_count) {
  WeightView no_bias = w;
  no_bias.bias = nullptr;
  OutputView to_partial{};
  to_partial.y = at.partial;
  to_partial.ld = w.n;
  to_partial.col_offset = 0;
  if (LaunchMultiply(no_bias, geo, 3 * m, at.act, to_partial, status_word, stream, sm_count) == nullptr) {
    return false;
  }
  const bool vector_ok = (w.n % 4) == 0 && (out.ld % 4) == 0 && (out.col_offset % 4) == 0 &&
                         (reinterpret_cast<std::uintptr_t>(out.y) & 15u) == 0 &&
                         (reinterpret_cast<std::uintptr_t>(w.bias) & 15u) == 0;
  if (vector_ok) {
    const std::int64_t n4 = w.n / 4;
    std::int64_t blocks_x = (n4 + 255) / 256;
    blocks_x = blocks_x > 148 ? 148 : blocks_x;
    nbits_digits_combine_vec_kernel<<<dim3(static_cast<unsigned>(blocks_x), static_cast<unsigned>(m)), 256, 0, stream>>>(
        reinterpret_cast<const float4 *>(at.partial), reinterpret_cast<const float4 *>(w.bias), n4, out);
  } else {
    const std::int64_t total = m * w.n;
    std::int64_t blocks = (total + 255) / 256;
    blocks = blocks > 148 * 8 ? 148 * 8 : blocks;
    nbits_digits_combine_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(at.partial, w.bias,
                                                                                static_cast<int>(m), w.n, out);
  }
  if (cudaGetLastError() != cudaSuccess) {
    return false;
  }
  CountLaunch();
  return true;
}

} // namespace

std::size_t DigitsInt8MmaScratchBytes(const WeightView &w, std::int64_t m) {
  const ImmaGeometry geo = ImmaGeometryOf(w, 3 * m);
  if (!geo.ok) {
    return 0;
  }
  return AlignUp(static_cast<std::size_t>(geo.passes) * geo.pass_bytes) + AlignUp(3 * m * sizeof(float)) +
         static_cast<std::size_t>(3 * m) * w.n * sizeof(float);
}

const char *LaunchDigitsInt8Mma(const WeightView &w, const float *a, std::int64_t m, unsigned char *scratch,
                                OutputView out, int *status_word, cudaStream_t stream, int sm_count) {
  return LaunchDigitsInt8MmaGroup(&w, &out, 1, a, m, scratch, status_word, stream, sm_count);
}

// Sibling nodes: the digit rows are made once; `scratch` holds DigitsInt8MmaScratchBytes of the
// node with the most columns.
const char *LaunchDigitsInt8MmaGroup(const WeightView *nodes, const OutputView *outs, int count, const float *a,
                                     std::int64_t m, unsigned char *scratch, int *status_word, cudaStream_t stream,
                                     int sm_count) {
  if (count < 1 || count > kMaxGroupedNodes || scratch == nullptr || m < 1 || m > 16) {
    return nullptr;
  }
  const WeightView &w = nodes[0];
  const ImmaGeometry geo = ImmaGeometryOf(w, 3 * m);
  if (!geo.ok) {
    return nullptr;
  }
  for (int i = 0; i < count; ++i) {
    if (nodes[i].meta == nullptr || !SameActivationLayout(w, geo, nodes[i], ImmaGeometryOf(nodes[i], 3 * m))) {
      return nullptr;
    }
  }
  const DigitsScratch at = DigitsScratchOf(geo, m, scratch);
  if (!LaunchDigitRows(w, geo, a, m, at, stream)) {
    return nullptr;
  }
  for (int i = 0; i < count; ++i) {
    if (!LaunchDigitsNode(nodes[i], ImmaGeometryOf(nodes[i], 3 * m), m, at, outs[i], status_word, stream, sm_count)) {
      return nullptr;
    }
  }
  return "nbits_int8_mma_kernel(digits)";
}

} // namespace mnb
