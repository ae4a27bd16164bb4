// Decode path of MatMulNBits for ONE activation row (accuracy_level 0, 4-bit weights, block_size
// 128) whose packed weights are asked for by a producer warp in a few large TMA copies.
//
// At M = 1 a node is a 30 MB stream that lasts a few microseconds, and what decides its time is
// how soon after the launch the memory system is saturated and whether it stays so. Measured on
// the way here (decoder projection N = 14336, K = 4096, launches back to back in a CUDA graph):
//  * a warp that keeps its own ring of loads in flight finds its activation loads queued behind
//    its own weight requests (the load pipe serves requests in order), and a ring that holds part
//    of a tile costs a memory round trip, about 2 us under load, each time it wraps;
//  * a response from L2 also queues behind whatever the SM asked for before: with the whole
//    share of an SM (200 KB) requested ahead of the 16 KB of activations the digits were ready
//    3.4 us after the previous kernel had finished, with the activations requested first 2.0 us;
//  * the TMA unit of an SM works on one copy at a time and a copy costs about 0.15 us whatever its
//    size: 36 copies per CTA (weights, scales and zero points of twelve tiles) took as long as
//    the whole stream at the HBM rate. Hence few, large copies.
//
// Structure. One CTA per SM owns a contiguous range of eight-row tiles. Consumer warp w works on
// one tile at a time; G consecutive warps form a group whose tiles are fetched together: one 3-D
// TMA box {128 B, 8 G rows, chunks of K} with the 128-byte swizzle for the packed weights, one 2-D
// box each for the scales and the prepared zero-point bytes of those rows (rows beyond N are
// filled with zeros by the TMA unit). A group has `slots_per_group` slots; with N = 14336 and K =
// 4096 every group of a CTA has a slot of its own except the thirteenth tile of sixteen CTAs. The
// consumer warps issue no weight loads: they wait for the previous kernel of the stream
// (programmatic dependent launch), ask for the activations, release the producer (which has asked
// for `early_groups` groups before), stage the activations as digit rows and work on their tiles
// as the groups land.
//
// With the MMA rows permuted (row g of the MMA is row (g & 1) * 4 + g / 2 of the tile) the 128-bit
// loads of a quarter warp fall on 32 different banks of the swizzled slot.
//
// MMA use ("row pair"): MMA rows 0..7 see the even 128-k segment of a chunk, rows 8..15 the odd
// one; columns 0..2 / 3..5 carry the three digits of the even / odd segment. Arithmetic and
// exactness: see nbits_digits.cuh. Every wait is bounded and reports through the status word.
//
// Conventions: packed-INT4 nibble order of
// onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:60-93; "stream B once, split N"
// partition of onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258.

#include "nbits_common.cuh"

#include <cstdint>
#include <memory>
#include <mutex>
#include <utility>
#include <vector>

#include "nbits_digits.cuh"
#include "nbits_ptx.cuh"
#include "nbits_tma.cuh"

namespace mnb {
namespace {

constexpr int kMaxConsumerWarps = 14;
constexpr int kMaxGroupSlots = 32;
constexpr int kProducerLanes = 4;         // lanes of the producer warp that issue copies
constexpr int kChunkRowsBytes = 8 * 128;  // one tile's share of a chunk in shared memory: 8 rows x 128 B

// One launch serves up to three nodes that take the same activations (the q / k / v or the gate /
// up projections of a decoder layer): their tile groups form one sequence, node after node, that
// goes round the CTAs, so the activations are staged once and no kernel boundary separates the
// nodes' weight streams.
struct ResidentNode {
  WeightView w;
  OutputView out;
  int tiles;            // eight-row tiles of the node
  int groups_end;       // tile groups of the launch below this number belong to this node or an earlier one
  int group_boxes;      // 1: a full group is fetched by one copy per operand (needs N % 8 == 0)
};

struct ResidentParams {
  ResidentNode node[kMaxGroupedNodes];
  int nodes;
  const float *a;
  int *status;
  int k;
  int steps_per_task;   // 128-byte chunks of a row per task = MMA steps of two segments each
  int parts;            // tasks per tile group (parts of K)
  int group_tiles;      // G: tiles (= consumer warps) whose weights one copy fetches
  int groups;           // consumer warp groups (G warps each)
  int slots_per_group;
  int early_groups;     // first-round group tasks the producer asks for before the consumers have asked for A
  int segs;             // 128-k segments per weight row
  int table_ints;
  GatherTail tail;      // gathered step (ranks > 0, single node): rows pushed to the peers, flags by the last CTA
};

__device__ __forceinline__ void TmaLoadBox3D(std::uint32_t smem_dst, const void *tensor_map, int x, int y, int z,
                                             std::uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_dst),
               "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(ptx::SmemAddr(bar))
               : "memory");
}

__device__ __forceinline__ void TmaLoadBox2D(std::uint32_t smem_dst, const void *tensor_map, int x, int y,
                                             std::uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_dst),
               "l"(tensor_map), "r"(x), "r"(y), "r"(ptx::SmemAddr(bar))
               : "memory");
}

template <int OFFSET>
__device__ __forceinline__ uint4 LoadSlot16(std::uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4 + %5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr), "n"(OFFSET));
  return v;
}

__device__ __forceinline__ uint4 LoadSlot16At(std::uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

__device__ __forceinline__ uint2 LoadSlot8At(std::uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

__device__ __forceinline__ void TmaLoadBox4D(std::uint32_t smem_dst, const void *tensor_map, int x, int y, int z,
                                             int w, std::uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(smem_dst),
               "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(ptx::SmemAddr(bar))
               : "memory");
}

// The six tensor maps of a node: packed weights, scales and prepared zero-point bytes, each for a
// whole group of tiles (one copy) and for a single tile (the last, short group of a node).
struct ResidentNodeMaps {
  CUtensorMap w_group;  // 4-D {32 words, 8 rows, chunks, tiles}, box {32, 8, steps, G}
  CUtensorMap w_tile;   // 3-D {32 words, rows, chunks}, box {32, 8, steps}
  CUtensorMap s_group;  // 2-D {blocks, rows}, box {2 steps, 8 G}
  CUtensorMap s_tile;   //                     box {2 steps, 8}
  CUtensorMap z_group;
  CUtensorMap z_tile;
};

struct ResidentMaps {
  ResidentNodeMaps node[kMaxGroupedNodes];
};

// A tile group of the launch: whose it is, its first tile there and how many tiles it has.
struct GroupPlace {
  int node;
  int tile0;
  int count;
};

__device__ __forceinline__ void LoadMatrixX4(std::uint32_t addr, std::uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// BPS: quantization blocks per 128-k segment: 1 (block_size 128) or 4 (block_size 32). With four,
// an MMA covers one 32-k block of a row's even segment (MMA rows 0-7) and of its odd segment (rows
// 8-15): ldmatrix hands lane t of a quad word t of each 16-byte unit (= block) of the row, the low
// nibbles of that word fill k slots 4t.. and the high nibbles slots 16 + 4t.., the staged digits are
// kept block by block in the same order, and every block's exact int32 sums leave through its own
// scale and zero point. Scales arrive as 128-byte-swizzled boxes of four steps (eight rows read by
// a quarter warp fall on different banks), zero-point bytes as plain rows.
template <bool HAS_ZP, int BPS>
__global__ void __launch_bounds__((kMaxConsumerWarps + 1) * 32, 1)
    nbits_decode_resident_kernel(const __grid_constant__ ResidentMaps maps, const ResidentParams p) {
  const int G = p.group_tiles;
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  // the weight slots need 1024-byte alignment (swizzle atom); align inside the shared window
  unsigned char *base = smem_dyn + ((1024u - (ptx::SmemAddr(smem_dyn) & 1023u)) & 1023u);
  const int groups = p.groups;
  const int consumers = groups * G;
  const int slots = groups * p.slots_per_group;
  const int steps = p.steps_per_task;
  const int weight_tile_bytes = steps * kChunkRowsBytes;      // [chunk][8 rows][128 B] per tile
  const int scale_tile_bytes = steps * 64 * BPS;              // [8 rows][2 segments per step][BPS] floats
  // zero points: [8 rows][2 segments per step] prepared bytes, or (blocks of 32) the operator's own
  // packed nibbles, [8 rows][8 blocks per step] = four bytes per row and step
  const int zero_tile_bytes = HAS_ZP ? (BPS == 1 ? steps * 16 : steps * 32) : 0;
  const int weight_slot_bytes = G * weight_tile_bytes;        // a slot holds the G tiles of a group, tile-major
  const int scale_slot_bytes = G * scale_tile_bytes;
  const int zero_slot_bytes = G * zero_tile_bytes;
  unsigned char *weight_slots = base;
  unsigned char *scale_slots = weight_slots + static_cast<size_t>(slots) * weight_slot_bytes;
  unsigned char *zero_slots = scale_slots + static_cast<size_t>(slots) * scale_slot_bytes;
  unsigned char *digits = zero_slots + static_cast<size_t>(slots) * zero_slot_bytes;
  int *table = reinterpret_cast<int *>(digits + static_cast<size_t>(p.segs) * (kDigits * kChunkBytes));
  float *undo = reinterpret_cast<float *>(table + p.table_ints);
  float *red = undo + kMaxTokens;
  std::uint64_t *full_bar = reinterpret_cast<std::uint64_t *>(red + kMaxTokens * kMaxWarps);
  std::uint64_t *empty_bar = full_bar + kMaxGroupSlots;

  // the next kernel of the stream may be scheduled onto this SM as soon as this CTA has left
  ptx::GridDependencyLaunch();

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int grid = static_cast<int>(gridDim.x);
  const int cta = static_cast<int>(blockIdx.x);
  // the launch's tile groups cta, cta + grid, ... are this CTA's; the last group of a node may be short
  const int total_groups = p.node[p.nodes - 1].groups_end;
  const int my_groups = cta < total_groups ? (total_groups - cta + grid - 1) / grid : 0;
  auto place_of = [&](int local_group) {
    const int id = cta + local_group * grid;
    GroupPlace at{0, 0, 0};
    int first = 0;
#pragma unroll
    for (int i = 0; i + 1 < kMaxGroupedNodes; ++i) {
      if (i + 1 < p.nodes && id >= p.node[i].groups_end) {
        at.node = i + 1;
        first = p.node[i].groups_end;
      }
    }
    at.tile0 = (id - first) * G;
    const int left = p.node[at.node].tiles - at.tile0;
    at.count = left < G ? left : G;
    return at;
  };
  // round r gives consumer group j the CTA's local tile group r * groups + j
  const int rounds = (my_groups + groups - 1) / groups;
  const int consumer_threads = consumers * 32;

  if (warp == consumers) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      for (int s = 0; s < slots; ++s) {
        ptx::MbarInit(&full_bar[s], 1);
        ptx::MbarInit(&empty_bar[s], static_cast<std::uint32_t>(G));  // released by every warp of the group
      }
      ptx::FenceMbarInit();
    }
    __syncwarp();
    // barriers initialised: the consumers may go on (they meet the producer at barrier 2 behind
    // their staging)
    asm volatile("bar.arrive 2, %0;" ::"r"(consumer_threads + 32) : "memory");
    const std::uint32_t tile_bytes =
        static_cast<std::uint32_t>(weight_tile_bytes + scale_tile_bytes + zero_tile_bytes);
    bool ok = true;
    // The q-th task of group j is part q % parts of its tiles of round q / parts; it goes to slot
    // q % slots_per_group of the group. A lane serves the groups lane, lane + kProducerLanes, ...
    auto issue_tasks = [&](int q, int j_begin, int j_end) -> bool {
      bool any = false;
      for (int j = j_begin + lane; j < j_end && ok; j += kProducerLanes) {
        const int local_group = (q / p.parts) * groups + j;
        if (local_group >= my_groups) {
          continue;
        }
        any = true;
        const GroupPlace at = place_of(local_group);
        const ResidentNodeMaps &node_maps = maps.node[at.node];
        const int part = q % p.parts;
        const int slot = j * p.slots_per_group + (q % p.slots_per_group);
        const int use = q / p.slots_per_group;  // how often this slot has been filled before
        if (use > 0 && !ptx::MbarWait(&empty_bar[slot], static_cast<std::uint32_t>(use - 1) & 1u)) {
          ReportStatus(p.status, kDeviceTimeoutEmptyBarrier);
          ok = false;
          break;
        }
        const int count = at.count;
        const int tile0 = at.tile0;
        const std::uint32_t w_at = ptx::SmemAddr(weight_slots) + slot * weight_slot_bytes;
        const std::uint32_t s_at = ptx::SmemAddr(scale_slots) + slot * scale_slot_bytes;
        const std::uint32_t z_at = ptx::SmemAddr(zero_slots) + slot * zero_slot_bytes;
        ptx::MbarArriveExpectTx(&full_bar[slot], static_cast<std::uint32_t>(count) * tile_bytes);
        if (count == G && p.node[at.node].group_boxes != 0) {
          // the whole group in one copy per operand
          TmaLoadBox4D(w_at, &node_maps.w_group, 0, 0, part * steps, tile0, &full_bar[slot]);
          if constexpr (BPS == 1) {
            TmaLoadBox2D(s_at, &node_maps.s_group, part * steps * 2, tile0 * 8, &full_bar[slot]);
          } else {
            TmaLoadBox4D(s_at, &node_maps.s_group, 0, 0, part * steps / 4, tile0, &full_bar[slot]);
          }
          if constexpr (HAS_ZP) {
            TmaLoadBox2D(z_at, &node_maps.z_group, BPS == 1 ? part * steps * 2 : part * steps * 4, tile0 * 8,
                         &full_bar[slot]);
          }
        } else {
          // a short group (the end of this CTA's range): tile by tile, same places in the slot
          for (int i = 0; i < count; ++i) {
            const int row0 = (tile0 + i) * 8;
            TmaLoadBox3D(w_at + i * weight_tile_bytes, &node_maps.w_tile, 0, row0, part * steps, &full_bar[slot]);
            if constexpr (BPS == 1) {
              TmaLoadBox2D(s_at + i * scale_tile_bytes, &node_maps.s_tile, part * steps * 2, row0, &full_bar[slot]);
            } else {
              TmaLoadBox3D(s_at + i * scale_tile_bytes, &node_maps.s_tile, 0, row0, part * steps / 4, &full_bar[slot]);
            }
            if constexpr (HAS_ZP) {
              TmaLoadBox2D(z_at + i * zero_tile_bytes, &node_maps.z_tile,
                           BPS == 1 ? part * steps * 2 : part * steps * 4, row0, &full_bar[slot]);
            }
          }
        }
      }
      return any;
    };
    const int early = p.early_groups < groups ? p.early_groups : groups;
    if (lane < kProducerLanes) {
      for (int i = 0; i < p.nodes; ++i) {
        ptx::PrefetchTensorMap(&maps.node[i].w_group);
        ptx::PrefetchTensorMap(&maps.node[i].s_group);
        ptx::PrefetchTensorMap(&maps.node[i].w_tile);
        ptx::PrefetchTensorMap(&maps.node[i].s_tile);
        if constexpr (HAS_ZP) {
          ptx::PrefetchTensorMap(&maps.node[i].z_group);
          ptx::PrefetchTensorMap(&maps.node[i].z_tile);
        }
      }
      issue_tasks(0, 0, early);
    }
    // The bulk of the copies starts once the consumers have ASKED for the activations (barrier 3):
    // a response from L2 queues behind whatever the SM asked for earlier.
    asm volatile("bar.sync 3, %0;" ::"r"(consumer_threads + 32) : "memory");
    if (lane < kProducerLanes) {
      issue_tasks(0, early, groups);
      const int total = rounds * p.parts;
      for (int q = 1; q < total && ok; ++q) {
        issue_tasks(q, 0, groups);
      }
      // Stay until every copy this lane asked for has been consumed (bounded), so that none lands
      // after the CTA has left: the last use of each of this lane's slots.
      for (int j = lane; j < groups && ok; j += kProducerLanes) {
        // tasks of group j: rounds in which it has at least one tile, times parts
        int my_rounds = 0;
        for (int r = 0; r < rounds; ++r) {
          if (r * groups + j < my_groups) {
            ++my_rounds;
          }
        }
        const int tasks = my_rounds * p.parts;
        for (int d = 0; d < p.slots_per_group && ok; ++d) {
          const int uses = tasks > d ? (tasks - d + p.slots_per_group - 1) / p.slots_per_group : 0;
          if (uses > 0 &&
              !ptx::MbarWait(&empty_bar[j * p.slots_per_group + d], static_cast<std::uint32_t>(uses - 1) & 1u)) {
            ok = false;
          }
        }
      }
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  // A (and Y) may be produced / still read by the previous kernel in the stream: from here on the
  // consumers depend on it. The producer above only touches the constant weights.
  ptx::GridDependencyWait();
  const DigitGeometry geometry{p.k, p.segs, kDigits * kChunkBytes, p.table_ints};
  StageDigits<true, BPS == 4>(
      geometry, p.a, 1, 1, digits, table, undo, red, tid, consumer_threads,
      [&] { asm volatile("bar.sync 1, %0;" ::"r"(consumer_threads) : "memory"); },
      [&] { asm volatile("bar.arrive 3, %0;" ::"r"(consumer_threads + 32) : "memory"); });
  // barriers initialised (the producer has arrived long ago)
  asm volatile("bar.sync 2, %0;" ::"r"(consumer_threads + 32) : "memory");

  const int g = lane >> 2;
  const int t = lane & 3;
  const int group = warp / G;
  const int member = warp - group * G;  // which tile of the group's box this warp works on
  // Gathered step: the arithmetic stores locally only; once all consumer warps of the CTA are done,
  // the rows of its tile groups go to the same place of every peer's buffer and the CTA counts
  // itself in; the last CTA of the grid publishes this rank's flags.
  auto finish_gathered_step = [&](bool rows_already_pushed) {
    if (p.tail.ranks <= 0) {
      return;
    }
    if (rows_already_pushed) {
      PublishWhenGridDone(p.tail, tid, consumer_threads, 4, gridDim.x, p.status);
      return;
    }
    asm volatile("bar.sync 4, %0;" ::"r"(consumer_threads) : "memory");
    // (single node) the CTA's tile groups are cta, cta + grid, ...: G * 8 consecutive rows each; all of
    // them in one pass over the consumer threads, consecutive lanes on consecutive rows
    const ResidentNode &node = p.node[0];
    const int rows_per_group = G * 8;
    const float *local = node.out.y + node.out.col_offset;
    for (int item = tid; item < my_groups * rows_per_group && p.tail.n_peers > 0; item += consumer_threads) {
      const int local_group = item / rows_per_group;
      const std::int64_t row = static_cast<std::int64_t>(cta + local_group * grid) * rows_per_group +
                               (item - local_group * rows_per_group);
      if (row < node.w.n) {
        const float v = __ldcg(local + row);
        for (int r = 0; r < p.tail.n_peers; ++r) {
          p.tail.peers[r][node.out.col_offset + row] = v;
        }
      }
    }
    PublishWhenGridDone(p.tail, tid, consumer_threads, 4, gridDim.x, p.status);
  };
  if constexpr (BPS == 4) {
    // ---- blocks of 32: one MMA per block, MMA row g = row g of the tile ----
    const int matrix = lane >> 3;  // ldmatrix: this lane names row (lane & 7) of matrix (lane >> 3) = unit of the segment
    const int mrow = lane & 7;
    const std::uint32_t lo_lane = member * weight_tile_bytes + mrow * 128 + ((matrix ^ mrow) << 4);
    const std::uint32_t hi_lane = member * weight_tile_bytes + mrow * 128 + (((4 + matrix) ^ mrow) << 4);
    const int column = g < 6 ? g : g - 4;  // MMA columns 6 and 7 are not used: they read columns 2 and 3 again
    const std::uint32_t digits_lane = LaunderAfterBarrier(ptx::SmemAddr(digits) + column * 32 + t * 8);
    const std::uint32_t table_lane = LaunderAfterBarrier(ptx::SmemAddr(table) + t * 8);
    const std::uint32_t weights_group = ptx::SmemAddr(weight_slots) + group * p.slots_per_group * weight_slot_bytes;
    const std::uint32_t scales_row = ptx::SmemAddr(scale_slots) + group * p.slots_per_group * scale_slot_bytes +
                                     member * scale_tile_bytes + g * 128;
    const std::uint32_t zeros_row = ptx::SmemAddr(zero_slots) + group * p.slots_per_group * zero_slot_bytes +
                                    member * zero_tile_bytes + g * (steps * 4);
    const int supers = steps / kStepsPerSuper;
    const ZeroQuad zero = MakeZeroQuad();
    int q = 0;  // this group's task counter
    for (int round = 0; round < rounds; ++round) {
      const int local_group = round * groups + group;
      if (local_group >= my_groups) {
        break;
      }
      const GroupPlace at = place_of(local_group);
      const bool has_tile = member < at.count;
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      bool dead = false;
      for (int part = 0; part < p.parts; ++part, ++q) {
        const int d = q % p.slots_per_group;
        const int slot = group * p.slots_per_group + d;
        if (!dead && !ptx::MbarWait(&full_bar[slot], static_cast<std::uint32_t>(q / p.slots_per_group) & 1u)) {
          ReportStatus(p.status, kDeviceTimeoutFullBarrier);
          dead = true;
        }
        if (dead) {
          continue;
        }
        if (has_tile) {
          std::uint32_t lo_at = weights_group + d * weight_slot_bytes + lo_lane;
          std::uint32_t hi_at = weights_group + d * weight_slot_bytes + hi_lane;
          std::uint32_t scales_at = scales_row + d * scale_slot_bytes;
          std::uint32_t zeros_at = zeros_row + d * zero_slot_bytes;
          std::uint32_t digits_at = digits_lane + part * steps * (4 * kBlock32Bytes);
          std::uint32_t table_at = table_lane + part * steps * (4 * 32);
#pragma unroll 1
          for (int super = 0; super < supers; ++super) {
            uint4 z_super = make_uint4(0u, 0u, 0u, 0u);
            if constexpr (HAS_ZP) {
              z_super = LoadSlot16At(zeros_at);  // one word per step: the nibbles of its eight blocks, in k order
            }
            auto do_step = [&](auto step_tag) {
              constexpr int i = decltype(step_tag)::value;
              std::uint32_t lo[4], hi[4];
              LoadMatrixX4(lo_at + i * kChunkRowsBytes, lo);
              LoadMatrixX4(hi_at + i * kChunkRowsBytes, hi);
              // scales of the four blocks of the even segment and of the odd one (16-byte units 2i and
              // 2i + 1 of the row's 128 bytes, swizzled with the row)
              const uint4 u_lo = LoadSlot16At(scales_at + (((2 * i) ^ g) << 4));
              const uint4 u_hi = LoadSlot16At(scales_at + (((2 * i + 1) ^ g) << 4));
              const std::uint32_t s_lo_bits[4] = {u_lo.x, u_lo.y, u_lo.z, u_lo.w};
              const std::uint32_t s_hi_bits[4] = {u_hi.x, u_hi.y, u_hi.z, u_hi.w};
              const std::uint32_t z_word = i == 0 ? z_super.x : (i == 1 ? z_super.y : (i == 2 ? z_super.z : z_super.w));
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const std::uint32_t a0 = lo[u] & 0x0f0f0f0fu;
                const std::uint32_t a1 = hi[u] & 0x0f0f0f0fu;
                const std::uint32_t a2 = (lo[u] >> 4) & 0x0f0f0f0fu;
                const std::uint32_t a3 = (hi[u] >> 4) & 0x0f0f0f0fu;
                const uint2 b = LoadSlot8At(digits_at + (i * 4 + u) * kBlock32Bytes);
                const uint2 sums_bits = LoadSlot8At(table_at + (i * 4 + u) * 32);
                const int sums_x = static_cast<int>(sums_bits.x);
                const int sums_y = static_cast<int>(sums_bits.y);
                int dot[4];
                ImmaFresh(dot, a0, a1, a2, a3, b.x, b.y, zero);
                int z_lo = 8, z_hi = 8;
                if constexpr (HAS_ZP) {
                  z_lo = static_cast<int>((z_word >> (4 * u)) & 0xfu);
                  z_hi = static_cast<int>((z_word >> (16 + 4 * u)) & 0xfu);
                }
                // block sum - zp * digit sum: exact (the table holds -sum); times 16 with the scale,
                // because the row's factor takes a sixteenth out again
                const float s_lo = __uint_as_float(s_lo_bits[u]) * 16.0f;
                const float s_hi = __uint_as_float(s_hi_bits[u]) * 16.0f;
                acc[0] = fmaf(s_lo, static_cast<float>(z_lo * sums_x + dot[0]), acc[0]);
                acc[1] = fmaf(s_lo, static_cast<float>(z_lo * sums_y + dot[1]), acc[1]);
                acc[2] = fmaf(s_hi, static_cast<float>(z_hi * sums_x + dot[2]), acc[2]);
                acc[3] = fmaf(s_hi, static_cast<float>(z_hi * sums_y + dot[3]), acc[3]);
              }
            };
            ForEachIndex<kStepsPerSuper>(do_step);
            lo_at += kStepsPerSuper * kChunkRowsBytes;
            hi_at += kStepsPerSuper * kChunkRowsBytes;
            scales_at += 1024;
            zeros_at += kStepsPerSuper * 4;
            digits_at += kStepsPerSuper * 4 * kBlock32Bytes;
            table_at += kStepsPerSuper * 4 * 32;
          }
        }
        __syncwarp();
        if (lane == 0) {
          ptx::MbarArrive(&empty_bar[slot]);
        }
      }
      if (!has_tile) {
        continue;
      }
      float v = t == 0   ? fmaf(16384.0f, acc[0], 128.0f * acc[1])
                : t == 1 ? fmaf(16384.0f, acc[3], acc[0])
                : t == 2 ? fmaf(128.0f, acc[2], acc[3])
                         : 0.0f;
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      const ResidentNode &node = p.node[at.node];
      const std::int64_t row = static_cast<std::int64_t>(at.tile0 + member) * 8 + g;
      float result = 0.0f;
      if (!dead && t == 0 && row < node.w.n) {
        const float bias = node.w.bias != nullptr ? __ldg(node.w.bias + row) : 0.0f;
        result = fmaf(v, undo[0], bias);
        StoreOutput(node.out, node.out.col_offset + row, result);
      }
      if (p.tail.ranks > 0 && p.tail.n_peers > 0) {
        // gathered step: the tile's eight outputs go to the peers right away, from one lane, as two
        // 16-byte stores per peer where the place allows it (the copies are long done when the CTA
        // counts itself in at the end)
        float out8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          out8[j] = __shfl_sync(0xffffffffu, result, 4 * j);
        }
        const std::int64_t row0 = static_cast<std::int64_t>(at.tile0 + member) * 8;
        const std::int64_t at0 = node.out.col_offset + row0;
        if (lane == 0 && !dead) {
          const bool whole = row0 + 8 <= node.w.n;
          for (int r = 0; r < p.tail.n_peers; ++r) {
            float *dst = p.tail.peers[r] + at0;
            if (whole && (reinterpret_cast<std::uintptr_t>(dst) & 15u) == 0) {
              reinterpret_cast<float4 *>(dst)[0] = make_float4(out8[0], out8[1], out8[2], out8[3]);
              reinterpret_cast<float4 *>(dst)[1] = make_float4(out8[4], out8[5], out8[6], out8[7]);
            } else {
              for (int j = 0; j < 8 && row0 + j < node.w.n; ++j) {
                dst[j] = out8[j];
              }
            }
          }
        }
      }
    }
    finish_gathered_step(true);
    return;
  }
  // MMA row g is row `rho` of the tile: the two rows a quarter warp reads together then differ in
  // bit 2, and the 128-byte swizzle (16-byte unit ^ row) puts them on different halves of the banks
  const int rho = ((g & 1) << 2) | (g >> 1);
  const std::uint32_t lo_offset = member * weight_tile_bytes + rho * 128 + ((t ^ rho) << 4);        // units 0..3
  const std::uint32_t hi_offset = member * weight_tile_bytes + rho * 128 + (((4 + t) ^ rho) << 4);  // units 4..7
  const int column = g < 6 ? g : g - 6;
  const int second = column >= kDigits ? 1 : 0;
  const int digit_of_column = column - second * kDigits;
  const int swizzle = (second + digit_of_column) & 1;
  const std::uint32_t digits_column =
      LaunderAfterBarrier(ptx::SmemAddr(digits) + (second * kDigits + digit_of_column) * kChunkBytes);
  const std::uint32_t digits_even = digits_column + (((2 * t) ^ swizzle) << 4);
  const std::uint32_t digits_odd = digits_column + (((2 * t + 1) ^ swizzle) << 4);
  const std::uint32_t table_lane = LaunderAfterBarrier(ptx::SmemAddr(table) + t * 8);
  const std::uint32_t weights_group = ptx::SmemAddr(weight_slots) + group * p.slots_per_group * weight_slot_bytes;
  const std::uint32_t scales_group = ptx::SmemAddr(scale_slots) + group * p.slots_per_group * scale_slot_bytes +
                                     (member * 8 + rho) * (steps * 8);
  const std::uint32_t zeros_group =
      ptx::SmemAddr(zero_slots) + group * p.slots_per_group * zero_slot_bytes + (member * 8 + rho) * (steps * 2);
  const int supers = steps / kStepsPerSuper;
  const ZeroQuad zero = MakeZeroQuad();
  const int sixteen = static_cast<int>(LaunderAfterBarrier(16u));  // a register: keeps 16 * even + odd one instruction

  int q = 0;  // this group's task counter
  for (int round = 0; round < rounds; ++round) {
    const int local_group = round * groups + group;
    if (local_group >= my_groups) {
      break;  // the whole group is done (all its warps see the same)
    }
    const GroupPlace at = place_of(local_group);
    const bool has_tile = member < at.count;  // the last group of a node may be short of tiles
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    bool dead = false;
    for (int part = 0; part < p.parts; ++part, ++q) {
      const int d = q % p.slots_per_group;
      const int slot = group * p.slots_per_group + d;
      if (!dead && !ptx::MbarWait(&full_bar[slot], static_cast<std::uint32_t>(q / p.slots_per_group) & 1u)) {
        ReportStatus(p.status, kDeviceTimeoutFullBarrier);
        dead = true;
      }
      if (dead) {
        continue;
      }
      if (has_tile) {
        std::uint32_t lo_at = weights_group + d * weight_slot_bytes + lo_offset;
        std::uint32_t hi_at = weights_group + d * weight_slot_bytes + hi_offset;
        std::uint32_t scales_at = scales_group + d * scale_slot_bytes;
        std::uint32_t zeros_at = zeros_group + d * zero_slot_bytes;
        const int step0 = part * steps;
        std::uint32_t even_at = digits_even + step0 * kTileColumnBytes;
        std::uint32_t odd_at = digits_odd + step0 * kTileColumnBytes;
        std::uint32_t table_at = table_lane + step0 * 32;
#pragma unroll 1
        for (int super = 0; super < supers; ++super) {
          // scales and zero points of the eight segments of this superstep, row rho of the tile
          const uint4 u0 = LoadSlot16At(scales_at);
          const uint4 u1 = LoadSlot16At(scales_at + 16);
          const float4 s_first =
              make_float4(__uint_as_float(u0.x), __uint_as_float(u0.y), __uint_as_float(u0.z), __uint_as_float(u0.w));
          const float4 s_second =
              make_float4(__uint_as_float(u1.x), __uint_as_float(u1.y), __uint_as_float(u1.z), __uint_as_float(u1.w));
          uint2 z = make_uint2(0u, 0u);
          if constexpr (HAS_ZP) {
            z = LoadSlot8At(zeros_at);
          }
          auto do_step = [&](auto step_tag) {
            constexpr int i = decltype(step_tag)::value;
            const float s_lo = Component(i < 2 ? s_first : s_second, (2 * i) & 3);
            const float s_hi = Component(i < 2 ? s_first : s_second, (2 * i + 1) & 3);
            int z_lo = 128, z_hi = 128;  // 16 x the default zero point 8
            if constexpr (HAS_ZP) {
              z_lo = static_cast<int>(__byte_perm(i < 2 ? z.x : z.y, 0u, 0x4440u + ((2 * i) & 3)));
              z_hi = static_cast<int>(__byte_perm(i < 2 ? z.x : z.y, 0u, 0x4440u + ((2 * i + 1) & 3)));
            }
            const uint4 be = LoadSharedConst16<i * kTileColumnBytes>(even_at);
            const uint4 bo = LoadSharedConst16<i * kTileColumnBytes>(odd_at);
            const int2 sums = LoadSharedConst8<i * 32>(table_at);
            const uint4 lo = LoadSlot16<i * kChunkRowsBytes>(lo_at);
            const uint4 hi = LoadSlot16<i * kChunkRowsBytes>(hi_at);
            const std::uint32_t wl[4] = {lo.x, lo.y, lo.z, lo.w};
            const std::uint32_t wh[4] = {hi.x, hi.y, hi.z, hi.w};
            std::uint32_t el[4], ol[4], eh[4], oh[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              el[x] = wl[x] & 0x0f0f0f0fu;
              ol[x] = wl[x] & 0xf0f0f0f0u;
              eh[x] = wh[x] & 0x0f0f0f0fu;
              oh[x] = wh[x] & 0xf0f0f0f0u;
            }
            int de[4], dd[4];
            ImmaFresh(de, el[0], eh[0], el[1], eh[1], be.x, be.y, zero);
            ImmaFresh(dd, ol[0], oh[0], ol[1], oh[1], bo.x, bo.y, zero);
            ImmaAdd(de, el[2], eh[2], el[3], eh[3], be.z, be.w);
            ImmaAdd(dd, ol[2], oh[2], ol[3], oh[3], bo.z, bo.w);
            // 16 * (even + odd block sum - zp * digit sum): exact, below 2^24 (the table holds -sum)
            const int c0 = z_lo * sums.x + (de[0] * sixteen + dd[0]);
            const int c1 = z_lo * sums.y + (de[1] * sixteen + dd[1]);
            const int c2 = z_hi * sums.x + (de[2] * sixteen + dd[2]);
            const int c3 = z_hi * sums.y + (de[3] * sixteen + dd[3]);
            acc[0] = fmaf(s_lo, static_cast<float>(c0), acc[0]);
            acc[1] = fmaf(s_lo, static_cast<float>(c1), acc[1]);
            acc[2] = fmaf(s_hi, static_cast<float>(c2), acc[2]);
            acc[3] = fmaf(s_hi, static_cast<float>(c3), acc[3]);
          };
          ForEachIndex<kStepsPerSuper>(do_step);
          lo_at += kStepsPerSuper * kChunkRowsBytes;
          hi_at += kStepsPerSuper * kChunkRowsBytes;
          scales_at += kStepsPerSuper * 8;
          zeros_at += kStepsPerSuper * 2;
          even_at += kStepsPerSuper * kTileColumnBytes;
          odd_at += kStepsPerSuper * kTileColumnBytes;
          table_at += kStepsPerSuper * 32;
        }
      }
      // the slot may be refilled once every warp of the group has said so
      __syncwarp();
      if (lane == 0) {
        ptx::MbarArrive(&empty_bar[slot]);
      }
    }
    if (!has_tile) {
      continue;
    }
    // ---- the tile is complete: rows g see columns 0..2 (even segments), rows g + 8 columns 3..5 ----
    float v = t == 0   ? fmaf(16384.0f, acc[0], 128.0f * acc[1])
              : t == 1 ? fmaf(16384.0f, acc[3], acc[0])
              : t == 2 ? fmaf(128.0f, acc[2], acc[3])
                       : 0.0f;
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    const ResidentNode &node = p.node[at.node];
    const std::int64_t row = static_cast<std::int64_t>(at.tile0 + member) * 8 + rho;
    if (!dead && t == 0 && row < node.w.n) {
      const float bias = node.w.bias != nullptr ? __ldg(node.w.bias + row) : 0.0f;
      StoreOutput(node.out, node.out.col_offset + row, fmaf(v, undo[0], bias));
    }
  }
  finish_gathered_step(false);
}

bool EncodeWeightTileMap(CUtensorMap *map, const WeightView &w, int steps) {
  EncodeTiledFn encode = GetEncodeTiled();
  if (encode == nullptr) {
    return false;
  }
  // a packed row seen as [chunks][32 words]; dimension order: word, row, chunk
  const cuuint64_t dims[3] = {32, static_cast<cuuint64_t>(w.n), static_cast<cuuint64_t>(w.row_bytes / 128)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(w.row_bytes), 128};
  const cuuint32_t box[3] = {32, 8, static_cast<cuuint32_t>(steps)};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<std::uint8_t *>(w.b), dims, strides, box,
                elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same bytes seen as [tiles][chunks][8 rows][32 words] (N a multiple of 8): a box of several
// tiles lands tile by tile, each laid out like a single-tile box.
bool EncodeWeightGroupMap(CUtensorMap *map, const WeightView &w, int steps, int tiles_per_box) {
  EncodeTiledFn encode = GetEncodeTiled();
  if (encode == nullptr || (w.n % 8) != 0) {
    return false;
  }
  const cuuint64_t dims[4] = {32, 8, static_cast<cuuint64_t>(w.row_bytes / 128), static_cast<cuuint64_t>(w.n / 8)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(w.row_bytes), 128, static_cast<cuuint64_t>(w.row_bytes) * 8};
  const cuuint32_t box[4] = {32, 8, static_cast<cuuint32_t>(steps), static_cast<cuuint32_t>(tiles_per_box)};
  const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, const_cast<std::uint8_t *>(w.b), dims, strides, box,
                elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Scales of a node with blocks of 32: a row's scales seen as [chunks of 32][32 floats] (= four MMA
// steps), fetched like the weights in 128-byte-swizzled boxes of eight rows.
bool EncodeScaleTileMap32(CUtensorMap *map, const WeightView &w, int steps) {
  EncodeTiledFn encode = GetEncodeTiled();
  if (encode == nullptr) {
    return false;
  }
  const cuuint64_t dims[3] = {32, static_cast<cuuint64_t>(w.n), static_cast<cuuint64_t>(w.n_blocks / 32)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(w.n_blocks) * 4, 128};
  const cuuint32_t box[3] = {32, 8, static_cast<cuuint32_t>(steps / 4)};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(w.scales), dims, strides, box,
                elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool EncodeScaleGroupMap32(CUtensorMap *map, const WeightView &w, int steps, int tiles_per_box) {
  EncodeTiledFn encode = GetEncodeTiled();
  if (encode == nullptr || (w.n % 8) != 0) {
    return false;
  }
  const cuuint64_t row = static_cast<cuuint64_t>(w.n_blocks) * 4;
  const cuuint64_t dims[4] = {32, 8, static_cast<cuuint64_t>(w.n_blocks / 32), static_cast<cuuint64_t>(w.n / 8)};
  const cuuint64_t strides[3] = {row, 128, row * 8};
  const cuuint32_t box[4] = {32, 8, static_cast<cuuint32_t>(steps / 4), static_cast<cuuint32_t>(tiles_per_box)};
  const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(w.scales), dims, strides, box,
                elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

} // namespace

// One token, 4-bit, block_size 128 or 32, whole 128-byte chunks per row in multiples of four (K a
// multiple of 1024; of 2048 with zero points and block_size 128, whose prepared bytes must exist).
bool DecodeResidentSupports(const WeightView &w, std::int64_t m) {
  if (m == 1 && w.bits == 4 && w.block_size == 32) {
    // zero points come straight from the operator's packed nibbles: K / 64 bytes per row
    return (w.k % 1024) == 0 && w.n_blocks * 32 == w.k &&
           (w.zp == nullptr || (w.zp_row_bytes * 2 == w.n_blocks && (reinterpret_cast<std::uintptr_t>(w.zp) & 15u) == 0)) &&
           (reinterpret_cast<std::uintptr_t>(w.b) & 15u) == 0 && (reinterpret_cast<std::uintptr_t>(w.scales) & 15u) == 0 &&
           w.n < (std::int64_t{1} << 31);
  }
  return m == 1 && w.bits == 4 && w.block_size == 128 && (w.n_blocks % (2 * kStepsPerSuper)) == 0 &&
         (w.zp == nullptr || (w.zp16 != nullptr && (w.n_blocks % 16) == 0)) &&
         (reinterpret_cast<std::uintptr_t>(w.b) & 15u) == 0 &&
         (reinterpret_cast<std::uintptr_t>(w.scales) & 15u) == 0 && (reinterpret_cast<std::uintptr_t>(w.zp16) & 15u) == 0 &&
         w.n < (std::int64_t{1} << 31);
}

bool DecodeResidentPreferred(const WeightView &w) {
  // at least four eight-row tiles per CTA of a 148-SM part: with fewer, most of its warps have no tile
  // and a tile is a long chain of steps on one warp; rows of up to 2048 k are short enough for that
  // not to matter (block 32: N = 4096 3.7 against 6.3 us on the fp16 kernel, N = 1024 5.1 against
  // 5.7; block 128: N = 4096 3.4-3.6 against 3.9 us on the direct kernel, N = 1024 4.7 against 3.0)
  const int chunks = w.row_bytes / 128;
  return chunks <= 16 && (w.n >= 4736 || (chunks <= 8 && (w.block_size == 32 || w.n >= 4096)));
}

bool DecodeResidentGroupPreferred(const WeightView *nodes, int count) {
  return count >= 1 && nodes[0].row_bytes / 128 <= 16;
}

namespace {

// Everything of a launch that depends on the nodes only: slot shape, tensor maps, grid. Built once
// per node group (six cuTensorMapEncodeTiled calls per node and a cudaFuncSetAttribute cost several
// microseconds, as much as the kernel's share of a host-buffer call) and kept until the weights go.
struct ResidentPlan {
  ResidentMaps maps;
  ResidentParams params;  // a, the outputs and status are filled per launch
  size_t smem = 0;
  int ctas = 0;
  int threads = 0;
};

struct PlanKey {
  const void *b[kMaxGroupedNodes];
  const void *scales[kMaxGroupedNodes];
  const void *zp16[kMaxGroupedNodes];
  std::int64_t n[kMaxGroupedNodes];
  std::int64_t k;
  int nodes;
  int sms;
  bool operator==(const PlanKey &o) const {
    if (nodes != o.nodes || k != o.k || sms != o.sms) {
      return false;
    }
    for (int i = 0; i < nodes; ++i) {
      if (b[i] != o.b[i] || scales[i] != o.scales[i] || zp16[i] != o.zp16[i] || n[i] != o.n[i]) {
        return false;
      }
    }
    return true;
  }
};

std::mutex g_plan_mutex;
std::vector<std::pair<PlanKey, std::unique_ptr<ResidentPlan>>> g_plans;

bool BuildPlan(const WeightView *nodes, int count, int sms, ResidentPlan *plan) {
  ResidentParams &p = plan->params;
  p = ResidentParams{};
  const WeightView &w = nodes[0];  // K, block size and the presence of zero points are the group's
  p.nodes = count;
  p.k = static_cast<int>(w.k);
  const int bps = 128 / w.block_size;  // quantization blocks per 128-k segment: 1 or 4
  p.segs = static_cast<int>((w.k + 127) / 128);  // the last one may be part padding (block_size 128 only)
  p.table_ints = (p.segs / 2) * 8 * bps;
  std::int64_t tiles = 0;
  for (int i = 0; i < count; ++i) {
    p.node[i].w = nodes[i];
    p.node[i].tiles = static_cast<int>((nodes[i].n + 7) / 8);
    tiles += p.node[i].tiles;
  }
  // one CTA per SM: two CTAs of half the slots each (so that the next launch's CTAs could move in
  // as this launch's leave) measured 11.7 against 8.3 us per node: twice the staging, half the warps
  const int ctas = sms < tiles ? sms : static_cast<int>(tiles);
  const int tiles_per_cta = static_cast<int>((tiles + ctas - 1) / ctas);
  const int chunks = w.row_bytes / 128;  // MMA steps of a whole row
  const size_t fixed = static_cast<size_t>(p.segs) * kDigits * kChunkBytes + static_cast<size_t>(p.table_ints) * 4 +
                       (kMaxTokens + kMaxTokens * kMaxWarps) * sizeof(float) +
                       2 * kMaxGroupSlots * sizeof(std::uint64_t) + 1024;  // + alignment slack
  const size_t limit = 227 * 1024;
  // per tile and chunk: weights, scales, zero points (prepared bytes, or packed nibbles with blocks of 32)
  const size_t per_step = kChunkRowsBytes + 64 * bps + (w.zp != nullptr ? (bps == 1 ? 16 : 32) : 0);
  const int min_steps = (w.zp != nullptr && bps == 1) ? 8 : 4;  // the zero-point box needs 16 bytes per row
  auto fits = [&](int warps, int slots, int s) {
    return fixed + static_cast<size_t>(warps) * slots * s * per_step <= limit;
  };
  auto most_warps = [&](int slots, int s, int multiple) {
    int c = tiles_per_cta < kMaxConsumerWarps ? tiles_per_cta : kMaxConsumerWarps;
    c = (c + multiple - 1) / multiple * multiple;
    if (c > kMaxConsumerWarps) {
      c -= multiple;
    }
    while (c > 0 && !fits(c, slots, s)) {
      c -= multiple;
    }
    return c;
  };
  // First choice: a whole row of K per task, tiles fetched in groups of two, one slot per group;
  // a CTA with more tile groups than slots refills a slot as soon as its group has released it
  // (with twelve warps at work about half of the slots are in flight at any time, which covers the
  // memory latency). Rows too long for that: tasks of at most sixteen chunks, single tiles, two
  // slots each.
  // Measured on the decoder projection (N = 14336, K = 4096, us per launch in a CUDA graph, one
  // box): groups of 2 / 4 / 1 tiles 8.47 / 8.48 / 8.95 with the groups going round the CTAs, 9.5 /
  // 9.6 / 9.1 with a contiguous range of tiles per CTA; 2 groups asked for before the activations
  // 8.47, 1: 8.71, 3: 9.07, none: 9.5. Two such nodes in one launch (25 tiles per CTA): 6.77 per
  // node with this shape, 7.55 with the two-slot shape.
  int group_tiles = 2;
  int steps = chunks;
  int slots_per_group = 1;
  int warps = chunks <= 256 ? most_warps(1, steps, group_tiles) : 0;
  // Long rows leave room for few whole-row slots (K = 14336: two warps, 24.9 against 11.9 us on the
  // direct kernel): then tasks of part of a row, single tiles, two slots per warp, with the longest
  // task that still lets ten warps (or one per tile of the CTA) work.
  const int enough = tiles_per_cta < 8 ? tiles_per_cta : 8;
  if (warps < enough || warps < group_tiles) {
    int best_steps = 0;
    int best_warps = 0;
    const int wanted = tiles_per_cta < 10 ? tiles_per_cta : 10;
    for (int s = 16; s >= min_steps; s -= kStepsPerSuper) {
      if ((chunks % s) != 0) {
        continue;
      }
      const int w2 = most_warps(2, s, 1);
      if (w2 > best_warps) {
        best_warps = w2;
        best_steps = s;
      }
      if (w2 >= wanted) {
        break;
      }
    }
    if (best_warps > warps || warps < group_tiles) {
      if (best_steps == 0 || best_warps < 1) {
        return false;
      }
      group_tiles = 1;
      slots_per_group = 2;
      steps = best_steps;
      warps = best_warps;
    }
  }
  if ((chunks % steps) != 0 || (steps % kStepsPerSuper) != 0 || steps > 256) {
    return false;
  }
  p.steps_per_task = steps;
  p.parts = chunks / steps;
  p.group_tiles = group_tiles;
  p.groups = warps / group_tiles;
  p.slots_per_group = slots_per_group;
  if (p.groups * slots_per_group > kMaxGroupSlots) {
    return false;
  }
  p.early_groups = 2;
  plan->smem = fixed + static_cast<size_t>(warps) * slots_per_group * steps * per_step;
  plan->ctas = ctas;
  plan->threads = (warps + 1) * 32;

  int groups_end = 0;
  for (int i = 0; i < count; ++i) {
    const WeightView &node = nodes[i];
    ResidentNodeMaps &maps = plan->maps.node[i];
    groups_end += (p.node[i].tiles + group_tiles - 1) / group_tiles;
    p.node[i].groups_end = groups_end;
    if (!EncodeWeightTileMap(&maps.w_tile, node, steps)) {
      return false;
    }
    p.node[i].group_boxes =
        (group_tiles > 1 && EncodeWeightGroupMap(&maps.w_group, node, steps, group_tiles)) ? 1 : 0;
    if (p.node[i].group_boxes == 0) {
      maps.w_group = maps.w_tile;
    }
    auto rows_map = [&](CUtensorMap *map, bool zero_points, int rows) {
      if (zero_points && bps == 4) {
        return EncodeMap2D(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, node.zp, static_cast<std::uint64_t>(node.zp_row_bytes),
                           static_cast<std::uint64_t>(node.n), static_cast<std::uint64_t>(node.zp_row_bytes),
                           static_cast<std::uint32_t>(4 * steps), static_cast<std::uint32_t>(rows),
                           CU_TENSOR_MAP_SWIZZLE_NONE);
      }
      return zero_points
                 ? EncodeMap2D(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, node.zp16,
                               static_cast<std::uint64_t>(node.n_blocks), static_cast<std::uint64_t>(node.n),
                               static_cast<std::uint64_t>(node.n_blocks), static_cast<std::uint32_t>(2 * steps),
                               static_cast<std::uint32_t>(rows), CU_TENSOR_MAP_SWIZZLE_NONE)
                 : EncodeMap2D(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, node.scales,
                               static_cast<std::uint64_t>(node.n_blocks), static_cast<std::uint64_t>(node.n),
                               static_cast<std::uint64_t>(node.n_blocks) * 4, static_cast<std::uint32_t>(2 * steps),
                               static_cast<std::uint32_t>(rows), CU_TENSOR_MAP_SWIZZLE_NONE);
    };
    if (bps == 4) {
      if (!EncodeScaleTileMap32(&maps.s_tile, node, steps)) {
        return false;
      }
      if (p.node[i].group_boxes == 0 || !EncodeScaleGroupMap32(&maps.s_group, node, steps, group_tiles)) {
        p.node[i].group_boxes = 0;
        maps.w_group = maps.w_tile;
        maps.s_group = maps.s_tile;
      }
    } else if (!rows_map(&maps.s_tile, false, 8) || !rows_map(&maps.s_group, false, 8 * group_tiles)) {
      return false;
    }
    maps.z_tile = maps.s_tile;
    maps.z_group = maps.s_group;
    if (node.zp != nullptr && (!rows_map(&maps.z_tile, true, 8) || !rows_map(&maps.z_group, true, 8 * group_tiles))) {
      return false;
    }
  }
  for (int i = count; i < kMaxGroupedNodes; ++i) {
    plan->maps.node[i] = plan->maps.node[0];
    p.node[i] = p.node[0];
    p.node[i].groups_end = groups_end;
  }
  // The function attribute belongs to the kernel, not to the node: it is raised to the most any
  // plan can ask for, so that plans of different sizes do not undo one another.
  const int most = static_cast<int>(limit);
  cudaError_t err = cudaErrorInvalidValue;
  if (bps == 4) {
    err = w.zp != nullptr
              ? cudaFuncSetAttribute(nbits_decode_resident_kernel<true, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, most)
              : cudaFuncSetAttribute(nbits_decode_resident_kernel<false, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
  } else {
    err = w.zp != nullptr
              ? cudaFuncSetAttribute(nbits_decode_resident_kernel<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, most)
              : cudaFuncSetAttribute(nbits_decode_resident_kernel<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
  }
  return err == cudaSuccess;
}

// The plan of a node group, built on first use. nullptr when the shape has none.
const ResidentPlan *PlanFor(const WeightView *nodes, int count, int sms) {
  PlanKey key{};
  key.nodes = count;
  key.k = nodes[0].k;
  key.sms = sms;
  for (int i = 0; i < count; ++i) {
    key.b[i] = nodes[i].b;
    key.scales[i] = nodes[i].scales;
    key.zp16[i] = nodes[i].zp != nullptr ? nodes[i].zp16 : nullptr;
    key.n[i] = nodes[i].n;
  }
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  for (const auto &entry : g_plans) {
    if (entry.first == key) {
      return entry.second.get();
    }
  }
  auto plan = std::make_unique<ResidentPlan>();
  if (!BuildPlan(nodes, count, sms, plan.get())) {
    cudaGetLastError();
    return nullptr;
  }
  g_plans.emplace_back(key, std::move(plan));
  return g_plans.back().second.get();
}

} // namespace

// Called when a node's weights are destroyed: the plans it takes part in name their addresses.
void ForgetDecodeResidentPlans(const WeightView &w) {
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  for (size_t i = 0; i < g_plans.size();) {
    bool names = false;
    for (int x = 0; x < g_plans[i].first.nodes; ++x) {
      names = names || g_plans[i].first.b[x] == w.b;
    }
    if (names) {
      g_plans.erase(g_plans.begin() + static_cast<std::ptrdiff_t>(i));
    } else {
      ++i;
    }
  }
}

bool DecodeResidentGroupSupports(const WeightView *nodes, int count, std::int64_t m) {
  if (count < 1 || count > kMaxGroupedNodes) {
    return false;
  }
  for (int i = 0; i < count; ++i) {
    if (!DecodeResidentSupports(nodes[i], m) || nodes[i].k != nodes[0].k || nodes[i].block_size != nodes[0].block_size ||
        (nodes[i].zp != nullptr) != (nodes[0].zp != nullptr)) {
      return false;
    }
  }
  return true;
}

const char *LaunchDecodeResidentGroup(const WeightView *nodes, const OutputView *outs, int count, const float *a,
                                      std::int64_t m, int *status_word, cudaStream_t stream, int sm_count,
                                      const GatherTail *tail) {
  if (!DecodeResidentGroupSupports(nodes, count, m) || (tail != nullptr && count != 1)) {
    return nullptr;
  }
  const ResidentPlan *plan = PlanFor(nodes, count, sm_count > 0 ? sm_count : 148);
  if (plan == nullptr) {
    return nullptr;
  }
  ResidentParams p = plan->params;
  for (int i = 0; i < kMaxGroupedNodes; ++i) {
    const int from = i < count ? i : 0;
    p.node[i].w = nodes[from];  // bias may differ between calls; the addresses in the maps do not
    p.node[i].out = outs[from];
  }
  p.a = a;
  p.status = status_word;
  p.tail = tail != nullptr ? *tail : GatherTail{};
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(plan->ctas), 1, 1);
  config.blockDim = dim3(static_cast<unsigned>(plan->threads), 1, 1);
  config.dynamicSmemBytes = plan->smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  cudaError_t err = cudaErrorInvalidValue;
  if (nodes[0].block_size == 32) {
    err = nodes[0].zp != nullptr ? cudaLaunchKernelEx(&config, nbits_decode_resident_kernel<true, 4>, plan->maps, p)
                                 : cudaLaunchKernelEx(&config, nbits_decode_resident_kernel<false, 4>, plan->maps, p);
  } else {
    err = nodes[0].zp != nullptr ? cudaLaunchKernelEx(&config, nbits_decode_resident_kernel<true, 1>, plan->maps, p)
                                 : cudaLaunchKernelEx(&config, nbits_decode_resident_kernel<false, 1>, plan->maps, p);
  }
  if (err != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  CountLaunch();
  return "nbits_decode_resident_kernel";
}

const char *LaunchDecodeResident(const WeightView &w, const float *a, std::int64_t m, OutputView out, int *status_word,
                                 cudaStream_t stream, int sm_count, const GatherTail *tail) {
  return LaunchDecodeResidentGroup(&w, &out, 1, a, m, status_word, stream, sm_count, tail);
}

} // namespace mnb
