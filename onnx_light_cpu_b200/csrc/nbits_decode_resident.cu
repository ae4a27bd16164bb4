// Decode path of MatMulNBits for ONE activation row (accuracy_level 0, 4-bit weights, block_size
// 128) whose packed weights are all asked for at kernel start.
//
// At M = 1 a node is a 30 MB stream that lasts a few microseconds, and what decides its time is
// how soon after the launch the memory system is saturated and whether it stays so. A warp that
// keeps its own ring of loads in flight has two problems at that scale: its activation loads
// queue behind its own weight requests (the load pipe serves requests in order), and a ring
// that holds part of a tile costs a memory round trip (about 2 us under load) every time it
// wraps. Here the copies are made by the TMA engine on behalf of one producer warp, into
// shared-memory slots that are only written once in the common case: a CTA (one per SM) owns
// `slots` = consumer warps x slots-per-warp task slots, and for a node of the size of a decoder
// projection (N = 14336, K = 4096: twelve or thirteen eight-row tiles of 16 KB per SM) every task
// of the CTA has a slot of its own, so the producer asks for the whole share of the SM before any
// consumer has looked at the activations. The consumer warps issue no weight loads at all: they
// wait for the previous kernel of the stream (programmatic dependent launch), stage the
// activations as digit rows, and work on tasks as they land.
//
// A task is eight weight rows x `steps_per_task` 128-byte chunks of K, fetched as one 3-D TMA box
// {128 B, 8 rows, chunks} with the 128-byte swizzle, plus the scales and the prepared zero-point
// bytes of those rows and blocks as 2-D boxes (rows beyond N are filled with zeros by the TMA
// unit). With the MMA rows permuted (row g of the MMA is row (g & 1) * 4 + g / 2 of the tile) the
// 128-bit loads of a quarter warp fall on 32 different banks.
//
// MMA use ("row pair"): MMA rows 0..7 see the even 128-k segment of a chunk, rows 8..15 the odd
// one; columns 0..2 / 3..5 carry the three digits of the even / odd segment. Arithmetic and
// exactness: see nbits_digits.cuh. Every wait is bounded and reports through the status word.
//
// Conventions: packed-INT4 nibble order of
// onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:60-93; "stream B once, split N"
// partition of onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258.

#include "nbits_common.cuh"
#include "nbits_digits.cuh"
#include "nbits_ptx.cuh"
#include "nbits_tma.cuh"

#include <cstdint>
#include <cstdlib>

#ifdef MNB_TIMELINE
__device__ unsigned long long g_resident_timeline[512 * 16 * 8];
__device__ __forceinline__ unsigned long long GlobalTimerR() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define MNB_MARKR(slot)                                                                            \
  if ((threadIdx.x & 31) == 0) {                                                                   \
    g_resident_timeline[(blockIdx.x * 16 + (threadIdx.x >> 5)) * 8 + (slot)] = GlobalTimerR();     \
  }
extern "C" int mnb_debug_copy_resident_timeline(unsigned long long *out, int count) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_resident_timeline, sizeof(unsigned long long) * count));
}
#else
#define MNB_MARKR(slot)
#endif

namespace mnb {
namespace {

constexpr int kMaxConsumerWarps = 14;
constexpr int kMaxSlots = 4 * kMaxConsumerWarps;
constexpr int kProducerLanes = 4;  // lanes of the producer warp that issue copies (one warp each, round robin)
constexpr int kChunkRowsBytes = 8 * 128;  // one chunk of a task in shared memory: 8 rows x 128 B

struct ResidentParams {
  WeightView w;
  const float *a;
  OutputView out;
  int *status;
  int tiles;           // eight-row tiles of the node
  int steps_per_task;  // 128-byte chunks of a row per task = MMA steps of two segments each
  int parts;           // tasks per tile
  int slots_per_warp;
  int consumer_warps;
  int early_tasks;     // first-round tasks the producer asks for before the consumers have asked for A
  int segs;            // 128-k segments per weight row
  int table_ints;
};

__device__ __forceinline__ void TmaLoadBox3D(std::uint32_t smem_dst, const void *tensor_map, int x, int y, int z,
                                             std::uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_dst),
               "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(ptx::SmemAddr(bar))
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

__device__ __forceinline__ void CopyAsyncMeta16(std::uint32_t smem_addr, const void *gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr));
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

template <bool HAS_ZP>
__global__ void __launch_bounds__((kMaxConsumerWarps + 1) * 32, 1)
    nbits_decode_resident_kernel(const __grid_constant__ CUtensorMap map_w, const ResidentParams p) {
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  // the weight slots need 1024-byte alignment (swizzle atom); align inside the shared window
  unsigned char *base = smem_dyn + ((1024u - (ptx::SmemAddr(smem_dyn) & 1023u)) & 1023u);
  const int consumers = p.consumer_warps;
  const int slots = consumers * p.slots_per_warp;
  const int steps = p.steps_per_task;
  const int weight_slot_bytes = steps * kChunkRowsBytes;
  // scales and zero points of a warp's current tile (all of K), fetched by the warp itself:
  // eight rows of n_blocks floats, 16 bytes of padding per row (the two rows a quarter warp reads
  // then sit on different banks), then eight rows of n_blocks prepared zero-point bytes
  const int scale_row_bytes = p.segs * 4 + 16;
  const int meta_warp_bytes = 8 * scale_row_bytes + (HAS_ZP ? 8 * p.segs : 0);
  unsigned char *weight_slots = base;
  unsigned char *meta = weight_slots + static_cast<size_t>(slots) * weight_slot_bytes;
  unsigned char *digits = meta + static_cast<size_t>(consumers) * meta_warp_bytes;
  int *table = reinterpret_cast<int *>(digits + static_cast<size_t>(p.segs) * (kDigits * kChunkBytes));
  float *undo = reinterpret_cast<float *>(table + p.table_ints);
  float *red = undo + kMaxTokens;
  std::uint64_t *full_bar = reinterpret_cast<std::uint64_t *>(red + kMaxTokens * kMaxWarps);
  std::uint64_t *empty_bar = full_bar + kMaxSlots;

  // the next kernel of the stream may be scheduled onto this SM as soon as this CTA has left
  ptx::GridDependencyLaunch();
  MNB_MARKR(0)

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int grid = static_cast<int>(gridDim.x);
  const int cta = static_cast<int>(blockIdx.x);
  // this CTA's tiles: cta, cta + grid, ...; its consumer warp w takes the local tiles w, w + consumers, ...
  const int local_tiles = cta < p.tiles ? (p.tiles - cta + grid - 1) / grid : 0;
  const int consumer_threads = consumers * 32;

  if (warp == consumers) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      for (int s = 0; s < slots; ++s) {
        ptx::MbarInit(&full_bar[s], 1);
        ptx::MbarInit(&empty_bar[s], 1);
      }
      ptx::FenceMbarInit();
    }
    __syncwarp();
    // barriers initialised: the consumers may go on (they arrive at barrier 2 without waiting
    // for anything else), the producer lanes start copying at once
    asm volatile("bar.arrive 2, %0;" ::"r"(consumer_threads + 32) : "memory");
    const std::uint32_t task_bytes = static_cast<std::uint32_t>(weight_slot_bytes);
    bool ok = true;
    // Rounds of tasks: in round q every consumer warp gets its q-th task. A lane serves the warps
    // lane, lane + kProducerLanes, ... Returns false when no warp had a q-th task.
    auto issue_round = [&](int q, int w_begin, int w_end) -> bool {
      bool any = false;
      for (int w = w_begin + lane; w < w_end && ok; w += kProducerLanes) {
        const int local_tile = w + (q / p.parts) * consumers;
        if (local_tile >= local_tiles) {
          continue;
        }
        any = true;
        const int part = q % p.parts;
        const int slot = w * p.slots_per_warp + (q % p.slots_per_warp);
        const int use = q / p.slots_per_warp;  // how often this slot has been filled before
        if (use > 0 && !ptx::MbarWait(&empty_bar[slot], static_cast<std::uint32_t>(use - 1) & 1u)) {
          ReportStatus(p.status, kDeviceTimeoutEmptyBarrier);
          ok = false;
          break;
        }
        const int row0 = (cta + local_tile * grid) * 8;
        ptx::MbarArriveExpectTx(&full_bar[slot], task_bytes);
        TmaLoadBox3D(ptx::SmemAddr(weight_slots) + slot * weight_slot_bytes, &map_w, 0, row0, part * steps,
                     &full_bar[slot]);
      }
      return any;
    };
    int q = 0;
    (void)q;
    if (lane < kProducerLanes) {
      ptx::PrefetchTensorMap(&map_w);
      issue_round(0, 0, p.early_tasks < consumers ? p.early_tasks : consumers);
    }
    // The bulk of the copies starts once the consumers have ASKED for the activations (barrier 3):
    // a response from L2 queues behind whatever the SM asked for earlier, and 200 KB of weights in
    // front of the 16 KB of activations delayed the digits by more than three microseconds.
    asm volatile("bar.sync 3, %0;" ::"r"(consumer_threads + 32) : "memory");
    if (lane < kProducerLanes) {
      if (p.early_tasks < consumers) {
        issue_round(0, p.early_tasks, consumers);
      }
      for (q = 1; ok; ++q) {
        if (!issue_round(q, 0, consumers)) {
          break;
        }
      }
      MNB_MARKR(1)
      // Stay until every copy this lane asked for has been consumed (bounded), so that none lands
      // after the CTA has left: the last use of each of this lane's slots.
      for (int w = lane; w < consumers && ok; w += kProducerLanes) {
        const int my_tiles = w < local_tiles ? (local_tiles - w + consumers - 1) / consumers : 0;
        const int tasks = my_tiles * p.parts;
        for (int d = 0; d < p.slots_per_warp && ok; ++d) {
          // tasks of this warp that went through slot d: q = d, d + D, ...
          const int uses = tasks > d ? (tasks - d + p.slots_per_warp - 1) / p.slots_per_warp : 0;
          if (uses > 0 && !ptx::MbarWait(&empty_bar[w * p.slots_per_warp + d], static_cast<std::uint32_t>(uses - 1) & 1u)) {
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
  MNB_MARKR(1)
  ptx::GridDependencyWait();
  MNB_MARKR(2)
  const std::uint32_t meta_warp = ptx::SmemAddr(meta) + warp * meta_warp_bytes;
  // Asks for the scales and zero points of all of K of one of this warp's tiles (16-byte pieces,
  // one asynchronous-copy group; rows beyond N repeat the last row, their results are not stored).
  auto fetch_meta = [&](int local_tile) {
    const int row0 = (cta + local_tile * grid) * 8;
    const int last_row = static_cast<int>(p.w.n) - 1;
    const int pieces_per_row = p.segs / 4;
    for (int i = lane; i < 8 * pieces_per_row; i += 32) {
      const int r = i / pieces_per_row;
      const int c = i - r * pieces_per_row;
      const int row = row0 + r < last_row ? row0 + r : last_row;
      CopyAsyncMeta16(meta_warp + r * scale_row_bytes + c * 16,
                      p.w.scales + static_cast<std::int64_t>(row) * p.segs + c * 4);
    }
    if constexpr (HAS_ZP) {
      const int zero_pieces = p.segs / 16;
      for (int i = lane; i < 8 * zero_pieces; i += 32) {
        const int r = i / zero_pieces;
        const int c = i - r * zero_pieces;
        const int row = row0 + r < last_row ? row0 + r : last_row;
        CopyAsyncMeta16(meta_warp + 8 * scale_row_bytes + r * p.segs + c * 16,
                        p.w.zp16 + static_cast<std::int64_t>(row) * p.segs + c * 16);
      }
    }
    asm volatile("cp.async.commit_group;" ::);
  };
  const DigitGeometry geometry{static_cast<int>(p.w.k), p.segs, kDigits * kChunkBytes, p.table_ints};
  StageDigits<true>(
      geometry, p.a, 1, 1, digits, table, undo, red, tid, consumer_threads,
      [&] { asm volatile("bar.sync 1, %0;" ::"r"(consumer_threads) : "memory"); },
      [&] {
        // behind the request for A: the producer's bulk of copies and this warp's own small ones
        asm volatile("bar.arrive 3, %0;" ::"r"(consumer_threads + 32) : "memory");
        if (warp < local_tiles) {
          fetch_meta(warp);
        }
      });
  // barriers initialised (the producer has arrived long ago)
  asm volatile("bar.sync 2, %0;" ::"r"(consumer_threads + 32) : "memory");
  MNB_MARKR(3)

  const int g = lane >> 2;
  const int t = lane & 3;
  // MMA row g is row `rho` of the tile: the two rows a quarter warp reads together then differ in
  // bit 2, and the 128-byte swizzle (16-byte unit ^ row) puts them on different halves of the banks
  const int rho = ((g & 1) << 2) | (g >> 1);
  const std::uint32_t lo_offset = rho * 128 + ((t ^ rho) << 4);        // even segment: units 0..3 of the row
  const std::uint32_t hi_offset = rho * 128 + (((4 + t) ^ rho) << 4);  // odd segment: units 4..7
  const int column = g < 6 ? g : g - 6;
  const int second = column >= kDigits ? 1 : 0;
  const int digit_of_column = column - second * kDigits;
  const int swizzle = (second + digit_of_column) & 1;
  const std::uint32_t digits_column =
      LaunderAfterBarrier(ptx::SmemAddr(digits) + (second * kDigits + digit_of_column) * kChunkBytes);
  const std::uint32_t digits_even = digits_column + (((2 * t) ^ swizzle) << 4);
  const std::uint32_t digits_odd = digits_column + (((2 * t + 1) ^ swizzle) << 4);
  const std::uint32_t table_lane = LaunderAfterBarrier(ptx::SmemAddr(table) + t * 8);
  const std::uint32_t weights_warp = ptx::SmemAddr(weight_slots) + warp * p.slots_per_warp * weight_slot_bytes;
  const std::uint32_t scales_lane = meta_warp + rho * scale_row_bytes;
  const std::uint32_t zeros_lane = meta_warp + 8 * scale_row_bytes + rho * p.segs;
  const int supers = steps / kStepsPerSuper;

  const ZeroQuad zero = MakeZeroQuad();
  const int sixteen = static_cast<int>(LaunderAfterBarrier(16u));  // a register: keeps 16 * even + odd one instruction
  int q = 0;  // this warp's task counter
  for (int local_tile = warp; local_tile < local_tiles; local_tile += consumers) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    bool dead = false;
    // this tile's scales / zero points: asked for at the start (first tile) or at the end of the
    // tile before; every lane waits for its own pieces, then the warp meets
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    for (int part = 0; part < p.parts; ++part, ++q) {
      const int d = q % p.slots_per_warp;
      const int slot = warp * p.slots_per_warp + d;
      if (!dead && !ptx::MbarWait(&full_bar[slot], static_cast<std::uint32_t>(q / p.slots_per_warp) & 1u)) {
        ReportStatus(p.status, kDeviceTimeoutFullBarrier);
        dead = true;
      }
      if (dead) {
        continue;
      }
      if (q == 0) { MNB_MARKR(4) }
      std::uint32_t lo_at = weights_warp + d * weight_slot_bytes + lo_offset;
      std::uint32_t hi_at = weights_warp + d * weight_slot_bytes + hi_offset;
      const int step0 = part * steps;
      std::uint32_t scales_at = scales_lane + step0 * 8;
      std::uint32_t zeros_at = zeros_lane + step0 * 2;
      std::uint32_t even_at = digits_even + step0 * kTileColumnBytes;
      std::uint32_t odd_at = digits_odd + step0 * kTileColumnBytes;
      std::uint32_t table_at = table_lane + step0 * 32;
#pragma unroll 1
      for (int super = 0; super < supers; ++super) {
        // scales and zero points of the eight segments of this superstep, row rho
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
      // the slot may be refilled
      __syncwarp();
      if (lane == 0) {
        ptx::MbarArrive(&empty_bar[slot]);
      }
    }
    // ---- the tile is complete: rows g see columns 0..2 (even segments), rows g + 8 columns 3..5 ----
    float v = t == 0   ? fmaf(16384.0f, acc[0], 128.0f * acc[1])
              : t == 1 ? fmaf(16384.0f, acc[3], acc[0])
              : t == 2 ? fmaf(128.0f, acc[2], acc[3])
                       : 0.0f;
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    const std::int64_t row = static_cast<std::int64_t>(cta + local_tile * grid) * 8 + rho;
    if (!dead && t == 0 && row < p.w.n) {
      const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + row) : 0.0f;
      StoreOutput(p.out, p.out.col_offset + row, fmaf(v, undo[0], bias));
    }
    if (local_tile == warp) { MNB_MARKR(5) }
    if (local_tile + consumers < local_tiles) {
      __syncwarp();  // every lane has read this tile's scales
      fetch_meta(local_tile + consumers);
    }
  }
  MNB_MARKR(7)
}

bool EncodeWeightMap(CUtensorMap *map, const WeightView &w, int steps) {
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

} // namespace

// One token, 4-bit, block_size 128, whole 128-byte chunks per row in multiples of four (K a
// multiple of 1024), prepared zero-point bytes when the node has zero points.
bool DecodeResidentSupports(const WeightView &w, std::int64_t m) {
  return m == 1 && w.bits == 4 && w.block_size == 128 && (w.n_blocks % (2 * kStepsPerSuper)) == 0 &&
         (w.zp == nullptr || (w.zp16 != nullptr && (w.n_blocks % 16) == 0)) &&
         (reinterpret_cast<std::uintptr_t>(w.b) & 15u) == 0 &&
         (reinterpret_cast<std::uintptr_t>(w.scales) & 15u) == 0 && (reinterpret_cast<std::uintptr_t>(w.zp16) & 15u) == 0 &&
         w.n < (std::int64_t{1} << 31);
}

const char *LaunchDecodeResident(const WeightView &w, const float *a, std::int64_t m, OutputView out, int *status_word,
                                 cudaStream_t stream, int sm_count) {
  if (!DecodeResidentSupports(w, m)) {
    return nullptr;
  }
  const int sms = sm_count > 0 ? sm_count : 148;
  ResidentParams p{};
  p.w = w;
  p.a = a;
  p.out = out;
  p.status = status_word;
  p.segs = w.n_blocks;
  p.table_ints = (p.segs / 2) * 8;
  p.tiles = static_cast<int>((w.n + 7) / 8);
  int ctas = sms < p.tiles ? sms : p.tiles;
  const int tiles_per_cta = (p.tiles + ctas - 1) / ctas;
  const int chunks = w.row_bytes / 128;  // MMA steps of a whole row
  const size_t fixed = static_cast<size_t>(p.segs) * kDigits * kChunkBytes + static_cast<size_t>(p.table_ints) * 4 +
                       (kMaxTokens + kMaxTokens * kMaxWarps) * sizeof(float) + 2 * kMaxSlots * sizeof(std::uint64_t) +
                       1024;  // + alignment slack
  const size_t limit = 227 * 1024;
  if (fixed + 16 * 1024 > limit) {
    return nullptr;
  }
  const size_t per_step = kChunkRowsBytes;
  const size_t per_warp = 8 * (static_cast<size_t>(w.n_blocks) * 4 + 16) + (w.zp != nullptr ? 8 * w.n_blocks : 0);
  // Shape of the slots. First choice: a whole row of K per task and one slot per consumer warp,
  // with as many consumer warps as shared memory holds; taken when (nearly) every tile of the CTA
  // then has a slot of its own, so that nothing (or one tile) waits for a slot to be released.
  // Else tasks of 8 ... 16 chunks and two slots per warp, so that a warp's next task is on its way
  // while it works.
  const int min_steps = kStepsPerSuper;
  auto fits = [&](int c, int d, int s) {
    return fixed + static_cast<size_t>(c) * (static_cast<size_t>(d) * s * per_step + per_warp) <= limit;
  };
  auto most_consumers = [&](int d, int s) {
    int c = tiles_per_cta < kMaxConsumerWarps ? tiles_per_cta : kMaxConsumerWarps;
    while (c > 0 && !fits(c, d, s)) {
      --c;
    }
    return c;
  };
  // A resident tile arrives in parts of `steps` chunks, each with a slot of its own, all first parts
  // before all second parts: a warp works on part p while part p + 1 streams, and what is left to
  // do after the last copy has landed is one part, not one tile.
  static const int exp_part = std::getenv("MNB_X_PART") ? std::atoi(std::getenv("MNB_X_PART")) : 16;
  int steps = chunks;
  if (exp_part >= min_steps && (exp_part % kStepsPerSuper) == 0 && (chunks % exp_part) == 0 &&
      chunks / exp_part <= 4) {
    steps = exp_part;
  }
  int slots_per_warp = chunks / steps;
  int consumers = chunks <= 256 ? most_consumers(slots_per_warp, steps) : 0;
  if (consumers < 1 || tiles_per_cta > consumers + consumers / 4) {
    slots_per_warp = 2;
    steps = 0;
    for (int s = 16; s >= min_steps; s -= kStepsPerSuper) {
      if ((chunks % s) == 0) {
        steps = s;
        break;
      }
    }
    if (steps == 0) {
      return nullptr;
    }
    consumers = most_consumers(2, steps);
    if (consumers < 1) {
      return nullptr;
    }
  }
  if ((chunks % steps) != 0 || (steps % kStepsPerSuper) != 0 || steps > 256) {
    return nullptr;
  }
  p.steps_per_task = steps;
  p.parts = chunks / steps;
  p.consumer_warps = consumers;
  p.slots_per_warp = slots_per_warp;
  static const int exp_early = std::getenv("MNB_X_EARLY") ? std::atoi(std::getenv("MNB_X_EARLY")) : 0;
  p.early_tasks = exp_early;
  const size_t smem =
      fixed + static_cast<size_t>(consumers) * (static_cast<size_t>(slots_per_warp) * steps * per_step + per_warp);

  CUtensorMap map_w;
  if (!EncodeWeightMap(&map_w, w, steps)) {
    return nullptr;
  }
  auto launch = [&](auto kernel) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) {
      return err;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
    config.blockDim = dim3(static_cast<unsigned>((consumers + 1) * 32), 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, map_w, p);
  };
  const cudaError_t err =
      w.zp != nullptr ? launch(nbits_decode_resident_kernel<true>) : launch(nbits_decode_resident_kernel<false>);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  CountLaunch();
  return "nbits_decode_resident_kernel";
}

} // namespace mnb
