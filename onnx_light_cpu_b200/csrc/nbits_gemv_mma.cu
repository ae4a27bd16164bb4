// Decode path of MatMulNBits on warp-level tensor-core MMA with fp32-grade accuracy.
//
// Why tensor cores for a GEMV: on CUDA cores every 4-bit code costs one integer extraction
// plus two floating-point operations per activation row, and the integer pipe (half rate)
// becomes the limit before HBM does. Here a code costs 5/8 integer operation and half an
// fp16x2 operation, and the multiply-accumulate is free: the weights are the MMA "A" operand
// (16 rows x 16 k per step) and the activations the "B" operand.
//
// Exactness. (q - zp) is an integer of magnitude < 256: exact in fp16. Each activation row is
// scaled by a power of two so that its largest magnitude is in [2^14, 2^15) and split into
// two fp16 pieces a = h1 + h2 (22 significant bits; what is dropped is below 2^-22 |a| or
// 2^-39 max|a|), which occupy two MMA columns. fp16 x fp16 products are exact in the fp32
// accumulator; accumulators are restarted per quantization block and the block sums are
// combined in ordinary fp32 arithmetic: acc += scale * (D[piece 0] + D[piece 1]). The result
// differs from a sequential fp32 evaluation by less than the 1e-5 bar of the CUDA-core path.
//
// Columns of the 16x8 MMA tile = (token, block-inside-supergroup, piece). A "supergroup" is
// 128 consecutive k (each of the four lanes of a quad loads 16 bytes = 32 codes of a row).
// For block_size 32 / 64 the four lanes' codes lie in different quantization blocks; the
// activation fragment of a lane is zero except in the column of its own block, so every
// column accumulates exactly one block and the per-block scale can be applied afterwards.
//
// Data movement: persistent CTA per SM; a producer warp fills a ring of task slots with 1-D
// bulk (TMA) copies - 16 weight rows x 16 quantization blocks per task plus that task's
// scales / zero points from a prepared, task-major side array - completed on mbarriers.
// Eight consumer warps own whole 16-row tiles (no cross-warp reduction). All waits bounded.
//
// Conventions: packed-INT4 nibble order of
// onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:60-93; "stream B once, split N"
// partition of onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258.

#include "nbits_common.cuh"
#include "nbits_ptx.cuh"
#include "nbits_mma_common.cuh"
#include "nbits_tma.cuh"

#include <cuda_fp16.h>

#include <cstdint>
#include <cstdlib>

namespace mnb {
namespace {

using namespace mma_decode;


constexpr int kPairs = 8;                 // 16-row tiles in flight per CTA
constexpr int kWarps = 2 * kPairs;        // consumer warps: two per tile, alternating k slices
constexpr int kConsumerThreads = kWarps * 32;
// Up to four producer warps can share the tasks (one issuing thread sustains 4.4 TB/s on long
// streams, four 6.7 TB/s); at decode sizes a single paced issuer is faster, see WantedProducers().
constexpr int kProducers = 4;
constexpr int kThreads = (kWarps + kProducers) * 32;
constexpr int kMaxSlots = 16;
constexpr int kMaxTokens = 4;             // most activation rows handled per CTA pass
#ifndef MNB_MMA_UNROLL
#define MNB_MMA_UNROLL 4
#endif
constexpr int kUnroll = MNB_MMA_UNROLL;   // supergroups per loop round (1, 2 or 4)
constexpr int kZeroBytes = 256 * kUnroll + 64; // what an inactive lane reads in one loop round

struct MmaParams {
  WeightView w;
  const float *a;
  int m_total;
  OutputView out;
  int *status;
  int half_tiles;       // ceil(n / 8)
  int bpt;              // quantization blocks per task
  int slices;           // tasks per row tile = ceil(n_blocks / bpt)
  int slice_b_bytes;    // packed bytes of one row inside a task
  int sg_per_task;      // 128-k supergroups per task
  int sg_per_block;     // supergroups per quantization block (block_size >= 128), else 1
  int rec_bytes;        // bytes of one prepared meta record (bpt blocks x 8 rows)
  int rec_scale_bytes;  // scale part of a record
  int slot_bytes;
  int num_slots;
  int full_rows;        // 1: a task is 16 whole weight rows (all of K), one contiguous bulk copy, shared
                        //    by the two warps of a pair; 0: 16 rows x one 2048-k slice through a TMA box
  int row_stride;       // bytes between weight rows inside a slot
  int weight_bytes;     // bytes of the weight part of a slot
  int producers;        // producer warps in use (num_slots is a multiple of it)
  int act_row_bytes;    // bytes between activation piece rows in shared memory
  int k_pad;            // activation positions per piece row (all tasks, zero beyond K)
  int tokens_per_pass;  // activation rows per grid.y pass (8 columns / blocks-per-supergroup / 2)
  std::uint32_t magic;  // 0x64006400, passed at run time so that it stays in a register
  GatherTail tail;      // flag exchange of a gathered step, run by the last CTA (ranks == 0: none)
};

// NB_SG_LOG2: log2 of quantization blocks per 128-k supergroup (block 128+: 0, 64: 1, 32: 2).
// BIG_BLOCK: a block spans several supergroups (block_size >= 256).
template <int NB_SG_LOG2, bool BIG_BLOCK, bool HAS_ZP>
__global__ void __launch_bounds__(kThreads, 1)
    nbits_gemv_mma_kernel(const __grid_constant__ CUtensorMap map_b, const MmaParams p) {
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  // keep the pointer in the shared address space (no integer round trip) while aligning it
  unsigned char *smem_raw = smem_dyn + ((128u - (ptx::SmemAddr(smem_dyn) & 127u)) & 127u);
  // layout: [slots][activation piece rows: 2 per token][per-token 2^-e][amax scratch]
  //         [pair exchange: kPairs x 32 lanes x 2][barriers]
  unsigned char *slots = smem_raw;
  unsigned char *act = smem_raw + static_cast<size_t>(p.num_slots) * p.slot_bytes;
  float *inv_scale = reinterpret_cast<float *>(act + 2 * p.tokens_per_pass * p.act_row_bytes + kZeroBytes);
  float *scratch = inv_scale + kMaxTokens;          // [2][kWarps], alternating with the token index
  float2 *pair_buf = reinterpret_cast<float2 *>(scratch + 2 * kWarps); // [kPairs][32]
  std::uint64_t *full_bar = reinterpret_cast<std::uint64_t *>(pair_buf + kPairs * 32);
  std::uint64_t *empty_bar = full_bar + kMaxSlots;
  // task index currently assigned to each slot. A slot is consumed by different warps in
  // successive rounds, and an mbarrier phase parity only tells two neighbouring phases apart,
  // so a consumer first waits until the producer has assigned ITS task to the slot (which
  // happens after the previous round was released) and only then waits on the parity.
  volatile int *slot_task = reinterpret_cast<volatile int *>(empty_bar + kMaxSlots);

  constexpr int kNbSg = 1 << NB_SG_LOG2;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int m_base = blockIdx.y * p.tokens_per_pass;
  int tokens = p.m_total - m_base;
  if (tokens > p.tokens_per_pass) {
    tokens = p.tokens_per_pass;
  }

  // this CTA's half tiles (8 rows each), split as evenly as the grid allows
  const int h_begin = static_cast<int>(static_cast<std::int64_t>(blockIdx.x) * p.half_tiles / gridDim.x);
  const int h_end = static_cast<int>(static_cast<std::int64_t>(blockIdx.x + 1) * p.half_tiles / gridDim.x);
  const int n_tiles = (h_end - h_begin + 1) >> 1;
  const std::int64_t row_limit =
      static_cast<std::int64_t>(h_end) * 8 < p.w.n ? static_cast<std::int64_t>(h_end) * 8 : p.w.n;

  // the next kernel in the stream may start filling SMs as they free up
  ptx::GridDependencyLaunch();

  if (warp >= kWarps) {
    // ------------------------------ producers ------------------------------
    // One lane per producer warp issues, per task, one 2-D tiled TMA load of the weight tile (16
    // rows x the slice; rows past the matrix end are zero-filled) and one bulk copy of the
    // task's scale / zero-point records (two consecutive half tiles of the same slice).
    // Producer j takes the tasks with index % producers == j. num_slots is a multiple of the
    // number of producers, so all rounds of a slot belong to the same producer and its parity
    // waits on that slot follow each other in order.
    const int producer = warp - kWarps;
    if (producer == 0 && lane == 0) {
      for (int s = 0; s < p.num_slots; ++s) {
        ptx::MbarInit(&full_bar[s], 1);
        ptx::MbarInit(&empty_bar[s], p.full_rows != 0 ? 2 : 1); // released by both warps of the pair
        slot_task[s] = -1;
      }
      ptx::FenceMbarInit();
    }
    // barriers initialised: the producers go on at once; the consumers join barrier 10 after
    // staging the activations, the producers only arrive there
    asm volatile("bar.sync 11, %0;" ::"n"(kProducers * 32) : "memory");
    asm volatile("bar.arrive 10, %0;" ::"n"(kThreads) : "memory");
    if (lane == 0 && producer < p.producers) {
      ptx::PrefetchTensorMap(&map_b);
      int task = 0;
      int slot = 0;              // task % num_slots, kept incrementally
      std::uint32_t round = 0;   // task / num_slots
      int turn = 0;              // task % producers
      bool ok = true;
      const std::uint32_t box_bytes = 16u * static_cast<std::uint32_t>(p.slice_b_bytes);
      const int x_step = p.slice_b_bytes / 4;
      const std::int64_t meta_slice_stride = static_cast<std::int64_t>(p.half_tiles) * p.rec_bytes;
      if (p.full_rows != 0) {
        // one task per row tile: 16 whole rows are contiguous in memory, so one large bulk copy
        // brings them (a single issuing thread sustains 6.4 TB/s with 32 KB copies against
        // 4.4 TB/s with 16 KB boxes), plus the tile's scale / zero-point records of every slice
        for (; task < n_tiles && ok; ++task) {
          if (turn == producer) {
            if (round != 0 && !ptx::MbarWait(&empty_bar[slot], (round & 1u) ^ 1u)) {
              ReportStatus(p.status, kDeviceTimeoutEmptyBarrier);
              ok = false;
              break;
            }
            const int h0 = h_begin + 2 * task;
            const std::int64_t first_row = static_cast<std::int64_t>(h0) * 8;
            const std::int64_t rows_left = p.w.n - first_row;
            const std::uint32_t row_bytes_total =
                static_cast<std::uint32_t>(rows_left < 16 ? rows_left : 16) * static_cast<std::uint32_t>(p.row_stride);
            const std::uint32_t meta_bytes = (h0 + 1 < p.half_tiles ? 2u : 1u) * static_cast<std::uint32_t>(p.rec_bytes);
            unsigned char *dst = slots + static_cast<size_t>(slot) * p.slot_bytes;
            slot_task[slot] = task;
            ptx::MbarArriveExpectTx(&full_bar[slot], row_bytes_total + static_cast<std::uint32_t>(p.slices) * meta_bytes);
            ptx::BulkLoad(dst, p.w.b + first_row * p.row_stride, row_bytes_total, &full_bar[slot]);
            const unsigned char *meta_src = p.w.meta + static_cast<std::int64_t>(h0) * p.rec_bytes;
            for (int s = 0; s < p.slices; ++s, meta_src += meta_slice_stride) {
              ptx::BulkLoad(dst + p.weight_bytes + s * 2 * p.rec_bytes, meta_src, meta_bytes, &full_bar[slot]);
            }
          }
          if (++turn == p.producers) {
            turn = 0;
          }
          if (++slot == p.num_slots) {
            slot = 0;
            ++round;
          }
        }
      }
      for (int wave0 = 0; p.full_rows == 0 && wave0 < n_tiles && ok; wave0 += kPairs) {
        const int wave_tiles = n_tiles - wave0 < kPairs ? n_tiles - wave0 : kPairs;
        const unsigned char *meta_slice = p.w.meta + static_cast<std::int64_t>(h_begin + 2 * wave0) * p.rec_bytes;
        for (int s = 0; s < p.slices && ok; ++s, meta_slice += meta_slice_stride) {
          int h0 = h_begin + 2 * wave0;
          const unsigned char *meta_src = meta_slice;
          for (int wt = 0; wt < wave_tiles; ++wt, ++task, h0 += 2, meta_src += 2 * p.rec_bytes) {
            if (turn == producer) {
              if (round != 0 && !ptx::MbarWait(&empty_bar[slot], (round & 1u) ^ 1u)) {
                ReportStatus(p.status, kDeviceTimeoutEmptyBarrier);
                ok = false;
                break;
              }
              const std::uint32_t meta_bytes = (h0 + 1 < p.half_tiles ? 2u : 1u) * static_cast<std::uint32_t>(p.rec_bytes);
              unsigned char *dst = slots + static_cast<size_t>(slot) * p.slot_bytes;
              slot_task[slot] = task;
              ptx::MbarArriveExpectTx(&full_bar[slot], box_bytes + meta_bytes);
              ptx::TmaLoad2D(dst, &map_b, s * x_step, h0 * 8, &full_bar[slot]);
              ptx::BulkLoad(dst + box_bytes, meta_src, meta_bytes, &full_bar[slot]);
            }
            if (++turn == p.producers) {
              turn = 0;
            }
            if (++slot == p.num_slots) {
              slot = 0;
              ++round;
            }
          }
        }
      }
      // stay until every copy this lane issued has been consumed (bounded), so none lands after exit
      const int first = task - p.num_slots < 0 ? 0 : task - p.num_slots;
      for (int i = first; i < task && ok; ++i) {
        if ((i % p.producers) == producer &&
            !ptx::MbarWait(&empty_bar[i % p.num_slots], static_cast<std::uint32_t>(i / p.num_slots) & 1u)) {
          break;
        }
      }
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  // Activation staging: per token a power-of-two scale, two fp16 pieces, permuted order.
  // A thread owns whole 8-k words (one 16-byte store per piece); up to four words per thread
  // stay in registers between the max reduction and the split, so A is read once.
  // A (and Y) may be produced / still read by the previous kernel in the stream: from here on
  // the consumers depend on it. The producer warp above only touches the constant weights.
  ptx::GridDependencyWait();
  // lanes whose MMA column takes no part read zeros: a small region that they re-read every
  // round (their pointer does not advance), not a whole row
  unsigned char *zero_row = act + 2 * p.tokens_per_pass * p.act_row_bytes;
  for (int i = tid; i < (kZeroBytes >> 4); i += kConsumerThreads) {
    reinterpret_cast<uint4 *>(zero_row)[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  // all rows at once, one group of warps per row (rows beyond `tokens` are never read: their
  // lanes point at the zero region)
  StageActivations<kWarps>(p.a + static_cast<std::int64_t>(m_base) * p.w.k, tokens, static_cast<int>(p.w.k), p.k_pad,
                           act, p.act_row_bytes, inv_scale, scratch, tid);
  // activations staged and (through the producer's arrival) barriers initialised
  asm volatile("bar.sync 10, %0;" ::"n"(kThreads) : "memory");

  const int g = lane >> 2;
  const int t = lane & 3;
  const int pair = warp >> 1;   // which tile of a wave this warp works on
  const int parity = warp & 1;  // which k slices of that tile
  // role of this lane's column (g) in the activation fragment
  const int pc_b = g >> 1;
  const int piece_b = g & 1;
  const int m_b = pc_b >> NB_SG_LOG2;
  const int blk_b = pc_b & (kNbSg - 1);
  // block-in-supergroup of this lane's own codes: lane t holds k = 32t .. 32t+31
  const int tb = NB_SG_LOG2 == 2 ? t : (NB_SG_LOG2 == 1 ? t >> 1 : 0);
  const bool b_active = m_b < tokens && blk_b == tb;
  // lanes whose column takes no part read a row of zeros, so the loads need no predicate
  const unsigned char *act_lane =
      (b_active ? act + (2 * m_b + piece_b) * p.act_row_bytes : zero_row) + t * 16;
  const int lane_step = b_active ? 256 : 0; // bytes per supergroup in this lane's activation row
  // role of this lane's accumulator columns (2t, 2t+1)
  const int m_d = t >> NB_SG_LOG2;
  const int blk_d = t & (kNbSg - 1);

  const std::uint32_t magic = p.magic;
  const std::uint32_t sixteenth = 0x2c002c00u;  // fp16 1/16 twice
  const std::uint32_t plus960 = 0x63806380u;    // fp16 960 twice
  const std::uint32_t default_offs = 0x64086408u; // fp16 1024 + 8 twice
  // meta record: float scale[8 rows][row floats] (rows padded where they would share a bank),
  // then uint8 zp[8 rows][bpt]
  const int scale_row_bytes = p.rec_scale_bytes / 8;
  constexpr int kNb = kNbSg; // quantization blocks per supergroup (1 when a block spans several)

  int tile_count = 0;
  bool dead = false; // a bounded wait gave up: skip the math but keep the pair barrier protocol
  for (int tile = pair; tile < n_tiles; tile += kPairs, ++tile_count) {
    const int wave0 = tile - pair;
    const int wave_tiles = n_tiles - wave0 < kPairs ? n_tiles - wave0 : kPairs;
    const int h0 = h_begin + 2 * tile;
    const std::int64_t row0 = static_cast<std::int64_t>(h0) * 8;
    float acc0 = 0.0f, acc1 = 0.0f; // rows g and g + 8, accumulator column pair t
    float da[4], db[4];

    // waits (bounded) until `task` has landed in its slot; false after a time-out
    auto wait_task = [&](int task, int slot) {
      const std::uint32_t round = static_cast<std::uint32_t>(task / p.num_slots);
      // first use of a slot: its barrier is still in phase 0, no tag needed
      bool assigned = round == 0;
      for (std::uint32_t spin = 0; !assigned && spin < ptx::kSpinLimit; ++spin) {
        assigned = slot_task[slot] == task;
        if (!assigned) {
          __nanosleep(256);
        }
      }
      if (!assigned || !ptx::MbarWait(&full_bar[slot], round & 1u)) {
        ReportStatus(p.status, kDeviceTimeoutFullBarrier);
        return false;
      }
      return true;
    };
    // whole-row tasks: the tile is one task, which both warps of the pair wait for and release
    int slot = tile % p.num_slots;
    if (p.full_rows != 0 && !wait_task(tile, slot)) {
      dead = true;
    }

    for (int s = parity; s < p.slices && !dead; s += 2) {
      const int task = p.full_rows != 0 ? tile : wave0 * p.slices + s * wave_tiles + pair;
      if (p.full_rows == 0) {
        slot = task % p.num_slots;
        if (!wait_task(task, slot)) {
          dead = true;
          break;
        }
      }
      const unsigned char *sb = slots + static_cast<size_t>(slot) * p.slot_bytes;
      const unsigned char *row_lo =
          sb + g * p.row_stride + (p.full_rows != 0 ? s * p.slice_b_bytes : 0) + t * 16;
      const unsigned char *row_hi = row_lo + 8 * p.row_stride;
      const unsigned char *meta0 = sb + p.weight_bytes + (p.full_rows != 0 ? s * 2 * p.rec_bytes : 0); // rows 0..7
      const unsigned char *meta1 = meta0 + p.rec_bytes;  // rows 8..15
      const float *sc0 = reinterpret_cast<const float *>(meta0 + g * scale_row_bytes);
      const float *sc1 = reinterpret_cast<const float *>(meta1 + g * scale_row_bytes);
      const unsigned char *zr0 = meta0 + p.rec_scale_bytes + g * p.bpt;
      const unsigned char *zr1 = meta1 + p.rec_scale_bytes + g * p.bpt;
      const unsigned char *act_task = act_lane + static_cast<size_t>(s) * p.sg_per_task * lane_step;

      for (int sg0 = 0; sg0 < p.sg_per_task; sg0 += kUnroll) {
        // scales / zero points of the supergroups of this round
        float s0v[kUnroll], s1v[kUnroll];
        std::uint32_t z0v[kUnroll], z1v[kUnroll];
        if constexpr (!BIG_BLOCK && NB_SG_LOG2 == 0 && kUnroll == 4) {
          // one block per supergroup: four consecutive blocks, one vector load each
          const float4 a4 = *reinterpret_cast<const float4 *>(sc0 + sg0);
          const float4 b4 = *reinterpret_cast<const float4 *>(sc1 + sg0);
          s0v[0] = a4.x, s0v[1] = a4.y, s0v[2] = a4.z, s0v[3] = a4.w;
          s1v[0] = b4.x, s1v[1] = b4.y, s1v[2] = b4.z, s1v[3] = b4.w;
          if constexpr (HAS_ZP) {
            const std::uint32_t za = *reinterpret_cast<const std::uint32_t *>(zr0 + sg0);
            const std::uint32_t zb = *reinterpret_cast<const std::uint32_t *>(zr1 + sg0);
            z0v[0] = __byte_perm(za, 0x64646464u, 0x4040), z1v[0] = __byte_perm(zb, 0x64646464u, 0x4040);
            z0v[1] = __byte_perm(za, 0x64646464u, 0x4141), z1v[1] = __byte_perm(zb, 0x64646464u, 0x4141);
            z0v[2] = __byte_perm(za, 0x64646464u, 0x4242), z1v[2] = __byte_perm(zb, 0x64646464u, 0x4242);
            z0v[3] = __byte_perm(za, 0x64646464u, 0x4343), z1v[3] = __byte_perm(zb, 0x64646464u, 0x4343);
          }
        } else {
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const int sg = sg0 + u;
            const int blk_codes = BIG_BLOCK ? sg / p.sg_per_block : sg * kNb + tb;
            const int blk_acc = BIG_BLOCK ? blk_codes : sg * kNb + blk_d;
            s0v[u] = sc0[blk_acc];
            s1v[u] = sc1[blk_acc];
            if constexpr (HAS_ZP) {
              z0v[u] = __byte_perm(static_cast<std::uint32_t>(zr0[blk_codes]), 0x64646464u, 0x4040);
              z1v[u] = __byte_perm(static_cast<std::uint32_t>(zr1[blk_codes]), 0x64646464u, 0x4040);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const uint4 q0 = *reinterpret_cast<const uint4 *>(row_lo + u * 64);
          const uint4 q1 = *reinterpret_cast<const uint4 *>(row_hi + u * 64);
          const std::uint32_t offs0 = HAS_ZP ? z0v[u] : default_offs; // (1024 + zp) twice
          const std::uint32_t offs1 = HAS_ZP ? z1v[u] : default_offs;
          const std::uint32_t offs0_16 = Hsub2(plus960, offs0); // -(64 + zp)
          const std::uint32_t offs1_16 = Hsub2(plus960, offs1);
          uint4 bf[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            bf[i] = *reinterpret_cast<const uint4 *>(act_task + u * 256 + i * 64);
          }
          const std::uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w};
          const std::uint32_t w1[4] = {q1.x, q1.y, q1.z, q1.w};
          // a block that spans several supergroups keeps accumulating; otherwise start afresh
          const bool fresh = BIG_BLOCK ? ((sg0 + u) % p.sg_per_block) == 0 : true;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            std::uint32_t pa[4], pb[4];
            Dequant8(w0[i], magic, offs0, offs0_16, sixteenth, pa);
            Dequant8(w1[i], magic, offs1, offs1_16, sixteenth, pb);
            // two accumulator sets halve the dependent chain of MMAs
            if (i == 0 && fresh) {
              MmaF16Zero(da, pa[0], pb[0], pa[1], pb[1], bf[i].x, bf[i].y);
              MmaF16Zero(db, pa[2], pb[2], pa[3], pb[3], bf[i].z, bf[i].w);
            } else {
              MmaF16(da, pa[0], pb[0], pa[1], pb[1], bf[i].x, bf[i].y);
              MmaF16(db, pa[2], pb[2], pa[3], pb[3], bf[i].z, bf[i].w);
            }
          }
          const bool block_done = BIG_BLOCK ? ((sg0 + u + 1) % p.sg_per_block) == 0 : true;
          if (block_done) {
            acc0 = fmaf(s0v[u], (da[0] + da[1]) + (db[0] + db[1]), acc0);
            acc1 = fmaf(s1v[u], (da[2] + da[3]) + (db[2] + db[3]), acc1);
          }
        }
        row_lo += 64 * kUnroll;
        row_hi += 64 * kUnroll;
        act_task += lane_step * kUnroll;
      }
      __syncwarp();
      if (lane == 0 && p.full_rows == 0) {
        ptx::MbarArrive(&empty_bar[slot]);
      }
    }
    if (p.full_rows != 0 && !dead) {
      __syncwarp();
      if (lane == 0) {
        ptx::MbarArrive(&empty_bar[slot]);
      }
    }
    // blocks of one supergroup sit in neighbouring lanes of the quad: add them up
    if (NB_SG_LOG2 >= 1) {
      acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
      acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    }
    if (NB_SG_LOG2 >= 2) {
      acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
      acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    }
    // the odd warp of the pair hands its half of K to the even warp (one buffer per pair: the
    // second barrier keeps the next tile's value from overwriting one that is still being read)
    float2 *exchange = pair_buf + pair * 32 + lane;
    if (parity == 1) {
      *exchange = make_float2(acc0, acc1);
    }
    asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");
    float2 other = make_float2(0.0f, 0.0f);
    if (parity == 0) {
      other = *exchange;
    }
    asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");
    if (parity == 0) {
      acc0 += other.x;
      acc1 += other.y;
      if (blk_d == 0 && m_d < tokens) {
        const float undo = inv_scale[m_d];
        const std::int64_t m = m_base + m_d;
        const std::int64_t r_lo = row0 + g;
        const std::int64_t r_hi = row0 + g + 8;
        if (r_lo < row_limit) {
          const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + r_lo) : 0.0f;
          StoreOutput(p.out, m * p.out.ld + p.out.col_offset + r_lo, fmaf(acc0, undo, bias));
        }
        if (r_hi < row_limit) {
          const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + r_hi) : 0.0f;
          StoreOutput(p.out, m * p.out.ld + p.out.col_offset + r_hi, fmaf(acc1, undo, bias));
        }
      }
    }
  }
  // ---- gathered step: the last CTA of the grid publishes this rank's flags --------------------
  if (p.tail.ranks > 0) {
    // gathered step: the arithmetic stored locally only; now this CTA's rows go to the peers
    asm volatile("bar.sync 12, %0;" ::"n"(kConsumerThreads) : "memory");
    PushRowsToPeers(p.out, p.tail, m_base, tokens, static_cast<std::int64_t>(h_begin) * 8, row_limit, tid, kConsumerThreads);
    PublishWhenGridDone(p.tail, tid, kConsumerThreads, 12, gridDim.x * gridDim.y, p.status);
  }
}

// ---- prepared side array -----------------------------------------------------------------
// meta[(slice * half_tiles + half_tile)] = { float scale[8 rows][scale_row_floats] ; uint8 zp[8 rows][bpt] }
// (the zero-point part only when the node has zero points). Rows beyond N and blocks beyond
// n_blocks get scale 0.
__global__ void __launch_bounds__(256) nbits_prepare_meta_kernel(const WeightView w, int bpt, int scale_row_floats,
                                                                 int half_tiles,
                                                                 int rec_bytes, int rec_scale_bytes,
                                                                 unsigned char *meta, std::int64_t records) {
  const std::int64_t per_record = 8 * bpt;
  const std::int64_t total = records * per_record;
  for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
    const std::int64_t record = i / per_record;
    const int within = static_cast<int>(i - record * per_record);
    const int r = within / bpt;
    const int b = within - r * bpt;
    const int slice = static_cast<int>(record / half_tiles);
    const std::int64_t half_tile = record - static_cast<std::int64_t>(slice) * half_tiles;
    const std::int64_t row = half_tile * 8 + r;
    const int block = slice * bpt + b;
    float scale = 0.0f;
    int zp = 0;
    if (row < w.n && block < w.n_blocks) {
      scale = w.scales[row * w.n_blocks + block];
      zp = ZeroPointOf(w, row, block);
    }
    unsigned char *rec = meta + record * rec_bytes;
    reinterpret_cast<float *>(rec)[r * scale_row_floats + b] = scale;
    if (w.zp != nullptr) {
      rec[rec_scale_bytes + r * bpt + b] = static_cast<unsigned char>(zp);
    }
  }
}

} // namespace


MetaGeometry MetaGeometryOf(const WeightView &w) {
  MetaGeometry geo{};
  if (w.bits != 4 || w.block_size < 32 || w.block_size > 1024 || (w.row_bytes % 16) != 0 ||
      GetEncodeTiled() == nullptr) {
    return geo; // unsupported: bytes == 0
  }
  // a task covers 2048 k of 16 rows (16 KB of packed weights): 64 / 32 / 16 / 8 ... blocks
  int bpt = 2048 / w.block_size;
  geo.bpt = bpt;
  geo.slices = (w.n_blocks + bpt - 1) / bpt;
  geo.scale_row_floats = bpt + (((bpt * 4) % 128) == 0 ? 4 : 0);
  geo.rec_scale_bytes = 8 * geo.scale_row_floats * 4;
  geo.rec_bytes = geo.rec_scale_bytes + (w.zp != nullptr ? 8 * bpt : 0);
  geo.half_tiles = static_cast<int>((w.n + 7) / 8);
  geo.bytes = static_cast<std::size_t>(geo.half_tiles) * geo.slices * geo.rec_bytes;
  return geo;
}

bool LaunchPrepareMeta(const WeightView &w, unsigned char *meta, cudaStream_t stream) {
  const MetaGeometry geo = MetaGeometryOf(w);
  if (geo.bytes == 0 || meta == nullptr) {
    return false;
  }
  const std::int64_t records = static_cast<std::int64_t>(geo.half_tiles) * geo.slices;
  std::int64_t blocks = (records * 8 * geo.bpt + 255) / 256;
  if (blocks > 148 * 8) {
    blocks = 148 * 8;
  }
  nbits_prepare_meta_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      w, geo.bpt, geo.scale_row_floats, geo.half_tiles, geo.rec_bytes, geo.rec_scale_bytes, meta, records);
  if (cudaGetLastError() != cudaSuccess) {
    return false;
  }
  CountLaunch();
  return true;
}

const char *LaunchGemvMma(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                          int *status_word, cudaStream_t stream, int sm_count, const GatherTail *tail) {
  const MetaGeometry geo = MetaGeometryOf(w);
  if (geo.bytes == 0 || w.meta == nullptr || m < 1 || (reinterpret_cast<std::uintptr_t>(w.b) & 15u) != 0) {
    return nullptr;
  }
  MmaParams p{};
  p.w = w;
  p.a = a;
  p.m_total = static_cast<int>(m);
  p.out = out;
  p.status = status_word;
  p.magic = 0x64006400u;
  if (tail != nullptr) {
    p.tail = *tail;
  }
  p.half_tiles = geo.half_tiles;
  p.bpt = geo.bpt;
  p.slices = geo.slices;
  p.rec_bytes = geo.rec_bytes;
  p.rec_scale_bytes = geo.rec_scale_bytes;
  p.slice_b_bytes = geo.bpt * w.block_size / 2;
  p.sg_per_task = geo.bpt * w.block_size / 128;
  int nb_sg_log2 = 0;
  if (w.block_size >= 128) {
    p.sg_per_block = w.block_size / 128;
  } else {
    p.sg_per_block = 1;
    nb_sg_log2 = Log2Of(128 / w.block_size);
  }
  // tokens per pass: columns = tokens * blocks-per-supergroup * 2 pieces <= 8
  int tokens_per_pass = kMaxTokens >> nb_sg_log2;
  if (m > 16 || tokens_per_pass < 1) {
    return nullptr;
  }
  if (tokens_per_pass > m) {
    tokens_per_pass = static_cast<int>(m);
  }
  p.tokens_per_pass = tokens_per_pass;
  p.k_pad = p.slices * p.sg_per_task * 128;
  if (p.k_pad < w.k || (p.sg_per_task % 4) != 0) {
    return nullptr;
  }
  p.act_row_bytes = p.k_pad * 2 + 64; // 64: bank spread between the two piece rows
  // Whole-row tasks when a row is exactly one or two slices long (K = 2048 or 4096): 16 rows are
  // then one contiguous copy of 16 or 32 KB (13 % faster than sliced boxes on K = 4096).
  p.full_rows = (w.row_bytes == p.slices * p.slice_b_bytes && p.slices <= 2 &&
                 w.row_bytes >= 1024) ? 1 : 0;
  if (p.full_rows != 0) {
    p.row_stride = w.row_bytes;
    p.weight_bytes = 16 * w.row_bytes;
    p.slot_bytes = (p.weight_bytes + p.slices * 2 * p.rec_bytes + 127) & ~127;
  } else {
    p.row_stride = p.slice_b_bytes;
    p.weight_bytes = 16 * p.slice_b_bytes;
    p.slot_bytes = (p.weight_bytes + 2 * p.rec_bytes + 127) & ~127;
  }
  const size_t fixed = static_cast<size_t>(2 * tokens_per_pass) * p.act_row_bytes + kZeroBytes +
                       (kMaxTokens + 2 * kWarps) * sizeof(float) + kPairs * 32 * sizeof(float2) +
                       2 * kMaxSlots * sizeof(std::uint64_t) + kMaxSlots * sizeof(int) + 128;
  const size_t limit = 227 * 1024 - 128; // the most a CTA can ask for, less the alignment slack
  if (fixed + 2 * static_cast<size_t>(p.slot_bytes) > limit) {
    return nullptr;
  }
  int slots = static_cast<int>((limit - fixed) / p.slot_bytes);
  if (slots > kMaxSlots) {
    slots = kMaxSlots;
  }
  // four producers need a ring that is a multiple of four deep (see the producer loop)
  const int wanted_producers = WantedProducers(1);
  if (wanted_producers > 1 && slots >= wanted_producers) {
    slots -= slots % wanted_producers;
    p.producers = wanted_producers;
  } else {
    p.producers = 1;
  }
  p.num_slots = slots;
  const size_t smem = static_cast<size_t>(slots) * p.slot_bytes + fixed + 128; // + alignment slack

  int ctas = sm_count > 0 ? sm_count : 148;
  const int tiles = (geo.half_tiles + 1) / 2;
  if (ctas > tiles) {
    ctas = tiles;
  }
  CUtensorMap map_b;
  if (!EncodeMap2D(&map_b, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, w.b, static_cast<std::uint64_t>(w.row_bytes / 4),
                   static_cast<std::uint64_t>(w.n), static_cast<std::uint64_t>(w.row_bytes),
                   static_cast<std::uint32_t>(p.slice_b_bytes / 4), 16, CU_TENSOR_MAP_SWIZZLE_NONE)) {
    return nullptr;
  }
  dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>((m + tokens_per_pass - 1) / tokens_per_pass), 1);
  cudaError_t err = cudaErrorInvalidValue;
#define MNB_MMA_CASE(LOG2_, BIG_, ZP_)                                                           \
  if (nb_sg_log2 == LOG2_ && (p.sg_per_block > 1) == BIG_ && (w.zp != nullptr) == ZP_) {         \
    auto kernel = nbits_gemv_mma_kernel<LOG2_, BIG_, ZP_>;                                       \
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,              \
                               static_cast<int>(smem));                                          \
    if (err == cudaSuccess) {                                                                    \
      cudaLaunchConfig_t config = {};                                                            \
      config.gridDim = grid;                                                                     \
      config.blockDim = dim3(kThreads, 1, 1);                                                    \
      config.dynamicSmemBytes = smem;                                                            \
      config.stream = stream;                                                                    \
      cudaLaunchAttribute attribute[1];                                                          \
      attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                      \
      attribute[0].val.programmaticStreamSerializationAllowed = 1;                               \
      config.attrs = attribute;                                                                  \
      config.numAttrs = DependentLaunchHint() ? 1 : 0;                                                                     \
      err = cudaLaunchKernelEx(&config, kernel, map_b, p);                                       \
    }                                                                                            \
  }
  MNB_MMA_CASE(0, false, true)
  MNB_MMA_CASE(0, false, false)
  MNB_MMA_CASE(0, true, true)
  MNB_MMA_CASE(0, true, false)
  MNB_MMA_CASE(1, false, true)
  MNB_MMA_CASE(1, false, false)
  MNB_MMA_CASE(2, false, true)
  MNB_MMA_CASE(2, false, false)
#undef MNB_MMA_CASE
  if (err != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return "nbits_gemv_mma_kernel";
}

} // namespace mnb
