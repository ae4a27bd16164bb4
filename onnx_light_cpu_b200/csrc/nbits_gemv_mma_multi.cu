// Decode path of MatMulNBits on warp-level tensor-core MMA for several tokens per pass over the
// weights. Same arithmetic as the single-column-tile kernel in nbits_gemv_mma.cu (weights as the
// MMA "A" operand in fp16, every activation row scaled by a power of two and split into two
// fp16 pieces, fp32 accumulators restarted per quantization block; columns of a 16x8 tile =
// (token, block-inside-supergroup, piece)), with NT column tiles sharing each dequantized
// weight fragment: 8 / 4 / 2 tokens per pass for NT = 2 and block sizes >= 128 / 64 / 32, twice
// that for NT = 4, where that kernel would need one pass per 4 / 2 / 1 tokens.
//
// Data movement: persistent CTA per SM; four producer lanes fill a ring of task slots - one 2-D
// tiled TMA load of 16 weight rows x 2048 k plus one bulk copy of that task's scales / zero
// points from the prepared, task-major side array - completed on mbarriers. All sixteen consumer
// warps work on the same task, one 128-k supergroup each: every warp is busy whatever the
// number of row tiles of the CTA, and the ring only has to cover the memory latency. Once per
// row tile the sixteen partial sums are added through shared memory by NT warps (rotating with
// the tile index) while the others go on. All waits on data are bounded.
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


constexpr int kWarps = 16;                // consumer warps = 128-k supergroups of a task
constexpr int kConsumerThreads = kWarps * 32;
// A single thread cannot keep enough tile loads in flight for the full memory bandwidth (one
// issuing thread measured 4.4 TB/s with 16 KB boxes whatever the ring depth, four 6.7 TB/s):
// four producer warps issue the tasks round-robin.
constexpr int kProducers = 4;
constexpr int kThreads = (kWarps + kProducers) * 32;
constexpr int kMaxSlots = 16;
constexpr int kMaxTokens = 16;            // most activation rows handled per CTA pass
constexpr int kTaskK = kWarps * 128;      // k per task

struct MultiParams {
  WeightView w;
  const float *a;
  int m_total;
  OutputView out;
  int *status;
  int half_tiles;       // ceil(n / 8)
  int bpt;              // quantization blocks per task
  int slices;           // tasks per row tile = ceil(n_blocks / bpt)
  int slice_b_bytes;    // packed bytes of one row inside a task
  int sg_per_block;     // supergroups per quantization block (block_size >= 128), else 1
  int rec_bytes;        // bytes of one prepared meta record (bpt blocks x 8 rows)
  int rec_scale_bytes;  // scale part of a record
  int slot_bytes;
  int num_slots;
  int producers;       // producer warps in use: min(kProducers, num_slots), see the producer loop
  int act_row_bytes;    // bytes between activation piece rows in shared memory
  int k_pad;            // activation positions per piece row (all tasks, zero beyond K)
  int tokens_per_pass;  // activation rows per grid.y pass: NT * (4 / blocks-per-supergroup)
  int token_rows;       // activation rows staged in shared memory: min(M, tokens_per_pass)
  std::uint32_t magic;  // 0x64006400, passed at run time so that it stays in a register
  GatherTail tail;      // gathered step: the last CTA publishes this rank's flags (ranks == 0: none)
};

// NB_SG_LOG2: log2 of quantization blocks per 128-k supergroup (block 128+: 0, 64: 1, 32: 2).
// NT: 8-column tiles of tokens per pass; a column tile holds 4 >> NB_SG_LOG2 tokens.
template <int NB_SG_LOG2, bool HAS_ZP, int NT>
__global__ void __launch_bounds__(kThreads, 1)
    nbits_gemv_mma_multi_kernel(const __grid_constant__ CUtensorMap map_b, const MultiParams p) {
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  // keep the pointer in the shared address space (no integer round trip) while aligning it
  unsigned char *smem_raw = smem_dyn + ((128u - (ptx::SmemAddr(smem_dyn) & 127u)) & 127u);
  // layout: [slots][activation piece rows: 2 per token, then a row of zeros][per-token 2^-e]
  //         [amax scratch][partial sums: 2 x kWarps x NT x 32 lanes][barriers]
  unsigned char *slots = smem_raw;
  unsigned char *act = smem_raw + static_cast<size_t>(p.num_slots) * p.slot_bytes;
  float *inv_scale = reinterpret_cast<float *>(act + (2 * p.token_rows + 1) * p.act_row_bytes);
  float *scratch = inv_scale + kMaxTokens;          // [2][kWarps], alternating with the token index
  float2 *partial = reinterpret_cast<float2 *>(scratch + 2 * kWarps); // [2][kWarps][NT][32]
  std::uint64_t *full_bar = reinterpret_cast<std::uint64_t *>(partial + 2 * kWarps * NT * 32);
  std::uint64_t *empty_bar = full_bar + kMaxSlots;

  constexpr int kNbSg = 1 << NB_SG_LOG2;
  constexpr int kTileTokens = 4 >> NB_SG_LOG2; // tokens per column tile
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
    // One lane per producer warp issues, per task, one 2-D tiled TMA load of the weight tile
    // (16 rows x the slice; rows past the matrix end are zero-filled) and one bulk copy of the
    // task's scale / zero-point records (two consecutive half tiles of the same slice).
    // Producer j takes tasks j, j + kProducers, ...
    const int producer = warp - kWarps;
    if (producer == 0 && lane == 0) {
      for (int s = 0; s < p.num_slots; ++s) {
        ptx::MbarInit(&full_bar[s], 1);
        ptx::MbarInit(&empty_bar[s], kWarps);
      }
      ptx::FenceMbarInit();
    }
    // barriers initialised: the producers go on at once, the consumers join barrier 10 after
    // staging the activations
    asm volatile("bar.sync 11, %0;" ::"n"(kProducers * 32) : "memory");
    asm volatile("bar.arrive 10, %0;" ::"n"(kThreads) : "memory");
    if (lane == 0) {
      ptx::PrefetchTensorMap(&map_b);
      const int total = n_tiles * p.slices;
      const std::uint32_t box_bytes = 16u * static_cast<std::uint32_t>(p.slice_b_bytes);
      const int x_step = p.slice_b_bytes / 4;
      const std::int64_t meta_slice_stride = static_cast<std::int64_t>(p.half_tiles) * p.rec_bytes;
      bool ok = true;
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
        if (round != 0 && !ptx::MbarWait(&empty_bar[slot], (round & 1u) ^ 1u)) {
          ReportStatus(p.status, kDeviceTimeoutEmptyBarrier);
          ok = false;
          break;
        }
        const int h0 = h_begin + 2 * tile;
        const unsigned char *meta_src =
            p.w.meta + static_cast<std::int64_t>(h0) * p.rec_bytes + s * meta_slice_stride;
        const std::uint32_t meta_bytes = (h0 + 1 < p.half_tiles ? 2u : 1u) * static_cast<std::uint32_t>(p.rec_bytes);
        unsigned char *dst = slots + static_cast<size_t>(slot) * p.slot_bytes;
        ptx::MbarArriveExpectTx(&full_bar[slot], box_bytes + meta_bytes);
        ptx::TmaLoad2D(dst, &map_b, s * x_step, h0 * 8, &full_bar[slot]);
        ptx::BulkLoad(dst + box_bytes, meta_src, meta_bytes, &full_bar[slot]);
      }
      // stay until every copy this lane issued has been consumed (bounded), so none lands after exit
      const int first = total - p.num_slots < 0 ? 0 : total - p.num_slots;
      for (int i = first; i < total && ok; ++i) {
        if (producer < p.producers && (i % p.producers) == producer &&
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
  unsigned char *zero_row = act + 2 * p.token_rows * p.act_row_bytes;
  for (int i = tid; i < (p.act_row_bytes >> 4); i += kConsumerThreads) {
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
  // role of this lane's column (g) in the activation fragment of column tile nt
  const int pc_b = g >> 1;
  const int piece_b = g & 1;
  const int blk_b = pc_b & (kNbSg - 1);
  // block-in-supergroup of this lane's own codes: lane t holds k = 32t .. 32t+31
  const int tb = NB_SG_LOG2 == 2 ? t : (NB_SG_LOG2 == 1 ? t >> 1 : 0);
  // lanes whose column takes no part read a row of zeros, so the loads need no predicate
  const unsigned char *act_lane[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int m_b = nt * kTileTokens + (pc_b >> NB_SG_LOG2);
    const bool b_active = m_b < tokens && blk_b == tb;
    act_lane[nt] = (b_active ? act + (2 * m_b + piece_b) * p.act_row_bytes : zero_row) + t * 16 + warp * 256;
  }
  // role of this lane's accumulator columns (2t, 2t+1)
  const int blk_d = t & (kNbSg - 1);

  const std::uint32_t magic = p.magic;
  const std::uint32_t sixteenth = 0x2c002c00u;  // fp16 1/16 twice
  const std::uint32_t plus960 = 0x63806380u;    // fp16 960 twice
  const std::uint32_t default_offs = 0x64086408u; // fp16 1024 + 8 twice
  const int box_bytes = 16 * p.slice_b_bytes;
  // meta record: float scale[8 rows][row floats] (rows padded where they would share a bank),
  // then uint8 zp[8 rows][bpt]
  const int scale_row_bytes = p.rec_scale_bytes / 8;
  // this warp's supergroup of every task: block index (inside the task) of the lane's codes and
  // of the lane's accumulator columns
  const int blk_codes = NB_SG_LOG2 == 0 ? warp / p.sg_per_block : warp * kNbSg + tb;
  const int blk_acc = NB_SG_LOG2 == 0 ? blk_codes : warp * kNbSg + blk_d;
  const int weight_off = g * p.slice_b_bytes + warp * 64 + t * 16;
  const int act_task_bytes = kWarps * 256; // activation bytes of one task in a piece row

  int task = 0;
  int slot = 0;
  std::uint32_t round = 0;
  bool dead = false; // a bounded wait gave up: skip the math but keep the barrier protocol
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int h0 = h_begin + 2 * tile;
    const std::int64_t row0 = static_cast<std::int64_t>(h0) * 8;
    float acc0[NT], acc1[NT]; // rows g and g + 8, accumulator column pair t of each column tile
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      acc0[nt] = 0.0f;
      acc1[nt] = 0.0f;
    }

    for (int s = 0; s < p.slices; ++s, ++task) {
      if (!dead && !ptx::MbarWait(&full_bar[slot], round & 1u)) {
        ReportStatus(p.status, kDeviceTimeoutFullBarrier);
        dead = true;
      }
      if (!dead) {
        const unsigned char *sb = slots + static_cast<size_t>(slot) * p.slot_bytes;
        const uint4 q0 = *reinterpret_cast<const uint4 *>(sb + weight_off);
        const uint4 q1 = *reinterpret_cast<const uint4 *>(sb + weight_off + 8 * p.slice_b_bytes);
        const unsigned char *meta0 = sb + box_bytes;       // rows 0..7
        const unsigned char *meta1 = meta0 + p.rec_bytes;  // rows 8..15
        const float s0 = reinterpret_cast<const float *>(meta0 + g * scale_row_bytes)[blk_acc];
        const float s1 = reinterpret_cast<const float *>(meta1 + g * scale_row_bytes)[blk_acc];
        std::uint32_t offs0 = default_offs; // (1024 + zp) twice
        std::uint32_t offs1 = default_offs;
        if constexpr (HAS_ZP) {
          const std::uint32_t z0 = meta0[p.rec_scale_bytes + g * p.bpt + blk_codes];
          const std::uint32_t z1 = meta1[p.rec_scale_bytes + g * p.bpt + blk_codes];
          offs0 = __byte_perm(z0, 0x64646464u, 0x4040);
          offs1 = __byte_perm(z1, 0x64646464u, 0x4040);
        }
        // the weights are in registers: hand the slot back before the arithmetic
        __syncwarp();
        if (lane == 0) {
          ptx::MbarArrive(&empty_bar[slot]);
        }
        const std::uint32_t offs0_16 = Hsub2(plus960, offs0); // -(64 + zp)
        const std::uint32_t offs1_16 = Hsub2(plus960, offs1);
        const std::uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w};
        const std::uint32_t w1[4] = {q1.x, q1.y, q1.z, q1.w};
        float da[NT][4], db[NT][4];
        const int act_off = s * act_task_bytes;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          std::uint32_t pa[4], pb[4];
          Dequant8(w0[i], magic, offs0, offs0_16, sixteenth, pa);
          Dequant8(w1[i], magic, offs1, offs1_16, sixteenth, pb);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4 bf = *reinterpret_cast<const uint4 *>(act_lane[nt] + act_off + i * 64);
            // two accumulator sets halve the dependent chain of MMAs
            if (i == 0) {
              MmaF16Zero(da[nt], pa[0], pb[0], pa[1], pb[1], bf.x, bf.y);
              MmaF16Zero(db[nt], pa[2], pb[2], pa[3], pb[3], bf.z, bf.w);
            } else {
              MmaF16(da[nt], pa[0], pb[0], pa[1], pb[1], bf.x, bf.y);
              MmaF16(db[nt], pa[2], pb[2], pa[3], pb[3], bf.z, bf.w);
            }
          }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          acc0[nt] = fmaf(s0, (da[nt][0] + da[nt][1]) + (db[nt][0] + db[nt][1]), acc0[nt]);
          acc1[nt] = fmaf(s1, (da[nt][2] + da[nt][3]) + (db[nt][2] + db[nt][3]), acc1[nt]);
        }
      }
      if (++slot == p.num_slots) {
        slot = 0;
        ++round;
      }
    }

    // ---- sum over the sixteen warps -----------------------------------------------------------
    // Buffer b = tile % 2. Named barriers 2 + b ("partials of this tile written") and 4 + b
    // ("buffer read, may be overwritten"), all consumer threads each: the NT reducing warps of
    // a tile wait on the first and arrive on the second, everybody else the other way round.
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
    float2 *mine = partial + ((b * kWarps + warp) * NT) * 32 + lane;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      mine[nt * 32] = make_float2(acc0[nt], acc1[nt]);
    }
    if (!reduces) {
      asm volatile("bar.arrive %0, %1;" ::"r"(2 + b), "n"(kConsumerThreads) : "memory");
    } else {
      asm volatile("bar.sync %0, %1;" ::"r"(2 + b), "n"(kConsumerThreads) : "memory");
      const int nt = (warp - reducer0) & (kWarps - 1);
      const float2 *column = partial + (b * kWarps * NT + nt) * 32 + lane;
      float2 total = column[0];
#pragma unroll
      for (int w = 1; w < kWarps; ++w) {
        const float2 v = column[w * NT * 32];
        total.x += v.x;
        total.y += v.y;
      }
      if (tile + 2 < n_tiles) {
        asm volatile("bar.arrive %0, %1;" ::"r"(4 + b), "n"(kConsumerThreads) : "memory");
      }
      // blocks of one supergroup sit in neighbouring lanes of the quad: add them up
      if (NB_SG_LOG2 >= 1) {
        total.x += __shfl_xor_sync(0xffffffffu, total.x, 1);
        total.y += __shfl_xor_sync(0xffffffffu, total.y, 1);
      }
      if (NB_SG_LOG2 >= 2) {
        total.x += __shfl_xor_sync(0xffffffffu, total.x, 2);
        total.y += __shfl_xor_sync(0xffffffffu, total.y, 2);
      }
      const int m_d = nt * kTileTokens + (t >> NB_SG_LOG2);
      if (blk_d == 0 && m_d < tokens) {
        const float undo = inv_scale[m_d];
        const std::int64_t m = m_base + m_d;
        const std::int64_t r_lo = row0 + g;
        const std::int64_t r_hi = row0 + g + 8;
        if (r_lo < row_limit) {
          const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + r_lo) : 0.0f;
          StoreOutput(p.out, m * p.out.ld + p.out.col_offset + r_lo, fmaf(total.x, undo, bias));
        }
        if (r_hi < row_limit) {
          const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + r_hi) : 0.0f;
          StoreOutput(p.out, m * p.out.ld + p.out.col_offset + r_hi, fmaf(total.y, undo, bias));
        }
      }
    }
  }
  if (p.tail.ranks > 0) {
    // gathered step: the arithmetic stored locally only; now this CTA's rows go to the peers
    asm volatile("bar.sync 12, %0;" ::"n"(kConsumerThreads) : "memory");
    PushRowsToPeers(p.out, p.tail, m_base, tokens, static_cast<std::int64_t>(h_begin) * 8, row_limit, tid, kConsumerThreads);
    PublishWhenGridDone(p.tail, tid, kConsumerThreads, 12, gridDim.x * gridDim.y, p.status);
  }
}

} // namespace

const char *LaunchGemvMmaMulti(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                               int *status_word, cudaStream_t stream, int sm_count, const GatherTail *tail) {
  const MetaGeometry geo = MetaGeometryOf(w);
  if (geo.bytes == 0 || w.meta == nullptr || m < 1 || (reinterpret_cast<std::uintptr_t>(w.b) & 15u) != 0 ||
      geo.bpt * w.block_size != kTaskK) {
    return nullptr;
  }
  MultiParams p{};
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
  p.slice_b_bytes = kTaskK / 2;
  int nb_sg_log2 = 0;
  if (w.block_size >= 128) {
    p.sg_per_block = w.block_size / 128;
  } else {
    p.sg_per_block = 1;
    nb_sg_log2 = Log2Of(128 / w.block_size);
  }
  if (m > 16) {
    return nullptr;
  }
  p.k_pad = p.slices * kTaskK;
  if (p.k_pad < w.k) {
    return nullptr;
  }
  p.act_row_bytes = p.k_pad * 2 + 64; // 64: bank spread between the two piece rows
  p.slot_bytes = (16 * p.slice_b_bytes + 2 * p.rec_bytes + 127) & ~127;
  // column tiles per pass: as many as the tokens need (1, 2 or 4) and shared memory allows,
  // while at least three ring slots remain
  const int tile_tokens = 4 >> nb_sg_log2;
  const size_t limit = 225 * 1024;
  int nt = 4;
  while (nt > 1 && (nt / 2) * tile_tokens >= m) {
    nt /= 2;
  }
  size_t fixed = 0;
  for (;; nt /= 2) {
    p.tokens_per_pass = nt * tile_tokens;
    p.token_rows = m < p.tokens_per_pass ? static_cast<int>(m) : p.tokens_per_pass;
    fixed = static_cast<size_t>(2 * p.token_rows + 1) * p.act_row_bytes +
            (kMaxTokens + 2 * kWarps) * sizeof(float) + 2 * kWarps * nt * 32 * sizeof(float2) +
            2 * kMaxSlots * sizeof(std::uint64_t) + 128;
    if (fixed + 3 * static_cast<size_t>(p.slot_bytes) <= limit) {
      break;
    }
    if (nt == 1) {
      if (fixed + 2 * static_cast<size_t>(p.slot_bytes) > limit) {
        return nullptr;
      }
      break;
    }
  }
  if (nt < 2) {
    return nullptr; // one column tile: the kernel in nbits_gemv_mma.cu is the faster one
  }
  int slots = static_cast<int>((limit - fixed) / p.slot_bytes);
  if (slots > kMaxSlots) {
    slots = kMaxSlots;
  }
  p.num_slots = slots;
  p.producers = slots < WantedProducers(kProducers) ? slots : WantedProducers(kProducers);
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
  dim3 grid(static_cast<unsigned>(ctas),
            static_cast<unsigned>((m + p.tokens_per_pass - 1) / p.tokens_per_pass), 1);
  cudaError_t err = cudaErrorInvalidValue;
#define MNB_MMA_CASE(LOG2_, ZP_, NT_)                                                            \
  if (nb_sg_log2 == LOG2_ && (w.zp != nullptr) == ZP_ && nt == NT_) {                            \
    auto kernel = nbits_gemv_mma_multi_kernel<LOG2_, ZP_, NT_>;                                        \
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
      config.numAttrs = DependentLaunchHint() ? 1 : 0;                                            \
      err = cudaLaunchKernelEx(&config, kernel, map_b, p);                                       \
    }                                                                                            \
  }
#define MNB_MMA_CASES(LOG2_)                                                                     \
  MNB_MMA_CASE(LOG2_, true, 1)                                                                   \
  MNB_MMA_CASE(LOG2_, false, 1)                                                                  \
  MNB_MMA_CASE(LOG2_, true, 2)                                                                   \
  MNB_MMA_CASE(LOG2_, false, 2)                                                                  \
  MNB_MMA_CASE(LOG2_, true, 4)                                                                   \
  MNB_MMA_CASE(LOG2_, false, 4)
  MNB_MMA_CASES(0)
  MNB_MMA_CASES(1)
  MNB_MMA_CASES(2)
#undef MNB_MMA_CASES
#undef MNB_MMA_CASE
  if (err != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return "nbits_gemv_mma_multi_kernel";
}

} // namespace mnb
