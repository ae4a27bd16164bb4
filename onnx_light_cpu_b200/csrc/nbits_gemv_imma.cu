// Decode path of MatMulNBits for one or two activation rows on integer tensor-core MMA, with
// fp32-grade accuracy (accuracy_level 0).
//
// Why integers for a float GEMV: turning a 4-bit code into fp16 costs more than one instruction
// per code (mask, magic-number OR, subtract), and at M = 1 the instruction issue rate of the SM,
// not HBM, is what the fp16 form of this kernel runs into. As an unsigned byte a code costs
// 3/8 of an instruction (two masks and a shift per word of eight codes) and feeds
// mma.sync.m16n8k32 directly.
//
// Exactness. Each activation row is scaled so that its largest magnitude becomes kDigitRange and
// rounded to a 22-bit integer n = 16384 d0 + 128 d1 + d2 with balanced base-128 digits (d1, d2 in
// [-64, 63], |d0| <= 123). The three digits of a token occupy three MMA columns (two tokens = six
// of the eight columns). Code x digit products are exact in the int32 accumulator, which is
// restarted per quantization block; zero points are taken out afterwards with the digit sums of
// the block (D - zp * sum, the correction of
// onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:208-223), or, when the node has none,
// the codes enter as the signed bytes 16 (q - 8). Block results are converted to float (exact:
// below 2^24) and combined in fp32: acc[digit] += scale * float(dot). What is lost is the
// rounding of the activation to 22 bits of its row maximum (|error| <= max|a| / 4e6 per element),
// well inside the 1e-5 bar of the fp32 decode paths.
//
// Data movement is that of the fp16 tensor-core decode kernel: persistent CTA per SM, a producer
// lane fills a ring of task slots with bulk (TMA) copies of 16 weight rows (whole rows when a row
// is one or two tasks long, else one 2048-k slice through a 2-D tiled box) plus the prepared
// scale / zero-point records; warp pairs own 16-row tiles. All waits are bounded.
//
// Takes block_size 128 ... 1024 (a 128-k supergroup never straddles two quantization blocks, so
// the four lanes of a quad may hold codes 32 k apart). Smaller blocks stay on the fp16 kernel.
//
// Conventions: packed-INT4 nibble order of
// onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:60-93; "stream B once, split N"
// partition of onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258.

#include "nbits_common.cuh"
#include "nbits_ptx.cuh"
#include "nbits_tma.cuh"

#include <cstdint>
#include <cstdlib>

namespace mnb {
namespace {

constexpr int kPairs = 8;                 // 16-row tiles in flight per CTA
constexpr int kWarps = 2 * kPairs;        // consumer warps: two per tile, alternating halves of K
constexpr int kConsumerThreads = kWarps * 32;
constexpr int kProducers = 4;             // producer warps present (one issuing lane each; one used by default)
constexpr int kThreads = (kWarps + kProducers) * 32;
constexpr int kMaxSlots = 16;
constexpr int kMaxTokens = 2;             // activation rows per CTA pass: 3 digit columns each
constexpr int kDigits = 3;
constexpr int kUnroll = 4;                // supergroups per loop round
constexpr int kZeroBytes = 128;           // what the lanes of unused MMA columns read
constexpr float kDigitRange = 2.0e6f;     // the row maximum maps to this integer (< 123 * 16384)

struct ImmaParams {
  WeightView w;
  const float *a;
  int m_total;
  OutputView out;
  int *status;
  int half_tiles;       // ceil(n / 8)
  int bpt;              // quantization blocks per task
  int slices;           // tasks per row tile
  int slice_b_bytes;    // packed bytes of one row inside a task
  int sg_per_task;      // 128-k supergroups per task
  int sg_per_block;     // supergroups per quantization block
  int rec_bytes;        // bytes of one prepared meta record (bpt blocks x 8 rows)
  int rec_scale_bytes;  // scale part of a record
  int slot_bytes;
  int num_slots;
  int full_rows;        // 1: a task is 16 whole weight rows, one contiguous bulk copy; 0: one slice
  int row_stride;       // bytes between weight rows inside a slot
  int weight_bytes;     // bytes of the weight part of a slot
  int producers;        // producer warps in use (num_slots is a multiple of it)
  int act_row_bytes;    // bytes between digit rows in shared memory (k_pad + 16: bank spread)
  int k_pad;            // activation positions per digit row (all tasks, zero beyond K)
  int tokens_per_pass;  // activation rows per grid.y pass (1 or 2)
  int blocks_pad;       // quantization blocks covered by k_pad
};

// D (int32, 16 x 8) += A (16 x 32 bytes, weights) * B (32 x 8 signed bytes, activation digits).
template <bool SIGNED_A>
__device__ __forceinline__ void Imma(int (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                     std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  if constexpr (SIGNED_A) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// Same with a zero accumulator input: starts a fresh block sum.
template <bool SIGNED_A>
__device__ __forceinline__ void ImmaZero(int (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                         std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  if constexpr (SIGNED_A) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
  } else {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
  }
}

// The two MMA operands made of one word of eight codes: even codes (low nibbles) and odd codes
// (high nibbles), one byte each. With zero points the bytes are the codes themselves; without,
// the signed bytes 16 (q - 8), the factor 16 being undone in the epilogue.
template <bool SIGNED_A>
__device__ __forceinline__ void Split8(std::uint32_t w, std::uint32_t &even, std::uint32_t &odd) {
  if constexpr (SIGNED_A) {
    even = ((w << 4) & 0xf0f0f0f0u) ^ 0x80808080u;
    odd = (w & 0xf0f0f0f0u) ^ 0x80808080u;
  } else {
    even = w & 0x0f0f0f0fu;
    odd = (w >> 4) & 0x0f0f0f0fu;
  }
}

// Stages `tokens` (1 or 2) activation rows as three signed digit rows each and, when the node has
// zero points, the per-block digit sums. Row (3 * token + digit) starts at
// act + (3 * token + digit) * act_row_bytes. Byte order inside a row: supergroup-major (128 k), then
// the quad lane t = (k % 128) / 32 that holds the codes, the word i = (k % 32) / 8 inside its
// 16-byte load, then the eight k of a word with the even ones first (the order Split8 produces):
// position = (k & ~7) + 4 * (k & 1) + (k & 7) / 2. undo[token] is
// the factor that takes the integer result back (NaN for a row with a non-finite entry: every
// output of that row is then NaN). The consumer warps are split evenly between the tokens; a
// thread owns whole 8-k words and keeps up to kHeld of them in registers between the maximum
// and the rounding, so A is read once for K <= kHeld * 8 * threads per token.
// sums[block * 8 + column] (int32) is written only when `with_sums`. Uses named barrier 9 with
// kConsumerThreads participants, twice; every consumer thread must call it.
__device__ __forceinline__ void StageDigits(const float *a_rows, int tokens, int k, int k_pad, int block_size,
                                            int blocks_pad, unsigned char *act, int act_row_bytes, float *undo,
                                            float *scratch, int *sums, bool with_sums, int tid) {
  constexpr int kHeld = 4;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int warps_per_token = kWarps / tokens;
  const int token = warp / warps_per_token;
  const int group_threads = warps_per_token * 32;
  const int tg = tid - token * group_threads;
  const int words_total = k_pad >> 3;
  const float *src = a_rows + static_cast<std::int64_t>(token) * k;
  const bool fast = (reinterpret_cast<std::uintptr_t>(src) & 15u) == 0 && (k & 7) == 0;

  auto load_word = [&](int word, float (&x)[8]) {
    const int k0 = word << 3;
    if (fast) {
      float4 lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi = lo;
      if (k0 < k) {
        lo = __ldg(reinterpret_cast<const float4 *>(src + k0));
        hi = __ldg(reinterpret_cast<const float4 *>(src + k0 + 4));
      }
      x[0] = lo.x, x[1] = lo.y, x[2] = lo.z, x[3] = lo.w;
      x[4] = hi.x, x[5] = hi.y, x[6] = hi.z, x[7] = hi.w;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        x[e] = (k0 + e < k) ? __ldg(src + k0 + e) : 0.0f;
      }
    }
  };

  float v[kHeld][8];
  float amax = 0.0f;
  bool bad = false; // a NaN in the row (fmaxf would drop it)
#pragma unroll
  for (int j = 0; j < kHeld; ++j) {
    const int word = tg + j * group_threads;
    if (word < words_total) {
      load_word(word, v[j]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[j][e] = 0.0f;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kHeld; ++j) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      amax = fmaxf(amax, fabsf(v[j][e]));
      bad = bad || (v[j][e] != v[j][e]);
    }
  }
  for (int word = tg + kHeld * group_threads; word < words_total; word += group_threads) {
    float x[8];
    load_word(word, x);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      amax = fmaxf(amax, fabsf(x[e]));
      bad = bad || (x[e] != x[e]);
    }
  }
  if (bad) {
    amax = __int_as_float(0x7f800000); // treated like an infinite entry below
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  }
  if (lane == 0) {
    scratch[warp] = amax;
  }
  asm volatile("bar.sync 9, %0;" ::"n"(kConsumerThreads) : "memory");
  amax = scratch[token * warps_per_token];
  for (int i = 1; i < warps_per_token; ++i) {
    amax = fmaxf(amax, scratch[token * warps_per_token + i]);
  }
  const bool finite = amax < 3.0e38f;
  // rows of very small magnitude are lifted by an exact power of two first, so that the factor
  // below stays finite
  const float lift = amax < 1.0e-18f ? 1.8446744e19f /* 2^64 */ : 1.0f;
  const float lifted = amax * lift;
  const float up = (finite && lifted > 0.0f) ? kDigitRange / lifted : 0.0f; // applied to x * lift
  if (tg == 0) {
    undo[token] = finite ? (lifted / kDigitRange) / lift : __int_as_float(0x7fc00000);
  }
  unsigned char *row0 = act + (kDigits * token) * act_row_bytes;
  auto store_word = [&](int word, const float (&x)[8]) {
    std::uint32_t d0[2] = {0u, 0u}, d1[2] = {0u, 0u}, d2[2] = {0u, 0u};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      int n = __float2int_rn((x[e] * lift) * up);
      n = n > static_cast<int>(kDigitRange) ? static_cast<int>(kDigitRange)
                                            : (n < -static_cast<int>(kDigitRange) ? -static_cast<int>(kDigitRange) : n);
      const int low = ((n + 64) & 127) - 64;
      const int n1 = (n - low) >> 7;
      const int mid = ((n1 + 64) & 127) - 64;
      const int high = (n1 - mid) >> 7;
      const int pos = ((e & 1) << 2) + (e >> 1); // even k first
      const int shift = (pos & 3) * 8;
      d0[pos >> 2] |= static_cast<std::uint32_t>(high & 0xff) << shift;
      d1[pos >> 2] |= static_cast<std::uint32_t>(mid & 0xff) << shift;
      d2[pos >> 2] |= static_cast<std::uint32_t>(low & 0xff) << shift;
    }
    const int byte = word << 3;
    *reinterpret_cast<uint2 *>(row0 + byte) = make_uint2(d0[0], d0[1]);
    *reinterpret_cast<uint2 *>(row0 + act_row_bytes + byte) = make_uint2(d1[0], d1[1]);
    *reinterpret_cast<uint2 *>(row0 + 2 * act_row_bytes + byte) = make_uint2(d2[0], d2[1]);
  };
#pragma unroll
  for (int j = 0; j < kHeld; ++j) {
    const int word = tg + j * group_threads;
    if (word < words_total) {
      store_word(word, v[j]);
    }
  }
  for (int word = tg + kHeld * group_threads; word < words_total; word += group_threads) {
    float x[8];
    load_word(word, x);
    store_word(word, x);
  }
  asm volatile("bar.sync 9, %0;" ::"n"(kConsumerThreads) : "memory");
  if (with_sums) {
    // digit sums per (quantization block, MMA column); a block is a contiguous run of bytes
    const int columns = kDigits * tokens;
    for (int entry = tid; entry < blocks_pad * 8; entry += kConsumerThreads) {
      const int column = entry & 7;
      const int block = entry >> 3;
      int sum = 0;
      if (column < columns) {
        const uint4 *bytes =
            reinterpret_cast<const uint4 *>(act + column * act_row_bytes + block * block_size);
        for (int i = 0; i < (block_size >> 4); ++i) {
          const uint4 q = bytes[i];
          sum = __dp4a(static_cast<int>(q.x), 0x01010101, sum);
          sum = __dp4a(static_cast<int>(q.y), 0x01010101, sum);
          sum = __dp4a(static_cast<int>(q.z), 0x01010101, sum);
          sum = __dp4a(static_cast<int>(q.w), 0x01010101, sum);
        }
      }
      sums[entry] = sum;
    }
  }
}

// BIG_BLOCK: a quantization block spans several 128-k supergroups (block_size >= 256).
// HAS_ZP: the node has zero points (unsigned codes + correction); else signed codes 16 (q - 8).
template <bool BIG_BLOCK, bool HAS_ZP>
__global__ void __launch_bounds__(kThreads, 1)
    nbits_gemv_imma_kernel(const __grid_constant__ CUtensorMap map_b, const ImmaParams p) {
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  // keep the pointer in the shared address space (no integer round trip) while aligning it
  unsigned char *smem_raw = smem_dyn + ((128u - (ptx::SmemAddr(smem_dyn) & 127u)) & 127u);
  // layout: [slots][digit rows: 3 per token][zeros][digit sums][undo x4][amax scratch]
  //         [pair exchange: kPairs x 32 lanes x float4][barriers][slot tags]
  unsigned char *slots = smem_raw;
  unsigned char *act = smem_raw + static_cast<size_t>(p.num_slots) * p.slot_bytes;
  unsigned char *zero_row = act + kDigits * p.tokens_per_pass * p.act_row_bytes;
  int *sums = reinterpret_cast<int *>(zero_row + kZeroBytes);
  float *undo = reinterpret_cast<float *>(sums + p.blocks_pad * 8);
  float *scratch = undo + 4;
  float4 *pair_buf = reinterpret_cast<float4 *>(scratch + kWarps);
  std::uint64_t *full_bar = reinterpret_cast<std::uint64_t *>(pair_buf + kPairs * 32);
  std::uint64_t *empty_bar = full_bar + kMaxSlots;
  // task index currently assigned to each slot: a slot is used by different warps in successive
  // rounds and an mbarrier parity only tells neighbouring phases apart, so a consumer of round
  // >= 1 first waits until the producer has assigned ITS task to the slot
  volatile int *slot_task = reinterpret_cast<volatile int *>(empty_bar + kMaxSlots);

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
    // One lane per producer warp issues the copies of a task: the weight tile and the task's scale /
    // zero-point records. Producer j takes the tasks with index % producers == j; num_slots is a
    // multiple of the number of producers, so all rounds of a slot belong to the same producer.
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
        // one task per row tile: 16 whole rows are contiguous in memory, one large bulk copy
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
  // A (and Y) may be produced / still read by the previous kernel in the stream: from here on
  // the consumers depend on it. The producer warp above only touches the constant weights.
  ptx::GridDependencyWait();
  for (int i = tid; i < (kZeroBytes >> 4); i += kConsumerThreads) {
    reinterpret_cast<uint4 *>(zero_row)[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  StageDigits(p.a + static_cast<std::int64_t>(m_base) * p.w.k, tokens, static_cast<int>(p.w.k), p.k_pad,
              p.w.block_size, p.blocks_pad, act, p.act_row_bytes, undo, scratch, sums, HAS_ZP, tid);
  // digits staged and (through the producers' arrival) barriers initialised
  asm volatile("bar.sync 10, %0;" ::"n"(kThreads) : "memory");

  const int g = lane >> 2;
  const int t = lane & 3;
  const int pair = warp >> 1;   // which tile of a wave this warp works on
  const int parity = warp & 1;  // which half of K of that tile
  // this lane's MMA column g as activation operand: digit g % 3 of token g / 3
  const bool b_active = g < kDigits * tokens;
  const unsigned char *act_lane = b_active ? act + g * p.act_row_bytes + t * 32 : zero_row;
  const int lane_step = b_active ? 128 : 0; // bytes per supergroup in this lane's digit row
  // this lane's accumulator columns 2t and 2t + 1: what they add to token 0 and to token 1
  // (digit weights 16384, 128, 1; columns 6 and 7 are unused)
  float to_token0[2], to_token1[2];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int column = 2 * t + c;
    const int digit = column % kDigits;
    const float weight = digit == 0 ? 16384.0f : (digit == 1 ? 128.0f : 1.0f);
    to_token0[c] = column < kDigits ? weight : 0.0f;
    to_token1[c] = (column >= kDigits && column < 2 * kDigits) ? weight : 0.0f;
  }
  const int scale_row_bytes = p.rec_scale_bytes / 8;

  bool dead = false; // a bounded wait gave up: skip the math but keep the pair barrier protocol
  for (int tile = pair; tile < n_tiles; tile += kPairs) {
    const int wave0 = tile - pair;
    const int wave_tiles = n_tiles - wave0 < kPairs ? n_tiles - wave0 : kPairs;
    const int h0 = h_begin + 2 * tile;
    const std::int64_t row0 = static_cast<std::int64_t>(h0) * 8;
    // per-digit sums of rows g and g + 8, accumulator columns 2t and 2t + 1
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int d[4] = {0, 0, 0, 0};

    // waits (bounded) until `task` has landed in its slot; false after a time-out
    auto wait_task = [&](int task, int slot) {
      const std::uint32_t round = static_cast<std::uint32_t>(task / p.num_slots);
      bool assigned = round == 0; // first use of a slot: its barrier is still in phase 0
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
      const int *sums_task = sums + s * p.bpt * 8 + 2 * t;

      for (int sg0 = 0; sg0 < p.sg_per_task; sg0 += kUnroll) {
        // scales / zero points of the blocks this round touches
        float s0v[kUnroll], s1v[kUnroll];
        int z0v[kUnroll], z1v[kUnroll];
        if constexpr (!BIG_BLOCK) {
          // one block per supergroup: four consecutive blocks, one vector load each
          const float4 a4 = *reinterpret_cast<const float4 *>(sc0 + sg0);
          const float4 b4 = *reinterpret_cast<const float4 *>(sc1 + sg0);
          s0v[0] = a4.x, s0v[1] = a4.y, s0v[2] = a4.z, s0v[3] = a4.w;
          s1v[0] = b4.x, s1v[1] = b4.y, s1v[2] = b4.z, s1v[3] = b4.w;
          if constexpr (HAS_ZP) {
            const std::uint32_t za = *reinterpret_cast<const std::uint32_t *>(zr0 + sg0);
            const std::uint32_t zb = *reinterpret_cast<const std::uint32_t *>(zr1 + sg0);
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
              z0v[u] = static_cast<int>((za >> (8 * u)) & 0xffu);
              z1v[u] = static_cast<int>((zb >> (8 * u)) & 0xffu);
            }
          }
        } else {
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const int blk = (sg0 + u) / p.sg_per_block;
            s0v[u] = sc0[blk];
            s1v[u] = sc1[blk];
            if constexpr (HAS_ZP) {
              z0v[u] = zr0[blk];
              z1v[u] = zr1[blk];
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const uint4 q0 = *reinterpret_cast<const uint4 *>(row_lo + u * 64);
          const uint4 q1 = *reinterpret_cast<const uint4 *>(row_hi + u * 64);
          const uint4 ba = *reinterpret_cast<const uint4 *>(act_task + u * lane_step);
          const uint4 bb = *reinterpret_cast<const uint4 *>(act_task + u * lane_step + 16);
          const std::uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w};
          const std::uint32_t w1[4] = {q1.x, q1.y, q1.z, q1.w};
          const std::uint32_t bv[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
          // a block that spans several supergroups keeps accumulating; otherwise start afresh
          const bool fresh = BIG_BLOCK ? ((sg0 + u) % p.sg_per_block) == 0 : true;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            std::uint32_t e0, o0, e1, o1;
            Split8<!HAS_ZP>(w0[i], e0, o0);
            Split8<!HAS_ZP>(w1[i], e1, o1);
            if (i == 0 && fresh) {
              ImmaZero<!HAS_ZP>(d, e0, e1, o0, o1, bv[0], bv[1]);
            } else {
              Imma<!HAS_ZP>(d, e0, e1, o0, o1, bv[2 * i], bv[2 * i + 1]);
            }
          }
          const bool block_done = BIG_BLOCK ? ((sg0 + u + 1) % p.sg_per_block) == 0 : true;
          if (block_done) {
            int c0 = d[0], c1 = d[1], c2 = d[2], c3 = d[3];
            if constexpr (HAS_ZP) {
              const int blk = BIG_BLOCK ? (sg0 + u) / p.sg_per_block : sg0 + u;
              const int2 sum = *reinterpret_cast<const int2 *>(sums_task + blk * 8);
              c0 -= z0v[u] * sum.x;
              c1 -= z0v[u] * sum.y;
              c2 -= z1v[u] * sum.x;
              c3 -= z1v[u] * sum.y;
            }
            acc[0] = fmaf(s0v[u], static_cast<float>(c0), acc[0]);
            acc[1] = fmaf(s0v[u], static_cast<float>(c1), acc[1]);
            acc[2] = fmaf(s1v[u], static_cast<float>(c2), acc[2]);
            acc[3] = fmaf(s1v[u], static_cast<float>(c3), acc[3]);
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
    // digits -> tokens: this lane's two columns, then the four lanes of the quad (fixed order)
    float lo0 = acc[0] * to_token0[0] + acc[1] * to_token0[1]; // row g, token 0
    float lo1 = acc[0] * to_token1[0] + acc[1] * to_token1[1]; // row g, token 1
    float hi0 = acc[2] * to_token0[0] + acc[3] * to_token0[1]; // row g + 8, token 0
    float hi1 = acc[2] * to_token1[0] + acc[3] * to_token1[1]; // row g + 8, token 1
#pragma unroll
    for (int offset = 1; offset <= 2; offset <<= 1) {
      lo0 += __shfl_xor_sync(0xffffffffu, lo0, offset);
      lo1 += __shfl_xor_sync(0xffffffffu, lo1, offset);
      hi0 += __shfl_xor_sync(0xffffffffu, hi0, offset);
      hi1 += __shfl_xor_sync(0xffffffffu, hi1, offset);
    }
    // the odd warp of the pair hands its half of K to the even warp (one buffer per pair: the
    // second barrier keeps the next tile's value from overwriting one that is still being read)
    float4 *exchange = pair_buf + pair * 32 + lane;
    if (parity == 1) {
      *exchange = make_float4(lo0, lo1, hi0, hi1);
    }
    asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");
    float4 other = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (parity == 0) {
      other = *exchange;
    }
    asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");
    if (parity == 0 && t < tokens) {
      // lane t of the quad stores token t
      const float sum_lo = t == 0 ? lo0 + other.x : lo1 + other.y;
      const float sum_hi = t == 0 ? hi0 + other.z : hi1 + other.w;
      // signed codes carry a factor 16 (exact power of two)
      const float back = HAS_ZP ? undo[t] : undo[t] * 0.0625f;
      const std::int64_t m = m_base + t;
      const std::int64_t r_lo = row0 + g;
      const std::int64_t r_hi = row0 + g + 8;
      if (r_lo < row_limit) {
        const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + r_lo) : 0.0f;
        StoreOutput(p.out, m * p.out.ld + p.out.col_offset + r_lo, fmaf(sum_lo, back, bias));
      }
      if (r_hi < row_limit) {
        const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + r_hi) : 0.0f;
        StoreOutput(p.out, m * p.out.ld + p.out.col_offset + r_hi, fmaf(sum_hi, back, bias));
      }
    }
  }
}

} // namespace

// The integer decode kernel takes 4-bit weights with block_size 128 ... 1024 whose prepared
// scale / zero-point records exist (MetaGeometryOf), one or two tokens per pass over the weights.
bool GemvImmaSupports(const WeightView &w, std::int64_t m) {
  if (w.bits != 4 || w.block_size < 128 || w.block_size > 1024 || w.meta == nullptr || m < 1 ||
      (reinterpret_cast<std::uintptr_t>(w.b) & 15u) != 0) {
    return false;
  }
  return MetaGeometryOf(w).bytes != 0;
}

const char *LaunchGemvImma(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                           int *status_word, cudaStream_t stream, int sm_count) {
  if (!GemvImmaSupports(w, m) || m > 16) {
    return nullptr;
  }
  const MetaGeometry geo = MetaGeometryOf(w);
  ImmaParams p{};
  p.w = w;
  p.a = a;
  p.m_total = static_cast<int>(m);
  p.out = out;
  p.status = status_word;
  p.half_tiles = geo.half_tiles;
  p.bpt = geo.bpt;
  p.slices = geo.slices;
  p.rec_bytes = geo.rec_bytes;
  p.rec_scale_bytes = geo.rec_scale_bytes;
  p.slice_b_bytes = geo.bpt * w.block_size / 2;
  p.sg_per_task = geo.bpt * w.block_size / 128;
  p.sg_per_block = w.block_size / 128;
  p.tokens_per_pass = m < kMaxTokens ? static_cast<int>(m) : kMaxTokens;
  p.k_pad = p.slices * p.sg_per_task * 128;
  p.blocks_pad = p.slices * p.bpt;
  if (p.k_pad < w.k || (p.sg_per_task % kUnroll) != 0 || (p.sg_per_task % p.sg_per_block) != 0 ||
      ((geo.bpt % 4) != 0 && p.sg_per_block == 1)) {
    return nullptr;
  }
  p.act_row_bytes = p.k_pad + 16; // 16: the two digit rows read by a quarter warp fall on different banks
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
  const size_t fixed = static_cast<size_t>(kDigits * p.tokens_per_pass) * p.act_row_bytes + kZeroBytes +
                       static_cast<size_t>(p.blocks_pad) * 8 * sizeof(int) + (4 + kWarps) * sizeof(float) +
                       kPairs * 32 * sizeof(float4) + 2 * kMaxSlots * sizeof(std::uint64_t) +
                       kMaxSlots * sizeof(int) + 128;
  const size_t limit = 227 * 1024 - 128; // the most a CTA can ask for, less the alignment slack
  if (fixed + 2 * static_cast<size_t>(p.slot_bytes) > limit) {
    return nullptr;
  }
  int slots = static_cast<int>((limit - fixed) / p.slot_bytes);
  if (slots > kMaxSlots) {
    slots = kMaxSlots;
  }
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
  // Programmatic dependent launch (the weight stream starts while the previous kernel drains; A is
  // read after the dependency wait) only behind the host-buffer call's fetch kernel: between
  // consecutive nodes it measured slower (11.3-12.1 vs 10.2-10.5 us per node).
  dim3 grid(static_cast<unsigned>(ctas),
            static_cast<unsigned>((m + p.tokens_per_pass - 1) / p.tokens_per_pass), 1);
  cudaError_t err = cudaErrorInvalidValue;
#define MNB_IMMA_CASE(BIG_, ZP_)                                                                 \
  if ((p.sg_per_block > 1) == BIG_ && (w.zp != nullptr) == ZP_) {                                \
    auto kernel = nbits_gemv_imma_kernel<BIG_, ZP_>;                                             \
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
      config.numAttrs = DependentLaunchHint() ? 1 : 0;                                          \
      err = cudaLaunchKernelEx(&config, kernel, map_b, p);                                       \
    }                                                                                            \
  }
  MNB_IMMA_CASE(false, true)
  MNB_IMMA_CASE(false, false)
  MNB_IMMA_CASE(true, true)
  MNB_IMMA_CASE(true, false)
#undef MNB_IMMA_CASE
  if (err != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return "nbits_gemv_imma_kernel";
}

} // namespace mnb
