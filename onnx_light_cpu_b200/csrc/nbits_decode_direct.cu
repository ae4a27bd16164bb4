// Decode path of MatMulNBits (accuracy_level 0, 1 ... 16 activation rows, 4-bit weights,
// block_size 128) in which every warp streams its own packed weights from global memory.
//
// No producer, no shared slots, no hand-over between warps while the weights stream: every warp
// owns a row tile (or a contiguous part of its K range) and keeps a ring of "supersteps" (four
// MMA steps, 4 KB per warp) in flight, either in lane-private shared-memory places filled by
// cp.async (a lane reads back only what it asked for itself) or, when shared memory is full of
// activation digits, in registers. The first superstep is asked for before the dependency on
// the previous kernel of the stream is awaited (programmatic dependent launch); the rest of the
// ring follows BEHIND the request for the activations, because the load pipe serves requests in
// order and three stages per warp in front of A delayed the digits by two to four microseconds.
// With two resident CTAs per SM the weight stream of node n+1 starts while node n drains.
//
// Arithmetic and exactness: nbits_digits.cuh. Scales are read in their own layout; zero points from
// the prepared byte-per-block array (16 x zero point), which rides the same asynchronous copies.
//
// Two ways to fill the sixteen MMA rows:
//  * several tokens: sixteen weight rows x one 128-k segment per step; `ks` warps of a CTA share
//    a tile, each with a contiguous part of K, partial results added through shared memory in a
//    fixed order;
//  * one token ("row pair"): eight weight rows x two consecutive segments per step; MMA rows
//    0..7 see the even segment, rows 8..15 the odd one, columns 0..2 / 3..5 carry the digits of
//    the even / odd segment. An eight-row tile is 16 KB at K = 4096, which gives twice as many
//    tiles to spread over the SMs and needs no exchange between warps.
//
// Conventions: packed-INT4 nibble order of
// onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:60-93; "stream B once, split N"
// partition of onnx_light_cpu/impl/math/gemm_kernel.cc:1219-1258.

#include "nbits_common.cuh"
#include "nbits_digits.cuh"
#include "nbits_ptx.cuh"

#include <cstdint>
#include <type_traits>

namespace mnb {
namespace {

struct DirectParams {
  WeightView w;
  const float *a;
  OutputView out;
  int m_total;
  int tokens_per_pass;  // activation rows staged per CTA (one grid.y pass)
  int tiles;            // row tiles: 16 rows, or 8 in row-pair mode
  int ks;               // warps sharing a tile, each a contiguous part of K
  int supers_per_part;  // supersteps of one part
  int segs;             // 64-byte (128-k) segments per weight row
  int chunk_stride;     // bytes between consecutive segments of the staged digits
  int table_ints;       // ints of the digit-sum table
};

// 16 bytes of weights, streamed: read once, no reason to keep them in L1.
__device__ __forceinline__ uint4 LoadStream16(const unsigned char *ptr) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

__device__ __forceinline__ float4 LoadScales4(const float *ptr) {
  float4 v;
  asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(ptr));
  return v;
}

// One superstep of weights, scales and zero points in registers (register ring, RING == 0).
struct SuperRegs {
  uint4 w[kStepsPerSuper][2];  // [step][MMA rows 0..7 / 8..15]
  float4 s[2];
  uint2 z;
};

// Shared-memory ring, per warp and stage: weights [4 steps][2 loads][32 lanes][16 B], then the
// scale vectors [2][8 quads][16 B], then the zero points [8 quads][8 B].
constexpr int kStageWeightBytes = kStepsPerSuper * 2 * 32 * 16;
constexpr int kStageScaleBytes = 2 * 8 * 16;
constexpr int kStageZeroBytes = 8 * 8;
constexpr int kStageBytes = kStageWeightBytes + kStageScaleBytes + kStageZeroBytes + 64;  // 4480 = 35 * 128

// 16-byte asynchronous copy global -> shared; `bytes` is 16, or 0 for "write zeros, read nothing"
// (what the ring does once the warp has asked for everything: no branch in the loop).
__device__ __forceinline__ void CopyAsync16(std::uint32_t smem_addr, const void *gptr, std::uint32_t bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(bytes));
}

template <int SIZE>
__device__ __forceinline__ void CopyAsyncSmall(std::uint32_t smem_addr, const void *gptr, std::uint32_t bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(smem_addr), "l"(gptr), "n"(SIZE), "r"(bytes));
}

__device__ __forceinline__ void CopyAsyncCommit() { asm volatile("cp.async.commit_group;" ::); }

template <int PENDING>
__device__ __forceinline__ void CopyAsyncWait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

// Ring reads: volatile, so they stay in program order with the cp.async that refills the slot.
template <int OFFSET>
__device__ __forceinline__ uint4 LoadSharedVolatile16(std::uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4 + %5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr), "n"(OFFSET));
  return v;
}

__device__ __forceinline__ uint2 LoadSharedVolatile8(std::uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// ROWPAIR: one token, eight rows x two segments per step. NT: MMA column tiles (two tokens each).
// RING: 0 = one superstep of weights in flight in registers; n > 0 = n supersteps in flight in
// lane-private shared-memory slots filled by cp.async (a lane reads back only what it asked for
// itself, so no hand-over between lanes is needed; the four lanes of a quad copy the same scale
// vector and zero points to the same place).
template <bool ROWPAIR, int NT, bool HAS_ZP, int RING>
__global__ void __launch_bounds__(512, 1) nbits_decode_direct_kernel(const DirectParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char *digits = smem;
  int *table = reinterpret_cast<int *>(digits + static_cast<size_t>(p.segs) * p.chunk_stride);
  float *undo = reinterpret_cast<float *>(table + p.table_ints);
  float *red = undo + kMaxTokens;
  float *exchange = red + kMaxTokens * kMaxWarps;

  // the next kernel of the stream may start filling SMs as soon as this grid's CTAs leave
  ptx::GridDependencyLaunch();

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int warps = blockDim.x >> 5;
  const int groups = warps / p.ks;
  const int group = warp / p.ks;
  const int part = warp - group * p.ks;
  const int tile_step = groups * static_cast<int>(gridDim.x);
  const int tile_first = group * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x);
  const int my_tiles = tile_first < p.tiles ? (p.tiles - tile_first + tile_step - 1) / tile_step : 0;
  const int supers_per_part = p.supers_per_part;
  const int total_supers = my_tiles * supers_per_part;
  const int m_base = static_cast<int>(blockIdx.y) * p.tokens_per_pass;
  int tokens = p.m_total - m_base;
  if (tokens > p.tokens_per_pass) {
    tokens = p.tokens_per_pass;
  }

  constexpr int kRowsPerTile = ROWPAIR ? 8 : 16;
  constexpr int kSegsPerStep = ROWPAIR ? 2 : 1;
  constexpr int kSegsPerSuper = kSegsPerStep * kStepsPerSuper;
  constexpr int kStepBytes = 64 * kSegsPerStep;
  const int n_blocks = p.w.n_blocks;
  const int last_row = static_cast<int>(p.w.n - 1);
  const int first_seg_of_part = part * supers_per_part * kSegsPerSuper;

  // shared-memory ring of this warp (RING > 0)
  const std::uint32_t ring_warp =
      ptx::SmemAddr(exchange + static_cast<size_t>(warps) * NT * 32) + warp * ((RING > 0 ? RING : 1) * kStageBytes);
  const std::uint32_t ring_lane = ring_warp + lane * 16;
  const std::uint32_t ring_scales = ring_warp + kStageWeightBytes + g * 16;
  const std::uint32_t ring_zeros = ring_warp + kStageWeightBytes + kStageScaleBytes + g * 8;

  // ---- load cursor: the next superstep to ask for ----
  // One block index per MMA row group: row * n_blocks + segment. The packed weights of that
  // block start at 64 * index, its scale at 4 * index, its prepared zero point at index.
  int load_tile = tile_first;
  int load_super = 0;
  int loads_left = total_supers;
  int index_lo = 0, index_hi = 0;
  auto place_cursor = [&]() {
    int row_lo = load_tile * kRowsPerTile + g;
    int row_hi = ROWPAIR ? row_lo : row_lo + 8;
    row_lo = row_lo < last_row ? row_lo : last_row;
    row_hi = row_hi < last_row ? row_hi : last_row;
    index_lo = row_lo * n_blocks + first_seg_of_part;
    index_hi = ROWPAIR ? index_lo + 1 : row_hi * n_blocks + first_seg_of_part;
  };
  if (my_tiles > 0) {
    place_cursor();
  }
  SuperRegs regs;  // RING == 0 only
  const unsigned char *next_lo = p.w.b;
  const unsigned char *next_hi = p.w.b;
  std::uint32_t next_bytes = 0;  // 16 while there is something left to ask for, then 0
  // Asks for the scales / zero points of the cursor's superstep (ring stage at `stage_offset`)
  // and leaves the addresses of its weights in next_lo / next_hi. Once everything has been asked
  // for it turns into "copy nothing" (zero-size cp.async), so the loop carries no branch for it.
  auto begin_super_load = [&](std::uint32_t stage_offset) {
    next_bytes = loads_left > 0 ? 16u : 0u;
    --loads_left;
    next_lo = p.w.b + static_cast<std::int64_t>(index_lo) * 64 + t * 16;
    next_hi = p.w.b + static_cast<std::int64_t>(index_hi) * 64 + t * 16;
    const float *s_first = p.w.scales + index_lo;
    const float *s_second = ROWPAIR ? s_first + 4 : p.w.scales + index_hi;
    if constexpr (RING > 0) {
      CopyAsync16(ring_scales + stage_offset, s_first, next_bytes);
      CopyAsync16(ring_scales + stage_offset + 128, s_second, next_bytes);
      if constexpr (HAS_ZP) {
        if constexpr (ROWPAIR) {
          CopyAsyncSmall<8>(ring_zeros + stage_offset, p.w.zp16 + index_lo, next_bytes >> 1);
        } else {
          CopyAsyncSmall<4>(ring_zeros + stage_offset, p.w.zp16 + index_lo, next_bytes >> 2);
          CopyAsyncSmall<4>(ring_zeros + stage_offset + 4, p.w.zp16 + index_hi, next_bytes >> 2);
        }
      }
    } else {
      if (next_bytes != 0) {
        regs.s[0] = LoadScales4(s_first);
        regs.s[1] = LoadScales4(s_second);
        if constexpr (HAS_ZP) {
          if constexpr (ROWPAIR) {
            regs.z = *reinterpret_cast<const uint2 *>(p.w.zp16 + index_lo);
          } else {
            regs.z.x = *reinterpret_cast<const std::uint32_t *>(p.w.zp16 + index_lo);
            regs.z.y = *reinterpret_cast<const std::uint32_t *>(p.w.zp16 + index_hi);
          }
        }
      }
    }
    index_lo += kSegsPerSuper;
    index_hi += kSegsPerSuper;
    if (++load_super == supers_per_part) {
      load_super = 0;
      load_tile += tile_step;
      if (loads_left > 0) {
        place_cursor();
      } else {
        index_lo = index_hi = 0;  // nothing left: any valid address
      }
    }
  };
  auto load_step = [&](std::uint32_t stage_offset, int i) {
    if constexpr (RING > 0) {
      CopyAsync16(ring_lane + stage_offset + (2 * i) * 512, next_lo + i * kStepBytes, next_bytes);
      CopyAsync16(ring_lane + stage_offset + (2 * i + 1) * 512, next_hi + i * kStepBytes, next_bytes);
    } else {
      if (next_bytes != 0) {
        regs.w[i][0] = LoadStream16(next_lo + i * kStepBytes);
        regs.w[i][1] = LoadStream16(next_hi + i * kStepBytes);
      }
    }
  };

  // The first superstep is asked for before anything else: it touches the constant weights only.
  // The other ring stages follow behind the loads of A (see StageDigits).
  auto issue_stage = [&](int b) {
    begin_super_load(b * kStageBytes);
#pragma unroll
    for (int i = 0; i < kStepsPerSuper; ++i) {
      load_step(b * kStageBytes, i);
    }
    if constexpr (RING > 0) {
      CopyAsyncCommit();  // one group per stage, empty or not
    }
  };
  issue_stage(0);
  auto issue_rest = [&]() {
#pragma unroll
    for (int b = 1; b < RING; ++b) {
      issue_stage(b);
    }
  };

  // A (and Y) may be produced / still read by the previous kernel in the stream
  ptx::GridDependencyWait();
  const DigitGeometry geometry{static_cast<int>(p.w.k), p.segs, p.chunk_stride, p.table_ints};
  StageDigits<ROWPAIR>(geometry, p.a + static_cast<std::int64_t>(m_base) * p.w.k, tokens, NT, digits, table, undo, red,
                       tid, static_cast<int>(blockDim.x), [] { __syncthreads(); }, issue_rest);

  // ---- per-lane constants ----
  // MMA column g as activation operand: digit g % 3 of the first (g < 3) or second (3 <= g < 6)
  // token of the column tile (row-pair mode: of the even / odd segment); columns 6, 7 are
  // unused and read what columns 0, 1 read.
  const int column = g < 6 ? g : g - 6;
  const int second = column >= kDigits ? 1 : 0;
  const int digit_of_column = column - second * kDigits;
  const int swizzle = (second + digit_of_column) & 1;
  constexpr int kDigitsStepBytes = (ROWPAIR ? 1 : NT) * kTileColumnBytes;  // staged digits of one step
  constexpr int kTableStepBytes = (ROWPAIR ? 1 : NT) * 8 * 4;
  const std::uint32_t digits_column =
      LaunderAfterBarrier(ptx::SmemAddr(digits) + (second * kDigits + digit_of_column) * kChunkBytes);
  const std::uint32_t digits_even = digits_column + (((2 * t) ^ swizzle) << 4);      // even k of the lane's words
  const std::uint32_t digits_odd = digits_column + (((2 * t + 1) ^ swizzle) << 4);   // odd k
  const std::uint32_t table_lane = LaunderAfterBarrier(ptx::SmemAddr(table) + t * 8);

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
  }
  int tile = tile_first;
  int super = 0;
  std::uint32_t stage_offset = 0;
  const ZeroQuad zero = MakeZeroQuad();

#pragma unroll 1
  for (int it = 0; it < total_supers; ++it) {
    // this superstep's scales / zero points move out of the ring, which is refilled at once
    float4 s_first, s_second;
    uint2 z = make_uint2(0u, 0u);
    if constexpr (RING > 0) {
      CopyAsyncWait<RING - 1>();
      const uint4 u0 = LoadSharedVolatile16<0>(ring_scales + stage_offset);
      const uint4 u1 = LoadSharedVolatile16<128>(ring_scales + stage_offset);
      s_first = make_float4(__uint_as_float(u0.x), __uint_as_float(u0.y), __uint_as_float(u0.z), __uint_as_float(u0.w));
      s_second =
          make_float4(__uint_as_float(u1.x), __uint_as_float(u1.y), __uint_as_float(u1.z), __uint_as_float(u1.w));
      if constexpr (HAS_ZP) {
        z = LoadSharedVolatile8(ring_zeros + stage_offset);
      }
      __syncwarp();  // every lane has read the quad's scales before any lane asks for new ones
    } else {
      s_first = regs.s[0];
      s_second = regs.s[1];
      z = regs.z;
    }
    begin_super_load(stage_offset);
    const int step0 = (part * supers_per_part + super) * kStepsPerSuper;
    const std::uint32_t even_at = digits_even + step0 * kDigitsStepBytes;
    const std::uint32_t odd_at = digits_odd + step0 * kDigitsStepBytes;
    const std::uint32_t table_at = table_lane + step0 * kTableStepBytes;
    const std::uint32_t ring_at = ring_lane + stage_offset;
    auto do_step = [&](auto step_tag) {
      constexpr int i = decltype(step_tag)::value;
      float s_lo, s_hi;
      int z_lo = 128, z_hi = 128;  // 16 x the default zero point 8
      if constexpr (ROWPAIR) {
        s_lo = Component(i < 2 ? s_first : s_second, (2 * i) & 3);
        s_hi = Component(i < 2 ? s_first : s_second, (2 * i + 1) & 3);
        if constexpr (HAS_ZP) {
          z_lo = static_cast<int>(__byte_perm(i < 2 ? z.x : z.y, 0u, 0x4440u + ((2 * i) & 3)));
          z_hi = static_cast<int>(__byte_perm(i < 2 ? z.x : z.y, 0u, 0x4440u + ((2 * i + 1) & 3)));
        }
      } else {
        s_lo = Component(s_first, i);
        s_hi = Component(s_second, i);
        if constexpr (HAS_ZP) {
          z_lo = static_cast<int>(__byte_perm(z.x, 0u, 0x4440u + i));
          z_hi = static_cast<int>(__byte_perm(z.y, 0u, 0x4440u + i));
        }
      }
      uint4 lo, hi;
      if constexpr (RING > 0) {
        lo = LoadSharedVolatile16<(2 * i) * 512>(ring_at);
        hi = LoadSharedVolatile16<(2 * i + 1) * 512>(ring_at);
      } else {
        lo = regs.w[i][0];
        hi = regs.w[i][1];
      }
      const std::uint32_t wl[4] = {lo.x, lo.y, lo.z, lo.w};
      const std::uint32_t wh[4] = {hi.x, hi.y, hi.z, hi.w};
      std::uint32_t el[4], ol[4], eh[4], oh[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        el[q] = wl[q] & 0x0f0f0f0fu;
        ol[q] = wl[q] & 0xf0f0f0f0u;
        eh[q] = wh[q] & 0x0f0f0f0fu;
        oh[q] = wh[q] & 0xf0f0f0f0u;
      }
      load_step(stage_offset, i);
      auto do_tile = [&](auto tile_tag) {
        constexpr int j = decltype(tile_tag)::value;
        constexpr int kAt = i * kDigitsStepBytes + j * kTileColumnBytes;
        const uint4 be = LoadSharedConst16<kAt>(even_at);  // even k of the lane's words 0..3
        const uint4 bo = LoadSharedConst16<kAt>(odd_at);
        const int2 sums = LoadSharedConst8<i * kTableStepBytes + j * 32>(table_at);
        int de[4], dd[4];
        ImmaFresh(de, el[0], eh[0], el[1], eh[1], be.x, be.y, zero);
        ImmaFresh(dd, ol[0], oh[0], ol[1], oh[1], bo.x, bo.y, zero);
        ImmaAdd(de, el[2], eh[2], el[3], eh[3], be.z, be.w);
        ImmaAdd(dd, ol[2], oh[2], ol[3], oh[3], bo.z, bo.w);
        // 16 * (even + odd block sum - zp * digit sum): exact, below 2^24 (the table holds -sum)
        const int c0 = z_lo * sums.x + (de[0] * 16 + dd[0]);
        const int c1 = z_lo * sums.y + (de[1] * 16 + dd[1]);
        const int c2 = z_hi * sums.x + (de[2] * 16 + dd[2]);
        const int c3 = z_hi * sums.y + (de[3] * 16 + dd[3]);
        acc[j][0] = fmaf(s_lo, static_cast<float>(c0), acc[j][0]);
        acc[j][1] = fmaf(s_lo, static_cast<float>(c1), acc[j][1]);
        acc[j][2] = fmaf(s_hi, static_cast<float>(c2), acc[j][2]);
        acc[j][3] = fmaf(s_hi, static_cast<float>(c3), acc[j][3]);
      };
      ForEachIndex<NT>(do_tile);
    };
    ForEachIndex<kStepsPerSuper>(do_step);
    if constexpr (RING > 0) {
      CopyAsyncCommit();  // one group per superstep consumed, empty or not
      stage_offset = stage_offset + kStageBytes == RING * kStageBytes ? 0u : stage_offset + kStageBytes;
    }

    if (++super == supers_per_part) {
      super = 0;
      // ---- the tile (this warp's part of it) is complete ----
      if constexpr (ROWPAIR) {
        // rows g see columns 0..2 (even segments), rows g + 8 columns 3..5 (odd segments)
        float v = t == 0   ? fmaf(16384.0f, acc[0][0], 128.0f * acc[0][1])
                  : t == 1 ? fmaf(16384.0f, acc[0][3], acc[0][0])
                  : t == 2 ? fmaf(128.0f, acc[0][2], acc[0][3])
                           : 0.0f;
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if (p.ks > 1) {
          if (t == 0 && part != 0) {
            exchange[warp * 8 + g] = v;
          }
          asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(p.ks * 32) : "memory");
          if (part == 0) {
            for (int q = 1; q < p.ks; ++q) {
              v += exchange[(warp + q) * 8 + g];
            }
          }
          asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(p.ks * 32) : "memory");
        }
        const std::int64_t row = static_cast<std::int64_t>(tile) * 8 + g;
        if (part == 0 && t == 0 && row < p.w.n) {
          const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + row) : 0.0f;
          StoreOutput(p.out, static_cast<std::int64_t>(m_base) * p.out.ld + p.out.col_offset + row,
                      fmaf(v, undo[0], bias));
        }
      } else {
        // columns: 0..2 digits of the tile's first token, 3..5 of its second; this lane holds
        // columns 2t and 2t + 1 of rows g (acc 0, 1) and g + 8 (acc 2, 3)
        float v[NT][4];  // first token row g, second token row g, first token row g + 8, second ...
#pragma unroll
        for (int j = 0; j < NT; ++j) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float x = acc[j][2 * h], y = acc[j][2 * h + 1];
            v[j][2 * h] = t == 0 ? fmaf(16384.0f, x, 128.0f * y) : (t == 1 ? x : 0.0f);
            v[j][2 * h + 1] = t == 1 ? 16384.0f * y : (t == 2 ? fmaf(128.0f, x, y) : 0.0f);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[j][e] += __shfl_xor_sync(0xffffffffu, v[j][e], 1);
            v[j][e] += __shfl_xor_sync(0xffffffffu, v[j][e], 2);
          }
        }
        if (p.ks > 1) {
          float4 *mine = reinterpret_cast<float4 *>(exchange) + (warp * NT) * 8 + g;
          if (t == 0 && part != 0) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
              mine[j * 8] = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
            }
          }
          asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(p.ks * 32) : "memory");
          if (part == 0 && t == 0) {
            for (int q = 1; q < p.ks; ++q) {
#pragma unroll
              for (int j = 0; j < NT; ++j) {
                const float4 other = mine[(q * NT + j) * 8];
                v[j][0] += other.x;
                v[j][1] += other.y;
                v[j][2] += other.z;
                v[j][3] += other.w;
              }
            }
          }
          asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(p.ks * 32) : "memory");
        }
        if (part == 0 && t == 0) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const std::int64_t row = static_cast<std::int64_t>(tile) * 16 + 8 * h + g;
            if (row < p.w.n) {
              const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + row) : 0.0f;
#pragma unroll
              for (int j = 0; j < NT; ++j) {
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                  const int token = 2 * j + x;
                  if (token < tokens) {
                    StoreOutput(p.out, static_cast<std::int64_t>(m_base + token) * p.out.ld + p.out.col_offset + row,
                                fmaf(v[j][2 * h + x], undo[token], bias));
                  }
                }
              }
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
      }
      tile += tile_step;
    }
  }
  if constexpr (RING > 0) {
    CopyAsyncWait<0>();  // nothing of this thread is in flight when it leaves
  }
}

// out[row * n_blocks + block] = 16 * zero point, one byte per block: what the ring copies beside
// the scales (a byte per block instead of a nibble costs n * n_blocks / 2 more bytes per node).
__global__ void __launch_bounds__(256) nbits_expand_zero_points_kernel(const WeightView w, unsigned char *out) {
  const std::int64_t total = w.n * w.n_blocks;
  for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
    const std::int64_t row = i / w.n_blocks;
    const int block = static_cast<int>(i - row * w.n_blocks);
    out[i] = static_cast<unsigned char>(16 * ZeroPointOf(w, row, block));
  }
}

size_t SharedBytes(const DirectParams &p, int column_tiles, int warps, int ring) {
  return static_cast<size_t>(p.segs) * p.chunk_stride + static_cast<size_t>(p.table_ints) * sizeof(int) +
         (kMaxTokens + kMaxTokens * kMaxWarps) * sizeof(float) +
         static_cast<size_t>(warps) * column_tiles * 8 * sizeof(float4) +
         static_cast<size_t>(warps) * ring * kStageBytes + 128;
}

template <bool ROWPAIR, int NT, int RING>
cudaError_t LaunchOne(const DirectParams &p, dim3 grid, int threads, size_t smem, bool dependent,
                      cudaStream_t stream) {
  auto launch = [&](auto kernel) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
    if (err != cudaSuccess) {
      return err;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, p);
  };
  if (p.w.zp != nullptr) {
    return launch(nbits_decode_direct_kernel<ROWPAIR, NT, true, RING>);
  }
  return launch(nbits_decode_direct_kernel<ROWPAIR, NT, false, RING>);
}

template <bool ROWPAIR, int NT>
cudaError_t LaunchRing(int ring, const DirectParams &p, dim3 grid, int threads, size_t smem, bool dependent,
                       cudaStream_t stream) {
  switch (ring) {
  case 0:
    return LaunchOne<ROWPAIR, NT, 0>(p, grid, threads, smem, dependent, stream);
  case 2:
    return LaunchOne<ROWPAIR, NT, 2>(p, grid, threads, smem, dependent, stream);
  default:
    return cudaErrorInvalidValue;
  }
}

} // namespace

namespace {
bool GeometryFits(const WeightView &w) {
  return w.bits == 4 && w.block_size == 128 && (w.n_blocks % kStepsPerSuper) == 0 &&
         w.n * static_cast<std::int64_t>(w.n_blocks) < (std::int64_t{1} << 31);
}
} // namespace

bool DecodeDirectWantsZeroPointBytes(const WeightView &w) { return w.zp != nullptr && GeometryFits(w); }

bool LaunchExpandZeroPoints(const WeightView &w, unsigned char *out, cudaStream_t stream) {
  const std::int64_t total = w.n * w.n_blocks;
  std::int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 8) {
    blocks = 148 * 8;
  }
  nbits_expand_zero_points_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(w, out);
  if (cudaGetLastError() != cudaSuccess) {
    return false;
  }
  CountLaunch();
  return true;
}

bool DecodeDirectSupports(const WeightView &w, std::int64_t m) {
  // One column tile (two tokens). The same code with 2, 4 or 8 column tiles per pass was measured
  // against the fp16 tensor-core decode kernels on N = 14336, K = 4096 and lost from M = 2 on (M = 4:
  // 17.1 vs 15.3 us, M = 16: 54.4 vs 38.5 us), so only the one-tile form is built.
  if (!GeometryFits(w) || m < 1 || m > 2 || (w.zp != nullptr && w.zp16 == nullptr)) {
    return false;
  }
  return (reinterpret_cast<std::uintptr_t>(w.b) & 15u) == 0 && (reinterpret_cast<std::uintptr_t>(w.scales) & 15u) == 0 &&
         (reinterpret_cast<std::uintptr_t>(w.zp16) & 7u) == 0;
}

// `dependent`: launch with programmatic stream serialization (the kernel's weight loads then start
// while the previous kernel of the stream drains; it waits for that kernel before it reads A or
// writes Y).
const char *LaunchDecodeDirect(const WeightView &w, const float *a, std::int64_t m, OutputView out,
                               cudaStream_t stream, int sm_count, bool dependent) {
  if (!DecodeDirectSupports(w, m)) {
    return nullptr;
  }
  const int sms = sm_count > 0 ? sm_count : 148;
  DirectParams p{};
  p.w = w;
  p.a = a;
  p.out = out;
  p.m_total = static_cast<int>(m);
  p.segs = w.n_blocks;
  const bool row_pair = m == 1 && (w.n_blocks % (2 * kStepsPerSuper)) == 0;
  constexpr size_t kTwoPerSm = 112 * 1024;   // two CTAs of this size are resident per SM
  constexpr size_t kOnePerSm = 226 * 1024;

  const int rows_per_tile = row_pair ? 8 : 16;
  int column_tiles = 1;
  // Preference: two resident CTAs per SM (the next node's CTAs then start while this node
  // drains) with a deep shared-memory ring, then one large CTA, then the register ring; fewer
  // tokens per pass when even that does not fit.
  struct Shape {
    int threads;
    int ring;
  };
  // Measured (one token, N = 14336, K = 4096, us per launch in a CUDA graph): 256 threads with a
  // ring of two stages 9.0, 512 threads with the register ring 9.0, 512 / ring 2: 9.2, rings of
  // three stages 9.8 ... 10.2 (what a warp asks for ahead of time is also in front of its own later
  // requests).
  const Shape shapes[] = {{256, 2}, {512, 2}, {512, 0}};
  int threads = 0;
  int ring = 0;
  size_t smem = 0;
  for (;;) {
    p.chunk_stride = row_pair ? kDigits * kChunkBytes : column_tiles * kTileColumnBytes;
    p.table_ints = row_pair ? (p.segs / 2) * 8 : p.segs * column_tiles * 8;
    for (const Shape &shape : shapes) {
      const size_t need = SharedBytes(p, column_tiles, shape.threads / 32, shape.ring);
      if (need <= (shape.threads <= 256 ? kTwoPerSm : kOnePerSm)) {
        threads = shape.threads;
        ring = shape.ring;
        smem = need;
        break;
      }
    }
    if (threads != 0) {
      break;
    }
    if (column_tiles == 1) {
      return nullptr;  // K too long for one token pair in shared memory
    }
    column_tiles /= 2;
  }
  p.tokens_per_pass = row_pair ? 1 : 2 * column_tiles;
  if (p.tokens_per_pass > m) {
    p.tokens_per_pass = static_cast<int>(m);
  }
  const int passes = static_cast<int>((m + p.tokens_per_pass - 1) / p.tokens_per_pass);
  p.tiles = static_cast<int>((w.n + rows_per_tile - 1) / rows_per_tile);
  const int supers = p.segs / (kStepsPerSuper * (row_pair ? 2 : 1));
  const int warps = threads / 32;
  int ctas = sms * (threads <= 256 ? 2 : 1);
  // warps sharing a tile: enough parts to give most warps of the grid one, parts of whole supersteps
  int ks = 1;
  while (ks * 2 <= 8 && (warps % (ks * 2)) == 0 && (supers % (ks * 2)) == 0 &&
         static_cast<std::int64_t>(p.tiles) * ks * 4 < static_cast<std::int64_t>(ctas) * warps * 3) {
    ks *= 2;
  }
  p.ks = ks;
  p.supers_per_part = supers / ks;
  // tiles go round the CTAs first (tile = group * CTAs + CTA), so every SM gets its share whatever
  // the number of warp groups; only a node with fewer tiles than CTAs uses a smaller grid
  if (ctas > p.tiles) {
    ctas = p.tiles;
  }
  const dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>(passes), 1);
  cudaError_t err = cudaErrorInvalidValue;
  if (row_pair) {
    err = LaunchRing<true, 1>(ring, p, grid, threads, smem, dependent, stream);
  } else {
    err = LaunchRing<false, 1>(ring, p, grid, threads, smem, dependent, stream);
  }
  if (err != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  CountLaunch();
  return "nbits_decode_direct_kernel";
}

} // namespace mnb
