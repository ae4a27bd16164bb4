// Pieces shared by the integer-MMA decode kernels of MatMulNBits (accuracy_level 0): activations as
// three base-128 digit rows, the digit-sum table of the zero-point correction, the MMA wrappers.
//
// Arithmetic (exact integer products, fp32-grade result):
//  * A weight word holds eight codes. `w & 0x0f0f0f0f` are the even codes as bytes, `w & 0xf0f0f0f0`
//    the odd codes times 16 as bytes: one instruction per MMA operand register, no shift. Even and
//    odd codes go through separate mma.sync.m16n8k32.s32.u8.s8 accumulators, merged per
//    quantization block as 16 * even + odd (so every block sum carries a factor 16, undone at the
//    end, exactly).
//  * Each activation row is scaled so that its largest magnitude becomes kDigitRange and rounded
//    to a 22-bit integer n = 16384 d0 + 128 d1 + d2 with balanced base-128 digits; the digits are
//    three signed-byte MMA columns. One MMA column tile (8 columns) holds two tokens.
//  * Zero points leave through `block sum - zp * (sum of the block's digits)`, the correction of
//    onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:208-223; a node without zero points
//    uses the default 8.
//  * Block sums are exact int32 (< 2^24), converted to float and combined as
//    acc[digit] += scale * float(sum); the end computes (16384 acc0 + 128 acc1 + acc2) * undo + bias.
#pragma once

#include "nbits_common.cuh"
#include "nbits_ptx.cuh"

#include <cstdint>
#include <type_traits>

namespace mnb {
namespace {

constexpr int kDigits = 3;
constexpr float kDigitRange = 2.0e6f;  // the row maximum maps to this integer (< 123 * 16384)
constexpr float kDigitBias = 64.0f + 64.0f * 128.0f + 128.0f * 16384.0f;  // makes all three digits non-negative
constexpr int kMaxWarps = 16;
constexpr int kMaxTokens = 16;
constexpr int kStepsPerSuper = 4;      // steps that share one 128-bit load of scales
constexpr int kChunkBytes = 128;       // digits of one (segment, token, digit): one byte per k
constexpr int kTileColumnBytes = 6 * kChunkBytes;  // one MMA column tile: two tokens x three digits

// Activations: volatile so that the request is made where the statement stands (ahead of the
// weight prefetch queued behind it), not where the value is first used.
__device__ __forceinline__ float4 LoadActivations4(const float *ptr) {
  float4 v;
  asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(ptr));
  return v;
}

// Four registers that hold zero, as four separate values: the accumulator input of an MMA that
// starts a block sum. (Written as the same register four times, the compiler copied it into a
// register quad in front of every such MMA: eight moves per step.)
struct ZeroQuad {
  int v[4];
};

__device__ __forceinline__ ZeroQuad MakeZeroQuad() {
  ZeroQuad z;
  asm volatile("mov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;"
               : "=r"(z.v[0]), "=r"(z.v[1]), "=r"(z.v[2]), "=r"(z.v[3]));
  return z;
}

// D (int32, 16 x 8) = A (16 x 32 unsigned bytes) * B (32 x 8 signed bytes), fresh accumulator.
__device__ __forceinline__ void ImmaFresh(int (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                          std::uint32_t a3, std::uint32_t b0, std::uint32_t b1, const ZeroQuad &zero) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(zero.v[0]), "r"(zero.v[1]), "r"(zero.v[2]),
        "r"(zero.v[3]));
}

__device__ __forceinline__ void ImmaAdd(int (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                        std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Calls f(std::integral_constant<int, 0>{}) ... f(std::integral_constant<int, N - 1>{}): a loop
// whose index is a compile-time constant inside the body (immediate address offsets).
template <int N, int I = 0, typename F>
__device__ __forceinline__ void ForEachIndex(F &&f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    ForEachIndex<N, I + 1>(f);
  }
}

// max that returns NaN when either operand is NaN
__device__ __forceinline__ float MaxNan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

__device__ __forceinline__ float Component(const float4 &v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// Where the digits of (segment, token, digit) start and the swizzle bit of that chunk. A chunk is
// eight 16-byte units; unit u sits at position u ^ swizzle so that the two MMA columns a quarter
// warp reads together fall on different banks.
template <bool ROWPAIR>
__device__ __forceinline__ int ChunkOffset(int seg, int token, int digit, int chunk_stride, int *swizzle) {
  if constexpr (ROWPAIR) {
    *swizzle = ((seg & 1) + digit) & 1;
    return (seg >> 1) * kTileColumnBytes + ((seg & 1) * kDigits + digit) * kChunkBytes;
  } else {
    *swizzle = ((token & 1) + digit) & 1;
    return seg * chunk_stride + (token >> 1) * kTileColumnBytes + ((token & 1) * kDigits + digit) * kChunkBytes;
  }
}

// Rounds eight activations (one 8-k word) to their three digits and stores the six packed words.
// Biased integer u = n + 64 + 64 * 128 + 128 * 16384 (0 < u < 2^22): its plain base-128 digits are
// the balanced digits of n plus 64, 64 and 128. One fused multiply-add and one conversion per
// value; u << 1 and u << 2 put the middle and high digit on byte boundaries.
// sums[d] receives the sum of the eight digits d.
//
// BLOCK32 (row-pair mode, quantization blocks of 32): the digits are kept block by block instead,
// for MMAs that take one 32-k block each. A block is four words; (step, block u of the segment,
// MMA column c = 3 * (segment & 1) + digit, word t) holds eight bytes: the digits of the word's four
// even k, then of its four odd k, which is what lane t of a quad feeds into k slots 4t.. and
// 16 + 4t.. of the MMA. 192 bytes per (step, u).
constexpr int kBlock32Bytes = 6 * 32;

template <bool ROWPAIR, bool BLOCK32 = false>
__device__ __forceinline__ void ConvertWord(const float (&x)[8], float lift, float up, int word, int token,
                                            unsigned char *digits, int chunk_stride, int (&sums)[kDigits]) {
  std::uint32_t u0[8], u1[8], u2[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    u0[e] = static_cast<std::uint32_t>(__float2int_rn(fmaf(x[e] * lift, up, kDigitBias)));
    u1[e] = u0[e] << 1;
    u2[e] = u0[e] << 2;
  }
  std::uint32_t packed[kDigits][2];  // [digit][even k / odd k], four bytes each
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const std::uint32_t low =
        __byte_perm(__byte_perm(u0[h], u0[h + 2], 0x0040), __byte_perm(u0[h + 4], u0[h + 6], 0x0040), 0x5410);
    const std::uint32_t mid =
        __byte_perm(__byte_perm(u1[h], u1[h + 2], 0x0051), __byte_perm(u1[h + 4], u1[h + 6], 0x0051), 0x5410);
    const std::uint32_t high =
        __byte_perm(__byte_perm(u2[h], u2[h + 2], 0x0062), __byte_perm(u2[h + 4], u2[h + 6], 0x0062), 0x5410);
    // signed bytes: (d' + 64) ^ 0x80 = d' - 64 for d' in [0, 127]; d' ^ 0x80 = d' - 128
    packed[0][h] = high ^ 0x80808080u;
    packed[1][h] = ((mid & 0x7f7f7f7fu) + 0x40404040u) ^ 0x80808080u;
    packed[2][h] = ((low & 0x7f7f7f7fu) + 0x40404040u) ^ 0x80808080u;
  }
#pragma unroll
  for (int d = 0; d < kDigits; ++d) {
    sums[d] = __dp4a(static_cast<int>(packed[d][0]), 0x01010101, __dp4a(static_cast<int>(packed[d][1]), 0x01010101, 0));
  }
  const int seg = word >> 4;
  const int quad_lane = (word >> 2) & 3;
  const int word_in_lane = word & 3;
  if constexpr (BLOCK32) {
    unsigned char *at = digits + ((seg >> 1) * 4 + quad_lane) * kBlock32Bytes + (seg & 1) * kDigits * 32 + word_in_lane * 8;
#pragma unroll
    for (int d = 0; d < kDigits; ++d) {
      *reinterpret_cast<uint2 *>(at + d * 32) = make_uint2(packed[d][0], packed[d][1]);
    }
    return;
  }
  // the three chunks of a (segment, token) are 128 bytes apart and their swizzle bits alternate
  int swizzle;
  unsigned char *chunk = digits + ChunkOffset<ROWPAIR>(seg, token, 0, chunk_stride, &swizzle);
  unsigned char *even0 = chunk + (((2 * quad_lane) ^ swizzle) << 4) + word_in_lane * 4;
  unsigned char *odd0 = chunk + (((2 * quad_lane + 1) ^ swizzle) << 4) + word_in_lane * 4;
  *reinterpret_cast<std::uint32_t *>(even0) = packed[0][0];
  *reinterpret_cast<std::uint32_t *>(odd0) = packed[0][1];
  *reinterpret_cast<std::uint32_t *>(odd0 + kChunkBytes) = packed[1][0];   // swizzle flipped: even <-> odd place
  *reinterpret_cast<std::uint32_t *>(even0 + kChunkBytes) = packed[1][1];
  *reinterpret_cast<std::uint32_t *>(even0 + 2 * kChunkBytes) = packed[2][0];
  *reinterpret_cast<std::uint32_t *>(odd0 + 2 * kChunkBytes) = packed[2][1];
}

// What takes a row maximum to the digit scale: `up` multiplies the (lifted) activations, `undo`
// takes the integer result back (NaN for a row with a non-finite entry: all its outputs are NaN).
// Neither factor needs to be correctly rounded (a relative error of 1e-7 in `up` moves an integer
// that may reach kDigitRange by less than one, and the digits hold up to 2,023,359; `undo` scales
// every output of the row alike), so the reciprocal is the fast one.
__device__ __forceinline__ void DigitFactors(float amax, float *lift, float *up, float *undo) {
  const bool finite = amax < 3.0e38f;  // false for an infinite entry and for NaN
  // rows of very small magnitude are lifted by an exact power of two first, so that `up` stays finite
  const bool tiny = amax < 1.0e-18f;
  *lift = tiny ? 1.8446744e19f /* 2^64 */ : 1.0f;
  const float unlift = tiny ? 5.4210109e-20f /* 2^-64 */ : 1.0f;
  const float lifted = amax * *lift;
  *up = (finite && lifted > 0.0f) ? __fdividef(kDigitRange, lifted) : 0.0f;
  // the factor 16 of the merged even / odd block sums is taken out here
  *undo = finite ? (lifted * (1.0f / kDigitRange)) * unlift * 0.0625f : __int_as_float(0x7fc00000);
}

// Stages `tokens` activation rows as digit bytes and builds the digit-sum table. All threads of
// the CTA take part (two or three barriers). undo[token] takes the integer result back to the
// row's scale. Byte order inside a chunk (128 k of one segment): the lane t = k / 32 of a quad owns
// units 2t (even k) and 2t + 1 (odd k); inside a unit the word k % 32 / 8 owns four bytes.
// `issue_rest` is called once, right behind the first loads of A: the caller queues the rest of
// its weight prefetch there, BEHIND the activations. (Queued in front of them, as in a first
// version, three ring stages per warp delayed the activations by two to four microseconds: the
// load pipe serves requests in order.)
// `geo` describes the staged layout; `tid` / `threads` the threads that take part (all of them call
// this function) and `sync` their barrier.
struct DigitGeometry {
  int k;             // activations per row
  int segs;          // 128-k segments per padded row
  int chunk_stride;  // bytes between consecutive segments of the staged digits
  int table_ints;    // ints of the digit-sum table
};

template <bool ROWPAIR, bool BLOCK32 = false, typename Sync, typename IssueRest>
__device__ __forceinline__ void StageDigits(const DigitGeometry &geo, const float *a_rows, int tokens,
                                            int column_tiles, unsigned char *digits, int *table, float *undo,
                                            float *red, int tid, int threads, Sync &&sync, IssueRest &&issue_rest) {
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int warps = threads >> 5;
  const int k = geo.k;
  const int words_pad = geo.segs * 16;  // 8-k words per padded row
  const bool fast = (reinterpret_cast<std::uintptr_t>(a_rows) & 15u) == 0 && (k & 7) == 0;

  auto load_word = [&](const float *src, int word, float (&x)[8]) {
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

  constexpr int kHeld = 3;  // 8-k words a thread keeps in registers (one token, K <= 24 * threads)
  if (tokens == 1 && fast && words_pad <= kHeld * threads) {
    // one token: A is read once, into registers, ahead of the rest of the weight prefetch
    float held[kHeld][8];
#pragma unroll
    for (int j = 0; j < kHeld; ++j) {
      const int word = tid + j * threads;
      float4 lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi = lo;
      if ((word << 3) < k) {
        lo = LoadActivations4(a_rows + (word << 3));
        hi = LoadActivations4(a_rows + (word << 3) + 4);
      }
      held[j][0] = lo.x, held[j][1] = lo.y, held[j][2] = lo.z, held[j][3] = lo.w;
      held[j][4] = hi.x, held[j][5] = hi.y, held[j][6] = hi.z, held[j][7] = hi.w;
    }
    issue_rest();
    // the table entries nothing writes below (unused MMA columns) are cleared while A is on its way
    for (int entry = tid; entry < geo.table_ints; entry += threads) {
      table[entry] = 0;
    }
    float amax = 0.0f;  // NaN as soon as the row holds one (max.NaN)
#pragma unroll
    for (int j = 0; j < kHeld; ++j) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        amax = MaxNan(amax, fabsf(held[j][e]));
      }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      amax = MaxNan(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
    }
    if (lane == 0) {
      red[warp] = amax;
    }
    sync();
    amax = red[0];
    for (int i = 1; i < warps; ++i) {
      amax = MaxNan(amax, red[i]);
    }
    float lift, up, back;
    DigitFactors(amax, &lift, &up, &back);
    if (tid == 0) {
      undo[0] = back;
    }
    // digit sums ride along: a 128-k segment is sixteen words = one half warp
#pragma unroll
    for (int j = 0; j < kHeld; ++j) {
      const int word = tid + j * threads;
      const bool valid = word < words_pad;  // the same for the sixteen lanes of a segment
      int sums[kDigits] = {0, 0, 0};
      if (valid) {
        ConvertWord<ROWPAIR, BLOCK32>(held[j], lift, up, word, 0, digits, geo.chunk_stride, sums);
      }
      if constexpr (BLOCK32) {
        // a 32-k block is four words = four neighbouring lanes
#pragma unroll
        for (int offset = 2; offset > 0; offset >>= 1) {
#pragma unroll
          for (int d = 0; d < kDigits; ++d) {
            sums[d] += __shfl_xor_sync(0xffffffffu, sums[d], offset);
          }
        }
        if (valid && (lane & 3) == 0) {
          const int seg = word >> 4;
          int *entry = table + ((seg >> 1) * 4 + ((word >> 2) & 3)) * 8 + (seg & 1) * kDigits;
          entry[0] = -sums[0];
          entry[1] = -sums[1];
          entry[2] = -sums[2];
        }
        continue;
      }
#pragma unroll
      for (int offset = 8; offset > 0; offset >>= 1) {
#pragma unroll
        for (int d = 0; d < kDigits; ++d) {
          sums[d] += __shfl_xor_sync(0xffffffffu, sums[d], offset);
        }
      }
      if (valid && (lane & 15) == 0) {
        const int seg = word >> 4;
        // entry (step, column): row-pair mode keeps the even segment in columns 0..2, the odd one in 3..5
        int *entry = ROWPAIR ? table + (seg >> 1) * 8 + (seg & 1) * kDigits : table + seg * column_tiles * 8;
        entry[0] = -sums[0];
        entry[1] = -sums[1];
        entry[2] = -sums[2];
      }
    }
    sync();
    return;
  } else {
    for (int token = 0; token < tokens; ++token) {
      const float *src = a_rows + static_cast<std::int64_t>(token) * k;
      float amax = 0.0f;
      for (int word = tid; word < words_pad; word += threads) {
        float x[8];
        load_word(src, word, x);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          amax = MaxNan(amax, fabsf(x[e]));
        }
      }
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) {
        amax = MaxNan(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
      }
      if (lane == 0) {
        red[token * kMaxWarps + warp] = amax;
      }
    }
    issue_rest();
    sync();
    for (int token = 0; token < tokens; ++token) {
      const float *src = a_rows + static_cast<std::int64_t>(token) * k;
      float amax = red[token * kMaxWarps];
      for (int i = 1; i < warps; ++i) {
        amax = MaxNan(amax, red[token * kMaxWarps + i]);
      }
      float lift, up, back;
      DigitFactors(amax, &lift, &up, &back);
      if (tid == 0) {
        undo[token] = back;
      }
      for (int word = tid; word < words_pad; word += threads) {
        float x[8];
        load_word(src, word, x);
        int unused[kDigits];
        ConvertWord<ROWPAIR, BLOCK32>(x, lift, up, word, token, digits, geo.chunk_stride, unused);
      }
    }
  }
  sync();
  // digit sums: entry (step, column tile, MMA column) -> sum of the 128 digits that column sees in
  // that step (0 for the unused columns)
  for (int entry = tid; entry < geo.table_ints; entry += threads) {
    const int column = entry & 7;
    if constexpr (BLOCK32) {
      // entry ((step, u), column): the 32 digits of that block and column
      int sum = 0;
      if (column < 2 * kDigits) {
        const uint4 *bytes = reinterpret_cast<const uint4 *>(digits + (entry >> 3) * kBlock32Bytes + column * 32);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint4 q = bytes[i];
          sum = __dp4a(static_cast<int>(q.x), 0x01010101, sum);
          sum = __dp4a(static_cast<int>(q.y), 0x01010101, sum);
          sum = __dp4a(static_cast<int>(q.z), 0x01010101, sum);
          sum = __dp4a(static_cast<int>(q.w), 0x01010101, sum);
        }
      }
      table[entry] = -sum;
      continue;
    }
    int seg, token, digit;
    bool used = column < 2 * kDigits;
    digit = column % kDigits;
    if constexpr (ROWPAIR) {
      seg = 2 * (entry >> 3) + (column >= kDigits ? 1 : 0);
      token = 0;
    } else {
      const int tile = (entry >> 3) % column_tiles;
      seg = (entry >> 3) / column_tiles;
      token = 2 * tile + (column >= kDigits ? 1 : 0);
      used = used && token < tokens;
    }
    int sum = 0;
    if (used) {
      int swizzle;
      const uint4 *bytes =
          reinterpret_cast<const uint4 *>(digits + ChunkOffset<ROWPAIR>(seg, token, digit, geo.chunk_stride, &swizzle));
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 q = bytes[i];
        sum = __dp4a(static_cast<int>(q.x), 0x01010101, sum);
        sum = __dp4a(static_cast<int>(q.y), 0x01010101, sum);
        sum = __dp4a(static_cast<int>(q.z), 0x01010101, sum);
        sum = __dp4a(static_cast<int>(q.w), 0x01010101, sum);
      }
    }
    table[entry] = -sum;  // negated: the correction is then a multiply-add
  }
  sync();
}

// Shared-memory loads of the staged digits and their sums. Volatile: executed exactly once where
// they stand (a plain asm statement was duplicated by the compiler instead of keeping its result
// in registers: four extra loads per step).
template <int OFFSET>
__device__ __forceinline__ uint4 LoadSharedConst16(std::uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4 + %5];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "r"(addr), "n"(OFFSET));
  return v;
}

template <int OFFSET>
__device__ __forceinline__ int2 LoadSharedConst8(std::uint32_t addr) {
  int2 v;
  asm volatile("ld.shared.v2.s32 {%0, %1}, [%2 + %3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFFSET));
  return v;
}

__device__ __forceinline__ std::uint32_t LaunderAfterBarrier(std::uint32_t value) {
  std::uint32_t out;
  asm volatile("mov.u32 %0, %1;" : "=r"(out) : "r"(value) : "memory");
  return out;
}


} // namespace
} // namespace mnb
