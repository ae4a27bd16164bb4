// MatMulNBits decode for 8-bit weights, up to sixteen tokens, accuracy_level 0, on integer tensor cores.
//
// The arithmetic of the 4-bit digit kernels (nbits_digits.cuh) with nothing to unpack: an 8-bit code is
// an unsigned-byte MMA operand as it lies in B. Each activation row is scaled so that its largest
// magnitude becomes 2e6 and rounded to n = 16384 d0 + 128 d1 + d2 with balanced base-128 digits; the
// digits of the tokens are signed-byte MMA columns (digit-major: column tile d * NTOK + j holds digit
// d of tokens 8 j ... 8 j + 7, so the three digits of a token meet in one lane and register). Per
// quantization block the three int32 sums are exact (< 2^24 for blocks of up to 256); the zero point
// leaves as e - zp * (sum of the block's digits) in int32, for the high digit on its own and for
// 128 e1 + e2 together; 16384 f0 + f12 in fp32 and one FFMA applies the block's scale. The row factor max / 2e6 and the bias
// are applied at the end.
//
// Two launches: a small kernel writes the digit bytes, the per-block digit sums and the row factors
// of all tokens; the multiply kernel gives every warp sixteen weight rows and a part of K. The weights
// travel as loads of 2 rows x 256 contiguous bytes (a warp that reads its MMA fragments straight from
// global memory asks for 32 bytes from each of sixteen rows per load: 1 TB/s), wait in registers while
// the tile before is used, and are parked in a tile of shared memory of the warp's own; the digits come
// through L1. No barrier in the loop but the warp's own; one in front of the sum over the parts of K.
#include "nbits_common.cuh"
#include "nbits_digits.cuh"

#include <cstdint>

namespace mnb {
namespace {

constexpr int kU8Warps = 8;
constexpr int kU8MaxSteps = 1024;     // 32-k steps of a row the digit kernel keeps sums for: K <= 32768
constexpr int kU8DigitBiasInt = 64 + 64 * 128 + 128 * 16384;

struct U8Layout {
  int steps;              // 32-k steps of a packed row (padding included)
  int cols;               // MMA columns: 3 digits x 8 NTOK tokens
  std::size_t sums_offset;
  std::size_t undo_offset;
  std::size_t total;
};

U8Layout LayoutFor(const WeightView &w, int ntok) {
  U8Layout l{};
  l.steps = w.row_bytes / 32;
  l.cols = kDigits * 8 * ntok;
  const std::size_t digits = static_cast<std::size_t>(l.steps) * l.cols * 32;
  l.sums_offset = (digits + 255) & ~std::size_t{255};
  const std::size_t sums = static_cast<std::size_t>(w.n_blocks) * 2 * 8 * ntok * sizeof(int);
  l.undo_offset = (l.sums_offset + sums + 255) & ~std::size_t{255};
  l.total = l.undo_offset + 8 * ntok * sizeof(float);
  return l;
}

// One CTA of 1024 threads per token slot (tokens beyond M get zeros), a thread per four consecutive k.
// Digits: [step][column][32 k] signed bytes, column = digit * tokens_pad + token. Sums: [block][2][token]
// int32: the block's sum of the high digits, and 128 * (sum of the middle digits) + (sum of the low ones).
// undo: [token].
constexpr int kU8DigitThreads = 1024;

__global__ void __launch_bounds__(kU8DigitThreads)
    nbits_u8_digits_kernel(const float *a, int m_total, std::int64_t k_total, int steps, int cols, int tokens_pad,
                           int steps_per_block, int n_blocks, signed char *digits, int *sums, float *undo,
                           int a_vector) {
  __shared__ float reduce[kU8DigitThreads / 32];
  __shared__ int step_sums[kU8MaxSteps][kDigits];
  // the multiply kernel behind this one may start on its first tile of weights right away
  ptx::GridDependencyLaunch();
  const int token = blockIdx.x;
  const int tid = threadIdx.x;
  const bool live = token < m_total;
  const float *row = a + static_cast<std::int64_t>(live ? token : 0) * k_total;
  const int words = steps * 8;

  auto load_word = [&](int word) {
    const std::int64_t k0 = static_cast<std::int64_t>(word) * 4;
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (a_vector != 0 && k0 + 4 <= k_total) {
      v = __ldg(reinterpret_cast<const float4 *>(row + k0));
    } else {
      v.x = k0 + 0 < k_total ? __ldg(row + k0 + 0) : 0.0f;
      v.y = k0 + 1 < k_total ? __ldg(row + k0 + 1) : 0.0f;
      v.z = k0 + 2 < k_total ? __ldg(row + k0 + 2) : 0.0f;
      v.w = k0 + 3 < k_total ? __ldg(row + k0 + 3) : 0.0f;
    }
    return v;
  };

  float amax = 0.0f;
  if (live) {
    for (int word = tid; word < words; word += kU8DigitThreads) {
      const float4 v = load_word(word);
      amax = MaxNan(MaxNan(amax, MaxNan(fabsf(v.x), fabsf(v.y))), MaxNan(fabsf(v.z), fabsf(v.w)));
    }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    amax = MaxNan(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  }
  if ((tid & 31) == 0) {
    reduce[tid >> 5] = amax;
  }
  __syncthreads();
  amax = reduce[0];
#pragma unroll
  for (int i = 1; i < kU8DigitThreads / 32; ++i) {
    amax = MaxNan(amax, reduce[i]);
  }
  // a NaN or an infinity in the row ends in the row factor, and so in every output of the token
  const bool usable = live && amax > 0.0f && amax <= 3.0e38f;
  if (tid == 0) {
    undo[token] = live ? amax / kDigitRange : 0.0f;
  }
  // x * lift * up = x / amax * 2e6 without an overflow of the reciprocal for a tiny maximum
  const float lift = amax < 1.0e-30f ? 1.8446744e19f : 1.0f;   // 2^64, exact
  const float up = usable ? kDigitRange / (amax * lift) : 0.0f;

  for (int base = 0; base < words; base += kU8DigitThreads) {
    const int word = base + tid;
    int total[kDigits] = {0, 0, 0};
    if (word < words) {
      const float4 v = load_word(word);
      const float x[4] = {v.x, v.y, v.z, v.w};
      std::uint32_t packed[kDigits] = {0u, 0u, 0u};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = usable ? __float2int_rn(x[e] * lift * up) : 0;
        const int u = n + kU8DigitBiasInt;  // 0 < u < 2^22: its plain base-128 digits, minus 128 / 64 / 64
        const int d0 = (u >> 14) - 128;
        const int d1 = ((u >> 7) & 127) - 64;
        const int d2 = (u & 127) - 64;
        total[0] += d0, total[1] += d1, total[2] += d2;
        packed[0] |= static_cast<std::uint32_t>(d0 & 0xff) << (8 * e);
        packed[1] |= static_cast<std::uint32_t>(d1 & 0xff) << (8 * e);
        packed[2] |= static_cast<std::uint32_t>(d2 & 0xff) << (8 * e);
      }
      const int step = word >> 3;
#pragma unroll
      for (int d = 0; d < kDigits; ++d) {
        *reinterpret_cast<std::uint32_t *>(digits + (static_cast<std::size_t>(step) * cols + d * tokens_pad + token) * 32 +
                                           (word & 7) * 4) = packed[d];
      }
    }
    // the eight words of a step sit in eight neighbouring lanes
#pragma unroll
    for (int d = 0; d < kDigits; ++d) {
      total[d] += __shfl_xor_sync(0xffffffffu, total[d], 1);
      total[d] += __shfl_xor_sync(0xffffffffu, total[d], 2);
      total[d] += __shfl_xor_sync(0xffffffffu, total[d], 4);
    }
    if (word < words && (word & 7) == 0) {
#pragma unroll
      for (int d = 0; d < kDigits; ++d) {
        step_sums[word >> 3][d] = total[d];
      }
    }
  }
  __syncthreads();
  for (int block = tid; block < n_blocks; block += kU8DigitThreads) {
    int total[kDigits] = {0, 0, 0};
    for (int s = 0; s < steps_per_block; ++s) {
      const int step = block * steps_per_block + s;
      if (step < steps) {
#pragma unroll
        for (int d = 0; d < kDigits; ++d) {
          total[d] += step_sums[step][d];
        }
      }
    }
    sums[static_cast<std::size_t>(block) * 2 * tokens_pad + token] = total[0];
    sums[static_cast<std::size_t>(block) * 2 * tokens_pad + tokens_pad + token] = 128 * total[1] + total[2];
  }
}

// 16 bytes of weights that are used once: past L1, which keeps the digits.
__device__ __forceinline__ uint4 LoadStreaming16(const void *ptr) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

struct U8Params {
  WeightView w;
  const unsigned char *digits;
  const int *sums;
  const float *undo;
  OutputView out;
  int m_total;
  int parts;            // warps that share a row tile, each on a run of quantization blocks
  int blocks_per_part;
  int steps;
  int tiles;
};

constexpr int kU8Super = 8;                              // 32-k steps per tile of weights
constexpr int kU8TileRowBytes = kU8Super * 32 + 32;      // 256 bytes of a row, padded: fragment reads hit 32 banks
constexpr int kU8TileBytes = 16 * kU8TileRowBytes;

// SPB = 32-k steps per quantization block (1, 2, 4, 8): a part of K starts on a block and tiles are eight steps,
// so where a block starts and ends inside a tile is known at compile time (a fresh accumulator there, no
// clearing, no test per step).
template <int NTOK, int SPB>
__global__ void __launch_bounds__(kU8Warps * 32)
    nbits_gemv_u8_mma_kernel(const U8Params p) {
  static_assert(SPB == 1 || SPB == 2 || SPB == 4 || SPB == 8, "blocks of 32 ... 256");
  constexpr int NT = kDigits * NTOK;   // MMA column tiles
  constexpr int kCols = NT * 8;
  __shared__ __align__(16) unsigned char tiles[kU8Warps][kU8TileBytes];
  __shared__ float meet[kU8Warps][NTOK * 4][32];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int part = warp % p.parts;
  const int tile = blockIdx.x * (kU8Warps / p.parts) + warp / p.parts;
  const bool live = tile < p.tiles;
  const std::int64_t row0 = static_cast<std::int64_t>(live ? tile : 0) * 16;
  // rows beyond N repeat the last one; their sums are not written
  const std::int64_t r_lo = row0 + g < p.w.n ? row0 + g : p.w.n - 1;
  const std::int64_t r_hi = row0 + g + 8 < p.w.n ? row0 + g + 8 : p.w.n - 1;
  const float *scale_lo = p.w.scales + r_lo * p.w.n_blocks;
  const float *scale_hi = p.w.scales + r_hi * p.w.n_blocks;
  const std::uint8_t *zp_lo = p.w.zp != nullptr ? p.w.zp + r_lo * p.w.zp_row_bytes : nullptr;
  const std::uint8_t *zp_hi = p.w.zp != nullptr ? p.w.zp + r_hi * p.w.zp_row_bytes : nullptr;
  // digits of column g of every column tile, this lane's eight k of a step
  const unsigned char *digit_lane = p.digits + g * 32 + 8 * t;
  const int *sum_lane = p.sums + 2 * t;
  // the weights of sixteen rows x 256 k travel as eight loads of 2 rows x 256 bytes (sixteen lanes along K
  // per row), are parked in shared memory and read back as MMA fragments
  unsigned char *my_tile = tiles[warp];
  const int copy_row = lane >> 4;          // + 2 i
  const int copy_byte = (lane & 15) * 16;
  const unsigned char *frag_lo = my_tile + g * kU8TileRowBytes + 8 * t;
  const unsigned char *frag_hi = frag_lo + 8 * kU8TileRowBytes;

  float acc[NTOK][4];
#pragma unroll
  for (int j = 0; j < NTOK; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[j][i] = 0.0f;
    }
  }
  int block_begin = part * p.blocks_per_part;
  int block_end = block_begin + p.blocks_per_part < p.w.n_blocks ? block_begin + p.blocks_per_part : p.w.n_blocks;
  if (!live || block_begin > block_end) {
    block_begin = block_end = 0;
  }
  const int s_begin = block_begin * SPB;
  const int s_end = block_end * SPB < p.steps ? block_end * SPB : p.steps;

  uint4 next[kU8Super];
  auto request = [&](int s_first) {
    const int byte = s_first * 32 + copy_byte;
    const bool inside = byte + 16 <= s_end * 32;
#pragma unroll
    for (int i = 0; i < kU8Super; ++i) {
      const std::int64_t row = row0 + 2 * i + copy_row < p.w.n ? row0 + 2 * i + copy_row : p.w.n - 1;
      next[i] = make_uint4(0u, 0u, 0u, 0u);
      if (inside) {
        next[i] = LoadStreaming16(p.w.b + row * p.w.row_bytes + byte);
      }
    }
  };
  if (s_begin < s_end) {
    request(s_begin);
  }
  // the digits come from the kernel launched just before; the weights above do not depend on it
  ptx::GridDependencyWait();
  int d[NT][4];
  const ZeroQuad zero = MakeZeroQuad();
#pragma unroll 1
  for (int s0 = s_begin; s0 < s_end; s0 += kU8Super) {
    __syncwarp(); // the tile before has been read
#pragma unroll
    for (int i = 0; i < kU8Super; ++i) {
      *reinterpret_cast<uint4 *>(my_tile + (2 * i + copy_row) * kU8TileRowBytes + copy_byte) = next[i];
    }
    __syncwarp();
    if (s0 + kU8Super < s_end) {
      request(s0 + kU8Super);
    }
    // the digits of a step are asked for one step ahead (a step beyond the part reads the last one again)
    uint2 bq[2][NT];
    {
      const unsigned char *digit_step = digit_lane + s0 * (kCols * 32);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        bq[0][nt] = __ldg(reinterpret_cast<const uint2 *>(digit_step + nt * 256));
      }
    }
#pragma unroll
    for (int u = 0; u < kU8Super; ++u) {
      const int s = s0 + u;
      if (s < s_end) {
        const uint2 lo = *reinterpret_cast<const uint2 *>(frag_lo + u * 32);
        const uint2 hi = *reinterpret_cast<const uint2 *>(frag_hi + u * 32);
        if (u + 1 < kU8Super) {
          const int ahead = s + 1 < s_end ? s + 1 : s;
          const unsigned char *digit_step = digit_lane + ahead * (kCols * 32);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            bq[(u + 1) & 1][nt] = __ldg(reinterpret_cast<const uint2 *>(digit_step + nt * 256));
          }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          // k slots 4 t ... of the MMA: bytes 8 t ... 8 t + 3 of the step; slots 16 + 4 t ...: bytes 8 t + 4 ...
          if (u % SPB == 0) {
            ImmaFresh(d[nt], lo.x, hi.x, lo.y, hi.y, bq[u & 1][nt].x, bq[u & 1][nt].y, zero);
          } else {
            ImmaAdd(d[nt], lo.x, hi.x, lo.y, hi.y, bq[u & 1][nt].x, bq[u & 1][nt].y);
          }
        }
        if ((u + 1) % SPB == 0) {
          // a quantization block is complete
          const int block = s / SPB;
          const float ws_lo = __ldg(scale_lo + block);
          const float ws_hi = __ldg(scale_hi + block);
          const int z_lo = zp_lo != nullptr ? static_cast<int>(__ldg(zp_lo + block)) : 128;
          const int z_hi = zp_hi != nullptr ? static_cast<int>(__ldg(zp_hi + block)) : 128;
          const int *sum_block = sum_lane + block * (2 * 8 * NTOK);
#pragma unroll
          for (int j = 0; j < NTOK; ++j) {
            // high digit on its own, middle and low digit combined in int32 (|128 e1 + e2| < 2^30 for blocks
            // of up to 256), the zero point out of both in int32, then 16384 f0 + f12 in fp32
            const int2 s_high = __ldg(reinterpret_cast<const int2 *>(sum_block + j * 8));
            const int2 s_rest = __ldg(reinterpret_cast<const int2 *>(sum_block + (NTOK + j) * 8));
            const int *e0 = d[j];
            const int *e1 = d[NTOK + j];
            const int *e2 = d[2 * NTOK + j];
            const float f0 = fmaf(16384.0f, static_cast<float>(e0[0] - z_lo * s_high.x),
                                  static_cast<float>(128 * e1[0] + e2[0] - z_lo * s_rest.x));
            const float f1 = fmaf(16384.0f, static_cast<float>(e0[1] - z_lo * s_high.y),
                                  static_cast<float>(128 * e1[1] + e2[1] - z_lo * s_rest.y));
            const float f2 = fmaf(16384.0f, static_cast<float>(e0[2] - z_hi * s_high.x),
                                  static_cast<float>(128 * e1[2] + e2[2] - z_hi * s_rest.x));
            const float f3 = fmaf(16384.0f, static_cast<float>(e0[3] - z_hi * s_high.y),
                                  static_cast<float>(128 * e1[3] + e2[3] - z_hi * s_rest.y));
            acc[j][0] = fmaf(ws_lo, f0, acc[j][0]);
            acc[j][1] = fmaf(ws_lo, f1, acc[j][1]);
            acc[j][2] = fmaf(ws_hi, f2, acc[j][2]);
            acc[j][3] = fmaf(ws_hi, f3, acc[j][3]);
          }
        }
      }
    }
  }

  // the parts of K of a row tile meet in shared memory; the first part's warp writes the rows
#pragma unroll
  for (int j = 0; j < NTOK; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      meet[warp][j * 4 + i][lane] = acc[j][i];
    }
  }
  __syncthreads();
  if (live && part == 0) {
#pragma unroll
    for (int j = 0; j < NTOK; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float total = acc[j][i];
        for (int other = 1; other < p.parts; ++other) {
          total += meet[warp + other][j * 4 + i][lane];
        }
        const int token = 8 * j + 2 * t + (i & 1);
        const std::int64_t row = row0 + g + (i >> 1) * 8;
        if (token < p.m_total && row < p.w.n) {
          const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + row) : 0.0f;
          p.out.y[static_cast<std::int64_t>(token) * p.out.ld + p.out.col_offset + row] =
              fmaf(total, __ldg(p.undo + token), bias);
        }
      }
    }
  }
}

// ---- accuracy_level 4 on the same structure -----------------------------------------------------------
// The quantized activations (signed bytes, one scale per token and block) are the MMA columns themselves:
// one column tile per eight tokens, e - zp * (sum of the block's quantized activations) in int32, one
// conversion and one FFMA with activation scale x weight scale per output and block.

// sums[token][block] of the quantized activations; aq rows are zero beyond K.
__global__ void __launch_bounds__(256)
    nbits_u8_aq_sums_kernel(const signed char *aq, int m_total, int n_blocks, int block_size, std::int64_t aq_ld,
                            int *sums) {
  const int item = blockIdx.x * 256 + threadIdx.x;
  if (item >= m_total * n_blocks) {
    return;
  }
  const int token = item / n_blocks;
  const int block = item - token * n_blocks;
  const uint4 *src = reinterpret_cast<const uint4 *>(aq + token * aq_ld + static_cast<std::int64_t>(block) * block_size);
  int total = 0;
  for (int i = 0; i < block_size / 16; ++i) {
    const uint4 v = __ldg(src + i);
    total = __dp4a(static_cast<int>(v.x), 0x01010101, total);
    total = __dp4a(static_cast<int>(v.y), 0x01010101, total);
    total = __dp4a(static_cast<int>(v.z), 0x01010101, total);
    total = __dp4a(static_cast<int>(v.w), 0x01010101, total);
  }
  sums[item] = total;
}

struct U8Int8Params {
  WeightView w;
  const signed char *aq;   // [m][aq_ld], aq_ld = n_blocks * block_size
  std::int64_t aq_ld;
  const float *a_scales;   // [m][n_blocks]
  const int *sums;         // [m][n_blocks]
  OutputView out;
  int m_total;
  int parts;
  int blocks_per_part;
  int steps;
  int tiles;
};

template <int NTOK, int SPB>
__global__ void __launch_bounds__(kU8Warps * 32)
    nbits_gemv_u8_int8_mma_kernel(const U8Int8Params p) {
  static_assert(SPB == 1 || SPB == 2 || SPB == 4 || SPB == 8, "blocks of 32 ... 256");
  __shared__ __align__(16) unsigned char tiles[kU8Warps][kU8TileBytes];
  __shared__ float meet[kU8Warps][NTOK * 4][32];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int part = warp % p.parts;
  const int tile = blockIdx.x * (kU8Warps / p.parts) + warp / p.parts;
  const bool live = tile < p.tiles;
  const std::int64_t row0 = static_cast<std::int64_t>(live ? tile : 0) * 16;
  const std::int64_t r_lo = row0 + g < p.w.n ? row0 + g : p.w.n - 1;
  const std::int64_t r_hi = row0 + g + 8 < p.w.n ? row0 + g + 8 : p.w.n - 1;
  const float *scale_lo = p.w.scales + r_lo * p.w.n_blocks;
  const float *scale_hi = p.w.scales + r_hi * p.w.n_blocks;
  const std::uint8_t *zp_lo = p.w.zp != nullptr ? p.w.zp + r_lo * p.w.zp_row_bytes : nullptr;
  const std::uint8_t *zp_hi = p.w.zp != nullptr ? p.w.zp + r_hi * p.w.zp_row_bytes : nullptr;
  // MMA column g of tile j is token 8 j + g; outputs of this lane are tokens 8 j + 2 t and 8 j + 2 t + 1.
  // Tokens beyond M repeat the last one; their sums are not written.
  const signed char *act_lane[NTOK];
  int token_a[NTOK], token_b[NTOK];
#pragma unroll
  for (int j = 0; j < NTOK; ++j) {
    const int column = 8 * j + g < p.m_total ? 8 * j + g : p.m_total - 1;
    act_lane[j] = p.aq + column * p.aq_ld + 8 * t;
    token_a[j] = 8 * j + 2 * t < p.m_total ? 8 * j + 2 * t : p.m_total - 1;
    token_b[j] = 8 * j + 2 * t + 1 < p.m_total ? 8 * j + 2 * t + 1 : p.m_total - 1;
  }
  unsigned char *my_tile = tiles[warp];
  const int copy_row = lane >> 4;
  const int copy_byte = (lane & 15) * 16;
  const unsigned char *frag_lo = my_tile + g * kU8TileRowBytes + 8 * t;
  const unsigned char *frag_hi = frag_lo + 8 * kU8TileRowBytes;

  float acc[NTOK][4];
#pragma unroll
  for (int j = 0; j < NTOK; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[j][i] = 0.0f;
    }
  }
  int block_begin = part * p.blocks_per_part;
  int block_end = block_begin + p.blocks_per_part < p.w.n_blocks ? block_begin + p.blocks_per_part : p.w.n_blocks;
  if (!live || block_begin > block_end) {
    block_begin = block_end = 0;
  }
  const int s_begin = block_begin * SPB;
  const int s_end = block_end * SPB < p.steps ? block_end * SPB : p.steps;

  uint4 next[kU8Super];
  auto request = [&](int s_first) {
    const int byte = s_first * 32 + copy_byte;
    const bool inside = byte + 16 <= s_end * 32;
#pragma unroll
    for (int i = 0; i < kU8Super; ++i) {
      const std::int64_t row = row0 + 2 * i + copy_row < p.w.n ? row0 + 2 * i + copy_row : p.w.n - 1;
      next[i] = make_uint4(0u, 0u, 0u, 0u);
      if (inside) {
        next[i] = LoadStreaming16(p.w.b + row * p.w.row_bytes + byte);
      }
    }
  };
  if (s_begin < s_end) {
    request(s_begin);
  }
  int d[NTOK][4];
  const ZeroQuad zero = MakeZeroQuad();
#pragma unroll 1
  for (int s0 = s_begin; s0 < s_end; s0 += kU8Super) {
    __syncwarp(); // the tile before has been read
#pragma unroll
    for (int i = 0; i < kU8Super; ++i) {
      *reinterpret_cast<uint4 *>(my_tile + (2 * i + copy_row) * kU8TileRowBytes + copy_byte) = next[i];
    }
    __syncwarp();
    if (s0 + kU8Super < s_end) {
      request(s0 + kU8Super);
    }
#pragma unroll
    for (int u = 0; u < kU8Super; ++u) {
      const int s = s0 + u;
      if (s < s_end) {
        const uint2 lo = *reinterpret_cast<const uint2 *>(frag_lo + u * 32);
        const uint2 hi = *reinterpret_cast<const uint2 *>(frag_hi + u * 32);
#pragma unroll
        for (int j = 0; j < NTOK; ++j) {
          const uint2 bq = __ldg(reinterpret_cast<const uint2 *>(act_lane[j] + s * 32));
          if (u % SPB == 0) {
            ImmaFresh(d[j], lo.x, hi.x, lo.y, hi.y, bq.x, bq.y, zero);
          } else {
            ImmaAdd(d[j], lo.x, hi.x, lo.y, hi.y, bq.x, bq.y);
          }
        }
        if ((u + 1) % SPB == 0) {
          // a quantization block is complete
          const int block = s / SPB;
          const float ws_lo = __ldg(scale_lo + block);
          const float ws_hi = __ldg(scale_hi + block);
          const int z_lo = zp_lo != nullptr ? static_cast<int>(__ldg(zp_lo + block)) : 128;
          const int z_hi = zp_hi != nullptr ? static_cast<int>(__ldg(zp_hi + block)) : 128;
#pragma unroll
          for (int j = 0; j < NTOK; ++j) {
            const float sa_a = __ldg(p.a_scales + token_a[j] * p.w.n_blocks + block);
            const float sa_b = __ldg(p.a_scales + token_b[j] * p.w.n_blocks + block);
            const int sum_a = __ldg(p.sums + token_a[j] * p.w.n_blocks + block);
            const int sum_b = __ldg(p.sums + token_b[j] * p.w.n_blocks + block);
            acc[j][0] = fmaf(sa_a * ws_lo, static_cast<float>(d[j][0] - z_lo * sum_a), acc[j][0]);
            acc[j][1] = fmaf(sa_b * ws_lo, static_cast<float>(d[j][1] - z_lo * sum_b), acc[j][1]);
            acc[j][2] = fmaf(sa_a * ws_hi, static_cast<float>(d[j][2] - z_hi * sum_a), acc[j][2]);
            acc[j][3] = fmaf(sa_b * ws_hi, static_cast<float>(d[j][3] - z_hi * sum_b), acc[j][3]);
          }
        }
      }
    }
  }

#pragma unroll
  for (int j = 0; j < NTOK; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      meet[warp][j * 4 + i][lane] = acc[j][i];
    }
  }
  __syncthreads();
  if (live && part == 0) {
#pragma unroll
    for (int j = 0; j < NTOK; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float total = acc[j][i];
        for (int other = 1; other < p.parts; ++other) {
          total += meet[warp + other][j * 4 + i][lane];
        }
        const int token = 8 * j + 2 * t + (i & 1);
        const std::int64_t row = row0 + g + (i >> 1) * 8;
        if (token < p.m_total && row < p.w.n) {
          const float bias = p.w.bias != nullptr ? __ldg(p.w.bias + row) : 0.0f;
          p.out.y[static_cast<std::int64_t>(token) * p.out.ld + p.out.col_offset + row] = total + bias;
        }
      }
    }
  }
}

// Warps per row tile: towards sixteen warps per SM, every part at least four blocks.
int PartsFor(const WeightView &w, int tiles, int sm_count) {
  const std::int64_t wanted = std::int64_t{16} * (sm_count > 0 ? sm_count : 148);
  int parts = 1;
  while (parts < kU8Warps && static_cast<std::int64_t>(tiles) * parts < wanted && w.n_blocks >= 8 * parts) {
    parts *= 2;
  }
  return parts;
}

template <int NTOK>
cudaError_t LaunchU8Int8(const U8Int8Params &p, int steps_per_block, unsigned grid, cudaStream_t stream) {
  switch (steps_per_block) {
  case 1: nbits_gemv_u8_int8_mma_kernel<NTOK, 1><<<grid, kU8Warps * 32, 0, stream>>>(p); break;
  case 2: nbits_gemv_u8_int8_mma_kernel<NTOK, 2><<<grid, kU8Warps * 32, 0, stream>>>(p); break;
  case 4: nbits_gemv_u8_int8_mma_kernel<NTOK, 4><<<grid, kU8Warps * 32, 0, stream>>>(p); break;
  case 8: nbits_gemv_u8_int8_mma_kernel<NTOK, 8><<<grid, kU8Warps * 32, 0, stream>>>(p); break;
  default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

} // namespace

const char *LaunchGemvU8Int8Mma(const WeightView &w, const std::int8_t *aq, const float *a_scales, std::int64_t m,
                                int *sums, OutputView out, cudaStream_t stream, int sm_count) {
  if (!GemvU8MmaSupports(w, m) || sums == nullptr || (reinterpret_cast<std::uintptr_t>(aq) & 15u) != 0) {
    return nullptr;
  }
  const std::int64_t aq_ld = static_cast<std::int64_t>(w.n_blocks) * w.block_size;
  const int items = static_cast<int>(m) * w.n_blocks;
  nbits_u8_aq_sums_kernel<<<(items + 255) / 256, 256, 0, stream>>>(reinterpret_cast<const signed char *>(aq),
                                                                   static_cast<int>(m), w.n_blocks, w.block_size, aq_ld,
                                                                   sums);
  if (cudaGetLastError() != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  U8Int8Params p{};
  p.w = w;
  p.aq = reinterpret_cast<const signed char *>(aq);
  p.aq_ld = aq_ld;
  p.a_scales = a_scales;
  p.sums = sums;
  p.out = out;
  p.m_total = static_cast<int>(m);
  p.steps = w.row_bytes / 32;
  p.tiles = static_cast<int>((w.n + 15) / 16);
  p.parts = PartsFor(w, p.tiles, sm_count);
  p.blocks_per_part = (w.n_blocks + p.parts - 1) / p.parts;
  const int tiles_per_cta = kU8Warps / p.parts;
  const unsigned grid = static_cast<unsigned>((p.tiles + tiles_per_cta - 1) / tiles_per_cta);
  const cudaError_t launched = m <= 8 ? LaunchU8Int8<1>(p, w.block_size / 32, grid, stream)
                                      : LaunchU8Int8<2>(p, w.block_size / 32, grid, stream);
  if (launched != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  CountLaunch();
  return "nbits_gemv_u8_int8_mma_kernel";
}

bool GemvU8MmaSupports(const WeightView &w, std::int64_t m) {
  return w.bits == 8 && m >= 1 && m <= 16 && w.block_size >= 32 && w.block_size <= 256 && w.n >= 1 && w.k >= 1 &&
         w.row_bytes / 32 <= kU8MaxSteps && (reinterpret_cast<std::uintptr_t>(w.b) & 15u) == 0;
}

std::size_t GemvU8MmaScratchBytes(const WeightView &w, std::int64_t m) {
  if (!GemvU8MmaSupports(w, m)) {
    return 0;
  }
  return LayoutFor(w, m <= 8 ? 1 : 2).total;
}

const char *LaunchGemvU8Mma(const WeightView &w, const float *a, std::int64_t m, unsigned char *scratch, OutputView out,
                            cudaStream_t stream, int sm_count) {
  if (!GemvU8MmaSupports(w, m) || scratch == nullptr) {
    return nullptr;
  }
  const int ntok = m <= 8 ? 1 : 2;
  const U8Layout layout = LayoutFor(w, ntok);
  const int steps_per_block = w.block_size / 32;
  const int a_vector = (w.k % 4) == 0 && (reinterpret_cast<std::uintptr_t>(a) & 15u) == 0 ? 1 : 0;
  nbits_u8_digits_kernel<<<8 * ntok, kU8DigitThreads, 0, stream>>>(
      a, static_cast<int>(m), w.k, layout.steps, layout.cols, 8 * ntok, steps_per_block, w.n_blocks,
      reinterpret_cast<signed char *>(scratch), reinterpret_cast<int *>(scratch + layout.sums_offset),
      reinterpret_cast<float *>(scratch + layout.undo_offset), a_vector);
  if (cudaGetLastError() != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();

  U8Params p{};
  p.w = w;
  p.digits = scratch;
  p.sums = reinterpret_cast<const int *>(scratch + layout.sums_offset);
  p.undo = reinterpret_cast<const float *>(scratch + layout.undo_offset);
  p.out = out;
  p.m_total = static_cast<int>(m);
  p.steps = layout.steps;
  p.tiles = static_cast<int>((w.n + 15) / 16);
  const int parts = PartsFor(w, p.tiles, sm_count);
  p.parts = parts;
  p.blocks_per_part = (w.n_blocks + parts - 1) / parts;
  const int tiles_per_cta = kU8Warps / parts;
  const unsigned grid = static_cast<unsigned>((p.tiles + tiles_per_cta - 1) / tiles_per_cta);
  // programmatic dependent launch: the multiply kernel asks for its first weights while the digit kernel runs
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kU8Warps * 32);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  cudaError_t launched = cudaErrorInvalidValue;
  if (ntok == 1) {
    switch (steps_per_block) {
    case 1: launched = cudaLaunchKernelEx(&config, nbits_gemv_u8_mma_kernel<1, 1>, p); break;
    case 2: launched = cudaLaunchKernelEx(&config, nbits_gemv_u8_mma_kernel<1, 2>, p); break;
    case 4: launched = cudaLaunchKernelEx(&config, nbits_gemv_u8_mma_kernel<1, 4>, p); break;
    case 8: launched = cudaLaunchKernelEx(&config, nbits_gemv_u8_mma_kernel<1, 8>, p); break;
    default: break;
    }
  } else {
    switch (steps_per_block) {
    case 1: launched = cudaLaunchKernelEx(&config, nbits_gemv_u8_mma_kernel<2, 1>, p); break;
    case 2: launched = cudaLaunchKernelEx(&config, nbits_gemv_u8_mma_kernel<2, 2>, p); break;
    case 4: launched = cudaLaunchKernelEx(&config, nbits_gemv_u8_mma_kernel<2, 4>, p); break;
    case 8: launched = cudaLaunchKernelEx(&config, nbits_gemv_u8_mma_kernel<2, 8>, p); break;
    default: break;
    }
  }
  if (launched != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  CountLaunch();
  return "nbits_gemv_u8_mma_kernel";
}

} // namespace mnb
