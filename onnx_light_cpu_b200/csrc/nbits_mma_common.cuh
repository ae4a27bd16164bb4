// Device helpers shared by the tensor-core decode kernels (one column tile per pass, and several):
// 4-bit code -> fp16 conversion, the fp16 MMA wrappers and the activation layout.
#pragma once

#include <cuda_fp16.h>

#include <cstdint>
#include <cmath>

namespace mnb {
namespace mma_decode {

__device__ __forceinline__ std::uint32_t AndOr(std::uint32_t a, std::uint32_t mask, std::uint32_t c) {
  std::uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(c));
  return d;
}

__device__ __forceinline__ std::uint32_t Hsub2(std::uint32_t a, std::uint32_t b) {
  std::uint32_t d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ std::uint32_t Hfma2(std::uint32_t a, std::uint32_t b, std::uint32_t c) {
  std::uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ void MmaF16(float (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                       std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same with a zero accumulator input: starts a fresh sum without clearing registers first.
__device__ __forceinline__ void MmaF16Zero(float (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                           std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// Eight codes of `w` minus the zero point, as four fp16 pairs (code j, code j+4), j = 0..3.
// `offs` = (1024 + zp) x2, `offs16` = -(64 + zp) x2, `sixteenth` = (1/16) x2.
__device__ __forceinline__ void Dequant8(std::uint32_t w, std::uint32_t magic, std::uint32_t offs,
                                         std::uint32_t offs16, std::uint32_t sixteenth,
                                         std::uint32_t (&p)[4]) {
  const std::uint32_t w8 = w >> 8;
  p[0] = Hsub2(AndOr(w, 0x000f000fu, magic), offs);
  p[1] = Hfma2(AndOr(w, 0x00f000f0u, magic), sixteenth, offs16);
  p[2] = Hsub2(AndOr(w8, 0x000f000fu, magic), offs);
  p[3] = Hfma2(AndOr(w8, 0x00f000f0u, magic), sixteenth, offs16);
}

// Position (in fp16 elements) of activation k inside a piece row: supergroup-major, then the
// word index i = (k % 32) / 8, the quad lane t = (k % 128) / 32, then the eight k of a word in
// the order 0,4,1,5,2,6,3,7 (the order the pair extraction produces).
__device__ __forceinline__ int ActPosition(int k) {
  const int sg = k >> 7;
  const int rem = k & 127;
  const int t = rem >> 5;
  const int i = (rem & 31) >> 3;
  const int j = rem & 7;
  const int pos = j < 4 ? 2 * j : 2 * (j - 4) + 1;
  return (sg << 7) + (i << 5) + (t << 3) + pos;
}

// Stages `tokens` activation rows for the fp16 MMA decode kernels: per row a power-of-two scale
// (largest magnitude into [2^14, 2^15)), two fp16 pieces, the k order of ActPosition, written to
// act + (2 * token + piece) * act_row_bytes; inv_scale[token] = the inverse factor. All rows
// are staged at once: the WARPS consumer warps are split into `tokens` groups, one row each, so
// the prologue costs the same for one row or sixteen. A thread owns whole 8-k words (one 16-byte
// store per piece); when a group has at least one thread per eight words the row stays in
// registers between the max reduction and the split and A is read once, otherwise twice
// (vector loads, several in flight: the second read comes from L2).
// `scratch` holds WARPS floats. Uses named barrier 9 with WARPS * 32 participants, once; every
// consumer thread must call it.
template <int WARPS>
__device__ __forceinline__ void StageActivations(const float *a_rows, int tokens, int k, int k_pad,
                                                 unsigned char *act, int act_row_bytes, float *inv_scale,
                                                 float *scratch, int tid) {
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int warps_per_token = WARPS / tokens; // tokens <= WARPS
  const int token = warp / warps_per_token;
  const bool working = token < tokens;
  const int group_threads = warps_per_token * 32;
  const int tg = tid - token * group_threads; // index inside the group
  const int words_total = k_pad >> 3;
  constexpr int kHeld = 8; // words a thread can keep in registers
  const bool in_registers = words_total <= kHeld * group_threads;
  const float *src = a_rows + static_cast<std::int64_t>(token) * k;
  const bool vector_ok = (reinterpret_cast<std::uintptr_t>(src) & 15u) == 0;
  float v[kHeld][8];
  float amax = 0.0f;
  // whole 8-k words only and 16-byte aligned rows: plain predicated vector loads, all in flight
  const bool fast = vector_ok && (k & 7) == 0;
  if (working && in_registers) {
    if (fast) {
      float4 lo[kHeld], hi[kHeld];
#pragma unroll
      for (int j = 0; j < kHeld; ++j) {
        const int k0 = (tg + j * group_threads) << 3;
        lo[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        hi[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (k0 < k) {
          lo[j] = __ldg(reinterpret_cast<const float4 *>(src + k0));
          hi[j] = __ldg(reinterpret_cast<const float4 *>(src + k0 + 4));
        }
      }
#pragma unroll
      for (int j = 0; j < kHeld; ++j) {
        v[j][0] = lo[j].x, v[j][1] = lo[j].y, v[j][2] = lo[j].z, v[j][3] = lo[j].w;
        v[j][4] = hi[j].x, v[j][5] = hi[j].y, v[j][6] = hi[j].z, v[j][7] = hi[j].w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < kHeld; ++j) {
        const int k0 = (tg + j * group_threads) << 3;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          v[j][e] = (k0 + e < k) ? __ldg(src + k0 + e) : 0.0f;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kHeld; ++j) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        amax = fmaxf(amax, fabsf(v[j][e]));
      }
    }
  } else if (working) {
#pragma unroll 4
    for (int word = tg; word < words_total; word += group_threads) {
      const int k0 = word << 3;
      if (fast) {
        float4 lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi = lo;
        if (k0 < k) {
          lo = __ldg(reinterpret_cast<const float4 *>(src + k0));
          hi = __ldg(reinterpret_cast<const float4 *>(src + k0 + 4));
        }
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(lo.x), fabsf(lo.y)), fmaxf(fabsf(lo.z), fabsf(lo.w))));
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(hi.x), fabsf(hi.y)), fmaxf(fabsf(hi.z), fabsf(hi.w))));
      } else {
        for (int e = 0; e < 8; ++e) {
          if (k0 + e < k) {
            amax = fmaxf(amax, fabsf(__ldg(src + k0 + e)));
          }
        }
      }
    }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  }
  if (lane == 0) {
    scratch[warp] = amax;
  }
  asm volatile("bar.sync 9, %0;" ::"n"(WARPS * 32) : "memory");
  if (!working) {
    return;
  }
  amax = scratch[token * warps_per_token];
  for (int i = 1; i < warps_per_token; ++i) {
    amax = fmaxf(amax, scratch[token * warps_per_token + i]);
  }
  int e2 = 0;
  if (amax > 0.0f && amax < 3.0e38f) {
    e2 = 14 - ilogbf(amax);
    e2 = e2 > 100 ? 100 : (e2 < -100 ? -100 : e2);
  }
  const float up = scalbnf(1.0f, e2);
  if (tg == 0) {
    inv_scale[token] = scalbnf(1.0f, -e2);
  }
  unsigned char *row_hi = act + (2 * token) * act_row_bytes;
  unsigned char *row_lo = act + (2 * token + 1) * act_row_bytes;
  // splits eight scaled activations into two fp16 pieces and stores both 16-byte words
  auto store_word = [&](int k0, const float (&x)[8]) {
    std::uint32_t hi[4], lo[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) { // stored order inside a word: k = 0,4,1,5,2,6,3,7
      const __half a_hi = __float2half_rn(x[q]);
      const __half b_hi = __float2half_rn(x[q + 4]);
      const __half a_lo = __float2half_rn(x[q] - __half2float(a_hi));
      const __half b_lo = __float2half_rn(x[q + 4] - __half2float(b_hi));
      hi[q] = static_cast<std::uint32_t>(__half_as_ushort(a_hi)) |
              (static_cast<std::uint32_t>(__half_as_ushort(b_hi)) << 16);
      lo[q] = static_cast<std::uint32_t>(__half_as_ushort(a_lo)) |
              (static_cast<std::uint32_t>(__half_as_ushort(b_lo)) << 16);
    }
    const int byte = ActPosition(k0) * 2;
    *reinterpret_cast<uint4 *>(row_hi + byte) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<uint4 *>(row_lo + byte) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  };
  if (in_registers) {
#pragma unroll
    for (int j = 0; j < kHeld; ++j) {
      const int word = tg + j * group_threads;
      if (word < words_total) {
        float x[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          x[e] = v[j][e] * up;
        }
        store_word(word << 3, x);
      }
    }
  } else {
#pragma unroll 4
    for (int word = tg; word < words_total; word += group_threads) {
      const int k0 = word << 3;
      float x[8];
      if (fast) {
        float4 lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi = lo;
        if (k0 < k) {
          lo = __ldg(reinterpret_cast<const float4 *>(src + k0));
          hi = __ldg(reinterpret_cast<const float4 *>(src + k0 + 4));
        }
        x[0] = lo.x * up, x[1] = lo.y * up, x[2] = lo.z * up, x[3] = lo.w * up;
        x[4] = hi.x * up, x[5] = hi.y * up, x[6] = hi.z * up, x[7] = hi.w * up;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          x[e] = (k0 + e < k) ? __ldg(src + k0 + e) * up : 0.0f;
        }
      }
      store_word(k0, x);
    }
  }
}

// log2 of a power of two
inline int Log2Of(int v) {
  int l = 0;
  while ((1 << l) < v) {
    ++l;
  }
  return l;
}

} // namespace mma_decode
} // namespace mnb
