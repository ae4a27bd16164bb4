// Device helpers shared by the tensor-core decode kernels (one column tile per pass, and several):
// 4-bit code -> fp16 conversion, the fp16 MMA wrappers and the activation layout.
#pragma once

#include <cuda_fp16.h>

#include <cstdint>

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
