// accuracy_level = 4 path of MatMulNBits for sm_100a: per-block int8 quantization of the
// activations, exact int32 block dot products against (q - zp), fp32 scaling.
//
// Definition (owned by this project; the reference has no counterpart):
//   sa[m,blk]  = max|A[m, blk]| / 127            (IEEE fp32 division, 0 for an all-zero block)
//   aq[m,k]    = clamp(rne(A[m,k] / sa), -127, 127)
//   dot[m,n,b] = sum_{k in b} aq[m,k] * (q[n,k] - zp[n,b])        int32, exact
//   Y[m,n]     = sum_b sa[m,b] * scale[n,b] * float(dot[m,n,b]) + bias[n]
// The integer part follows the exact modulo-2^32 integer GEMM conventions of
// onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:48-56 (u8 x s8 dot) and :208-223
// (zero-point correction through row sums), here with dp4a.

#include "nbits_common.cuh"

#include <cstdint>

namespace mnb {
namespace {

// One warp per (row, block).
__global__ void __launch_bounds__(256)
    nbits_quantize_a_kernel(const float *a, int m_total, std::int64_t k, int block_size,
                            int n_blocks, std::int64_t aq_ld, std::int8_t *aq, float *a_scales) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const std::int64_t item = static_cast<std::int64_t>(blockIdx.x) * 8 + warp;
  if (item >= static_cast<std::int64_t>(m_total) * n_blocks) {
    return;
  }
  const int row = static_cast<int>(item / n_blocks);
  const int block = static_cast<int>(item % n_blocks);
  const std::int64_t k0 = static_cast<std::int64_t>(block) * block_size;
  const float *src = a + static_cast<std::int64_t>(row) * k;
  float amax = 0.0f;
  bool bad = false;  // a NaN or an infinity in the block
  for (int e = lane; e < block_size; e += 32) {
    if (k0 + e < k) {
      const float v = fabsf(src[k0 + e]);
      amax = fmaxf(amax, v);
      bad = bad || !(v <= 3.4028235e38f);
    }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  }
  bad = __any_sync(0xffffffffu, bad);
  // A block with a non-finite activation has no int8 form: its scale is NaN and its codes are 0,
  // so that every output of the token comes out NaN (what accuracy_level 0 gives for such a row).
  const float sa = bad ? __int_as_float(0x7fc00000) : __fdiv_rn(amax, 127.0f);
  if (lane == 0) {
    a_scales[static_cast<std::int64_t>(row) * n_blocks + block] = sa;
  }
  std::int8_t *dst = aq + static_cast<std::int64_t>(row) * aq_ld;
  for (int e = lane; e < block_size; e += 32) {
    const std::int64_t kk = k0 + e;
    if (kk < aq_ld) {
      int q = 0;
      if (kk < k && sa > 0.0f) {
        const float r = rintf(__fdiv_rn(src[kk], sa));
        q = static_cast<int>(fminf(127.0f, fmaxf(-127.0f, r)));
      }
      dst[kk] = static_cast<std::int8_t>(q);
    }
  }
}

// Exact dot of 8 consecutive int8 activations (two words) with the 8 nibbles of `w`.
__device__ __forceinline__ int Dot8Nibbles(std::uint32_t w, std::uint32_t a_lo, std::uint32_t a_hi) {
  // even elements live in the low nibbles, odd elements in the high nibbles
  const std::uint32_t even = w & 0x0f0f0f0fu;
  const std::uint32_t odd = (w >> 4) & 0x0f0f0f0fu;
  const std::uint32_t a_even = __byte_perm(a_lo, a_hi, 0x6420);
  const std::uint32_t a_odd = __byte_perm(a_lo, a_hi, 0x7531);
  int acc = __dp4a(static_cast<int>(a_even), static_cast<int>(even), 0);
  return __dp4a(static_cast<int>(a_odd), static_cast<int>(odd), acc);
}

__device__ __forceinline__ int Sum4(std::uint32_t a) {
  return __dp4a(static_cast<int>(a), 0x01010101, 0);
}

// dots[(m*N + n)*n_blocks + blk], one thread per (n, blk), loops over m. Parity hook.
__global__ void __launch_bounds__(128)
    nbits_int8_block_dots_kernel(const WeightView w, const std::int8_t *aq, int m_total,
                                 std::int32_t *dots) {
  const std::int64_t item = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= w.n * w.n_blocks) {
    return;
  }
  const std::int64_t col = item / w.n_blocks;
  const int block = static_cast<int>(item % w.n_blocks);
  const int zp = ZeroPointOf(w, col, block);
  const std::int64_t k0 = static_cast<std::int64_t>(block) * w.block_size;
  for (int row = 0; row < m_total; ++row) {
    int acc = 0;
    for (int e = 0; e < w.block_size; ++e) {
      const std::int64_t kk = k0 + e;
      if (kk < w.k) {
        acc += static_cast<int>(aq[static_cast<std::int64_t>(row) * w.k + kk]) * (CodeOf(w, col, kk) - zp);
      }
    }
    dots[(static_cast<std::int64_t>(row) * w.n + col) * w.n_blocks + block] = acc;
  }
}

constexpr int kInt8Mt = 8;

// One warp per output column; lanes stride over 16-byte chunks of the packed row. `aq` is
// zero padded to n_blocks*block_size columns (leading dimension aq_ld), so weight padding
// beyond K multiplies zeros.
template <int BITS>
__global__ void __launch_bounds__(256)
    nbits_int8_matmul_kernel(const WeightView w, const std::int8_t *aq, std::int64_t aq_ld,
                             const float *a_scales, int m_total, OutputView out, int block_shift) {
  constexpr int kW = BITS == 4 ? 32 : 16; // weights per 16-byte chunk
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const std::int64_t col = static_cast<std::int64_t>(blockIdx.x) * 8 + warp;
  const int m_base = blockIdx.y * kInt8Mt;
  if (col >= w.n) {
    return;
  }
  float acc[kInt8Mt];
#pragma unroll
  for (int mi = 0; mi < kInt8Mt; ++mi) {
    acc[mi] = 0.0f;
  }
  const int chunks = w.row_bytes / 16;
  const uint4 *row = reinterpret_cast<const uint4 *>(w.b + col * w.row_bytes);
  for (int c = lane; c < chunks; c += 32) {
    const uint4 q = __ldg(row + c);
    const int block = (c * kW) >> block_shift;
    const float scale = w.scales[col * w.n_blocks + block];
    const int zp = ZeroPointOf(w, col, block);
    const std::uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int mi = 0; mi < kInt8Mt; ++mi) {
      const int m = m_base + mi;
      if (m < m_total) {
        const std::int8_t *arow = aq + static_cast<std::int64_t>(m) * aq_ld + static_cast<std::int64_t>(c) * kW;
        int dot = 0;
        int asum = 0;
        if constexpr (BITS == 4) {
          const uint4 a0 = *reinterpret_cast<const uint4 *>(arow);
          const uint4 a1 = *reinterpret_cast<const uint4 *>(arow + 16);
          const std::uint32_t av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            dot += Dot8Nibbles(words[i], av[2 * i], av[2 * i + 1]);
            asum += Sum4(av[2 * i]) + Sum4(av[2 * i + 1]);
          }
        } else {
          const uint4 a0 = *reinterpret_cast<const uint4 *>(arow);
          const std::uint32_t av[4] = {a0.x, a0.y, a0.z, a0.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // signed activations x unsigned codes
            int part;
            asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(part) : "r"(av[i]), "r"(words[i]), "r"(0));
            dot += part;
            asum += Sum4(av[i]);
          }
        }
        const int exact = dot - zp * asum; // sum aq * (q - zp) over this chunk
        const float sa = a_scales[static_cast<std::int64_t>(m) * w.n_blocks + block];
        acc[mi] = fmaf(sa * scale, static_cast<float>(exact), acc[mi]);
      }
    }
  }
#pragma unroll
  for (int mi = 0; mi < kInt8Mt; ++mi) {
    float v = acc[mi];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      v += __shfl_xor_sync(0xffffffffu, v, offset);
    }
    if (lane == 0 && m_base + mi < m_total) {
      const float bias = w.bias != nullptr ? w.bias[col] : 0.0f;
      out.y[static_cast<std::int64_t>(m_base + mi) * out.ld + out.col_offset + col] = v + bias;
    }
  }
}

// The same product for rows the 16-byte chunks do not fit (4-bit weights with block_size 16, where a
// chunk would span two blocks, and packed rows that are not a multiple of 16 bytes): lanes stride
// over groups of eight codes, 4 bytes of a 4-bit row or 8 of an 8-bit one, against 8 bytes of `aq`.
template <int BITS>
__global__ void __launch_bounds__(256)
    nbits_int8_words_kernel(const WeightView w, const std::int8_t *aq, std::int64_t aq_ld, const float *a_scales,
                            int m_total, OutputView out, int block_shift) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const std::int64_t col = static_cast<std::int64_t>(blockIdx.x) * 8 + warp;
  const int m_base = blockIdx.y * kInt8Mt;
  if (col >= w.n) {
    return;
  }
  float acc[kInt8Mt];
#pragma unroll
  for (int mi = 0; mi < kInt8Mt; ++mi) {
    acc[mi] = 0.0f;
  }
  const int groups = w.row_bytes / BITS;
  const unsigned char *row = w.b + col * w.row_bytes;
  for (int g = lane; g < groups; g += 32) {
    std::uint32_t q_lo;
    std::uint32_t q_hi = 0;
    if constexpr (BITS == 4) {
      q_lo = __ldg(reinterpret_cast<const std::uint32_t *>(row) + g);
    } else {
      const uint2 q = __ldg(reinterpret_cast<const uint2 *>(row) + g);
      q_lo = q.x;
      q_hi = q.y;
    }
    const int block = (g * 8) >> block_shift;
    const float scale = w.scales[col * w.n_blocks + block];
    const int zp = ZeroPointOf(w, col, block);
#pragma unroll
    for (int mi = 0; mi < kInt8Mt; ++mi) {
      const int m = m_base + mi;
      if (m < m_total) {
        const uint2 av = *reinterpret_cast<const uint2 *>(aq + static_cast<std::int64_t>(m) * aq_ld +
                                                          static_cast<std::int64_t>(g) * 8);
        int dot;
        if constexpr (BITS == 4) {
          dot = Dot8Nibbles(q_lo, av.x, av.y);
        } else {
          asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(dot) : "r"(av.x), "r"(q_lo), "r"(0));
          asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(dot) : "r"(av.y), "r"(q_hi), "r"(dot));
        }
        const int exact = dot - zp * (Sum4(av.x) + Sum4(av.y)); // sum aq * (q - zp) over this group
        const float sa = a_scales[static_cast<std::int64_t>(m) * w.n_blocks + block];
        acc[mi] = fmaf(sa * scale, static_cast<float>(exact), acc[mi]);
      }
    }
  }
#pragma unroll
  for (int mi = 0; mi < kInt8Mt; ++mi) {
    float v = acc[mi];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      v += __shfl_xor_sync(0xffffffffu, v, offset);
    }
    if (lane == 0 && m_base + mi < m_total) {
      const float bias = w.bias != nullptr ? w.bias[col] : 0.0f;
      out.y[static_cast<std::int64_t>(m_base + mi) * out.ld + out.col_offset + col] = v + bias;
    }
  }
}

int Log2Of(int v) {
  int l = 0;
  while ((1 << l) < v) {
    ++l;
  }
  return l;
}

} // namespace

const char *LaunchQuantizeA(const float *a, std::int64_t m, std::int64_t k, int block_size,
                            std::int8_t *aq, float *a_scales, cudaStream_t stream) {
  // natural layout: leading dimension k
  const int n_blocks = static_cast<int>((k + block_size - 1) / block_size);
  const std::int64_t items = m * n_blocks;
  if (items <= 0) {
    return nullptr;
  }
  nbits_quantize_a_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, stream>>>(
      a, static_cast<int>(m), k, block_size, n_blocks, k, aq, a_scales);
  if (cudaGetLastError() != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return "nbits_quantize_a_kernel";
}

const char *LaunchInt8BlockDots(const WeightView &w, const std::int8_t *aq, std::int64_t m,
                                std::int32_t *dots, cudaStream_t stream) {
  const std::int64_t items = w.n * w.n_blocks;
  if (items <= 0 || m < 1) {
    return nullptr;
  }
  nbits_int8_block_dots_kernel<<<static_cast<unsigned>((items + 127) / 128), 128, 0, stream>>>(
      w, aq, static_cast<int>(m), dots);
  if (cudaGetLastError() != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return "nbits_int8_block_dots_kernel";
}

// `aq` here is the padded internal layout: [m, n_blocks*block_size] int8 followed by nothing;
// `a_scales` is [m, n_blocks]. The C ABI layer produces both with QuantizeAPadded below.
const char *LaunchInt8Matmul(const WeightView &w, const std::int8_t *aq, const float *a_scales,
                             std::int64_t m, OutputView out, cudaStream_t stream, int sm_count) {
  (void)sm_count;
  if (m < 1 || (w.bits != 4 && w.bits != 8) || w.block_size < 16) {
    return nullptr;
  }
  const std::int64_t aq_ld = static_cast<std::int64_t>(w.n_blocks) * w.block_size;
  dim3 grid(static_cast<unsigned>((w.n + 7) / 8), static_cast<unsigned>((m + kInt8Mt - 1) / kInt8Mt), 1);
  const int shift = Log2Of(w.block_size);
  const bool chunked = (w.row_bytes % 16) == 0 && (reinterpret_cast<std::uintptr_t>(w.b) & 15u) == 0 &&
                       !(w.bits == 4 && w.block_size < 32);
  if (!chunked) {
    // groups of eight codes: one aligned 4-byte (4-bit) or 8-byte (8-bit) load each; `aq` rows are a
    // multiple of 16 bytes in the padded layout
    const std::uintptr_t group_bytes = static_cast<std::uintptr_t>(w.bits);
    if ((reinterpret_cast<std::uintptr_t>(w.b) % group_bytes) != 0 || (w.row_bytes % group_bytes) != 0 ||
        (reinterpret_cast<std::uintptr_t>(aq) & 7u) != 0) {
      return nullptr;
    }
    if (w.bits == 4) {
      nbits_int8_words_kernel<4><<<grid, 256, 0, stream>>>(w, aq, aq_ld, a_scales, static_cast<int>(m), out, shift);
    } else {
      nbits_int8_words_kernel<8><<<grid, 256, 0, stream>>>(w, aq, aq_ld, a_scales, static_cast<int>(m), out, shift);
    }
    if (cudaGetLastError() != cudaSuccess) {
      return nullptr;
    }
    CountLaunch();
    return w.bits == 4 ? "nbits_int8_words_kernel<4>" : "nbits_int8_words_kernel<8>";
  }
  if (w.bits == 4) {
    nbits_int8_matmul_kernel<4><<<grid, 256, 0, stream>>>(w, aq, aq_ld, a_scales, static_cast<int>(m), out, shift);
  } else {
    nbits_int8_matmul_kernel<8><<<grid, 256, 0, stream>>>(w, aq, aq_ld, a_scales, static_cast<int>(m), out, shift);
  }
  if (cudaGetLastError() != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return w.bits == 4 ? "nbits_int8_matmul_kernel<4>" : "nbits_int8_matmul_kernel<8>";
}

// Internal: quantize into the zero-padded layout used by LaunchInt8Matmul.
const char *LaunchQuantizeAPadded(const float *a, std::int64_t m, std::int64_t k, int block_size,
                                  std::int8_t *aq_padded, float *a_scales, cudaStream_t stream) {
  const int n_blocks = static_cast<int>((k + block_size - 1) / block_size);
  const std::int64_t items = m * n_blocks;
  if (items <= 0) {
    return nullptr;
  }
  nbits_quantize_a_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, stream>>>(
      a, static_cast<int>(m), k, block_size, n_blocks,
      static_cast<std::int64_t>(n_blocks) * block_size, aq_padded, a_scales);
  if (cudaGetLastError() != cudaSuccess) {
    return nullptr;
  }
  CountLaunch();
  return "nbits_quantize_a_kernel";
}

} // namespace mnb
