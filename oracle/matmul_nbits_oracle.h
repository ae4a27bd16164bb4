// TEST INFRASTRUCTURE ONLY. CPU restatement of com.microsoft.MatMulNBits used as the
// checker for the CUDA path. Nothing in the shipped library links or calls this file; only
// the test-suite, the smoke check and the CPU-baseline leg of the benchmark load it.
//
// PARITY STATUS: the reference project (xadupre/onnx-light-cpu 0.1.16) ships no MatMulNBits
// kernel, so the operator semantics restated here are PARITY UNPINNED against a reference
// MatMulNBits. What IS pinned against reference code (compiled from the reference sources
// into oracle/_ref and against its unit-test vectors) is every integer convention the
// operator rests on:
//   * nibble order (element 2i = low nibble of byte i, unused final high nibble ignored)
//     - onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.h:42-47,
//       onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:60-93
//   * exact (q - zero_point) integers and exact int32 block dot products
//     - onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:164-224 (4-bit),
//       :97-162 (8-bit), modulo-2^32 accumulation :48-56
//   * bf16 round-to-nearest-even with NaN quieting
//     - onnx_light_cpu/impl/math/half_conversion.h:80-87
//
// Operator contract restated here (public com.microsoft.MatMulNBits schema):
//   attrs  K, N, bits in {4, 8}, block_size (power of two >= 16), accuracy_level in {0, 4}
//   A      fp32 [M, K]
//   B      uint8 [N, n_blocks, block_size*bits/8], n_blocks = ceil(K / block_size)
//   scales fp32 [N * n_blocks]
//   zero_points (optional) uint8 [N, ceil(n_blocks*bits/8)]; default 2^(bits-1)
//   bias   (optional) fp32 [N]
//   Y[m,n] = sum_k A[m,k] * (q[n,k] - zp[n, k/block_size]) * scale[n, k/block_size] + bias[n]
#pragma once

#include <cstdint>

extern "C" {

// Integer dequantization: out[n*K + k] = q[n,k] - zp[n, k / block_size]. Exact.
int nbits_oracle_dequant_int(const std::uint8_t *b, const std::uint8_t *zero_points,
                             std::int64_t n, std::int64_t k, int bits, int block_size,
                             std::int32_t *out);

// fp32 path, fixed order: for each output, k ascending, w = float(q - zp) * scale (one
// rounding), acc = fmaf(a, w, acc); bias added last.
int nbits_oracle_matmul_f32(const float *a, const std::uint8_t *b, const float *scales,
                            const std::uint8_t *zero_points, const float *bias, std::int64_t m,
                            std::int64_t n, std::int64_t k, int bits, int block_size, float *y,
                            int threads);

// Same value accumulated in double (the "true" result used for error-bound reporting).
int nbits_oracle_matmul_f64(const float *a, const std::uint8_t *b, const float *scales,
                            const std::uint8_t *zero_points, const float *bias, std::int64_t m,
                            std::int64_t n, std::int64_t k, int bits, int block_size, double *y,
                            int threads);

// Tensor-core model: A and the dequantized weight are each rounded to bf16 (RNE), products
// accumulated in double, bias added in double. The GPU accumulates in fp32 in a different
// order; the documented tolerance for that path is 2e-2.
int nbits_oracle_matmul_bf16(const float *a, const std::uint8_t *b, const float *scales,
                             const std::uint8_t *zero_points, const float *bias, std::int64_t m,
                             std::int64_t n, std::int64_t k, int bits, int block_size, double *y,
                             int threads);

// accuracy_level = 4, definition owned by this project: per (row, block)
//   sa = max|A_block| / 127 (fp32 division; 0 when the block is all zero)
//   aq = clamp(rne(A / sa), -127, 127)  (fp32 division, round-half-even), 0 when sa == 0.
int nbits_oracle_quantize_a(const float *a, std::int64_t m, std::int64_t k, int block_size,
                            std::int8_t *aq, float *a_scales);

// dots[(m*N + n)*n_blocks + blk] = sum_{k in blk} aq[m,k] * (q[n,k] - zp[n,blk]), int32 exact.
int nbits_oracle_int8_block_dots(const std::int8_t *aq, const std::uint8_t *b,
                                 const std::uint8_t *zero_points, std::int64_t m, std::int64_t n,
                                 std::int64_t k, int bits, int block_size, std::int32_t *dots,
                                 int threads);

// Y[m,n] = sum_blk fmaf(sa[m,blk] * scale[n,blk], float(dot), acc), blocks ascending, + bias.
int nbits_oracle_matmul_int8(const float *a, const std::uint8_t *b, const float *scales,
                             const std::uint8_t *zero_points, const float *bias, std::int64_t m,
                             std::int64_t n, std::int64_t k, int bits, int block_size, float *y,
                             int threads);

// Throughput-oriented fp32 CPU implementation (blockwise unpack + vectorizable dot, N column
// panels split across `threads` std::threads). Same math as nbits_oracle_matmul_f32 up to
// summation order. This is the timed "CPU port" baseline.
int nbits_oracle_matmul_f32_fast(const float *a, const std::uint8_t *b, const float *scales,
                                 const std::uint8_t *zero_points, const float *bias,
                                 std::int64_t m, std::int64_t n, std::int64_t k, int bits,
                                 int block_size, float *y, int threads);

// bf16 helpers (RNE, NaN quieted).
std::uint16_t nbits_oracle_float_to_bf16_bits(float value);
float nbits_oracle_bf16_bits_to_float(std::uint16_t bits);

int nbits_oracle_hardware_threads();
}
