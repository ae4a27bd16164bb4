// TEST INFRASTRUCTURE ONLY. C-ABI bridge over the reference's own compiled sources so that
// Python tests can call the real reference functions that pin this project's integer
// conventions. Compiled by oracle/Makefile together with the reference translation units,
// read in place from the reference checkout (never copied), into oracle/_ref/.
//
// Reference entry points bridged:
//   IntegerMatMul4Bit2D  onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:276-299
//   IntegerMatMul2D      onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.cc:236-274
//   FloatToBFloat16Bits  onnx_light_cpu/impl/math/half_conversion.h:80-87

#include "onnx_light_cpu/impl/math/gemm/vnni/integer_gemm_vnni.h"
#include "onnx_light_cpu/impl/math/half_conversion.h"

#include <cstdint>

extern "C" {

void ref_integer_matmul_4bit_2d(const std::uint8_t *a, int a_signed, const std::uint8_t *b,
                                int b_signed, std::int32_t *c, std::int64_t rows,
                                std::int64_t cols, std::int64_t depth,
                                const std::int32_t *a_zero_point, std::int64_t a_zero_point_count,
                                const std::int32_t *b_zero_point,
                                std::int64_t b_zero_point_count) {
  onnx_light_cpu::IntegerMatMul4Bit2D(a, a_signed != 0, b, b_signed != 0, c, rows, cols, depth,
                                      a_zero_point, a_zero_point_count, b_zero_point,
                                      b_zero_point_count);
}

void ref_integer_matmul_2d(const std::uint8_t *a, int a_signed, const std::uint8_t *b,
                           int b_signed, std::int32_t *c, std::int64_t rows, std::int64_t cols,
                           std::int64_t depth, const std::int32_t *a_zero_point,
                           std::int64_t a_zero_point_count, const std::int32_t *b_zero_point,
                           std::int64_t b_zero_point_count) {
  onnx_light_cpu::IntegerMatMul2D(a, a_signed != 0, b, b_signed != 0, c, rows, cols, depth,
                                  a_zero_point, a_zero_point_count, b_zero_point,
                                  b_zero_point_count);
}

std::uint16_t ref_float_to_bf16_bits(float value) {
  return onnx_light_cpu::detail::FloatToBFloat16Bits(value);
}

int ref_uses_vnni() { return onnx_light_cpu::IntegerMatMul2DUsesVnni() ? 1 : 0; }
}
