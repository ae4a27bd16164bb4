"""Hand-computable MatMulNBits cases and self-consistency of the CPU checker."""

import numpy as np
import pytest

from oracle import nbits_oracle as o
from onnx_light_cpu_b200.tools import synthetic as syn


def test_tiny_known_answer_default_zero_point():
    # K=32, N=2, one block. Row 0 codes all 9 -> (9-8)=1; row 1 codes k%16.
    k, n, bs = 32, 2, 32
    codes = np.stack([np.full(k, 9), np.arange(k) % 16])
    b = np.stack([o.pack4(r) for r in codes]).reshape(n, 1, bs // 2)
    scales = np.array([0.5, 2.0], np.float32)
    a = np.ones((1, k), np.float32)
    y = o.matmul_f32(a, b, scales, None, None, n, k, 4, bs)
    assert y[0, 0] == pytest.approx(0.5 * 32)
    assert y[0, 1] == pytest.approx(2.0 * float(((np.arange(k) % 16) - 8).sum()))


def test_zero_point_row_with_padding_nibble_and_bias():
    # three blocks -> zero-point row is 2 bytes, the last high nibble is padding (set to 0xF)
    k, n, bs = 48, 1, 16
    codes = np.concatenate([np.full(16, 3), np.full(16, 7), np.full(16, 15)])
    b = o.pack4(codes).reshape(1, 3, 8)
    zp = np.array([[0x21, 0xF4]], np.uint8)  # zp = 1, 2, 4 and a padding nibble
    scales = np.array([1.0, 10.0, 100.0], np.float32)
    bias = np.array([0.25], np.float32)
    a = np.ones((2, k), np.float32)
    a[1] = 2.0
    y = o.matmul_f32(a, b, scales, zp, bias, n, k, 4, bs)
    expect = 16 * ((3 - 1) * 1.0 + (7 - 2) * 10.0 + (15 - 4) * 100.0)
    assert y[0, 0] == pytest.approx(expect + 0.25)
    assert y[1, 0] == pytest.approx(2 * expect + 0.25)


def test_eight_bit_and_partial_last_block():
    k, n, bs = 40, 2, 32  # second block only 8 wide; blob padding must be ignored
    rng = np.random.default_rng(0)
    b = rng.integers(0, 256, size=(n, 2, bs), dtype=np.uint8)
    zp = np.array([[100, 128], [0, 255]], np.uint8)
    scales = np.array([1.0, 0.5, 0.25, 2.0], np.float32)
    a = rng.standard_normal((3, k)).astype(np.float32)
    y = o.matmul_f64(a, b, scales, zp, None, n, k, 8, bs)
    expect = np.zeros((3, n))
    for col in range(n):
        for kk in range(k):
            blk = kk // bs
            expect[:, col] += a[:, kk].astype(np.float64) * (int(b[col, blk, kk % bs]) - int(zp[col, blk])) * float(scales[col * 2 + blk])
    np.testing.assert_allclose(y, expect, rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("bits,bs,k", [(4, 16, 48), (4, 32, 200), (4, 128, 256), (8, 16, 40), (8, 64, 128)])
def test_cpp_checker_matches_numpy_restatement(bits, bs, k):
    c = syn.make_case("x", 3, k, 9, bits, bs, seed=bits * 1000 + bs + k, bias=True)
    y64 = o.matmul_f64(c.a, c.b, c.scales, c.zero_points, c.bias, c.n, c.k, bits, bs)
    ynp = o.np_matmul_f64(c.a, c.b, c.scales, c.zero_points, c.bias, c.n, c.k, bits, bs)
    np.testing.assert_allclose(y64, ynp, rtol=1e-12, atol=1e-12)
    scale = np.abs(y64).max()
    y32 = o.matmul_f32(c.a, c.b, c.scales, c.zero_points, c.bias, c.n, c.k, bits, bs)
    assert np.abs(y32 - y64).max() / scale < 1e-5
    fast = o.matmul_f32_fast(c.a, c.b, c.scales, c.zero_points, c.bias, c.n, c.k, bits, bs)
    assert np.abs(fast - y64).max() / scale < 1e-5
    ybf = o.matmul_bf16(c.a, c.b, c.scales, c.zero_points, c.bias, c.n, c.k, bits, bs)
    assert np.abs(ybf - y64).max() / scale < 2e-2


def test_activation_quantization_definition():
    a = np.array([[0.0] * 16 + [1.0, -2.0, 0.5, 127.0] + [0.0] * 12 + [1e-3] * 16], np.float32)
    aq, sa = o.quantize_a(a, 48, 16)
    assert sa[0, 0] == 0.0 and not aq[0, :16].any()          # all-zero block
    assert sa[0, 1] == np.float32(127.0) / np.float32(127.0)
    assert list(aq[0, 16:20]) == [1, -2, 0, 127]             # 0.5 rounds half-to-even to 0
    assert (aq[0, 32:] == 127).all()
    c = syn.make_case("q", 2, 96, 4, 4, 32, seed=9)
    aq, sa = o.quantize_a(c.a, 96, 32)
    dots = o.int8_block_dots(aq, c.b, c.zero_points, 4, 96, 4, 32)
    ints = o.dequant_int(c.b, c.zero_points, 4, 96, 4, 32)
    for blk in range(3):
        expect = aq[:, blk * 32:(blk + 1) * 32].astype(np.int64) @ ints[:, blk * 32:(blk + 1) * 32].T
        assert np.array_equal(dots[:, :, blk], expect)
    y = o.matmul_int8(c.a, c.b, c.scales, c.zero_points, None, 4, 96, 4, 32)
    expect = np.einsum("mb,nb,mnb->mn", sa.astype(np.float64), c.scales.reshape(4, 3).astype(np.float64), dots)
    np.testing.assert_allclose(y, expect, rtol=1e-5, atol=1e-7)


def test_config_shapes():
    c1 = syn.config1()
    assert c1.a.shape == (1, 4096) and c1.b.shape == (4096, 128, 16) and c1.scales.shape == (524288,)
    assert c1.zero_points is None and c1.bias is None and c1.scales.min() >= 1e-4
    c2 = syn.config2(4, n=64)
    assert c2.b.shape == (64, 32, 64) and c2.zero_points.shape == (64, 16) and c2.bias.shape == (64,)
    assert np.array_equal(c2.a, c2.a.astype(np.float16).astype(np.float32))
    c5 = syn.config5(1, 8, n=128)
    assert c5.b.shape == (128, 128, 32) and c5.zero_points.shape == (128, 128)
    shard = syn.shard_columns(c5, 4, 1)
    assert shard.n == 32 and shard.meta["col_offset"] == 32
    assert np.array_equal(shard.scales, c5.scales.reshape(128, 128)[32:64].reshape(-1))


def test_digit_split_invariants_of_the_integer_mma_decode_kernels():
    """The integer-MMA decode kernels (csrc/nbits_digits.cuh, csrc/nbits_gemv_u8_mma.cu) write an activation
    row as n = round(a / max|a| * 2e6) = 16384 d0 + 128 d1 + d2 with balanced base-128 digits taken from the
    plain digits of the biased integer n + 64 + 64 * 128 + 128 * 16384. Restated here in numpy: the identity,
    the signed-byte ranges, the int32 / 2^24 bounds the per-block sums rely on, and the accuracy of a product
    rebuilt from the digits against the float64 product."""
    rng = np.random.default_rng(2026)
    k, block = 4096, 256
    a = (rng.standard_normal(k) * np.exp(rng.uniform(-3, 3, size=k))).astype(np.float32)
    amax = np.abs(a).max()
    n = np.rint(a.astype(np.float64) / amax * 2.0e6).astype(np.int64)
    bias = 64 + 64 * 128 + 128 * 16384
    u = n + bias
    assert u.min() > 0 and u.max() < 2 ** 22
    d0, d1, d2 = (u >> 14) - 128, ((u >> 7) & 127) - 64, (u & 127) - 64
    assert np.array_equal(16384 * d0 + 128 * d1 + d2, n)
    assert np.abs(d0).max() <= 123 and d1.min() >= -64 and d1.max() <= 63 and d2.min() >= -64 and d2.max() <= 63
    # exact int32 block sums: 8-bit codes against digits, blocks of up to 256
    assert 255 * 123 * block < 2 ** 24
    # middle and low digit combined before the conversion, zero point taken out in int32
    worst = 128 * (255 * 64 * block) + 255 * 64 * block + 255 * (128 * 64 * block + 64 * block)
    assert worst < 2 ** 31
    # a product rebuilt from the digits is within 1e-5 of the float64 product (codes minus zero point)
    w = rng.integers(0, 256, size=k).astype(np.int64) - 128
    rebuilt = float((w * (16384 * d0 + 128 * d1 + d2)).sum()) * (float(amax) / 2.0e6)
    exact = float((w.astype(np.float64) * a.astype(np.float64)).sum())
    scale = float(np.abs(w.astype(np.float64) * a.astype(np.float64)).sum())
    assert abs(rebuilt - exact) <= 1e-6 * scale
