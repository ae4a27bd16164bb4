"""Pins the CPU checker to the reference: committed outputs of the reference's own functions
(tests/golden/reference_pins.npz, made by tests/golden/make_golden.py) and, where the
reference build oracle/_ref is present, the live functions."""

from pathlib import Path

import numpy as np
import pytest

from oracle import nbits_oracle as o

GOLDEN = np.load(Path(__file__).parent / "golden" / "reference_pins.npz")


def naive_int4(a, b, rows, cols, depth, azp, bzp):
    a = a.reshape(rows, depth).astype(np.int64)
    b = b.reshape(depth, cols).astype(np.int64)
    az = azp.astype(np.int64).reshape(-1, 1) if azp.size > 1 else np.int64(azp[0])
    bz = bzp.astype(np.int64).reshape(1, -1) if bzp.size > 1 else np.int64(bzp[0])
    wrapped = ((a - az) @ (b - bz)) & 0xFFFFFFFF  # modulo 2^32
    return wrapped.astype(np.uint32).view(np.int32).reshape(rows, cols)


def test_reference_int4_vectors_match_plain_integer_math():
    """The committed reference outputs equal (A - az)(B - bz) mod 2^32: the fixture is sane."""
    for case in range(int(GOLDEN["int4_cases"][0])):
        rows, cols, depth, _, _ = GOLDEN[f"int4_{case}_meta"]
        expect = naive_int4(GOLDEN[f"int4_{case}_a"], GOLDEN[f"int4_{case}_b"], rows, cols, depth,
                            GOLDEN[f"int4_{case}_azp"], GOLDEN[f"int4_{case}_bzp"])
        assert np.array_equal(GOLDEN[f"int4_{case}_c"], expect)
    assert int(GOLDEN["int4_kat_tail"][0, 0]) == 2 * 5 + 3 * 6 + 4 * 7


def test_oracle_nibble_order_matches_reference_vectors():
    """Unsigned cases of the reference's 4-bit test, replayed through the checker: each B column
    of the reference's [depth, cols] operand becomes one MatMulNBits weight row."""
    for case in range(int(GOLDEN["int4_cases"][0])):
        rows, cols, depth, a_signed, b_signed = GOLDEN[f"int4_{case}_meta"]
        if a_signed or b_signed:
            continue  # MatMulNBits codes are unsigned
        a = GOLDEN[f"int4_{case}_a"].reshape(rows, depth)
        b = GOLDEN[f"int4_{case}_b"].reshape(depth, cols)
        block = 16
        while block < depth:
            block *= 2
        packed = np.zeros((cols, block // 2), np.uint8)
        for col in range(cols):
            padded = np.zeros(block, np.int64)
            padded[:depth] = b[:, col]
            packed[col] = o.pack4(padded)
        bzp = GOLDEN[f"int4_{case}_bzp"]
        zp_codes = np.broadcast_to(bzp, (cols,)).astype(np.int64)
        zp_packed = (zp_codes & 0x0F).astype(np.uint8).reshape(cols, 1)
        ints = o.dequant_int(packed, zp_packed, cols, depth, 4, block)
        azp = np.broadcast_to(GOLDEN[f"int4_{case}_azp"], (rows,)).astype(np.int64)
        got = ((a.astype(np.int64) - azp[:, None]) @ ints.T.astype(np.int64))
        assert np.array_equal(got.astype(np.int32), GOLDEN[f"int4_{case}_c"])


def test_oracle_dequant_integers_match_reference():
    n, k, bs = GOLDEN["nbits_geometry"]
    ints = o.dequant_int(GOLDEN["nbits_b"], GOLDEN["nbits_zp"], int(n), int(k), 4, int(bs))
    assert np.array_equal(ints, GOLDEN["nbits_ints"])
    assert np.array_equal(o.np_dequant_int(GOLDEN["nbits_b"], GOLDEN["nbits_zp"], int(n), int(k), 4, int(bs)),
                          GOLDEN["nbits_ints"])


def test_oracle_int8_block_dots_match_reference():
    n, k, bs = (int(v) for v in GOLDEN["nbits_geometry"])
    dots = o.int8_block_dots(GOLDEN["nbits_aq"], GOLDEN["nbits_b"], GOLDEN["nbits_zp"], n, k, 4, bs)
    assert np.array_equal(dots, GOLDEN["nbits_dots"])


def test_oracle_bf16_rounding_matches_reference():
    for value, bits in zip(GOLDEN["bf16_in"], GOLDEN["bf16_bits"]):
        assert o.float_to_bf16_bits(float(value)) == int(bits), value


@pytest.mark.skipif(o.ref_lib() is None, reason="oracle/_ref not built (reference checkout absent)")
def test_live_reference_agrees_on_random_blocks():
    rng = np.random.default_rng(3)
    for bs in (16, 32, 64):
        n, nb = 5, 3
        k = nb * bs
        packed = rng.integers(0, 256, size=(n, nb, bs // 2), dtype=np.uint8)
        zp = rng.integers(0, 256, size=(n, (nb + 1) // 2), dtype=np.uint8)
        zp_values = o.np_zero_points(zp, n, k, 4, bs)
        ints = o.dequant_int(packed, zp, n, k, 4, bs)
        eye = o.pack4(np.eye(bs, dtype=np.int64).reshape(-1))
        for row in range(n):
            for blk in range(nb):
                c = o.ref_matmul_4bit(eye, False, packed[row, blk], False, bs, 1, bs, [0], [zp_values[row, blk]])
                assert np.array_equal(c[:, 0], ints[row, blk * bs:(blk + 1) * bs])
        aq = rng.integers(-127, 128, size=(2, k), dtype=np.int8)
        dots = o.int8_block_dots(aq, packed, zp, n, k, 4, bs)
        codes = o.np_unpack_codes(packed, n, k, 4, bs).astype(np.uint8)
        for blk in range(nb):
            ref = o.ref_matmul_8bit(np.ascontiguousarray(aq[:, blk * bs:(blk + 1) * bs]), True,
                                    np.ascontiguousarray(codes[:, blk * bs:(blk + 1) * bs].T), False, 2, n, bs,
                                    [0], zp_values[:, blk])
            assert np.array_equal(ref, dots[:, :, blk])
    for value in rng.standard_normal(200).astype(np.float32):
        assert o.float_to_bf16_bits(float(value)) == int(o.ref_lib().ref_float_to_bf16_bits(float(value)))
