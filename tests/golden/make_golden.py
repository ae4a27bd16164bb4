"""Generates tests/golden/reference_pins.npz from the reference's own code.

Run where the reference checkout is available (it builds oracle/_ref from the reference
sources): ``python tests/golden/make_golden.py``. The fixture holds inputs and the outputs
the REFERENCE functions produced for them, so the CPU tests can pin this project's checker
to the reference without the checkout:

* int4_*  - IntegerMatMul4Bit2D on the deterministic nibble fills and shapes of the
            reference's own unit test (unittests/cc/test_integer_gemm_vnni.cc:164-175,
            :343-352) and its known-answer case {2,3,4}.{5,6,7} = 56 (:354-364)
* nbits_* - a MatMulNBits-shaped weight: (q - zp) obtained from IntegerMatMul4Bit2D with
            an identity left operand, and int8 block dots from IntegerMatMul2D
* bf16_*  - FloatToBFloat16Bits on edge values (half_conversion.h:80-87)
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import nbits_oracle as o  # noqa: E402


def fill(count, mul, add, signed):
    nib = (np.arange(count) * mul + add) & 0x0F
    return np.where(signed & (nib >= 8), nib - 16, nib).astype(np.int32)


def main() -> None:
    o.build(reference=True)
    assert o.ref_lib() is not None, "reference build failed"
    out = {}
    shapes = [(1, 1, 1, False), (5, 7, 17, False), (4, 6, 64, True), (3, 5, 65, True)]
    case = 0
    for a_signed in (False, True):
        for b_signed in (False, True):
            for rows, cols, depth, per_axis in shapes:
                a = fill(rows * depth, 5, 3, a_signed)
                b = fill(depth * cols, 7, 1, b_signed)
                azp = np.array([(i % 16) - 8 if a_signed else i % 16 for i in range(rows if per_axis else 1)], np.int32)
                bzp = np.array([7 - (i % 16) if b_signed else 15 - (i % 16) for i in range(cols if per_axis else 1)], np.int32)
                c = o.ref_matmul_4bit(o.pack4(a), a_signed, o.pack4(b), b_signed, rows, cols, depth, azp, bzp)
                out[f"int4_{case}_meta"] = np.array([rows, cols, depth, int(a_signed), int(b_signed)], np.int64)
                out[f"int4_{case}_a"] = a
                out[f"int4_{case}_b"] = b
                out[f"int4_{case}_azp"] = azp
                out[f"int4_{case}_bzp"] = bzp
                out[f"int4_{case}_c"] = c
                case += 1
    out["int4_cases"] = np.array([case], np.int64)
    a = o.pack4([2, 3, 4])
    b = o.pack4([5, 6, 7])
    a[-1] |= 0xF0
    b[-1] |= 0x80
    out["int4_kat_tail"] = o.ref_matmul_4bit(a, False, b, False, 1, 1, 3, [0], [0])

    # MatMulNBits-shaped pins
    rng = np.random.default_rng(77)
    n, k, bs = 6, 96, 32
    nb = k // bs
    packed = rng.integers(0, 256, size=(n, nb, bs // 2), dtype=np.uint8)
    zp = rng.integers(0, 256, size=(n, (nb + 1) // 2), dtype=np.uint8)
    zp_values = o.np_zero_points(zp, n, k, 4, bs)
    ints = np.zeros((n, k), np.int32)
    eye = np.eye(bs, dtype=np.int32)
    eye_packed = o.pack4(eye.reshape(-1))
    for row in range(n):
        for blk in range(nb):
            # one block of one weight row is a packed [depth=bs, cols=1] right operand
            c = o.ref_matmul_4bit(eye_packed, False, packed[row, blk], False, bs, 1, bs, [0], [zp_values[row, blk]])
            ints[row, blk * bs:(blk + 1) * bs] = c[:, 0]
    out["nbits_b"] = packed
    out["nbits_zp"] = zp
    out["nbits_geometry"] = np.array([n, k, bs], np.int64)
    out["nbits_ints"] = ints
    m = 3
    aq = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    codes = o.np_unpack_codes(packed, n, k, 4, bs).astype(np.uint8)
    dots = np.zeros((m, n, nb), np.int32)
    for blk in range(nb):
        b_block = np.ascontiguousarray(codes[:, blk * bs:(blk + 1) * bs].T)  # [depth, cols]
        dots[:, :, blk] = o.ref_matmul_8bit(np.ascontiguousarray(aq[:, blk * bs:(blk + 1) * bs]), True, b_block,
                                            False, m, n, bs, [0], zp_values[:, blk])
    out["nbits_aq"] = aq
    out["nbits_dots"] = dots

    values = np.array([0.0, -0.0, 1.0, 1.00390625, 1.0039062, 1.0117188, 3.1415927, -2.7182817, 65504.0,
                       1e-40, 3.3895314e38, np.inf, -np.inf, np.nan, 0.3333333, 255.5, 256.5], np.float32)
    out["bf16_in"] = values
    out["bf16_bits"] = np.array([o.ref_lib().ref_float_to_bf16_bits(float(v)) for v in values], np.uint16)
    target = Path(__file__).resolve().parent / "reference_pins.npz"
    np.savez_compressed(target, **out)
    print(target, target.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
