"""Front door for DequantizeLinear (blocked) -> MatMul: operand conversion against the CPU checker
(no GPU), and the converted node on the GPU against a float64 evaluation of the original pair."""

import numpy as np
import pytest

import onnx_light_cpu_b200 as pkg
from onnx_light_cpu_b200 import qdq
from oracle import nbits_oracle as o


def _pair(k, n, bs, bits, signed, with_zp, seed):
    rng = np.random.default_rng(seed)
    nb = -(-k // bs)
    lo, hi = (-(1 << (bits - 1)), (1 << (bits - 1))) if signed else (0, 1 << bits)
    w_q = rng.integers(lo, hi, size=(k, n))
    scale = (np.abs(rng.normal(0.0, 0.02, size=(nb, n))) + 1e-4).astype(np.float32)
    zp = rng.integers(lo, hi, size=(nb, n)) if with_zp else None
    return w_q, scale, zp


def _dequantize(w_q, scale, zp, bs):
    """DequantizeLinear with axis=0 and block_size=bs, in float64."""
    k = w_q.shape[0]
    block = np.arange(k) // bs
    z = 0 if zp is None else zp[block].astype(np.float64)
    return (w_q.astype(np.float64) - z) * scale[block].astype(np.float64)


@pytest.mark.parametrize("k,n,bs,bits,signed,with_zp", [
    (64, 5, 16, 4, False, True),
    (96, 7, 32, 4, True, True),      # INT4 codes and zero points; three blocks: padded zero-point nibble
    (80, 3, 32, 4, False, False),    # K not a multiple of the block; ONNX default zero point 0
    (64, 4, 32, 4, True, False),     # signed, no zero point: becomes the operator's default 8
    (48, 6, 16, 8, False, True),
    (40, 2, 32, 8, True, False),
])
def test_converted_operands_match_the_pair(k, n, bs, bits, signed, with_zp):
    w_q, scale, zp = _pair(k, n, bs, bits, signed, with_zp, seed=k + n + bs + bits)
    ops = qdq.qdq_to_matmulnbits(w_q, scale, zp, block_size=bs, bits=bits, signed=signed)
    nb = -(-k // bs)
    assert ops["b"].shape == (n, nb, bs * bits // 8) and ops["scales"].shape == (n * nb,)
    if signed and not with_zp:
        assert ops["zero_points"] is None
    rng = np.random.default_rng(1)
    a = rng.normal(size=(3, k)).astype(np.float32)
    y = o.matmul_f64(a, ops["b"], ops["scales"], ops["zero_points"], None, n, k, bits, bs)
    ref = a.astype(np.float64) @ _dequantize(w_q, scale, zp, bs)
    assert np.abs(y - ref).max() <= 1e-12 * max(np.abs(ref).max(), 1.0)
    # the integer part, bit for bit
    ints = o.dequant_int(ops["b"], ops["zero_points"], n, k, bits, bs)
    expect = (w_q - (0 if zp is None else zp[np.arange(k) // bs])).T
    assert np.array_equal(ints[:, :k], expect)


def test_unpack_int4_follows_the_onnx_packing():
    packed = np.array([0x21, 0xF3, 0x08], dtype=np.uint8)      # elements 1, 2, 3, 15, 8, (unused 0)
    assert unpack(packed, (5,), False) == [1, 2, 3, 15, 8]
    assert unpack(packed, (5,), True) == [1, 2, 3, -1, -8]
    with pytest.raises(ValueError):
        qdq.unpack_int4(packed, (8,))


def unpack(packed, shape, signed):
    return qdq.unpack_int4(packed, shape, signed).tolist()


def test_rejects_bad_shapes_and_ranges():
    w_q, scale, zp = _pair(64, 4, 32, 4, False, True, seed=3)
    with pytest.raises(ValueError):
        qdq.qdq_to_matmulnbits(w_q, scale[:1], zp, block_size=32)
    with pytest.raises(ValueError):
        qdq.qdq_to_matmulnbits(w_q + 16, scale, zp, block_size=32)
    with pytest.raises(ValueError):
        qdq.qdq_to_matmulnbits(w_q, scale, zp, block_size=24)


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n,bs,signed,with_zp", [(1, 4096, 256, 128, False, True), (16, 4096, 128, 32, True, True),
                                                     (3, 2048, 77, 64, True, False)])
def test_pair_runs_on_the_matmulnbits_kernels(cuda_device, m, k, n, bs, signed, with_zp):
    w_q, scale, zp = _pair(k, n, bs, 4, signed, with_zp, seed=m + k + n + bs)
    rng = np.random.default_rng(5)
    a = rng.normal(size=(m, k)).astype(np.float32)
    bias = rng.normal(0.0, 0.1, size=n).astype(np.float32)
    pkg.register_kernels()
    session = qdq.QdqMatMulSession(w_q, scale, zp, bias, block_size=bs, signed=signed)
    y = session.run(a)
    ref = a.astype(np.float64) @ _dequantize(w_q, scale, zp, bs) + bias
    assert np.abs(y - ref).max() / np.abs(ref).max() <= 1e-5
    assert session.last_device_kernel.startswith("nbits_")
    session.close()
