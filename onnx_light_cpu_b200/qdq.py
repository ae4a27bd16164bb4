"""Front door for the standard-ONNX spelling of a weight-only quantized projection.

The reference's roadmap treats ``DequantizeLinear`` (blocked, 4-bit or 8-bit constant weight)
followed by ``MatMul`` as the contract of a quantized projection and ``com.microsoft.MatMulNBits``
as one way of spelling it (onnx_light_cpu docs/next_steps/2026/2026_08_qwen3_inference.rst:87-101,
262). This module turns the operands of such a pair into MatMulNBits operands once, at load time,
so that the pair runs on the same CUDA kernels:

    W_q   [K, N]            codes, blocked along axis 0 (the K axis of ``MatMul(A, W)``)
    scale [ceil(K/bs), N]   one scale per (block, column)
    zp    [ceil(K/bs), N]   optional zero points, same type as the codes

    B      [N, ceil(K/bs), bs * bits / 8]   column-major over K, two 4-bit codes per byte, low first
    scales [N * ceil(K/bs)]
    zero_points [N, ceil(ceil(K/bs) * bits / 8)]

Signed codes (INT4 / INT8) become unsigned by adding 2^(bits-1) to codes and zero points alike:
``q - zp`` is unchanged. Packed 4-bit ONNX tensors hold element 2i in the low nibble of byte i of
the row-major flattened tensor; :func:`unpack_int4` undoes that.
"""

from __future__ import annotations

import numpy as np

__all__ = ["QdqMatMulSession", "qdq_to_matmulnbits", "unpack_int4"]


def unpack_int4(packed: np.ndarray, shape: tuple[int, ...], signed: bool = False) -> np.ndarray:
    """Codes of a packed 4-bit ONNX tensor of logical ``shape`` (row-major, element 2i in the low
    nibble of byte i; an unused final high nibble is ignored). Returns int16 values: 0..15, or
    -8..7 for ``signed``."""
    count = int(np.prod(shape))
    raw = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
    if raw.size != (count + 1) // 2:
        raise ValueError(f"a packed 4-bit tensor of shape {shape} has {(count + 1) // 2} bytes, got {raw.size}")
    codes = np.empty(raw.size * 2, dtype=np.int16)
    codes[0::2] = raw & 0x0F
    codes[1::2] = raw >> 4
    codes = codes[:count]
    if signed:
        codes = np.where(codes >= 8, codes - 16, codes).astype(np.int16)
    return codes.reshape(shape)


def _pack_low_first(codes: np.ndarray) -> np.ndarray:
    """Packs the last axis (even length) two 4-bit codes per byte, even index in the low nibble."""
    codes = codes.astype(np.uint8)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def qdq_to_matmulnbits(w_q: np.ndarray, scale: np.ndarray, zero_point: np.ndarray | None = None, *,
                       block_size: int, bits: int = 4, signed: bool = False) -> dict:
    """MatMulNBits operands of ``MatMul(A, DequantizeLinear(w_q, scale, zero_point, axis=0,
    block_size=block_size))``.

    ``w_q``: integer codes ``[K, N]``, one per element (see :func:`unpack_int4` for packed 4-bit
    tensors), unsigned ``0 .. 2^bits - 1`` or, with ``signed``, ``-2^(bits-1) .. 2^(bits-1) - 1``.
    ``scale``: ``[ceil(K / block_size), N]``. ``zero_point``: same shape and signedness as the codes,
    or None (ONNX default 0; for unsigned codes that is NOT MatMulNBits' default of 2^(bits-1), so a
    zero-point tensor is always produced then).

    Returns a dict with ``b``, ``scales``, ``zero_points`` (or None), ``K``, ``N``, ``bits``,
    ``block_size``: keyword arguments of ``MatMulNBitsSession`` / ``MatMulNBitsWeights``.
    """
    if bits not in (4, 8):
        raise ValueError("MatMulNBits takes bits = 4 or 8")
    if block_size < 16 or (block_size & (block_size - 1)) != 0:
        raise ValueError("MatMulNBits takes a power-of-two block_size >= 16")
    w_q = np.asarray(w_q)
    if w_q.ndim != 2:
        raise ValueError("w_q must be [K, N]")
    k, n = w_q.shape
    n_blocks = -(-k // block_size)
    scale = np.asarray(scale, dtype=np.float32)
    if scale.shape != (n_blocks, n):
        raise ValueError(f"scale must be [{n_blocks}, {n}] for K={k}, block_size={block_size}; got {scale.shape}")
    half = 1 << (bits - 1)
    top = (1 << bits) - 1
    codes = w_q.astype(np.int32) + (half if signed else 0)
    if codes.min(initial=0) < 0 or codes.max(initial=0) > top:
        raise ValueError(f"codes outside the {bits}-bit range")
    if zero_point is None:
        zp = np.full((n_blocks, n), half if signed else 0, dtype=np.int32)
    else:
        zp = np.asarray(zero_point).astype(np.int32) + (half if signed else 0)
        if zp.shape != (n_blocks, n):
            raise ValueError(f"zero_point must be [{n_blocks}, {n}]; got {zp.shape}")
        if zp.min(initial=0) < 0 or zp.max(initial=0) > top:
            raise ValueError(f"zero points outside the {bits}-bit range")
    # K axis padded to whole blocks (the operator ignores codes beyond K), then column-major over K
    padded = np.zeros((n_blocks * block_size, n), dtype=np.uint8)
    padded[:k] = codes
    by_column = np.ascontiguousarray(padded.T).reshape(n, n_blocks, block_size)
    b = _pack_low_first(by_column) if bits == 4 else by_column
    zp_rows = np.ascontiguousarray(zp.T).astype(np.uint8)        # [N, n_blocks]
    if np.all(zp_rows == half):
        zero_points = None                                       # the operator's default
    elif bits == 4:
        if n_blocks % 2:
            zp_rows = np.concatenate([zp_rows, np.zeros((n, 1), dtype=np.uint8)], axis=1)
        zero_points = _pack_low_first(zp_rows)
    else:
        zero_points = zp_rows
    return {"b": np.ascontiguousarray(b), "scales": np.ascontiguousarray(scale.T).reshape(-1),
            "zero_points": zero_points, "K": int(k), "N": int(n), "bits": int(bits), "block_size": int(block_size)}


class QdqMatMulSession:
    """``Y = MatMul(A, DequantizeLinear(w_q, scale, zero_point, axis=0, block_size))`` (+ ``bias``)
    through the registered MatMulNBits kernel (``register_kernels()`` first, as for
    ``MatMulNBitsSession``): the operands are converted once, here."""

    def __init__(self, w_q, scale, zero_point=None, bias=None, *, block_size, bits=4, signed=False,
                 accuracy_level=0):
        from .matmul_nbits import MatMulNBitsSession

        ops = qdq_to_matmulnbits(w_q, scale, zero_point, block_size=block_size, bits=bits, signed=signed)
        self.operands = ops
        self._session = MatMulNBitsSession(ops["b"], ops["scales"], ops["zero_points"], bias, K=ops["K"], N=ops["N"],
                                           bits=ops["bits"], block_size=ops["block_size"],
                                           accuracy_level=accuracy_level)

    def run(self, a: np.ndarray) -> np.ndarray:
        return self._session.run(a)

    @property
    def last_device_kernel(self) -> str:
        return self._session.last_device_kernel

    def close(self) -> None:
        self._session.close()
