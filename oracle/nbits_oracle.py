"""TEST INFRASTRUCTURE ONLY. Python access to the CPU checker.

* ctypes binding of ``liboracle_nbits.so`` (the C++ restatement, matmul_nbits_oracle.cc)
* an independent numpy restatement of the same contract, used to cross-check the C++ one
* ctypes binding of ``_ref/libref_intgemm.so``: the reference's own integer GEMM compiled
  from its sources (IntegerMatMul4Bit2D / IntegerMatMul2D /  FloatToBFloat16Bits), present
  only where ``make -C oracle ref`` ran with the reference checkout available

PARITY STATUS: the reference has no MatMulNBits, so the operator-level semantics are PARITY
UNPINNED; nibble order, exact (q - zp) integers, exact int32 dots and bf16 rounding are
pinned against the reference functions above (tests/test_oracle_pins.py).
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_LIB = HERE / "liboracle_nbits.so"
REF_LIB = HERE / "_ref" / "libref_intgemm.so"

_oracle = None
_ref = None


def build(reference: bool = True) -> None:
    """Compiles the checker (and, when the reference checkout exists, oracle/_ref)."""
    targets = ["oracle"] + (["ref"] if reference else [])
    subprocess.run(["make", "-C", str(HERE), f"REFERENCE_ROOT={reference_root()}", *targets], check=True,
                   capture_output=True)


def lib() -> ctypes.CDLL:
    global _oracle
    if _oracle is None:
        if not ORACLE_LIB.exists():
            build(reference=False)
        _oracle = ctypes.CDLL(str(ORACLE_LIB))
        _oracle.nbits_oracle_bf16_bits_to_float.restype = ctypes.c_float
        _oracle.nbits_oracle_bf16_bits_to_float.argtypes = [ctypes.c_uint16]
        _oracle.nbits_oracle_float_to_bf16_bits.restype = ctypes.c_uint16
        _oracle.nbits_oracle_float_to_bf16_bits.argtypes = [ctypes.c_float]
    return _oracle


def ref_lib():
    """The reference's integer GEMM, or None when oracle/_ref was not built."""
    global _ref
    if _ref is None and REF_LIB.exists():
        _ref = ctypes.CDLL(str(REF_LIB))
        _ref.ref_float_to_bf16_bits.restype = ctypes.c_uint16
        _ref.ref_float_to_bf16_bits.argtypes = [ctypes.c_float]
    return _ref


def reference_root() -> Path:
    """The reference checkout: environment variable REFERENCE_ROOT, else ``reference`` beside the repository."""
    import os

    return Path(os.environ.get("REFERENCE_ROOT", HERE.parent.parent / "reference"))


def use_reference_execute_ranges(enable: bool = True) -> bool:
    """Routes the column panels of the threaded checker functions through the reference's own
    ``ExecuteRanges`` (onnx_light_cpu/impl/execution.h:146-176) with a persistent ``std::thread``
    executor injected through ``ExecutionExecutorScope`` - how the reference's CPU kernels get their
    threads. Needs oracle/_ref; returns whether it is in effect. ``enable=False`` goes back to the
    checker's own persistent worker pool."""
    setter = lib().nbits_oracle_set_range_runner
    setter.argtypes = [ctypes.c_void_p]
    setter.restype = None
    ref = ref_lib() if enable else None
    if ref is None or not hasattr(ref, "ref_execute_ranges"):
        setter(None)
        return False
    setter(ctypes.cast(ref.ref_execute_ranges, ctypes.c_void_p))
    return True


def reference_execute_ranges_calls() -> int:
    ref = ref_lib()
    if ref is None or not hasattr(ref, "ref_execute_ranges_calls"):
        return 0
    ref.ref_execute_ranges_calls.restype = ctypes.c_longlong
    return int(ref.ref_execute_ranges_calls())


def _p(x):
    return None if x is None else ctypes.c_void_p(x.ctypes.data)


def _c(x, dtype):
    return None if x is None else np.ascontiguousarray(x, dtype=dtype)


def hardware_threads() -> int:
    return int(lib().nbits_oracle_hardware_threads())


def dequant_int(b, zero_points, n, k, bits, block_size) -> np.ndarray:
    b, zp = _c(b, np.uint8), _c(zero_points, np.uint8)
    out = np.empty((n, k), dtype=np.int32)
    rc = lib().nbits_oracle_dequant_int(_p(b), _p(zp), ctypes.c_int64(n), ctypes.c_int64(k), bits, block_size, _p(out))
    assert rc == 0
    return out


def _matmul(fn_name, out_dtype, a, b, scales, zero_points, bias, n, k, bits, block_size, threads):
    a = _c(a, np.float32).reshape(-1, k)
    m = a.shape[0]
    b, scales = _c(b, np.uint8), _c(scales, np.float32)
    zp, bias = _c(zero_points, np.uint8), _c(bias, np.float32)
    y = np.empty((m, n), dtype=out_dtype)
    rc = getattr(lib(), fn_name)(_p(a), _p(b), _p(scales), _p(zp), _p(bias), ctypes.c_int64(m),
                                 ctypes.c_int64(n), ctypes.c_int64(k), bits, block_size, _p(y), threads)
    assert rc == 0, fn_name
    return y


def matmul_f32(a, b, scales, zero_points, bias, n, k, bits, block_size, threads=0):
    return _matmul("nbits_oracle_matmul_f32", np.float32, a, b, scales, zero_points, bias, n, k, bits,
                   block_size, threads or hardware_threads())


def matmul_f64(a, b, scales, zero_points, bias, n, k, bits, block_size, threads=0):
    return _matmul("nbits_oracle_matmul_f64", np.float64, a, b, scales, zero_points, bias, n, k, bits,
                   block_size, threads or hardware_threads())


def matmul_bf16(a, b, scales, zero_points, bias, n, k, bits, block_size, threads=0):
    return _matmul("nbits_oracle_matmul_bf16", np.float64, a, b, scales, zero_points, bias, n, k, bits,
                   block_size, threads or hardware_threads())


def matmul_int8(a, b, scales, zero_points, bias, n, k, bits, block_size, threads=0):
    return _matmul("nbits_oracle_matmul_int8", np.float32, a, b, scales, zero_points, bias, n, k, bits,
                   block_size, threads or hardware_threads())


def matmul_f32_fast(a, b, scales, zero_points, bias, n, k, bits, block_size, threads=0):
    return _matmul("nbits_oracle_matmul_f32_fast", np.float32, a, b, scales, zero_points, bias, n, k, bits,
                   block_size, threads or hardware_threads())


def quantize_a(a, k, block_size):
    a = _c(a, np.float32).reshape(-1, k)
    m = a.shape[0]
    n_blocks = -(-k // block_size)
    aq = np.empty((m, k), dtype=np.int8)
    sa = np.empty((m, n_blocks), dtype=np.float32)
    rc = lib().nbits_oracle_quantize_a(_p(a), ctypes.c_int64(m), ctypes.c_int64(k), block_size, _p(aq), _p(sa))
    assert rc == 0
    return aq, sa


def int8_block_dots(aq, b, zero_points, n, k, bits, block_size, threads=0):
    aq = _c(aq, np.int8).reshape(-1, k)
    m = aq.shape[0]
    b, zp = _c(b, np.uint8), _c(zero_points, np.uint8)
    n_blocks = -(-k // block_size)
    dots = np.empty((m, n, n_blocks), dtype=np.int32)
    rc = lib().nbits_oracle_int8_block_dots(_p(aq), _p(b), _p(zp), ctypes.c_int64(m), ctypes.c_int64(n),
                                            ctypes.c_int64(k), bits, block_size, _p(dots),
                                            threads or hardware_threads())
    assert rc == 0
    return dots


def float_to_bf16_bits(x: float) -> int:
    return int(lib().nbits_oracle_float_to_bf16_bits(ctypes.c_float(x)))


# ---- independent numpy restatement ---------------------------------------------------------

def np_unpack_codes(b, n, k, bits, block_size) -> np.ndarray:
    """Codes q[n, k] as int32. Element 2i of a 4-bit blob is the low nibble of byte i."""
    n_blocks = -(-k // block_size)
    blob = np.asarray(b, dtype=np.uint8).reshape(n, n_blocks, block_size * bits // 8)
    if bits == 8:
        codes = blob.astype(np.int32)
    else:
        codes = np.empty((n, n_blocks, block_size), dtype=np.int32)
        codes[:, :, 0::2] = blob & 0x0F
        codes[:, :, 1::2] = blob >> 4
    return codes.reshape(n, n_blocks * block_size)[:, :k]


def np_zero_points(zero_points, n, k, bits, block_size) -> np.ndarray:
    n_blocks = -(-k // block_size)
    if zero_points is None:
        return np.full((n, n_blocks), 1 << (bits - 1), dtype=np.int32)
    z = np.asarray(zero_points, dtype=np.uint8).reshape(n, -1)
    if bits == 8:
        return z[:, :n_blocks].astype(np.int32)
    out = np.empty((n, z.shape[1] * 2), dtype=np.int32)
    out[:, 0::2] = z & 0x0F
    out[:, 1::2] = z >> 4
    return out[:, :n_blocks]


def np_dequant_int(b, zero_points, n, k, bits, block_size) -> np.ndarray:
    codes = np_unpack_codes(b, n, k, bits, block_size)
    zp = np_zero_points(zero_points, n, k, bits, block_size)
    return codes - np.repeat(zp, block_size, axis=1)[:, :k]


def np_matmul_f64(a, b, scales, zero_points, bias, n, k, bits, block_size) -> np.ndarray:
    n_blocks = -(-k // block_size)
    ints = np_dequant_int(b, zero_points, n, k, bits, block_size).astype(np.float64)
    s = np.repeat(np.asarray(scales, dtype=np.float32).reshape(n, n_blocks).astype(np.float64), block_size, axis=1)[:, :k]
    y = np.asarray(a, dtype=np.float32).reshape(-1, k).astype(np.float64) @ (ints * s).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32).astype(np.float64)[None, :]
    return y


# ---- reference functions (oracle/_ref) -------------------------------------------------------

def ref_matmul_4bit(a_packed, a_signed, b_packed, b_signed, rows, cols, depth, a_zp, b_zp) -> np.ndarray:
    """IntegerMatMul4Bit2D from the reference build. A [rows, depth], B [depth, cols] packed."""
    r = ref_lib()
    a_packed, b_packed = _c(a_packed, np.uint8), _c(b_packed, np.uint8)
    a_zp, b_zp = _c(a_zp, np.int32), _c(b_zp, np.int32)
    c = np.zeros((rows, cols), dtype=np.int32)
    r.ref_integer_matmul_4bit_2d(_p(a_packed), int(a_signed), _p(b_packed), int(b_signed), _p(c),
                                 ctypes.c_int64(rows), ctypes.c_int64(cols), ctypes.c_int64(depth),
                                 _p(a_zp), ctypes.c_int64(a_zp.size), _p(b_zp), ctypes.c_int64(b_zp.size))
    return c


def ref_matmul_8bit(a, a_signed, b, b_signed, rows, cols, depth, a_zp, b_zp) -> np.ndarray:
    """IntegerMatMul2D from the reference build. A [rows, depth] bytes, B [depth, cols] bytes."""
    r = ref_lib()
    a = np.ascontiguousarray(a).view(np.uint8)
    b = np.ascontiguousarray(b).view(np.uint8)
    a_zp, b_zp = _c(a_zp, np.int32), _c(b_zp, np.int32)
    c = np.zeros((rows, cols), dtype=np.int32)
    r.ref_integer_matmul_2d(_p(a), int(a_signed), _p(b), int(b_signed), _p(c), ctypes.c_int64(rows),
                            ctypes.c_int64(cols), ctypes.c_int64(depth), _p(a_zp),
                            ctypes.c_int64(a_zp.size), _p(b_zp), ctypes.c_int64(b_zp.size))
    return c


def pack4(values) -> np.ndarray:
    """Packs logical 4-bit values: even index -> low nibble, odd -> high nibble, pad 0."""
    v = np.asarray(values, dtype=np.int64).reshape(-1) & 0x0F
    if v.size % 2:
        v = np.concatenate([v, [0]])
    return (v[0::2] | (v[1::2] << 4)).astype(np.uint8)
