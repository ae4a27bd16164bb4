"""ctypes binding of the C ABI declared in ``include/matmulnbits_b200.h``.

The product path is the CUDA library: importing this module without the built
``libmatmulnbits_b200.so`` raises, and there is no CPU fallback behind any function here.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import os

PACKAGE_DIR = Path(__file__).resolve().parent
# MNB_LIBRARY_PATH selects another build of the same C ABI (e.g. an instrumented one).
CUDA_LIB_PATH = Path(os.environ.get("MNB_LIBRARY_PATH", PACKAGE_DIR / "libmatmulnbits_b200.so"))

MNB_OK = 0
MNB_ERR_INVALID_ARGUMENT = 1
MNB_ERR_CUDA = 2
MNB_ERR_UNSUPPORTED = 3
MNB_ERR_DEVICE_TIMEOUT = 4

PATH_AUTO = 0
PATH_GEMV = 1
PATH_TCGEN05 = 2
PATH_INT8 = 3
PATH_GEMV_MMA = 4
PATH_TCGEN05_WIDE = 5
PATH_INT8_MMA = 6
PATH_GEMV_MMA_MULTI = 7
PATH_GEMV_IMMA = 8
PATH_GEMV_DIGITS = 9
PATH_GEMV_DIRECT = 10
PATH_GEMV_RESIDENT = 11
IPC_HANDLE_BYTES = 64
MAX_GATHER_RANKS = 8

# every symbol include/matmulnbits_b200.h declares
EXPORTED_SYMBOLS = (
    "mnb_last_error",
    "mnb_device_count",
    "mnb_version",
    "mnb_weights_create",
    "mnb_weights_wrap_device",
    "mnb_weights_destroy",
    "mnb_algorithmic_bytes",
    "mnb_matmul_host",
    "mnb_matmul_device",
    "mnb_matmul_device_strided",
    "mnb_matmul_device_group",
    "mnb_peer_buffer_create",
    "mnb_peer_buffer_open",
    "mnb_peer_buffer_close",
    "mnb_peer_buffer_destroy",
    "mnb_matmul_device_gather",
    "mnb_matmul_device_gather_ex",
    "mnb_gather_wait",
    "mnb_weights_poll_status",
    "mnb_dequant_int_device",
    "mnb_quantize_a_device",
    "mnb_int8_block_dots_device",
    "mnb_int8_mma_block_dots_device",
    "mnb_matmul_int8_static",
    "mnb_launch_count",
    "mnb_last_kernel",
    "mnb_weights_n",
    "mnb_weights_k",
    "mnb_weights_bits",
    "mnb_weights_block_size",
)

_lib = None


class MatMulNBitsError(RuntimeError):
    """A C ABI call failed; ``status`` is the mnb_status code."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def load() -> ctypes.CDLL:
    """Loads the CUDA library (building nothing). Raises OSError when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not CUDA_LIB_PATH.exists():
        raise OSError(
            f"{CUDA_LIB_PATH} is missing: build it with `python -m onnx_light_cpu_b200.build` "
            "(there is no CPU fallback)"
        )
    lib = ctypes.CDLL(str(CUDA_LIB_PATH), mode=ctypes.RTLD_GLOBAL)
    c = ctypes
    vp, i64, i32 = c.c_void_p, c.c_int64, c.c_int
    lib.mnb_last_error.restype = c.c_char_p
    lib.mnb_version.restype = c.c_char_p
    lib.mnb_last_kernel.restype = c.c_char_p
    lib.mnb_device_count.argtypes = [c.POINTER(i32)]
    lib.mnb_weights_create.argtypes = [i32, vp, vp, vp, vp, i64, i64, i32, i32, c.POINTER(vp)]
    lib.mnb_weights_wrap_device.argtypes = [i32, vp, vp, vp, vp, i64, i64, i32, i32, c.POINTER(vp)]
    lib.mnb_weights_destroy.argtypes = [vp]
    lib.mnb_algorithmic_bytes.argtypes = [i64, i64, i64, i32, i32, i32, i32]
    lib.mnb_algorithmic_bytes.restype = i64
    lib.mnb_matmul_host.argtypes = [vp, vp, i64, i32, i32, vp]
    lib.mnb_matmul_device.argtypes = [vp, vp, i64, i32, i32, vp, vp]
    lib.mnb_matmul_device_strided.argtypes = [vp, vp, i64, i32, i32, vp, i64, i64, vp]
    lib.mnb_matmul_device_group.argtypes = [c.POINTER(vp), i32, vp, i64, i32, c.POINTER(vp), vp]
    lib.mnb_peer_buffer_create.argtypes = [i32, c.c_size_t, c.POINTER(vp), vp]
    lib.mnb_peer_buffer_open.argtypes = [i32, vp, c.POINTER(vp)]
    lib.mnb_peer_buffer_close.argtypes = [i32, vp]
    lib.mnb_peer_buffer_destroy.argtypes = [i32, vp]
    lib.mnb_matmul_device_gather.argtypes = [vp, vp, i64, c.POINTER(vp), c.POINTER(vp), i32, i32, i64, i64, i32, vp]
    lib.mnb_matmul_device_gather_ex.argtypes = [vp, vp, i64, i32, c.POINTER(vp), c.POINTER(vp), i32, i32, i64, i64, i32,
                                                i32, vp]
    lib.mnb_gather_wait.argtypes = [vp, c.POINTER(vp), c.POINTER(i32), i32, i32, vp]
    lib.mnb_weights_poll_status.argtypes = [vp, c.POINTER(i32)]
    lib.mnb_dequant_int_device.argtypes = [vp, vp, vp]
    lib.mnb_quantize_a_device.argtypes = [vp, i64, i64, i32, vp, vp, vp]
    lib.mnb_int8_block_dots_device.argtypes = [vp, vp, i64, vp, vp]
    lib.mnb_int8_mma_block_dots_device.argtypes = [vp, vp, i64, vp, vp, vp]
    lib.mnb_matmul_int8_static.argtypes = [vp, vp, i64, vp, vp]
    lib.mnb_launch_count.restype = i64
    for name in ("mnb_weights_n", "mnb_weights_k"):
        getattr(lib, name).argtypes = [vp]
        getattr(lib, name).restype = i64
    for name in ("mnb_weights_bits", "mnb_weights_block_size"):
        getattr(lib, name).argtypes = [vp]
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != MNB_OK:
        raise MatMulNBitsError(status, load().mnb_last_error().decode())


def device_count() -> int:
    count = ctypes.c_int(0)
    check(load().mnb_device_count(ctypes.byref(count)))
    return count.value


def algorithmic_bytes(m, n, k, bits, block_size, has_zero_points, has_bias) -> int:
    return int(load().mnb_algorithmic_bytes(m, n, k, bits, block_size, int(has_zero_points), int(has_bias)))


def launch_count() -> int:
    return int(load().mnb_launch_count())


def last_kernel() -> str:
    return load().mnb_last_kernel().decode()
