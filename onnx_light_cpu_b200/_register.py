"""Python facade over the C++ registration layer.

Same functions as the reference's ``onnx_light_cpu._register``
(``register_kernels`` :63, ``registered_kernels`` :106, ``registered_kernel_names`` :142,
``used_kernel_names`` :157, ``clear_used_kernel_names`` :173), bound with ctypes to
``libonnx_light_cuda_kernels.so`` instead of a nanobind module.
"""

from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any

PACKAGE_DIR = Path(__file__).resolve().parent
HOST_LIB_PATH = PACKAGE_DIR / "libonnx_light_cuda_kernels.so"

_host = None


@dataclass(frozen=True)
class RegisteredKernel:
    """Immutable record describing one kernel registration of this library."""

    domain: str
    op_type: str
    device: str
    kernel_name: str
    types: tuple[int, ...]
    since_version: int | None
    until_version: int | None


def _host_lib() -> ctypes.CDLL:
    global _host
    if _host is not None:
        return _host
    if not HOST_LIB_PATH.exists():
        raise OSError(f"{HOST_LIB_PATH} is missing: build it with `python -m onnx_light_cpu_b200.build`")
    from . import _capi

    _capi.load()  # the kernels library links against the CUDA library
    lib = ctypes.CDLL(str(HOST_LIB_PATH))
    c = ctypes
    lib.olc_last_error.restype = c.c_char_p
    lib.olc_registered_kernels_json.restype = c.c_char_p
    lib.olc_used_kernel_names_json.restype = c.c_char_p
    lib.olc_dispatch_table_has.argtypes = [c.c_char_p]
    lib.olc_set_kernel_usage_recording.argtypes = [c.c_int]
    lib.olc_set_device.argtypes = [c.c_int]
    lib.olc_session_create.restype = c.c_void_p
    lib.olc_session_create.argtypes = [
        c.c_void_p, c.c_int64, c.c_void_p, c.c_int64, c.c_void_p, c.c_int64, c.c_void_p, c.c_int64,
        c.c_int64, c.c_int64, c.c_int64, c.c_int64, c.c_int64, c.c_int,
    ]
    lib.olc_session_run.argtypes = [c.c_void_p, c.c_void_p, c.POINTER(c.c_int64), c.c_int, c.c_void_p, c.c_int64]
    lib.olc_session_last_device_kernel.argtypes = [c.c_void_p]
    lib.olc_session_last_device_kernel.restype = c.c_char_p
    lib.olc_session_destroy.argtypes = [c.c_void_p]
    lib.olc_session_overwrite_b.argtypes = [c.c_void_p, c.c_void_p, c.c_int64]
    i64p, u64p = c.POINTER(c.c_int64), c.POINTER(c.c_uint64)
    lib.olc_peer_gather_layout.argtypes = [c.c_int, c.c_int, c.c_int64, c.c_int64, c.c_int, i64p]
    lib.olc_peer_gather_tables.argtypes = [c.c_int, c.c_int, c.c_int64, c.c_int64, c.c_int, c.c_int, u64p, u64p, u64p]
    lib.olc_shard_bounds.argtypes = [c.c_int64, c.c_int, c.c_int, i64p, i64p]
    lib.olc_peer_gather_create.restype = c.c_void_p
    lib.olc_peer_gather_create.argtypes = [c.c_int, c.c_int, c.c_int64, c.c_int64, c.c_int, c.c_int, c.c_void_p]
    lib.olc_peer_gather_open.argtypes = [c.c_void_p, c.c_void_p]
    lib.olc_peer_gather_result.restype = c.c_void_p
    lib.olc_peer_gather_result.argtypes = [c.c_void_p, c.c_int]
    lib.olc_peer_gather_run.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int64, c.c_int, c.c_int, c.c_int,
                                        c.c_void_p]
    lib.olc_peer_gather_wait.argtypes = [c.c_void_p, c.c_void_p, c.POINTER(c.c_int), c.c_int, c.c_void_p]
    lib.olc_peer_gather_close_peers.argtypes = [c.c_void_p]
    lib.olc_peer_gather_destroy.argtypes = [c.c_void_p]
    _host = lib
    return lib


def _raise_last(code: int) -> None:
    message = _host_lib().olc_last_error().decode()
    if code == 1:
        raise ValueError(message)  # std::invalid_argument
    raise RuntimeError(message)


def register_kernels(sess: Any = None) -> Any:
    """Registers this library's kernels (``com.microsoft.MatMulNBits``) into the process-wide
    kernel dispatch table. Idempotent. ``sess`` is returned unchanged so calls can be chained."""
    code = _host_lib().olc_register_all_kernels()
    if code != 0:
        _raise_last(code)
    return sess


def registered_kernels() -> tuple[RegisteredKernel, ...]:
    """One record per registration, sorted by (domain, op_type, device, kernel_name). Does not
    touch the dispatch table."""
    text = _host_lib().olc_registered_kernels_json()
    if text is None:
        _raise_last(2)
    return tuple(
        RegisteredKernel(
            domain=item["domain"],
            op_type=item["op_type"],
            device=item["device"],
            kernel_name=item["kernel_name"],
            types=tuple(item["types"]),
            since_version=item["since_version"],
            until_version=item["until_version"],
        )
        for item in json.loads(text.decode())
    )


def registered_kernel_names() -> dict[str, str]:
    """``{op_type: kernel name}`` for every kernel of this library."""
    return {record.op_type: record.kernel_name for record in registered_kernels()}


def used_kernel_names() -> list[str]:
    """Kernel class names that ran since the last clear, in invocation order."""
    return list(json.loads(_host_lib().olc_used_kernel_names_json().decode()))


def clear_used_kernel_names() -> None:
    _host_lib().olc_clear_used_kernel_names()


def set_kernel_usage_recording(enabled: bool) -> None:
    """Switches the usage log off for timing runs; dispatch is unchanged."""
    _host_lib().olc_set_kernel_usage_recording(1 if enabled else 0)
